"""Typed configuration of the Figalix decoder, read from its own config.json keys.

config.json gives every size and every constant that differs between models of the design:

    architecture "Figalix"; vocab, width; norm.eps; residual_mult; logit_softcap (optional)
    layers[i]: type "parallel":  mixer.left  {heads, kv_heads, dim, vdim, scale, mask {size, keep_first} (optional),
                                              rot {dims, base, scaling {factor, original, fast, slow} (optional)}}
                                 mixer.right {heads, dim, vdim, gate_cap}
               type "mamba2":    mixer {heads, vdim, state, groups, conv, norm_groups}
               mlp null | {kind "dense", ff} | {kind "moe", expert.ff, router {experts, top}, shared.ff (optional)}

What the design fixes (activation functions, where norms sit, how rotated pairs lie, the 1e-6 of the matrix memory's
denominator) is in the parts and in the builder.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Dict, List, Optional

from .errors import InvalidValue, MissingKey
from .rifizen import _get


@dataclass
class KeptWindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    keep_first: int
    rot_dims: int
    rot_base: Optional[float]
    rot_scaling: Optional[Dict[str, float]]


@dataclass
class MatrixMemoryConfig:
    heads: int
    dim: int
    vdim: int
    gate_cap: Optional[float]


@dataclass
class ParallelMixerConfig:
    left: KeptWindowAttentionConfig
    right: MatrixMemoryConfig


@dataclass
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int


@dataclass
class FigalixMlp:
    kind: str                      # "dense" | "moe"
    ff: int                        # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0
    shared_ff: Optional[int] = None


@dataclass
class FigalixLayer:
    type: str                      # "parallel" | "mamba2"
    mixer: object
    mlp: Optional[FigalixMlp]


@dataclass
class FigalixConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    residual_mult: float
    logit_softcap: Optional[float]
    layers: List[FigalixLayer]
    raw: dict = field(default_factory=dict, repr=False)

    ARCHITECTURE = "Figalix"

    @classmethod
    def from_dict(cls, raw: dict) -> "FigalixConfig":
        layers_raw = raw.get("layers")
        if layers_raw is None:
            raise MissingKey("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise InvalidValue("layers", layers_raw, "must be a non-empty list")
        layers: List[FigalixLayer] = []
        for i, L in enumerate(layers_raw):
            p = f"layers[{i}]"
            if not isinstance(L, dict):
                raise InvalidValue(p, L, "must be an object")
            kind = L.get("type")

            def g(path, k, L=L, p=p, **kw):
                return _get(L, path, k, where=p + ".", **kw)
            if kind == "parallel":
                mixer = ParallelMixerConfig(cls._left(L, g, p), cls._right(g, p))
            elif kind == "mamba2":
                mixer = StateSpaceConfig(heads=g("mixer.heads", int, minimum=1), vdim=g("mixer.vdim", int, minimum=1),
                                         state=g("mixer.state", int, minimum=1), groups=g("mixer.groups", int, minimum=1),
                                         taps=g("mixer.conv", int, minimum=1),
                                         norm_groups=g("mixer.norm_groups", int, optional=True, minimum=1) or 1)
                if mixer.heads % mixer.groups:
                    raise InvalidValue(f"{p}.mixer.groups", mixer.groups, f"must divide heads = {mixer.heads}")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise InvalidValue(f"{p}.mixer.norm_groups", mixer.norm_groups,
                                       f"must divide heads * vdim = {mixer.heads * mixer.vdim}")
                if mixer.taps > 16:
                    raise InvalidValue(f"{p}.mixer.conv", mixer.taps, "the convolution kernel takes up to 16 taps")
                if mixer.state > 256:
                    raise InvalidValue(f"{p}.mixer.state", mixer.state, "the recurrence kernel holds at most 256 rows of a state column")
            else:
                raise InvalidValue(f"{p}.type", kind, "this design has layers of type 'parallel' and 'mamba2'")
            layers.append(FigalixLayer(kind, mixer, cls._mlp(L, g, p)))
        return cls(architecture=str(raw.get("architecture") or cls.ARCHITECTURE),
                   vocab=_get(raw, "vocab", int, minimum=1), width=_get(raw, "width", int, minimum=1),
                   eps=_get(raw, "norm.eps", float, positive=True),
                   residual_mult=cls._or(_get(raw, "residual_mult", float, optional=True), 1.0),
                   logit_softcap=_get(raw, "logit_softcap", float, optional=True, positive=True),
                   layers=layers, raw=copy.deepcopy(raw))

    @staticmethod
    def _or(value, default):
        return default if value is None else value

    @staticmethod
    def _left(L, g, p) -> KeptWindowAttentionConfig:
        m = L.get("mixer", {}).get("left", {}) if isinstance(L.get("mixer"), dict) else {}
        rot = (m.get("rot") or {}) if isinstance(m, dict) else {}
        scaling = rot.get("scaling")
        if scaling is not None:
            scaling = {k: g(f"mixer.left.rot.scaling.{k}", float, positive=True) for k in ("factor", "original", "fast", "slow")}
        rot_dims = g("mixer.left.rot.dims", int, optional=True, minimum=0) or 0
        a = KeptWindowAttentionConfig(
            heads=g("mixer.left.heads", int, minimum=1), kv_heads=g("mixer.left.kv_heads", int, minimum=1),
            dim=g("mixer.left.dim", int, minimum=1), vdim=g("mixer.left.vdim", int, minimum=1),
            scale=g("mixer.left.scale", float, positive=True),
            window=g("mixer.left.mask.size", int, optional=True, minimum=1),
            keep_first=g("mixer.left.mask.keep_first", int, optional=True, minimum=0) or 0,
            rot_dims=rot_dims, rot_base=g("mixer.left.rot.base", float, positive=True) if rot_dims else None,
            rot_scaling=scaling if rot_dims else None)
        if a.heads % a.kv_heads:
            raise InvalidValue(f"{p}.mixer.left.kv_heads", a.kv_heads, f"must divide heads = {a.heads}")
        if a.rot_dims % 2 or a.rot_dims > a.dim:
            raise InvalidValue(f"{p}.mixer.left.rot.dims", a.rot_dims, f"must be even and at most dim = {a.dim}")
        if a.rot_dims and not a.rot_base > 1:
            raise InvalidValue(f"{p}.mixer.left.rot.base", a.rot_base, "must be larger than 1")
        return a

    @staticmethod
    def _right(g, p) -> MatrixMemoryConfig:
        r = MatrixMemoryConfig(heads=g("mixer.right.heads", int, minimum=1), dim=g("mixer.right.dim", int, minimum=1),
                               vdim=g("mixer.right.vdim", int, minimum=1),
                               gate_cap=g("mixer.right.gate_cap", float, optional=True, positive=True))
        if r.dim > 256:
            raise InvalidValue(f"{p}.mixer.right.dim", r.dim, "the recurrence kernel holds at most 256 rows of a state column")
        return r

    @staticmethod
    def _mlp(L, g, p) -> Optional[FigalixMlp]:
        mlp_raw = L.get("mlp")
        if mlp_raw is None:
            return None
        mk = mlp_raw.get("kind") if isinstance(mlp_raw, dict) else None
        if mk == "dense":
            return FigalixMlp("dense", g("mlp.ff", int, minimum=1))
        if mk != "moe":
            raise InvalidValue(f"{p}.mlp.kind", mk, "must be 'dense' or 'moe' (or mlp null)")
        mlp = FigalixMlp("moe", g("mlp.expert.ff", int, minimum=1), g("mlp.router.experts", int, minimum=1),
                         g("mlp.router.top", int, minimum=1), g("mlp.shared.ff", int, optional=True, minimum=1))
        if mlp.top > mlp.experts:
            raise InvalidValue(f"{p}.mlp.router.top", mlp.top, f"there are only {mlp.experts} experts")
        if mlp.top > 16 or mlp.experts > 1024:
            raise InvalidValue(f"{p}.mlp.router", mlp_raw.get("router"), "the routing kernels take up to 16 of up to 1024 experts")
        return mlp

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)
