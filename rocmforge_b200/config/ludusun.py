"""Typed configuration of the Ludusun decoder, read from its own config.json keys.

config.json gives every size and every constant that differs between models of the design:

    architecture "Ludusun"; vocab, width; norm.eps; embedding.scale; logit_softcap (optional)
    layers[i]: type "attention":         mixer {heads, kv_heads, dim, vdim, scale, rot {dims, base, scaling {factor,
                                         original, fast, slow} (optional)}, kv_from (optional: the layer whose keys and
                                         values this one reads)}
               type "latent_attention":  mixer {heads, dim, vdim, q_rank, kv_rank, scale, mask.size}
               type "parallel":          mixer {left {heads, kv_heads, dim, vdim, scale, q_temp {coef, every} (optional)},
                                         right {heads, kv_heads, dim, vdim, conv}, left_scale, right_scale}
               mlp null | {kind "dense", ff}

The ranks of the gated delta rule's two low-rank projections are no keys: they are the shapes of the layer's
``mix.right.a1`` and ``mix.right.g1`` tensors, which the loader hands to ``from_dict`` as ``shapes``.  What the design
fixes (activation functions, where norms sit, how rotated pairs lie, the 1e-6 of the unit vectors, the norm weights
stored around zero) is in the parts and in the builder.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

from .errors import InvalidValue, MissingKey
from .rifizen import _get


@dataclass
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: Optional[float]
    rot_scaling: Optional[Dict[str, float]]
    kv_from: Optional[int]


@dataclass
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]


@dataclass
class KeyValueAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, float]]


@dataclass
class DeltaRuleConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int
    decay_rank: int                # rows of mix.right.a1
    gate_rank: int                 # rows of mix.right.g1


@dataclass
class SideBySideConfig:
    left: KeyValueAttentionConfig
    right: DeltaRuleConfig
    left_scale: float
    right_scale: float


@dataclass
class LudusunLayer:
    type: str                      # "attention" | "latent_attention" | "parallel"
    mixer: object
    ff: Optional[int]              # width of the dense feed-forward; None: the layer has none


@dataclass
class LudusunConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_softcap: Optional[float]
    layers: List[LudusunLayer]
    raw: dict = field(default_factory=dict, repr=False)

    ARCHITECTURE = "Ludusun"
    DEFAULT_RANK = 16              # where no tensor shapes are at hand (a model made from a configuration alone)
    SHAPES_FROM_TENSORS = True     # the loader passes the folder's tensor shapes to from_dict

    @classmethod
    def from_dict(cls, raw: dict, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> "LudusunConfig":
        layers_raw = raw.get("layers")
        if layers_raw is None:
            raise MissingKey("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise InvalidValue("layers", layers_raw, "must be a non-empty list")
        ranks = raw.get("ranks") if isinstance(raw.get("ranks"), dict) else {}
        layers: List[LudusunLayer] = []
        for i, L in enumerate(layers_raw):
            p = f"layers[{i}]"
            if not isinstance(L, dict):
                raise InvalidValue(p, L, "must be an object")
            kind = L.get("type")

            def g(path, k, L=L, p=p, **kw):
                return _get(L, path, k, where=p + ".", **kw)
            if kind == "attention":
                # a layer that reads another layer's keys and values may leave out what it shares with that layer
                src = L.get("mixer", {}).get("kv_from") if isinstance(L.get("mixer"), dict) else None
                if isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i and isinstance(layers_raw[src].get("mixer"), dict):
                    L = dict(L, mixer={**{k: v for k, v in layers_raw[src]["mixer"].items() if k in ("kv_heads", "dim", "vdim", "rot")},
                                       **L["mixer"]})

                    def g(path, k, L=L, p=p, **kw):
                        return _get(L, path, k, where=p + ".", **kw)
                mixer = cls._attention(L, g, p, i, layers)
            elif kind == "latent_attention":
                mixer = LatentAttentionConfig(
                    heads=g("mixer.heads", int, minimum=1), dim=g("mixer.dim", int, minimum=1),
                    vdim=g("mixer.vdim", int, minimum=1), q_rank=g("mixer.q_rank", int, minimum=1),
                    kv_rank=g("mixer.kv_rank", int, minimum=1), scale=g("mixer.scale", float, positive=True),
                    window=g("mixer.mask.size", int, optional=True, minimum=1))
            elif kind == "parallel":
                def rank(name, i=i):
                    key = f"l{i}.mix.right.{name}"
                    if shapes is not None and key in shapes:
                        return int(shapes[key][0])
                    return int(ranks.get(key, cls.DEFAULT_RANK))
                qt = None
                if isinstance(L.get("mixer", {}).get("left", {}).get("q_temp"), dict):
                    qt = (g("mixer.left.q_temp.coef", float), g("mixer.left.q_temp.every", float, positive=True))
                left = KeyValueAttentionConfig(
                    heads=g("mixer.left.heads", int, minimum=1), kv_heads=g("mixer.left.kv_heads", int, minimum=1),
                    dim=g("mixer.left.dim", int, minimum=1), vdim=g("mixer.left.vdim", int, minimum=1),
                    scale=g("mixer.left.scale", float, positive=True), q_temp=qt)
                if left.heads % left.kv_heads:
                    raise InvalidValue(f"{p}.mixer.left.kv_heads", left.kv_heads, f"must divide heads = {left.heads}")
                if left.vdim != left.dim:
                    raise InvalidValue(f"{p}.mixer.left.vdim", left.vdim, f"the values are the keys: must equal dim = {left.dim}")
                right = DeltaRuleConfig(
                    heads=g("mixer.right.heads", int, minimum=1), kv_heads=g("mixer.right.kv_heads", int, minimum=1),
                    dim=g("mixer.right.dim", int, minimum=1), vdim=g("mixer.right.vdim", int, minimum=1),
                    taps=g("mixer.right.conv", int, minimum=1), decay_rank=rank("a1"), gate_rank=rank("g1"))
                if right.heads % right.kv_heads:
                    raise InvalidValue(f"{p}.mixer.right.kv_heads", right.kv_heads, f"must divide heads = {right.heads}")
                if right.dim > 256:
                    raise InvalidValue(f"{p}.mixer.right.dim", right.dim, "the recurrence kernel holds at most 256 rows of a state column")
                if right.taps > 16:
                    raise InvalidValue(f"{p}.mixer.right.conv", right.taps, "the convolution kernel takes up to 16 taps")
                mixer = SideBySideConfig(left, right, left_scale=g("mixer.left_scale", float),
                                         right_scale=g("mixer.right_scale", float))
            else:
                raise InvalidValue(f"{p}.type", kind, "this design has layers of type 'attention', 'latent_attention' and 'parallel'")
            mlp_raw = L.get("mlp")
            ff = None
            if mlp_raw is not None:
                mk = mlp_raw.get("kind") if isinstance(mlp_raw, dict) else None
                if mk != "dense":
                    raise InvalidValue(f"{p}.mlp.kind", mk, "must be 'dense' (or mlp null)")
                ff = g("mlp.ff", int, minimum=1)
            layers.append(LudusunLayer(kind, mixer, ff))
        scale = _get(raw, "embedding.scale", float, optional=True)
        return cls(architecture=str(raw.get("architecture") or cls.ARCHITECTURE),
                   vocab=_get(raw, "vocab", int, minimum=1), width=_get(raw, "width", int, minimum=1),
                   eps=_get(raw, "norm.eps", float, positive=True), embedding_scale=1.0 if scale is None else scale,
                   logit_softcap=_get(raw, "logit_softcap", float, optional=True, positive=True),
                   layers=layers, raw=copy.deepcopy(raw))

    @staticmethod
    def _attention(L, g, p, i, layers) -> SinkAttentionConfig:
        rot = (L.get("mixer", {}).get("rot") or {}) if isinstance(L.get("mixer"), dict) else {}
        rot_dims = g("mixer.rot.dims", int, optional=True, minimum=0) or 0
        scaling = rot.get("scaling") if rot_dims else None
        if scaling is not None:
            scaling = {k: g(f"mixer.rot.scaling.{k}", float, positive=True) for k in ("factor", "original", "fast", "slow")}
        m = SinkAttentionConfig(
            heads=g("mixer.heads", int, minimum=1), kv_heads=g("mixer.kv_heads", int, minimum=1),
            dim=g("mixer.dim", int, minimum=1), vdim=g("mixer.vdim", int, minimum=1),
            scale=g("mixer.scale", float, positive=True), rot_dims=rot_dims,
            rot_base=g("mixer.rot.base", float, positive=True) if rot_dims else None, rot_scaling=scaling,
            kv_from=g("mixer.kv_from", int, optional=True, minimum=0))
        if m.heads % m.kv_heads:
            raise InvalidValue(f"{p}.mixer.kv_heads", m.kv_heads, f"must divide heads = {m.heads}")
        if m.rot_dims % 2 or m.rot_dims > m.dim:
            raise InvalidValue(f"{p}.mixer.rot.dims", m.rot_dims, f"must be even and at most dim = {m.dim}")
        if m.rot_dims and not m.rot_base > 1:
            raise InvalidValue(f"{p}.mixer.rot.base", m.rot_base, "must be larger than 1")
        if m.kv_from is not None:
            j = m.kv_from
            src = layers[j] if j < i else None
            if src is None or src.type != "attention" or src.mixer.kv_from is not None:
                raise InvalidValue(f"{p}.mixer.kv_from", j, "must name an earlier attention layer with keys and values of its own")
            if not all(getattr(src.mixer, k) == getattr(m, k) for k in ("kv_heads", "dim", "vdim")):
                raise InvalidValue(f"{p}.mixer.kv_from", j, "the two layers' kv heads and head sizes must be equal")
        return m

    def to_dict(self) -> dict:
        """The configuration as config.json holds it; the ranks that were read from tensor shapes ride along under
        ``ranks`` so that a folder written from this dict alone (random weights) gets the same shapes."""
        out = copy.deepcopy(self.raw)
        ranks = {}
        for i, L in enumerate(self.layers):
            if L.type == "parallel":
                ranks[f"l{i}.mix.right.a1"] = L.mixer.right.decay_rank
                ranks[f"l{i}.mix.right.g1"] = L.mixer.right.gate_rank
        if ranks:
            out["ranks"] = ranks
        return out
