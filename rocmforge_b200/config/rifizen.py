"""Typed configuration of the Rifizen decoder, read from its own config.json keys.

config.json gives every size and every constant that differs between models of the design:

    architecture "Rifizen"; vocab, width; norm.eps
    layers[i]: type ("parallel"), mixer.left {heads, kv_heads, dim, vdim, scale, softcap, mask.size},
               mixer.right {heads, dim, vdim, decay[heads], rot {dims, base}},
               mlp null | {kind "dense", ff} | {kind "moe", expert.ff, router {experts, top}}
    loop {start, stop, times} (optional): layers start .. stop-1 run ``times`` times in a row

What the design fixes (activation functions, the slopes of the distance bias, where norms sit) is in the parts.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import List, Optional

from .errors import InvalidValue, MissingKey


def _get(raw: dict, path: str, kind, *, optional=False, minimum=None, positive=False, where: str = ""):
    """raw["a"]["b"] for path "a.b", checked: ``kind`` int or float.  ``where`` goes before the path in messages."""
    cur = raw
    for part in path.split("."):
        if not isinstance(cur, dict) or part not in cur or cur[part] is None:
            if optional:
                return None
            raise MissingKey(where + path)
        cur = cur[part]
    path = where + path
    if kind is int and isinstance(cur, float) and cur.is_integer():
        cur = int(cur)                      # a whole number written with a decimal point
    if isinstance(cur, bool) or not isinstance(cur, (int, float) if kind is float else int):
        raise InvalidValue(path, cur, "must be a number" if kind is float else "must be an integer")
    if minimum is not None and cur < minimum:
        raise InvalidValue(path, cur, f"must be >= {minimum}")
    if positive and not cur > 0:
        raise InvalidValue(path, cur, "must be positive")
    return kind(cur)


@dataclass
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    window: int


@dataclass
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: List[float]
    rot_dims: int
    rot_base: float


@dataclass
class FeedForwardConfig:
    kind: str                      # "dense" | "moe"
    ff: int
    experts: int = 0
    top: int = 0


@dataclass
class RifizenLayer:
    type: str
    left: WindowAttentionConfig
    right: RetentionConfig
    mlp: Optional[FeedForwardConfig]


@dataclass
class RifizenConfig:
    architecture: str
    vocab: int
    width: int
    eps: float
    layers: List[RifizenLayer]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    loop_given: bool = False       # config.json has a loop (its table of pass vectors exists even if the stretch is empty)
    raw: dict = field(default_factory=dict, repr=False)

    ARCHITECTURE = "Rifizen"

    @classmethod
    def from_dict(cls, raw: dict) -> "RifizenConfig":
        layers_raw = raw.get("layers")
        if layers_raw is None:
            raise MissingKey("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise InvalidValue("layers", layers_raw, "must be a non-empty list")
        layers = []
        for i, L in enumerate(layers_raw):
            p = f"layers[{i}]"
            if not isinstance(L, dict):
                raise InvalidValue(p, L, "must be an object")
            kind = L.get("type")
            if kind != "parallel":
                raise InvalidValue(f"{p}.type", kind, "this design has layers of type 'parallel' only")

            def g(path, k, L=L, p=p, **kw):
                return _get(L, path, k, where=p + ".", **kw)
            left = WindowAttentionConfig(
                heads=g("mixer.left.heads", int, minimum=1), kv_heads=g("mixer.left.kv_heads", int, minimum=1),
                dim=g("mixer.left.dim", int, minimum=1), vdim=g("mixer.left.vdim", int, minimum=1),
                scale=g("mixer.left.scale", float, positive=True),
                softcap=g("mixer.left.softcap", float, optional=True, positive=True),
                window=g("mixer.left.mask.size", int, minimum=1))
            if left.heads % left.kv_heads:
                raise InvalidValue(f"{p}.mixer.left.kv_heads", left.kv_heads, f"must divide heads = {left.heads}")
            decay = (L.get("mixer", {}).get("right", {}) or {}).get("decay")
            right = RetentionConfig(
                heads=g("mixer.right.heads", int, minimum=1), dim=g("mixer.right.dim", int, minimum=1),
                vdim=g("mixer.right.vdim", int, minimum=1), decay=[],
                rot_dims=g("mixer.right.rot.dims", int, minimum=0), rot_base=g("mixer.right.rot.base", float, positive=True))
            if not isinstance(decay, list) or len(decay) != right.heads or not all(
                    isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                raise InvalidValue(f"{p}.mixer.right.decay", decay, f"must list one number for each of the {right.heads} heads")
            right.decay = [float(d) for d in decay]
            if right.rot_dims % 2 or right.rot_dims > right.dim:
                raise InvalidValue(f"{p}.mixer.right.rot.dims", right.rot_dims, f"must be even and at most dim = {right.dim}")
            if right.dim > 256:
                raise InvalidValue(f"{p}.mixer.right.dim", right.dim, "the recurrence kernel holds at most 256 rows of a state column")
            mlp_raw = L.get("mlp")
            mlp = None
            if mlp_raw is not None:
                mk = mlp_raw.get("kind") if isinstance(mlp_raw, dict) else None
                if mk == "dense":
                    mlp = FeedForwardConfig("dense", g("mlp.ff", int, minimum=1))
                elif mk == "moe":
                    mlp = FeedForwardConfig("moe", g("mlp.expert.ff", int, minimum=1),
                                            experts=g("mlp.router.experts", int, minimum=1), top=g("mlp.router.top", int, minimum=1))
                    if mlp.top > mlp.experts:
                        raise InvalidValue(f"{p}.mlp.router.top", mlp.top, f"there are only {mlp.experts} experts")
                    if mlp.top > 16 or mlp.experts > 1024:
                        raise InvalidValue(f"{p}.mlp.router", mlp_raw.get("router"), "the routing kernels take up to 16 of up to 1024 experts")
                else:
                    raise InvalidValue(f"{p}.mlp.kind", mk, "must be 'dense' or 'moe' (or mlp null)")
            layers.append(RifizenLayer(kind, left, right, mlp))
        cfg = cls(architecture=str(raw.get("architecture") or cls.ARCHITECTURE),
                  vocab=_get(raw, "vocab", int, minimum=1), width=_get(raw, "width", int, minimum=1),
                  eps=_get(raw, "norm.eps", float, positive=True), layers=layers, raw=copy.deepcopy(raw))
        loop = raw.get("loop")
        if loop is not None:
            cfg.loop_given = True
            cfg.loop_start = _get(raw, "loop.start", int, minimum=0)
            cfg.loop_stop = _get(raw, "loop.stop", int, minimum=0)
            cfg.loop_times = _get(raw, "loop.times", int, minimum=1)
            if not cfg.loop_start <= cfg.loop_stop <= len(layers):
                raise InvalidValue("loop", loop, f"needs 0 <= start <= stop <= {len(layers)} layers")
        return cfg

    @property
    def has_loop(self) -> bool:
        return self.loop_stop > self.loop_start

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)
