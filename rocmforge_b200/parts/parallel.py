"""Mixers side by side."""
from __future__ import annotations

from typing import Dict

import torch

from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer, NormedMean, Part


class _OutWeights(Part):
    """The weights with which the halves' outputs are normed before they are averaged."""

    def __init__(self, hidden: int, names):
        self.hidden, self.names = hidden, list(names)
        self.weights: Dict[str, torch.Tensor] = {}

    def param_specs(self):
        return {n: ParamSpec((self.hidden,), kind="vector", init="ones") for n in self.names}

    def bind(self, params, compute_dtype):
        self.weights = dict(params)


@MIXERS.register("parallel")
class ParallelMixer(Mixer):
    """Several mixers read the same input; the result is the mean of their outputs, each first RMS-normed over the
    width with a weight of its own (used as stored):  mean_b( x_b / sqrt(mean(x_b^2) + eps) * w_b ).

    ``branches``: {name: mixer}; a branch's tensors lie under ``<name>.`` and its out-weight is ``<name>.out``
    (``out_name``).  Each branch keeps what it keeps: the cache request is the dict of the branches' requests, and
    the view this mixer receives is the dict of their views.  Two branches are merged in the kernel that adds the
    result to the stream (the mixer hands out a ``NormedMean``).

    ``scales`` = {name: factor}: the result is instead the plain weighted sum  sum_b factor_b x_b  (no norms, no
    out-weights).  It is formed in 32-bit by the kernel that adds it to the stream (``forward``), which also computes
    the norm that reads the stream next when the block names it (``stream.next_norm``).
    """

    prepares_next_norm = True        # forward() takes the block's hint and leaves that norm's result in stream.prepared

    def __init__(self, hidden: int, branches: Dict[str, Mixer], eps: float = 0.0, out_name: str = "out",
                 scales: Dict[str, float] = None):
        if len(branches) != 2:
            raise ValueError("parallel mixer: the merging kernel takes two branches")
        self.hidden, self.branches, self.eps, self.out_name = hidden, dict(branches), float(eps), out_name
        self.scales = None if scales is None else {name: float(scales[name]) for name in self.branches}
        self.outs = _OutWeights(hidden, [] if self.scales is not None else [f"{name}.{out_name}" for name in self.branches])

    # the halves are leaf parts of their own (their tensors have prefixes of their own)
    def leaf_parts(self) -> Dict[str, Part]:
        out: Dict[str, Part] = {f"{name}.": m for name, m in self.branches.items()}
        if self.scales is None:
            out[""] = self.outs
        return out

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def cache_request(self):
        return {name: m.cache_request() for name, m in self.branches.items()}

    def output(self, ctx, y, cache_view):
        if self.scales is not None:
            raise NotImplementedError("parallel mixer: a weighted sum is added to the stream by forward()")
        return NormedMean([(m.output(ctx, y, cache_view[name]), self.outs.weights[f"{name}.{self.out_name}"])
                           for name, m in self.branches.items()], self.eps)

    def forward(self, ctx, y, cache_view, stream):
        if self.scales is None:
            raise NotImplementedError("parallel mixer: its result is merged by the block that holds it (output)")
        from .. import kernels
        follows = stream.take_hint()
        addends = [(m.output(ctx, y, cache_view[name]), self.scales[name]) for name, m in self.branches.items()]
        nxt = follows.deferred_params() if follows is not None else None
        stream.flush()
        stream.prepared = None
        normed = kernels.weighted_add(stream.h, addends, ctx.compute_dtype, next_norm=nxt)
        if normed is not None:
            stream.prepared = (follows, normed)
