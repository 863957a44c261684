"""Gated feed-forward (SwiGLU)."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import FEED_FORWARDS, FeedForward
from .linear import Linear


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """x += W_down (act(W_gate y) * (W_up y)), no biases
    (maeddesg/ROCmForge src/gpu/forward.rs:1094-1161, hip_kernels/elementwise.hip:72-82).

    gate and up are fused into one matrix at load time with their rows interleaved
    (row 2j = gate_j, row 2j+1 = up_j), so that one product yields both and the
    activation reads neighbouring columns (the reference fuses gate, up and SiLU in its
    decode kernels, src/gpu/forward.rs:2485-2500).
    """

    accepts_scaled_rows = True

    def __init__(self, hidden: int, intermediate: int, activation: str = "silu", names: Optional[Dict[str, str]] = None):
        """``names``: the tensors' names below the part's prefix (keys gate, up, down)."""
        if activation != "silu":
            raise ValueError(f"gated_mlp: activation {activation!r} has no kernel")
        self.hidden, self.intermediate = hidden, intermediate
        self.names = {"gate": "gate_proj.weight", "up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.gate_up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            self.names["gate"]: ParamSpec((self.intermediate, self.hidden)),
            self.names["up"]: ParamSpec((self.intermediate, self.hidden)),
            self.names["down"]: ParamSpec((self.hidden, self.intermediate)),
        }

    def bind(self, params, compute_dtype):
        g, u = params[self.names["gate"]], params[self.names["up"]]
        gu = torch.stack([g, u], dim=1).reshape(2 * self.intermediate, self.hidden).contiguous()
        self.gate_up = Linear(gu)
        self.down = Linear(params[self.names["down"]])

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def forward(self, ctx, y, stream):
        a = ctx.gated_activation(y, self.gate_up)                           # [T, I]
        self.down.add_to_stream(ctx, a, stream)

    def output(self, ctx, y):
        return self.down.f32_parts(ctx, ctx.gated_activation(y, self.gate_up))


@FEED_FORWARDS.register("relu2_mlp")
class SquaredReluMLP(FeedForward):
    """W_down relu(W_up y)^2, no gate, no biases.  ``names``: the tensors' names below the part's prefix (up, down)."""

    def __init__(self, hidden: int, intermediate: int, names: Optional[Dict[str, str]] = None):
        self.hidden, self.intermediate = hidden, intermediate
        self.names = {"up": "up_proj.weight", "down": "down_proj.weight"}
        self.names.update(names or {})
        self.up: Optional[Linear] = None
        self.down: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.names["up"]: ParamSpec((self.intermediate, self.hidden)),
                self.names["down"]: ParamSpec((self.hidden, self.intermediate))}

    def bind(self, params, compute_dtype):
        self.up = Linear(params[self.names["up"]])
        self.down = Linear(params[self.names["down"]])

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def activated(self, ctx, y):
        from ..engine.stream import ScaledRows
        if isinstance(y, ScaledRows):
            y = y.materialize()
        return kernels.relu2(self.up(ctx, y))

    def forward(self, ctx, y, stream):
        self.down.add_to_stream(ctx, self.activated(ctx, y), stream)

    def output(self, ctx, y):
        return self.down.f32_parts(ctx, self.activated(ctx, y))


@FEED_FORWARDS.register("sum")
class SummedFeedForward(FeedForward):
    """Feed-forwards side by side on the same input whose results are added (routed experts and an expert that every token
    uses, say).  ``branches``: {prefix below this part's: feed-forward}; at most two.  The sum is formed by whoever adds
    the result to the stream (the part hands out a ``SumOf``)."""

    def __init__(self, branches: Dict[str, FeedForward]):
        if not 1 <= len(branches) <= 2:
            raise ValueError("summed feed-forward: one or two branches")
        self.branches = dict(branches)

    def leaf_parts(self):
        return dict(self.branches)

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def output(self, ctx, y):
        from ..engine.stream import ScaledRows
        from .base import SumOf
        if isinstance(y, ScaledRows):
            y = y.materialize()
        return SumOf([f.output(ctx, y) for f in self.branches.values()])

    def forward(self, ctx, y, stream):
        raise NotImplementedError("summed feed-forward: its result is added by the block that holds it (output)")
