"""Token embedding and output head."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..weights.spec import ParamSpec
from .base import Part
from .linear import Linear


class TokenEmbedding(Part):
    """x = E[token], no scaling (maeddesg/ROCmForge src/gpu/forward.rs:826-883); with ``scale``, x = E[token] * scale
    (formed in 32-bit on the way into the stream; a head tied to the table reads the table itself)."""

    def __init__(self, vocab: int, hidden: int, param_name: str = "weight", scale: Optional[float] = None):
        self.vocab, self.hidden, self.param_name = vocab, hidden, param_name
        self.scale = None if scale is None or float(scale) == 1.0 else float(scale)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.param_name: ParamSpec((self.vocab, self.hidden))}

    def bind(self, params, compute_dtype):
        self.weight = params[self.param_name]

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]

    def forward(self, ctx, token_ids: torch.Tensor) -> torch.Tensor:
        return kernels.embed(self.weight, token_ids, scale=self.scale)

    def forward_with(self, ctx, token_ids: torch.Tensor, positions: "LearnedPositions" = None, rounded: bool = False):
        """(x, y): x = E[token] (+ positions' vector of the token's position), and y = x in the compute dtype if
        ``rounded`` (for a first layer that reads the stream itself), else None; one kernel."""
        if self.scale is not None:
            raise NotImplementedError("a scaled embedding does not go with learned positions or a first layer that reads the stream")
        return kernels.embed_positions(self.weight, token_ids, positions.table if positions is not None else None,
                                       ctx.tok_pos if positions is not None else None,
                                       rounded=rounded and ctx.compute_dtype != torch.float32)


class LearnedPositions(Part):
    """A learned vector per position, [positions, hidden], added to the embedding (not scaled).  Sequences cannot grow
    beyond the table (the model's longest sequence is set from it)."""

    def __init__(self, positions: int, hidden: int, param_name: str = "weight"):
        self.positions, self.hidden, self.param_name = positions, hidden, param_name
        self.table: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.param_name: ParamSpec((self.positions, self.hidden))}

    def bind(self, params, compute_dtype):
        self.table = params[self.param_name]

    def cuda_modules(self, compute_dtype):
        return ["elementwise"]


class OutputHead(Part):
    """logits = W y in float32; with tied embeddings W is the embedding matrix itself
    (maeddesg/ROCmForge src/gpu/forward.rs:1313-1338; tie: src/gpu/weights.rs:868-886)."""

    def __init__(self, vocab: int, hidden: int, tied_to: Optional[str] = None, param_name: str = "weight",
                 softcap: Optional[float] = None):
        """``softcap``: logits <- softcap * tanh(logits / softcap), in 32-bit."""
        self.vocab, self.hidden, self.tied_to, self.param_name = vocab, hidden, tied_to, param_name
        self.softcap = float(softcap) if softcap else None
        self.linear: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.param_name: ParamSpec((self.vocab, self.hidden), tied_to=self.tied_to)}

    def bind(self, params, compute_dtype):
        self.linear = Linear(params[self.param_name])

    def cuda_modules(self, compute_dtype):
        return ["elementwise"] if self.softcap is not None else []

    def forward(self, ctx, y: torch.Tensor) -> torch.Tensor:
        logits = self.linear(ctx, y, out_f32=True)
        return kernels.softcap_(logits, self.softcap) if self.softcap is not None else logits
