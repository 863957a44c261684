"""Retention: linear attention with a fixed decay per head and a matrix state per sequence."""
from __future__ import annotations

from typing import Dict, Optional, Sequence

import numpy as np
import torch

from .. import kernels
from ..cache.requests import StateRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer
from .linear import Linear


def recurrence_chunk_table(batch, chunked_from: int) -> np.ndarray:
    """The table of the recurrences' chunked kernels: first[B+1] (index of each sequence's first chunk), then (sequence,
    first row) of every chunk of 64 new tokens; empty for steps that take the token-by-token kernel (decoding, and
    portions whose longest is below ``chunked_from`` tokens)."""
    if batch.is_decode or batch.max_new < chunked_from:
        return np.zeros((0,), dtype=np.int32)
    C = kernels.RETENTION_CHUNK
    counts = [(int(n) + C - 1) // C for n in batch.n_new]
    first = np.concatenate([[0], np.cumsum(counts)])
    pairs = [(b, q0) for b in range(batch.B) for q0 in range(0, int(batch.n_new[b]), C)]
    return np.concatenate([first, np.asarray(pairs, dtype=np.int64).reshape(-1)]).astype(np.int32)


@MIXERS.register("retention")
class Retention(Mixer):
    """Per head, with q, k of size ``dim`` and v of size ``vdim``:

        S_t = decay_h * S_(t-1) + k_t v_t^T        (S starts at zero, float32, kept per sequence as [vdim, dim])
        o_t = S_t^T q_t                            (no softmax, no denominator)
        out = W_o (concat_h(o_t / rms(o_t)) * silu(W_g x))

    q and k are rotated by ``position`` (a PositionEncoding: first rot_dim elements of a head), then k is multiplied
    by ``k_scale`` (default dim^-1/2).  rms(o) = sqrt(mean(o^2) + eps) per head, without a weight.  The projections
    (one fused product q | k | v | g) run in the compute dtype; the rotation, the state, o and its norm are 32-bit.
    ``names``: the tensors' names below the part's prefix (keys q, k, v, g, o).
    """

    def __init__(self, hidden: int, n_heads: int, dim: int, vdim: int, decay: Sequence[float], eps: float, *,
                 position=None, k_scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        if len(decay) != n_heads:
            raise ValueError(f"retention: {len(decay)} decays for {n_heads} heads")
        self.hidden, self.n_heads, self.dim, self.vdim = hidden, n_heads, dim, vdim
        self.decay = [float(d) for d in decay]
        self.eps = float(eps)
        self.position = position
        self.k_scale = float(k_scale) if k_scale is not None else float(dim) ** -0.5
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight"}
        self.names.update(names or {})
        self.qk_size, self.v_size = n_heads * dim, n_heads * vdim
        self.qkvg: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.decay_dev = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["q"]: ParamSpec((self.qk_size, self.hidden)), n["k"]: ParamSpec((self.qk_size, self.hidden)),
                n["v"]: ParamSpec((self.v_size, self.hidden)), n["g"]: ParamSpec((self.v_size, self.hidden)),
                n["o"]: ParamSpec((self.hidden, self.v_size))}

    def bind(self, params, compute_dtype):
        n = self.names
        w = torch.cat([params[n["q"]], params[n["k"]], params[n["v"]], params[n["g"]]], dim=0).contiguous()
        self.qkvg = Linear(w)
        self.o = Linear(params[n["o"]])
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=w.device)
        if self.position is not None:
            self.position.prepare(w.device)

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "retention"]

    def cache_request(self):
        return StateRequest.of(S=((self.n_heads, self.vdim, self.dim), torch.float32))

    # Prompts run the recurrence in chunks side by side; steps of few tokens per sequence run it token by token.
    CHUNKED_FROM = 17            # tokens of the step's longest portion from which the chunked kernels are taken

    def step_table_names(self):
        return ("retention_chunks",)

    def step_table(self, name, batch):
        return recurrence_chunk_table(batch, self.CHUNKED_FROM)

    def gated(self, ctx, y, state_view):
        """The gated, normed heads [T, heads*vdim] in the compute dtype (the output product's input)."""
        if isinstance(y, ScaledRows):
            y = y.materialize()
        p = self.qkvg(ctx, y)                                                # [T, q | k | v | g]
        rot = (self.position.rotation() if self.position is not None else None) or dict(inv_freq=None, rot_dim=0)
        if rot.get("interleaved"):
            raise NotImplementedError("retention: neighbouring pairs are not rotated by its kernel")
        qk = kernels.retention_prepare(p, 0, self.qk_size, self.n_heads, self.dim, rot["rot_dim"], rot["inv_freq"],
                                       ctx.tok_pos, self.k_scale)
        v = p[:, 2 * self.qk_size: 2 * self.qk_size + self.v_size]
        g = p[:, 2 * self.qk_size + self.v_size:]
        table = ctx.tables.get("retention_chunks")
        if table is not None and table.numel() > 0:
            o = kernels.retention_chunked(qk, v, state_view["S"], self.decay_dev, table, ctx.cu_q, ctx.seq_slot,
                                          self.n_heads, self.dim, self.vdim)
        else:
            o = kernels.retention_scan(qk, v, state_view["S"], self.decay_dev, ctx.cu_q, ctx.seq_slot, self.n_heads,
                                       self.dim, self.vdim)
        return kernels.retention_gate(o, g, self.n_heads, self.vdim, self.eps)

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.gated(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.gated(ctx, y, cache_view))
