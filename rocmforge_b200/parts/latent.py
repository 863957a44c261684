"""Attention whose queries, keys and values are made from narrow latents of the token."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..cache.requests import KVRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .attention import GQAAttention
from .base import MIXERS, Mixer
from .linear import Linear


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Softmax attention without positions whose heads are expanded from two latents of the mixer's input x:

        c_q = rms(W_dq x) * w_q            (``q_rank`` numbers)        q_h = W_uq c_q       (``dim`` per head)
        c   = rms(W_dkv x) * w_kv          (``kv_rank`` numbers)       k_h = W_uk c,  v_h = W_uv c   (``dim``, ``vdim`` per head)
        score = scale q_h . k_h over the last ``window`` positions (None: all earlier ones), ordinary softmax
        out = W_o concat_h(o_h * sigmoid(W_g x)_h)                     (``gate`` "sigmoid_head"; None: no gate)

    rms(x) = x / sqrt(mean(x^2) + eps), in 32-bit.  One product makes W_dq x | W_dkv x | W_g x, one kernel norms the two
    latents, two products expand them, and from there on the mixer is grouped-query attention with as many kv heads as
    heads: the expanded keys and values of the window go into the paged cache through the per-head writer, and the
    attention kernels, the gate and the output product are those of ``gqa_attention`` (an inner part without projections
    of its own).  Caching the expanded heads rather than c costs heads * (dim + vdim) instead of kv_rank numbers a
    position; a window bounds both.
    ``names``: the tensors' names below the part's prefix (keys dq, dq_norm, uq, dkv, dkv_norm, uk, uv, g, o).
    """

    def __init__(self, hidden: int, n_heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int, eps: float, *,
                 scale: Optional[float] = None, window: Optional[int] = None, gate: Optional[str] = "sigmoid_head",
                 names: Optional[Dict[str, str]] = None):
        if gate not in (None, "sigmoid_head"):
            raise ValueError(f"latent_attention: gate {gate!r} has no kernel (sigmoid_head)")
        self.hidden, self.n_heads, self.head_dim, self.v_head_dim = hidden, n_heads, head_dim, v_head_dim
        self.q_rank, self.kv_rank, self.eps, self.gate = int(q_rank), int(kv_rank), float(eps), gate
        self.names = {"dq": "q_a_proj.weight", "dq_norm": "q_a_norm.weight", "uq": "q_b_proj.weight",
                      "dkv": "kv_a_proj.weight", "dkv_norm": "kv_a_norm.weight", "uk": "k_b_proj.weight",
                      "uv": "v_b_proj.weight", "g": "g_proj.weight", "o": "o_proj.weight"}
        self.names.update(names or {})
        # the attention over the expanded heads: masks, kernel choice and tile tables are gqa_attention's
        self.inner = GQAAttention(hidden, n_heads, n_heads, head_dim, qkv_bias=False, window=window, position=None,
                                  scale=scale, v_head_dim=v_head_dim)
        self.q_size, self.k_size, self.v_size = n_heads * head_dim, n_heads * head_dim, n_heads * v_head_dim
        self.down: Optional[Linear] = None
        self.uq: Optional[Linear] = None
        self.ukv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        s = {n["dq"]: ParamSpec((self.q_rank, self.hidden)), n["dq_norm"]: ParamSpec((self.q_rank,), kind="vector", init="ones"),
             n["uq"]: ParamSpec((self.q_size, self.q_rank)),
             n["dkv"]: ParamSpec((self.kv_rank, self.hidden)), n["dkv_norm"]: ParamSpec((self.kv_rank,), kind="vector", init="ones"),
             n["uk"]: ParamSpec((self.k_size, self.kv_rank)), n["uv"]: ParamSpec((self.v_size, self.kv_rank)),
             n["o"]: ParamSpec((self.hidden, self.v_size))}
        if self.gate is not None:
            s[n["g"]] = ParamSpec((self.n_heads, self.hidden))
        return s

    @staticmethod
    def _padded(blocks, hidden):
        """The blocks stacked with every block's first row on a 16-byte boundary of the product's output rows (8 columns
        of bfloat16), and the columns at which they start."""
        out, cols, at = [], [], 0
        for b in blocks:
            pad = (-at) % 8
            if pad:
                out.append(b.new_zeros((pad, hidden)))
                at += pad
            cols.append(at)
            out.append(b)
            at += b.shape[0]
        if at % 8:
            out.append(blocks[0].new_zeros(((-at) % 8, hidden)))
        return torch.cat(out, dim=0).contiguous(), cols

    def bind(self, params, compute_dtype):
        n = self.names
        blocks = [params[n["dq"]], params[n["dkv"]]] + ([params[n["g"]]] if self.gate is not None else [])
        w, cols = self._padded(blocks, self.hidden)
        self.down = Linear(w)
        self.cq_col, self.c_col = cols[0], cols[1]
        self.gate_col = cols[2] if self.gate is not None else None
        self.dq_norm_w = params[n["dq_norm"]].contiguous()
        self.dkv_norm_w = params[n["dkv_norm"]].to(self.dq_norm_w.dtype).contiguous()
        self.uq = Linear(params[n["uq"]])
        self.ukv = Linear(torch.cat([params[n["uk"]], params[n["uv"]]], dim=0).contiguous())
        self.o = Linear(params[n["o"]])

    def cuda_modules(self, compute_dtype):
        return list(dict.fromkeys(["elementwise"] + self.inner.cuda_modules(compute_dtype)))

    def cache_request(self):
        return self.inner.cache_request()

    def step_table_names(self):
        return self.inner.step_table_names()

    def step_table(self, name, batch):
        return self.inner.step_table(name, batch)

    def heads_out(self, ctx, y, view):
        if isinstance(y, ScaledRows):
            y = y.materialize()
        p = self.down(ctx, y)                                                # [T, W_dq x | W_dkv x | W_g x]
        c_q, c = kernels.stretch_norm(p, [(self.cq_col, self.q_rank, self.dq_norm_w), (self.c_col, self.kv_rank, self.dkv_norm_w)],
                                      self.eps)
        q = self.uq(ctx, c_q)                                                # the queries need nothing more
        kv = self.ukv(ctx, c)                                                # [T, k heads | v heads]
        # keys and values into their pages, head by head (rows without query heads: nothing is normed or turned)
        kernels.head_norm_kv_write(kv, 0, self.n_heads, self.head_dim, self.v_head_dim, None, ctx.tok_seq, ctx.tok_pos,
                                   ctx.seq_slot, view.block_table, view.k_pages, view.v_pages, view.writes,
                                   compute_dtype=ctx.compute_dtype)
        o = self.inner.attend(ctx, q, view)
        if self.gate is not None:
            o = kernels.sigmoid_gate(o, p[:, self.gate_col:self.gate_col + self.n_heads], group=self.v_head_dim)
        return o

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.heads_out(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.heads_out(ctx, y, cache_view))
