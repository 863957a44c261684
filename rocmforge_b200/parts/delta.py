"""The gated delta rule: a matrix memory that is corrected towards each token's value instead of only added to."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..cache.requests import StateRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer
from .linear import Linear


@MIXERS.register("gated_delta")
class GatedDeltaRule(Mixer):
    """Per head, with q, k of size ``dim`` (``qk_heads`` of them; head h reads q/k head h // (heads / qk_heads)) and v of
    size ``vdim``:

        (q, k, v) <- silu(conv(W_q x | W_k x | W_v x))     a causal convolution per channel over the last ``taps`` tokens,
                                                            no bias, zeros before the sequence's start
        q <- q / sqrt(sum q^2 + unit_eps) * q_scale (default dim^-1/2),  k <- k / sqrt(sum k^2 + unit_eps)      per head
        beta = sigmoid(W_b x)                               one per head
        g = exp(-exp(A_log_h) softplus(W_a2 (W_a1 x) + dt_bias))        one per head and key channel, [heads, dim]
        S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q      (S is dim x vdim, starts at zero)
        out = W_o concat_h(rms(o_h) * w * sigmoid(W_g2 (W_g1 x))_h)     rms over vdim with ``eps``; w [vdim] for all heads

    One product makes q | k | v | W_b x | W_a1 x | W_g1 x in the compute dtype; the decay's second product stays 32-bit,
    and so do the convolution's result, the unit norms, beta, softplus, the decays, S, o and its norm.  Per sequence the
    mixer keeps S [heads, dim, vdim] and the convolution's last taps-1 inputs, so a prompt may be cut anywhere; the
    recurrence runs token by token in prompts too, so its sums do not depend on how a prompt is cut into portions (a token
    decoded alone takes another kernel form, whose sums differ by rounding).
    ``names``: the tensors' names below the part's prefix (keys q, k, v, q_conv, k_conv, v_conv, b, a_log, dt_bias, a1, a2,
    g1, g2, norm, o).
    """

    def __init__(self, hidden: int, n_heads: int, qk_heads: int, dim: int, vdim: int, taps: int, decay_rank: int,
                 gate_rank: int, eps: float, *, unit_eps: float = 1e-6, q_scale: Optional[float] = None,
                 names: Optional[Dict[str, str]] = None):
        if n_heads % qk_heads:
            raise ValueError(f"gated_delta: {n_heads} heads cannot share {qk_heads} q/k heads")
        if dim > 256:
            raise ValueError(f"gated_delta: the recurrence kernel holds at most 256 rows of a state column, got dim {dim}")
        if not 1 <= taps <= 16:
            raise ValueError(f"gated_delta: the convolution kernel takes 1 to 16 taps, got {taps}")
        if decay_rank < 1 or gate_rank < 1:
            raise ValueError("gated_delta: the low-rank projections need a rank of at least 1")
        self.hidden, self.n_heads, self.qk_heads, self.dim, self.vdim = hidden, n_heads, qk_heads, dim, vdim
        self.taps, self.decay_rank, self.gate_rank = int(taps), int(decay_rank), int(gate_rank)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.q_scale = float(q_scale) if q_scale is not None else float(dim) ** -0.5
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_conv": "q_conv.weight",
                      "k_conv": "k_conv.weight", "v_conv": "v_conv.weight", "b": "b_proj.weight", "a_log": "A_log",
                      "dt_bias": "dt_bias", "a1": "a_proj.0.weight", "a2": "a_proj.1.weight", "g1": "g_proj.0.weight",
                      "g2": "g_proj.1.weight", "norm": "norm.weight", "o": "o_proj.weight"}
        self.names.update(names or {})
        self.qk_size, self.v_size, self.decay_size = qk_heads * dim, n_heads * vdim, n_heads * dim
        self.channels = 2 * self.qk_size + self.v_size
        self.proj: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["q"]: ParamSpec((self.qk_size, self.hidden)), n["k"]: ParamSpec((self.qk_size, self.hidden)),
                n["v"]: ParamSpec((self.v_size, self.hidden)),
                # random-weights mode: taps that let earlier tokens count, decays spread between fast and slow channels
                n["q_conv"]: ParamSpec((self.qk_size, self.taps), kind="vector", init="normal", std=0.3),
                n["k_conv"]: ParamSpec((self.qk_size, self.taps), kind="vector", init="normal", std=0.3),
                n["v_conv"]: ParamSpec((self.v_size, self.taps), kind="vector", init="normal", std=0.3),
                n["b"]: ParamSpec((self.n_heads, self.hidden), std=0.1),
                n["a_log"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=0.5, mean=-1.0),
                n["dt_bias"]: ParamSpec((self.decay_size,), kind="vector", init="normal", std=1.0),
                n["a1"]: ParamSpec((self.decay_rank, self.hidden)),
                n["a2"]: ParamSpec((self.decay_size, self.decay_rank), std=1.0),
                n["g1"]: ParamSpec((self.gate_rank, self.hidden)),
                n["g2"]: ParamSpec((self.v_size, self.gate_rank), std=1.0),
                n["norm"]: ParamSpec((self.vdim,), kind="vector", init="ones"),
                n["o"]: ParamSpec((self.hidden, self.v_size))}

    def bind(self, params, compute_dtype):
        n = self.names

        def padded_rank(first, second, rank):
            """The narrow half padded to a multiple of 8 rows (zeros), the wide half to as many columns: the second
            product's input rows stay 16-byte aligned in bfloat16."""
            rp = (rank + 7) // 8 * 8
            if rp != rank:
                first = torch.cat([first, first.new_zeros((rp - rank, first.shape[1]))], dim=0)
                second = torch.cat([second, second.new_zeros((second.shape[0], rp - rank))], dim=1)
            return first, second.contiguous(), rp
        a1, a2, self.a_rank = padded_rank(params[n["a1"]], params[n["a2"]], self.decay_rank)
        g1, g2, self.g_rank = padded_rank(params[n["g1"]], params[n["g2"]], self.gate_rank)
        blocks, at, cols = [], 0, {}
        for name, b in (("qkv", torch.cat([params[n["q"]], params[n["k"]], params[n["v"]]], dim=0)), ("b", params[n["b"]]),
                        ("a1", a1), ("g1", g1)):
            pad = (-at) % 8                               # every block starts on a 16-byte boundary of the output rows
            if pad:
                blocks.append(b.new_zeros((pad, self.hidden)))
                at += pad
            cols[name] = at
            blocks.append(b)
            at += b.shape[0]
        if at % 8:
            blocks.append(blocks[0].new_zeros(((-at) % 8, self.hidden)))
        self.cols = cols
        self.proj = Linear(torch.cat(blocks, dim=0).contiguous())
        self.a2, self.g2 = Linear(a2), Linear(g2)
        self.conv_w = torch.cat([params[n["q_conv"]], params[n["k_conv"]].to(params[n["q_conv"]].dtype),
                                 params[n["v_conv"]].to(params[n["q_conv"]].dtype)], dim=0).contiguous()
        self.conv_b = torch.zeros((self.channels,), dtype=self.conv_w.dtype, device=self.conv_w.device)      # the design has none
        self.a_log = params[n["a_log"]].contiguous()
        self.dt_bias = params[n["dt_bias"]].to(self.a_log.dtype).contiguous()
        self.norm_w = params[n["norm"]].contiguous()
        self.o = Linear(params[n["o"]])
        self._no_conv_state = None

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "retention", "mamba2", "delta"]

    def cache_request(self):
        named = dict(S=((self.n_heads, self.dim, self.vdim), torch.float32))
        if self.taps > 1:
            named["conv"] = ((self.taps - 1, self.channels), torch.float32)
        return StateRequest.of(**named)

    def gated(self, ctx, y, state_view):
        """The normed, gated heads [T, heads*vdim] in the compute dtype (the output product's input)."""
        if isinstance(y, ScaledRows):
            y = y.materialize()
        c = self.cols
        p = self.proj(ctx, y)                                                # [T, q | k | v | b | a1 | g1]
        a = self.a2(ctx, p[:, c["a1"]:c["a1"] + self.a_rank], out_f32=True)  # [T, heads*dim], 32-bit
        gate = self.g2(ctx, p[:, c["g1"]:c["g1"] + self.g_rank])             # [T, heads*vdim]
        if self.taps > 1:
            conv_state = state_view["conv"]
        else:
            if self._no_conv_state is None:
                self._no_conv_state = torch.empty((0, 0, self.channels), dtype=torch.float32, device=p.device)
            conv_state = self._no_conv_state
        qkv = kernels.conv_silu(p, c["qkv"], self.channels, conv_state, self.conv_w, self.conv_b, ctx.tok_seq, ctx.cu_q,
                                ctx.seq_slot)                                # float32 [T, q | k | v]
        qn, kn, kq, decay, beta = kernels.delta_prepare(qkv, a, self.dt_bias, self.a_log, p[:, c["b"]:c["b"] + self.n_heads],
                                                        self.n_heads, self.qk_heads, self.dim, self.q_scale, self.unit_eps)
        o = kernels.delta_scan(qn, kn, kq, decay, beta, qkv[:, 2 * self.qk_size:], state_view["S"], ctx.cu_q, ctx.seq_slot,
                               self.n_heads, self.qk_heads, self.dim, self.vdim, one_token=ctx.is_decode)
        return kernels.retention_gate(o, gate, self.n_heads, self.vdim, self.eps, weight=self.norm_w, gate_fn="sigmoid")

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.gated(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.gated(ctx, y, cache_view))
