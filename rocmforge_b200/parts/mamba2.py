"""The Mamba-2 mixer (state-space duality): a matrix state per head that decays by one number per token, fed through a
short causal convolution."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import kernels
from ..cache.requests import StateRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer
from .linear import Linear
from .retention import recurrence_chunk_table


@MIXERS.register("mamba2")
class StateSpaceDuality(Mixer):
    """With inner = heads * vdim, N = ``state`` and G = ``groups`` (head h reads group h // (heads / G)):

        W_in x = [z: inner | u: inner | B: G N | C: G N | dt: heads]
        (u, B, C) <- silu(conv(u | B | C))           a causal convolution per channel over the last ``taps`` tokens
        dt_t = softplus(dt_t + dt_bias),  a_t = exp(-exp(A_log) dt_t)                       (per head, no clamp)
        S_t = a_t S_(t-1) + dt_t B_t u_t^T  (S is N x vdim, starts at zero),  y_t = S_t^T C_t + D u_t
        out = W_o (rms_parts(y * silu(z)) * w)       the gate first, then ``norm_groups`` equal parts of a row are each
                                                     divided by their own root mean square

    The product z | u | B | C runs in the compute dtype; dt comes from a second, small product whose result stays
    32-bit.  The convolution's result, dt, the decay, S and y are 32-bit.  Per sequence the mixer keeps S
    [heads, N, vdim] and the convolution's last taps-1 inputs [taps-1, inner + 2 G N], so that a prompt may be cut
    anywhere.  The recurrence is the scalar form of the gated linear attention's scan (``kernels.gated_scan``) with B as
    keys, C as queries and u as values.
    ``names``: the tensors' names below the part's prefix (keys in, conv, conv_bias, dt_bias, a_log, d, norm, o).
    """

    def __init__(self, hidden: int, n_heads: int, vdim: int, state: int, groups: int, taps: int, norm_groups: int,
                 eps: float, *, names: Optional[Dict[str, str]] = None):
        if n_heads % groups:
            raise ValueError(f"mamba2: {n_heads} heads cannot share {groups} groups")
        if (n_heads * vdim) % norm_groups:
            raise ValueError(f"mamba2: the norm's {norm_groups} parts must divide inner = {n_heads * vdim}")
        if not 1 <= taps <= 16:
            raise ValueError(f"mamba2: the convolution kernel takes 1 to 16 taps, got {taps}")
        if state > 256:
            raise ValueError(f"mamba2: the recurrence kernel holds at most 256 rows of a state column, got state {state}")
        self.hidden, self.n_heads, self.vdim, self.state, self.groups = hidden, n_heads, vdim, state, groups
        self.taps, self.norm_groups, self.eps = int(taps), int(norm_groups), float(eps)
        self.inner = n_heads * vdim
        self.bc = groups * state
        self.channels = self.inner + 2 * self.bc
        self.names = {"in": "in_proj.weight", "conv": "conv1d.weight", "conv_bias": "conv1d.bias", "dt_bias": "dt_bias",
                      "a_log": "A_log", "d": "D", "norm": "norm.weight", "o": "out_proj.weight"}
        self.names.update(names or {})
        self.proj: Optional[Linear] = None
        self.dt: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["in"]: ParamSpec((self.inner + self.channels + self.n_heads, self.hidden)),
                # random-weights mode: taps of a size that lets earlier tokens count, step sizes around softplus(0),
                # decays spread between fast and slow heads
                n["conv"]: ParamSpec((self.channels, self.taps), kind="vector", init="normal", std=0.3),
                n["conv_bias"]: ParamSpec((self.channels,), kind="vector", init="normal", std=0.1),
                n["dt_bias"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=1.0),
                n["a_log"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=1.0, mean=-1.0),
                n["d"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=0.5, mean=1.0),
                n["norm"]: ParamSpec((self.inner,), kind="vector", init="ones"),
                n["o"]: ParamSpec((self.hidden, self.inner))}

    def bind(self, params, compute_dtype):
        n = self.names
        w = params[n["in"]]
        split = self.inner + self.channels
        main = w[:split]
        pad = (-split) % 8                              # rows of the product stay 16-byte aligned in bfloat16
        if pad:
            main = torch.cat([main, w.new_zeros((pad, self.hidden))], dim=0)
        self.proj = Linear(main.contiguous())
        self.dt = Linear(w[split:].contiguous())
        self.conv_w = params[n["conv"]].contiguous()
        self.conv_b = params[n["conv_bias"]].to(self.conv_w.dtype).contiguous()
        self.a_log = params[n["a_log"]].contiguous()
        self.dt_bias = params[n["dt_bias"]].to(self.a_log.dtype).contiguous()
        self.norm_w = params[n["norm"]].contiguous()
        self.skip = params[n["d"]].to(self.norm_w.dtype).contiguous()
        self.o = Linear(params[n["o"]])
        self._no_conv_state = None

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "gla", "mamba2"]

    # Prompts run the recurrence in chunks side by side; steps of few tokens per sequence run it token by token.
    CHUNKED_FROM = 17            # tokens of the step's longest portion from which the chunked kernels are taken

    def step_table_names(self):
        return ("retention_chunks",)

    def step_table(self, name, batch):
        return recurrence_chunk_table(batch, self.CHUNKED_FROM)

    def cache_request(self):
        named = dict(S=((self.n_heads, self.state, self.vdim), torch.float32))
        if self.taps > 1:
            named["conv"] = ((self.taps - 1, self.channels), torch.float32)
        return StateRequest.of(**named)

    def gated(self, ctx, y, state_view):
        """The gated, normed inner activations [T, inner] in the compute dtype (the output product's input)."""
        if isinstance(y, ScaledRows):
            y = y.materialize()
        p = self.proj(ctx, y)                                                # [T, z | u | B | C]
        zdt = self.dt(ctx, y, out_f32=True)                                  # [T, heads], 32-bit
        if self.taps > 1:
            conv_state = state_view["conv"]
        else:
            if self._no_conv_state is None:
                self._no_conv_state = torch.empty((0, 0, self.channels), dtype=torch.float32, device=p.device)
            conv_state = self._no_conv_state
        ubc = kernels.conv_silu(p, self.inner, self.channels, conv_state, self.conv_w, self.conv_b, ctx.tok_seq,
                                ctx.cu_q, ctx.seq_slot)                      # float32 [T, u | B | C]
        ab = kernels.mamba_gates(zdt, self.dt_bias, self.a_log)              # (decay, dt)
        u = ubc[:, :self.inner]
        b = ubc[:, self.inner:self.inner + self.bc]
        c = ubc[:, self.inner + self.bc:]
        table = ctx.tables.get("retention_chunks")
        if table is not None and table.numel() > 0:
            s, _ = kernels.gated_chunked(c, b, ab, u, state_view["S"], table, ctx.cu_q, ctx.seq_slot, self.n_heads, self.state,
                                         self.vdim, qk_heads=self.groups)
        else:
            s, _ = kernels.gated_scan(c, b, ab, u, state_view["S"], ctx.cu_q, ctx.seq_slot, self.n_heads, self.state,
                                      self.vdim, qk_heads=self.groups, one_token=ctx.is_decode)
        return kernels.mamba_finish(s, u, p[:, :self.inner], self.skip, self.norm_w, self.norm_groups, self.vdim, self.eps)

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.gated(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.gated(ctx, y, cache_view))
