"""The matrix memory of xLSTM (mLSTM): linear attention whose state is gated by an exponential input gate and a sigmoid
forget gate, one pair per head and token, stabilised by a running maximum of the gates' logarithms."""
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


@MIXERS.register("mlstm")
class MatrixMemory(Mixer):
    """Per head, with q, k of size ``dim`` and v of size ``vdim``:

        li_t = cap tanh((W_i x_t + b_i) / cap),  lf_t = log sigmoid(cap tanh((W_f x_t + b_f) / cap))   (cap None: no cap)
        m_t = max(lf_t + m_(t-1), li_t)                                       (m starts at 0)
        S_t = exp(lf_t + m_(t-1) - m_t) S_(t-1) + exp(li_t - m_t) k_t v_t^T   (S, n start at zero)
        n_t = exp(lf_t + m_(t-1) - m_t) n_(t-1) + exp(li_t - m_t) k_t
        o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6),  q_t = W_q x_t * q_scale (default dim^-1/2)
        out = W_o (concat_h(rms(o_t)) * w * sigmoid(W_g x))                    (rms per head over vdim; w [heads*vdim])

    The product q | k | v | g runs in the compute dtype; the gates' pre-activations come from a second, small product
    whose result stays 32-bit.  The gates and their chain of maxima, q, k, S, n, m, o and its norm are 32-bit.  Per
    sequence the mixer keeps S [heads, dim, vdim], n [heads, dim] and m [heads].  The recurrence itself is the scalar form
    of the gated linear attention's scan (``kernels.gated_scan``) with n as one more column of the state.
    ``names``: the tensors' names below the part's prefix (keys q, k, v, g, o, i, i_bias, f, f_bias, norm).
    """

    def __init__(self, hidden: int, n_heads: int, dim: int, vdim: int, eps: float, *, gate_cap: Optional[float] = None,
                 q_scale: Optional[float] = None, names: Optional[Dict[str, str]] = None):
        if gate_cap is not None and not gate_cap > 0:
            raise ValueError(f"mlstm: the gates' cap must be positive, got {gate_cap}")
        if dim > 256:
            raise ValueError(f"mlstm: the recurrence kernel holds at most 256 rows of a state column, got dim {dim}")
        self.hidden, self.n_heads, self.dim, self.vdim = hidden, n_heads, dim, vdim
        self.eps = float(eps)
        self.gate_cap = float(gate_cap) if gate_cap is not None else None
        self.q_scale = float(q_scale) if q_scale is not None else float(dim) ** -0.5
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                      "o": "o_proj.weight", "i": "i_proj.weight", "i_bias": "i_proj.bias", "f": "f_proj.weight",
                      "f_bias": "f_proj.bias", "norm": "norm.weight"}
        self.names.update(names or {})
        self.qk_size, self.v_size = n_heads * dim, n_heads * vdim
        self.proj: Optional[Linear] = None
        self.gates: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.norm_w = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        return {n["q"]: ParamSpec((self.qk_size, self.hidden)), n["k"]: ParamSpec((self.qk_size, self.hidden)),
                n["v"]: ParamSpec((self.v_size, self.hidden)), n["g"]: ParamSpec((self.v_size, self.hidden)),
                n["o"]: ParamSpec((self.hidden, self.v_size)),
                # random-weights mode: gates that move (input gates around 0, forget gates that mostly keep)
                n["i"]: ParamSpec((self.n_heads, self.hidden), std=0.1),
                n["i_bias"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=1.0),
                n["f"]: ParamSpec((self.n_heads, self.hidden), std=0.1),
                n["f_bias"]: ParamSpec((self.n_heads,), kind="vector", init="normal", std=1.0, mean=3.0),
                n["norm"]: ParamSpec((self.v_size,), kind="vector", init="ones")}

    def bind(self, params, compute_dtype):
        n = self.names
        self.proj = Linear(torch.cat([params[n["q"]], params[n["k"]], params[n["v"]], params[n["g"]]], dim=0).contiguous())
        gw = torch.cat([params[n["i"]], params[n["f"]]], dim=0).contiguous()
        gb = torch.cat([params[n["i_bias"]].to(torch.float32), params[n["f_bias"]].to(torch.float32)]).contiguous()
        self.gates = Linear(gw, gb)
        self.o = Linear(params[n["o"]])
        self.norm_w = params[n["norm"]].contiguous()

    def cuda_modules(self, compute_dtype):
        return ["elementwise", "retention", "gla", "mlstm"]

    # Prompts run the recurrence in chunks side by side; steps of few tokens per sequence run it token by token.
    CHUNKED_FROM = 17            # tokens of the step's longest portion from which the chunked kernels are taken

    def step_table_names(self):
        return ("retention_chunks",)

    def step_table(self, name, batch):
        return recurrence_chunk_table(batch, self.CHUNKED_FROM)

    def cache_request(self):
        return StateRequest.of(S=((self.n_heads, self.dim, self.vdim), torch.float32),
                               n=((self.n_heads, self.dim), torch.float32), m=((self.n_heads,), torch.float32))

    def gated(self, ctx, y, state_view):
        """The normed, gated heads [T, heads*vdim] in the compute dtype (the output product's input)."""
        if isinstance(y, ScaledRows):
            y = y.materialize()
        p = self.proj(ctx, y)                                                # [T, q | k | v | g]
        z = self.gates(ctx, y, out_f32=True)                                 # [T, i | f] pre-activations, 32-bit
        qk = kernels.mlstm_prepare(p, 0, self.qk_size, self.qk_size, self.q_scale)
        ab, mt = kernels.mlstm_gates(z, state_view["m"], ctx.cu_q, ctx.seq_slot, self.n_heads, self.gate_cap or 0.0,
                                     ctx.max_new)
        v = p[:, 2 * self.qk_size: 2 * self.qk_size + self.v_size]
        g = p[:, 2 * self.qk_size + self.v_size: 2 * self.qk_size + 2 * self.v_size]
        table = ctx.tables.get("retention_chunks")
        if table is not None and table.numel() > 0:
            o, qn = kernels.gated_chunked(qk[0], qk[1], ab, v, state_view["S"], table, ctx.cu_q, ctx.seq_slot, self.n_heads,
                                          self.dim, self.vdim, nstate=state_view["n"])
        else:
            o, qn = kernels.gated_scan(qk[0], qk[1], ab, v, state_view["S"], ctx.cu_q, ctx.seq_slot, self.n_heads, self.dim,
                                       self.vdim, nstate=state_view["n"], one_token=ctx.is_decode)
        return kernels.retention_gate(o, g, self.n_heads, self.vdim, self.eps, weight=self.norm_w, gate_fn="sigmoid",
                                      denominator=(qn, mt))

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.gated(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.gated(ctx, y, cache_view))
