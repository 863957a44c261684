"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math
from typing import Dict, Optional

import numpy as np
import torch

from .. import kernels
from ..cache.requests import KVRequest
from ..engine.stream import ScaledRows
from ..weights.spec import ParamSpec
from .base import MIXERS, Mixer, POSITIONS
from .linear import Linear


@MIXERS.register("gqa_attention")
class GQAAttention(Mixer):
    """q/k/v projections (with or without bias), rotation of q and k, write of k and v into
    the cache, softmax attention of the new tokens over the cache, output projection.

    Order and formulas follow maeddesg/ROCmForge src/gpu/forward.rs:940-1079 (prefill) and
    :2361-2472 (decode): the bias is added after the product and before the rotation;
    head h reads kv head h // (heads / kv_heads); scores are scaled by 1/sqrt(head_dim)
    (forward.rs:583); a query at position p sees keys 0..=p, or the last ``window`` of them.
    The three projections are fused into one matrix at load time (the reference fuses them
    in its decode kernels, src/gpu/ops.rs:748-880).

    Options that other designs use, all off by default: ``v_head_dim`` (values of another size than keys),
    ``qk_norm_eps`` (every query and key head divided by its root mean square, x / sqrt(mean(x^2) + eps), no weight,
    before the rotation), ``softcap`` (score <- softcap * tanh(score / softcap) after scaling), ``distance_slopes``
    (one slope per head: after the cap a score is lowered by slope * (query position - key position)), ``names``
    (the tensors' names below the part's prefix, keys q, k, v, o, and g, q_norm, k_norm where they exist),
    ``qk_norm_weight`` (the normed query heads are multiplied by a weight [head_dim] shared by all of them, the key heads
    by another), ``chunk`` (position i sees j <= i only inside its own chunk of ``chunk`` positions, chunks counted from
    position 0 of the sequence, however the prompt is cut into steps), ``gate`` ("sigmoid": the concatenated heads are
    multiplied by sigmoid(W_g x) before the output projection; W_g reads the same input as q, k, v and is part of the same
    product), ``shares_kv`` (the mixer has no key and value tensors: the schedule lets it read another execution's
    cache, ``ScheduleEntry.kv_from``, with queries, mask and everything else of its own) and ``cache_keeps`` (what the
    cache must keep when other mixers read it with masks of their own: "all", or None for this mixer's own mask),
    ``keep_first`` (with a window: the first ``keep_first`` positions of a sequence stay visible to every later query, at
    their own positions; the cache keeps their pages) and ``gate`` "sigmoid_head" (one gate per head, W_g of ``heads``
    rows: head h's output is multiplied by sigmoid(W_g x)_h).  A position encoding whose rotation carries a ``magnitude``
    (sine and cosine times a factor) goes through the per-head writer as well.  Normed heads and values of another size go into the
    cache through the per-head writer.  ``sink``: a learned number per head (tensor ``names["sink"]``, [heads]) whose
    exponential counts once in the softmax's denominator, with no key, no value and no scaling.
    ``qk_norm_after_rotation``: the division of ``qk_norm_eps`` is applied to the heads as they are after the rotation.
    ``q_temperature`` = (coef, every): the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).
    ``values_are_keys``: the mixer has no value projection; its values are its keys as they lie in the cache, which then
    holds keys alone.  With any of these (as with normed heads) biases are added by the per-head writer.
    A cap, slopes and kept first positions are known to the generic attention and to the
    tcgen05 prompt attention and the clustered decode attention (heads of 64 or 128 with values of the same size), so such a mixer runs
    on the same kernels as one without them.
    """

    accepts_scaled_rows = True

    def __init__(self, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int, *, qkv_bias: bool,
                 o_bias: bool = False, window: Optional[int] = None, position=None,
                 scale: Optional[float] = None, v_head_dim: Optional[int] = None, qk_norm_eps: Optional[float] = None,
                 softcap: Optional[float] = None, distance_slopes=None, names: Optional[Dict[str, str]] = None,
                 qk_norm_weight: bool = False, chunk: Optional[int] = None, gate: Optional[str] = None,
                 shares_kv: bool = False, cache_keeps: Optional[str] = None, keep_first: int = 0, sink: bool = False,
                 qk_norm_after_rotation: bool = False, q_temperature=None, values_are_keys: bool = False):
        if n_heads % n_kv_heads:
            raise ValueError(f"{n_heads} heads cannot share {n_kv_heads} kv heads")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.qkv_bias, self.o_bias, self.window = qkv_bias, o_bias, window
        self.position = position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.v_head_dim = head_dim if v_head_dim is None else int(v_head_dim)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.softcap = float(softcap) if softcap else None
        self.distance_slopes = None if distance_slopes is None else [float(s) for s in distance_slopes]
        if self.distance_slopes is not None and len(self.distance_slopes) != n_heads:
            raise ValueError(f"{len(self.distance_slopes)} distance slopes for {n_heads} heads")
        self.slopes_dev = None
        self.names = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "o": "o_proj.weight",
                      "g": "g_proj.weight", "q_norm": "q_norm.weight", "k_norm": "k_norm.weight", "sink": "sinks",
                      "q_bias": "q_proj.bias", "k_bias": "k_proj.bias", "v_bias": "v_proj.bias"}
        self.names.update(names or {})
        self.chunk = int(chunk) if chunk else None
        if self.chunk is not None and window:
            raise ValueError("gqa_attention: a window or chunks, not both")
        if gate not in (None, "sigmoid", "sigmoid_head"):
            raise ValueError(f"gqa_attention: gate {gate!r} has no kernel (sigmoid, sigmoid_head)")
        self.keep_first = int(keep_first or 0)
        if self.keep_first < 0 or (self.keep_first and self.chunk is not None):
            raise ValueError("gqa_attention: keep_first is a number of first positions kept beside a window")
        if not window:
            self.keep_first = 0                           # without a window every earlier position is visible anyway
        if cache_keeps not in (None, "all"):
            raise ValueError(f"gqa_attention: cache_keeps {cache_keeps!r} (all, or None)")
        self.gate, self.shares_kv, self.cache_keeps = gate, bool(shares_kv), cache_keeps
        self.sink = bool(sink)
        self.sinks_dev = None
        self.norm_after = bool(qk_norm_after_rotation)
        if self.norm_after and qk_norm_eps is None:
            raise ValueError("gqa_attention: qk_norm_after_rotation goes with qk_norm_eps")
        self.q_temperature = None if q_temperature is None else (float(q_temperature[0]), float(q_temperature[1]))
        if self.q_temperature is not None and not self.q_temperature[1] > 0:
            raise ValueError("gqa_attention: the query temperature's step must be a positive number of positions")
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys and ((v_head_dim is not None and v_head_dim != head_dim) or shares_kv):
            raise ValueError("gqa_attention: keys that serve as values have the keys' size and a cache of their own")
        self.qk_norm_weight = bool(qk_norm_weight)
        if self.qk_norm_weight and qk_norm_eps is None:
            raise ValueError("gqa_attention: norm weights go with qk_norm_eps")
        self.q_norm_w = self.k_norm_w = None
        self.q_size = n_heads * head_dim
        self.kv_size = n_kv_heads * head_dim
        self.v_size = 0 if self.values_are_keys else n_kv_heads * self.v_head_dim
        self.o_in = n_heads * self.v_head_dim
        self.gate_rows = n_heads if gate == "sigmoid_head" else self.o_in
        self.magnitude = float(((position.rotation() if position is not None else None) or {}).get("magnitude", 1.0))
        # normed heads and values of another size: the per-head cache writer; a cap or slopes: no mma.sync kernel knows them
        self.plain_projection = (self.v_head_dim != head_dim or self.qk_norm_eps is not None or self.gate is not None
                                 or self.shares_kv or self.magnitude != 1.0 or self.q_temperature is not None
                                 or self.values_are_keys)
        self.shaped_scores = self.softcap is not None or self.distance_slopes is not None
        self.plain_only = self.plain_projection or self.shaped_scores
        if self.plain_only and o_bias:
            raise ValueError("gqa_attention: an output bias does not go with the per-head writer or shaped scores")
        if self.shaped_scores and qkv_bias and not self.plain_projection:
            raise ValueError("gqa_attention: biases with a score cap or distance slopes need the per-head writer")
        if qkv_bias and self.shares_kv:
            raise ValueError("gqa_attention: biases do not go with a borrowed cache")
        self.plain_bias = None
        self.qkv: Optional[Linear] = None
        self.o: Optional[Linear] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        n = self.names
        s = {n["q"]: ParamSpec((self.q_size, self.hidden)), n["o"]: ParamSpec((self.hidden, self.o_in))}
        if not self.shares_kv:
            s[n["k"]] = ParamSpec((self.kv_size, self.hidden))
            if not self.values_are_keys:
                s[n["v"]] = ParamSpec((self.v_size, self.hidden))
        if self.sink:
            s[n["sink"]] = ParamSpec((self.n_heads,), kind="vector", init="normal", std=1.0)
        if self.gate is not None:
            s[n["g"]] = ParamSpec((self.gate_rows, self.hidden))
        if self.qk_norm_weight:
            s[n["q_norm"]] = ParamSpec((self.head_dim,), kind="vector", init="ones")
            if not self.shares_kv:
                s[n["k_norm"]] = ParamSpec((self.head_dim,), kind="vector", init="ones")
        if self.qkv_bias:
            s[n["q_bias"]] = ParamSpec((self.q_size,), kind="vector")
            s[n["k_bias"]] = ParamSpec((self.kv_size,), kind="vector")
            if not self.values_are_keys:
                s[n["v_bias"]] = ParamSpec((self.v_size,), kind="vector")
        if self.o_bias:
            s["o_proj.bias"] = ParamSpec((self.hidden,), kind="vector")
        return s

    def bind(self, params, compute_dtype):
        n = self.names
        # one product for everything that reads the mixer's input: q | k | v | gate (k, v absent with a borrowed cache)
        blocks = [params[n["q"]]] + ([] if self.shares_kv else [params[n["k"]]] + ([] if self.values_are_keys else [params[n["v"]]]))
        self.gate_col = self.q_size + (0 if self.shares_kv else self.kv_size + self.v_size)
        if self.gate is not None:
            g = params[n["g"]]
            pad = (-self.gate_col) % 8                    # the gate's columns start on a 16-byte boundary
            if pad:
                blocks.append(g.new_zeros((pad, self.hidden)))
                self.gate_col += pad
            blocks.append(g)
            if (self.gate_col + self.gate_rows) % 8:      # and the rows of the product stay 16-byte aligned
                blocks.append(g.new_zeros(((-(self.gate_col + self.gate_rows)) % 8, self.hidden)))
        w = torch.cat(blocks, dim=0)
        if self.qk_norm_weight:
            self.q_norm_w = params[n["q_norm"]]
            self.k_norm_w = None if self.shares_kv else params[n["k_norm"]].to(self.q_norm_w.dtype)
        b = None
        if self.qkv_bias:
            bs = [params[n["q_bias"]], params[n["k_bias"]]] + ([] if self.values_are_keys else [params[n["v_bias"]]])
            dt = torch.float32 if any(x.dtype == torch.float32 for x in bs) else bs[0].dtype
            b = torch.cat([x.to(dt) for x in bs]).contiguous()
            if self.plain_projection:                     # the per-head writer adds it (the product may carry more columns)
                self.plain_bias, b = b, None
        if self.sink:
            self.sinks_dev = params[n["sink"]].to(torch.float32).contiguous()
        self.qkv = Linear(w.contiguous(), b)
        self.o = Linear(params[n["o"]], params.get("o_proj.bias"))
        if self.position is not None:
            self.position.prepare(w.device)
        if self.distance_slopes is not None:
            self.slopes_dev = torch.tensor(self.distance_slopes, dtype=torch.float32, device=w.device)

    def cuda_modules(self, compute_dtype):
        mods = ["elementwise", "attention_generic"]
        if compute_dtype == torch.bfloat16 and self.v_head_dim == self.head_dim:
            mods += ["attention_decode", "attention_prefill_tc"]
            if not self.shaped_scores and not self.keep_first and not self.sink:
                mods.append("attention_prefill")         # the mma.sync prompt kernel knows no cap and no slopes
        return mods

    def cache_request(self):
        if self.shares_kv:
            return None                                   # the schedule names the execution whose cache it reads
        keeps_all = self.cache_keeps == "all"
        return KVRequest(self.n_kv_heads, self.head_dim, None if keeps_all else self.window,
                         None if self.v_head_dim == self.head_dim else self.v_head_dim,
                         None if keeps_all else self.chunk, 0 if keeps_all else self.keep_first, self.values_are_keys)

    # rows of the query tiles of the two tiled prefill kernels (csrc/attention_prefill.cu, attention_prefill_tc.cu)
    TILE_ROWS = {"attention_tiles64": 64, "attention_tiles128": 128}

    def step_table_names(self):
        if self.v_head_dim != self.head_dim:
            return ()
        return ("attention_tiles128",) if self.keep_first or self.sink else tuple(self.TILE_ROWS)

    def step_table(self, name, batch):
        """(sequence, first row) of every query tile of the step's new tokens, sorted by the keys a tile sees (the
        kernels start with the heaviest): decided on the host so that the device never searches.  Steps of one token
        per sequence need none."""
        if batch.is_decode:
            return np.zeros((0,), dtype=np.int32)
        rows = self.TILE_ROWS[name]
        tiles = [(i, q0) for i in range(batch.B) for q0 in range(0, int(batch.n_new[i]), rows)]
        tiles.sort(key=lambda t: int(batch.starts[t[0]]) + t[1])
        return np.asarray(tiles, dtype=np.int32).reshape(-1)

    def forward(self, ctx, y, cache_view, stream):
        self.o.add_to_stream(ctx, self.heads_out(ctx, y, cache_view), stream)

    def output(self, ctx, y, cache_view):
        return self.o.f32_parts(ctx, self.heads_out(ctx, y, cache_view))

    def heads_out(self, ctx, y, cache_view):
        """The concatenated heads (gated, if the mixer has a gate): the output projection's input."""
        if self.shares_kv and (cache_view is None or cache_view.writes):
            raise RuntimeError("gqa_attention: a mixer without keys and values must be scheduled with kv_from")
        q = self.project_into_cache(ctx, y, cache_view)                     # rotated q; k, v are in the cache
        o = self.attend(ctx, q, cache_view)
        if self.gate is not None:
            o = kernels.sigmoid_gate(o, self._gate_cols, group=self.o_in // self.gate_rows)
        return o

    def _project_plain(self, ctx, y, view, rot, inv_freq):
        """The projection for heads that are normed or values of another size: one product (K-split partial sums with
        few tokens), then a warp per head norms, turns and writes."""
        tc = kernels.tensor_core
        w = self.qkv.weight
        if isinstance(y, ScaledRows):
            y = y.materialize()
        common = dict(compute_dtype=ctx.compute_dtype, rot_dim=rot["rot_dim"], interleaved=rot.get("interleaved", False),
                      unit_norm_eps=self.qk_norm_eps, q_norm_weight=self.q_norm_w, k_norm_weight=self.k_norm_w,
                      magnitude=self.magnitude, bias=self.plain_bias, norm_after_rotation=self.norm_after,
                      q_temperature=self.q_temperature, values_are_keys=self.values_are_keys)
        writes = view.writes and not self.shares_kv
        args = (self.n_heads, self.n_kv_heads, self.head_dim, self.v_head_dim, inv_freq, ctx.tok_seq, ctx.tok_pos,
                ctx.seq_slot, view.block_table, view.k_pages, view.v_pages, writes)
        if self.gate is None and y.shape[0] <= tc.SKINNY_MAX_TOKENS:        # (a gate is read from the product's own output)
            if ctx.uses_tensor_cores(y, w, tc.PARTIAL):
                splits = tc.split_k_for(w.shape[0], w.shape[1], tokens=y.shape[0])
                if splits > 1:
                    return kernels.head_norm_kv_write(tc.gemm_tc_skinny(y, w, mode=tc.PARTIAL, splits=splits), *args, **common)
            elif not ctx.uses_tensor_cores(y, w, tc.STORE):
                splits = kernels.split_k_for_simt(w.shape[0], w.shape[1])
                if splits > 1:
                    return kernels.head_norm_kv_write(kernels.gemm_simt(y, w, splits=splits), *args, **common)
        p = ctx.matmul(y, w)
        if self.gate is not None:
            self._gate_cols = p[:, self.gate_col:self.gate_col + self.gate_rows]
        return kernels.head_norm_kv_write(p, *args, **common)

    def project_into_cache(self, ctx, y, view):
        """q/k/v projection (+ bias), rotation, cache write; returns rotated q [T, >= heads*head_dim].

        With few tokens on the tensor-core path the product is K-split for parallelism and the
        rotation kernel sums the 32-bit partial sums (and the bias) itself, so q/k/v never
        exist as an intermediate bfloat16 tensor.
        """
        tc = kernels.tensor_core
        w, bias = self.qkv.weight, self.qkv.bias
        y, row_ss = ctx.unpack_rows(y, w, tc.PARTIAL)
        rot = dict((self.position.rotation() if self.position is not None else None) or dict(inv_freq=None, rot_dim=0))
        inv_freq = rot.pop("inv_freq")
        rot.pop("magnitude", None)
        if self.plain_projection:
            return self._project_plain(ctx, y, view, rot, inv_freq)
        rope = dict(rot_dim=rot["rot_dim"], interleaved=rot.get("interleaved", False), tok_seq=ctx.tok_seq, tok_pos=ctx.tok_pos, seq_slot=ctx.seq_slot,
                    block_table=view.block_table, k_pages=view.k_pages, v_pages=view.v_pages, write_kv=view.writes)
        if y.shape[0] <= tc.SKINNY_MAX_TOKENS and ctx.uses_tensor_cores(y, w, tc.PARTIAL):
            splits = tc.split_k_for(w.shape[0], w.shape[1], tokens=y.shape[0])
            if splits > 1:
                parts = tc.gemm_tc_skinny(y, w, mode=tc.PARTIAL, splits=splits, row_ss=row_ss)
                return kernels.rope_kv_write(parts, self.n_heads, self.n_kv_heads, self.head_dim,
                                             inv_freq, bias=bias, compute_dtype=ctx.compute_dtype,
                                             **rope)
        if row_ss is not None:
            y = ScaledRows(y, row_ss[0], row_ss[1], w.shape[1])
        elif y.shape[0] <= tc.SKINNY_MAX_TOKENS and not ctx.uses_tensor_cores(y, w, tc.STORE):
            splits = kernels.split_k_for_simt(w.shape[0], w.shape[1])
            if splits > 1:                           # CUDA-core product of few tokens: the same scheme
                parts = kernels.gemm_simt(y, w, splits=splits)
                return kernels.rope_kv_write(parts, self.n_heads, self.n_kv_heads, self.head_dim,
                                             inv_freq, bias=bias, compute_dtype=ctx.compute_dtype,
                                             **rope)
        qkv = ctx.matmul(y, w, bias)
        return kernels.rope_kv_write(qkv, self.n_heads, self.n_kv_heads, self.head_dim,
                                     inv_freq, **rope)

    def attend(self, ctx, q, view):
        """Attention of the step's tokens over the cache; q is the first heads*head_dim columns of ``q``."""
        nh, nkv, hd = self.n_heads, self.n_kv_heads, self.head_dim
        tiles64, tiles128 = ctx.tables.get("attention_tiles64"), ctx.tables.get("attention_tiles128")
        longest = ctx.model_cache_limit if ctx.replayed else ctx.max_end
        shaped = dict(softcap=self.softcap, slopes=self.slopes_dev, chunk=self.chunk)
        span = self.window or self.chunk                  # the most keys a query sees
        # kept first positions: the generic kernel, the tcgen05 prompt kernel and the clustered decode kernel walk the
        # pages that hold them before the window's
        kept = dict(keep_first=self.keep_first)
        shaped["sinks"] = self.sinks_dev                  # (None without): known to the same kernels as a cap and slopes
        if (self.v_head_dim != hd
                or ((self.shaped_scores or self.keep_first or self.sink) and ctx.compute_dtype != torch.bfloat16)):
            return kernels.attention_generic(q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos,
                                             ctx.seq_slot, view.block_table, self.scale, self.window,
                                             v_head_dim=self.v_head_dim, **shaped, **kept)
        if (ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and kernels.attention_decode_supported(nh, nkv, hd)):
            if ctx.options.clustered_decode:
                # a cluster of 1..8 CTAs per (sequence, kv head), every warp on its own tiles of keys, merged
                # through distributed shared memory: no scratch memory, no second pass, any context length
                return kernels.attention_decode_warps(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                    view.block_table, self.scale, self.window,
                    splits=kernels.decode_splits(ctx.B, nkv, longest, span), **shaped, **kept)
            if (not self.shaped_scores and not self.keep_first and not self.sink
                    and longest <= kernels.DECODE_CHUNK * kernels.DECODE_CHUNK):
                # the earlier kernel: one CTA per 128-key chunk, partial results merged through scratch memory
                need = max(1, (longest + kernels.DECODE_CHUNK - 1) // kernels.DECODE_CHUNK)
                max_chunks = 1
                while max_chunks < need:                   # powers of two: few distinct scratch sizes
                    max_chunks *= 2
                cap = 1
                while cap < ctx.B:
                    cap *= 2
                n_o, n_ml, n_c = kernels.attention_decode_scratch(cap, nh, nkv, hd, max_chunks)
                scratch = ctx.model.scratch
                return kernels.attention_decode(
                    q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos, ctx.seq_slot,
                    view.block_table, self.scale, self.window, max_chunks,
                    scratch("attn_decode_o", n_o, torch.float32), scratch("attn_decode_ml", n_ml, torch.float32),
                    kernels.tensor_core.register_counters(scratch("attn_decode_counters", n_c, torch.int32)),
                    chunk=self.chunk)
        if (not ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and ctx.options.tcgen05_attention and tiles128 is not None and tiles128.numel() > 0
                and kernels.attention_prefill_tc_supported(nh, nkv, hd)
                and q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0):
            return kernels.attention_prefill_tc(q, nh, nkv, hd, view.k_pages, view.v_pages, tiles128,
                                                ctx.seq_slot, ctx.seq_start, ctx.seq_nnew, ctx.cu_q,
                                                view.block_table, self.scale, self.window, **shaped, **kept)
        if self.shaped_scores or self.keep_first or self.sink:
            return kernels.attention_generic(q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos,
                                             ctx.seq_slot, view.block_table, self.scale, self.window, **shaped, **kept)
        if (not ctx.is_decode and ctx.compute_dtype == torch.bfloat16 and ctx.options.tuned_attention
                and tiles64 is not None and tiles64.numel() > 0 and kernels.attention_prefill_supported(nh, nkv, hd)
                and q.data_ptr() % 4 == 0 and q.stride(0) % 2 == 0):
            return kernels.attention_prefill(q, nh, nkv, hd, view.k_pages, view.v_pages, tiles64, ctx.seq_slot,
                                             ctx.seq_start, ctx.seq_nnew, ctx.cu_q, view.block_table, self.scale,
                                             self.window, chunk=self.chunk)
        return kernels.attention_generic(q, nh, nkv, hd, view.k_pages, view.v_pages, ctx.tok_seq, ctx.tok_pos,
                                         ctx.seq_slot, view.block_table, self.scale, self.window, chunk=self.chunk)

