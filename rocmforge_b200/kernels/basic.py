"""Python faces of the plain kernels: embedding, add+RMSNorm, rotation + cache write,
SwiGLU, the CUDA-core matrix product, the generic attention and argmax.

Each function checks shapes and dtypes, then launches on torch's current stream.
"""
from __future__ import annotations

import functools

import torch

from ._ffi import (KernelError, sm_count as device_sm_count, c_float, c_int, c_ll, c_void_p, check, dtype_code, fn, need, need_cuda,
                   ptr, stream)

PAGE = 64      # tokens per cache page (RF_PAGE in csrc/common.cuh)


@functools.lru_cache(None)
def _f(module, name, *argtypes):
    return fn(module, name, list(argtypes))


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """out[t] = table[ids[t]] widened to float32 (times ``scale``, the product formed in 32-bit)."""
    need_cuda(table, ids)
    need(table.dim() == 2 and table.is_contiguous(), "embed: table must be a contiguous matrix")
    need(ids.dtype == torch.int32 and ids.dim() == 1, "embed: ids must be a 1-d int32 tensor")
    V, H = table.shape
    T = ids.shape[0]
    if out is None:
        out = torch.empty((T, H), dtype=torch.float32, device=table.device)
    if scale is not None and float(scale) != 1.0:
        f = _f("elementwise", "rf_embed_scaled", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p)
        check(f(dtype_code(table.dtype), ptr(table), ptr(ids), ptr(out), T, H, V, float(scale), stream()), "embed")
        return out
    f = _f("elementwise", "rf_embed", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(table.dtype), ptr(table), ptr(ids), ptr(out), T, H, V, stream()), "embed")
    return out


def embed_positions(table: torch.Tensor, ids: torch.Tensor, pos_table: torch.Tensor | None, tok_pos: torch.Tensor | None,
                    rounded: bool = False):
    """(h, y): h[t] = table[ids[t]] (+ pos_table[tok_pos[t]], a learned vector per position) as float32, the sum formed
    in 32-bit; y is h in the table's dtype if ``rounded`` (for sub-layers that read the stream itself), else None."""
    need_cuda(table, ids, pos_table, tok_pos)
    need(table.dim() == 2 and table.is_contiguous(), "embed: table must be a contiguous matrix")
    need(ids.dtype == torch.int32 and ids.dim() == 1, "embed: ids must be a 1-d int32 tensor")
    V, H = table.shape
    T = ids.shape[0]
    P = 0
    if pos_table is not None:
        need(pos_table.dim() == 2 and pos_table.shape[1] == H and pos_table.is_contiguous() and pos_table.dtype == table.dtype,
             "embed: the position table must be [positions, H] of the embedding's dtype")
        need(tok_pos is not None and tok_pos.dtype == torch.int32 and tok_pos.shape == (T,), "embed: one int32 position per token")
        P = pos_table.shape[0]
    h = torch.empty((T, H), dtype=torch.float32, device=table.device)
    y = torch.empty((T, H), dtype=table.dtype, device=table.device) if rounded else None
    f = _f("elementwise", "rf_embed_pos", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int,
           c_void_p, c_void_p)
    check(f(dtype_code(table.dtype), ptr(table), ptr(ids), ptr(h), T, H, V, ptr(pos_table), ptr(tok_pos), P, ptr(y), stream()),
          "embed_positions")
    return h, y


def round_rows(h: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream rounded to ``dtype`` (a copy)."""
    need_cuda(h)
    need(h.dtype == torch.float32 and h.is_contiguous(), "round_rows: a contiguous float32 tensor")
    out = torch.empty(h.shape, dtype=dtype, device=h.device)
    f = _f("elementwise", "rf_round_rows", c_int, c_void_p, c_void_p, c_ll, c_void_p)
    check(f(dtype_code(dtype), ptr(h), ptr(out), h.numel(), stream()), "round_rows")
    return out


def clamped_glu(gu: torch.Tensor, limit: float, alpha: float, row_scale: torch.Tensor | None = None) -> torch.Tensor:
    """a[t, j] = g sigmoid(alpha g) (u + 1) with g = min(s gu[t, 2j], limit), u = clamp(s gu[t, 2j+1], -limit, limit) and
    s = row_scale[t] (float32 [T]; 1 without), evaluated in 32-bit."""
    need_cuda(gu, row_scale)
    need(gu.dim() == 2 and gu.is_contiguous() and gu.shape[1] % 2 == 0, "clamped_glu: input must be [T, 2I]")
    T, I2 = gu.shape
    need(row_scale is None or (row_scale.dtype == torch.float32 and row_scale.numel() >= T and row_scale.is_contiguous()),
         "clamped_glu: row_scale must be float32 [T]")
    out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    f = _f("elementwise", "rf_clamped_glu", c_int, c_void_p, c_void_p, c_int, c_int, c_float, c_float, c_void_p, c_void_p)
    check(f(dtype_code(gu.dtype), ptr(gu), ptr(out), T, I2 // 2, float(limit), float(alpha), ptr(row_scale), stream()), "clamped_glu")
    return out


def sigmoid_gate(x: torch.Tensor, gate: torch.Tensor, group: int = 1) -> torch.Tensor:
    """x * sigmoid(gate), 32-bit inside; x [T, W] and gate [T, W / group] views with unit inner stride: column c of x is
    gated by column c // group (``group`` 1: a gate per element; a head's size: one gate per head)."""
    need_cuda(x, gate)
    need(x.dim() == 2 and group >= 1 and x.shape[1] % group == 0 and gate.shape == (x.shape[0], x.shape[1] // group)
         and x.stride(1) == 1 and gate.stride(1) == 1 and x.dtype == gate.dtype,
         "sigmoid_gate: x [T, W] and gate [T, W / group] must share a dtype")
    T, W = x.shape
    out = torch.empty((T, W), dtype=x.dtype, device=x.device)
    f = _f("elementwise", "rf_sigmoid_gate", c_int, c_void_p, c_int, c_void_p, c_int, c_void_p, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(x.dtype), ptr(x), x.stride(0), ptr(gate), gate.stride(0), ptr(out), T, W, int(group), stream()),
          "sigmoid_gate")
    return out


def add_rmsnorm(h: torch.Tensor, weight: torch.Tensor, eps: float, compute_dtype: torch.dtype,
                pending: torch.Tensor | None = None, rows: torch.Tensor | None = None,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """y = rmsnorm(h + pending) * weight.

    ``h`` [T, H] float32 is the residual stream.  ``pending`` is None, a float32
    [S, T, H] stack of partial sums, or a [T, H] tensor of the compute dtype; without
    ``rows`` it is added into ``h`` in place.  With ``rows`` (int32 indices) only those
    rows are normalised and ``h`` is left untouched.
    """
    need_cuda(h, weight, pending, rows)
    need(h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous(), "add_rmsnorm: h must be [T,H] float32")
    T, H = h.shape
    need(weight.shape == (H,) and weight.dtype in (torch.float32, torch.bfloat16),
         "add_rmsnorm: weight must be [H] in float32 or bfloat16")
    kind, n_pending, pstride = 0, 0, 0
    if pending is not None:
        need(pending.is_contiguous(), "add_rmsnorm: pending must be contiguous")
        if pending.dtype == torch.float32 and pending.dim() == 3 and pending.shape[1:] == (T, H):
            kind, n_pending, pstride = 1, pending.shape[0], T * H
        elif pending.dtype == torch.float32 and pending.shape == (T, H) and compute_dtype == torch.float32:
            kind = 2
        elif pending.dtype == torch.float32 and pending.shape == (T, H):
            kind, n_pending, pstride = 1, 1, T * H
        elif pending.dtype == compute_dtype and pending.shape == (T, H):
            kind = 2
        else:
            raise KernelError(f"add_rmsnorm: pending of shape {tuple(pending.shape)} / {pending.dtype} "
                              f"does not fit h {tuple(h.shape)}")
    n_rows = T
    if rows is not None:
        need(rows.dtype == torch.int32 and rows.dim() == 1, "add_rmsnorm: rows must be 1-d int32")
        n_rows = rows.shape[0]
    if out is None:
        out = torch.empty((n_rows, H), dtype=compute_dtype, device=h.device)
    from .tensor_core import status_word
    f = _f("elementwise", "rf_add_rmsnorm", c_int, c_void_p, c_void_p, c_int, c_int, c_ll, c_void_p, c_int,
           c_float, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(pending), kind, n_pending, pstride, ptr(weight),
            int(weight.dtype == torch.float32), float(eps), ptr(out), ptr(rows), n_rows, H,
            ptr(status_word(h.device)), stream()),
          f"add_rmsnorm (H={H})")
    return out


def rope_kv_write(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, inv_freq: torch.Tensor,
                  tok_seq, tok_pos, seq_slot, block_table: torch.Tensor,
                  k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, write_kv: bool = True, *,
                  bias: torch.Tensor | None = None, compute_dtype: torch.dtype | None = None,
                  q_out: torch.Tensor | None = None, rot_dim: int | None = None,
                  interleaved: bool = False) -> torch.Tensor:
    """Rotate q and k by position; write rotated k and v into their cache pages; return q.

    The first ``rot_dim`` elements of every query and key head turn (default: the whole head; 0: none, and
    ``inv_freq`` may then be None), as pairs (i, i + rot_dim/2) or, ``interleaved``, (2i, 2i+1), pair i by the angle
    position * inv_freq[i]; the other elements pass through.

    ``qkv`` is [T, (heads + 2 kv_heads) * head_dim] in the compute dtype (q is then rotated in place and
    the returned q is a view of it), or a float32 stack [S, T, ...] of partial sums of a K-split product,
    to which ``bias`` is added (q then goes to a new [T, heads * head_dim] tensor of ``compute_dtype``).
    """
    need_cuda(qkv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, k_pages, v_pages, bias)
    width = (n_heads + 2 * n_kv_heads) * head_dim
    partials = qkv.dim() == 3
    if partials:
        need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[2] == width,
             "rope_kv_write: partial sums must be a contiguous float32 [S, T, width] stack")
        need(compute_dtype is not None, "rope_kv_write: partial sums need the compute dtype")
        S, T = qkv.shape[0], qkv.shape[1]
        dt = compute_dtype
        if q_out is None:
            q_out = torch.empty((T, n_heads * head_dim), dtype=dt, device=qkv.device)
        row_stride, pstride = width, T * width
    else:
        need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] == width,
             "rope_kv_write: qkv must be [T, (heads + 2 kv_heads) * head_dim]")
        need(bias is None, "rope_kv_write: a bias goes with partial sums only")
        S, T, dt = 0, qkv.shape[0], qkv.dtype
        q_out = qkv
        row_stride, pstride = qkv.stride(0), 0
    rot_dim = head_dim if rot_dim is None else int(rot_dim)
    need(0 <= rot_dim <= head_dim and rot_dim % 2 == 0, f"rope_kv_write: rot_dim {rot_dim} must be even and at most head_dim")
    need(rot_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2),
         "rope_kv_write: inv_freq must hold rot_dim/2 float32 frequencies")
    if write_kv:
        for p in (k_pages, v_pages):
            need(p is not None and p.dtype == dt and p.is_contiguous()
                 and tuple(p.shape[1:]) == (n_kv_heads, PAGE, head_dim),
                 "rope_kv_write: pages must be [n_pages, kv_heads, 64, head_dim] of the compute dtype")
    f = _f("elementwise", "rf_rope_kv_write", c_int, c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_void_p, c_int,
           c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int,
           c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(dt), ptr(qkv), row_stride, S, pstride, ptr(bias),
            int(bias is not None and bias.dtype == torch.float32), ptr(q_out), q_out.stride(0), n_heads, n_kv_heads,
            head_dim, ptr(inv_freq), ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table),
            block_table.shape[1], ptr(k_pages), ptr(v_pages), int(write_kv), T, rot_dim, int(interleaved), stream()),
          "rope_kv_write")
    return q_out


def swiglu(gu: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """a[t, j] = silu(gu[t, 2j]) * gu[t, 2j+1]."""
    need_cuda(gu)
    need(gu.dim() == 2 and gu.is_contiguous() and gu.shape[1] % 2 == 0, "swiglu: input must be [T, 2I]")
    T, I2 = gu.shape
    if out is None:
        out = torch.empty((T, I2 // 2), dtype=gu.dtype, device=gu.device)
    f = _f("elementwise", "rf_swiglu", c_int, c_void_p, c_void_p, c_int, c_int, c_void_p)
    check(f(dtype_code(gu.dtype), ptr(gu), ptr(out), T, I2 // 2, stream()), "swiglu")
    return out


def split_k_for_simt(N: int, K: int, sm_count: int | None = None) -> int:
    """K splits of a CUDA-core product of few tokens, from N and K alone (never from the batch): about two CTAs
    per SM, every split at least 4 blocks of 16."""
    sm_count = sm_count or device_sm_count()
    tiles = (N + 127) // 128
    kb = (K + 15) // 16
    if tiles >= 2 * sm_count or kb < 8:
        return 1
    splits = max(1, min((2 * sm_count) // tiles, kb // 4))
    per = (kb + splits - 1) // splits
    return (kb + per - 1) // per                   # no empty split


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *,
              out: torch.Tensor | None = None, out_f32: bool = False, accumulate: bool = False,
              splits: int = 0) -> torch.Tensor:
    """y = x @ w.T (+ bias) on CUDA cores with 32-bit sums.

    out_f32: the result is float32 whatever the inputs; accumulate: added into ``out`` (float32);
    splits >= 1: the result is the float32 stack [splits, M, N] of partial sums over K ranges (no bias).
    """
    need_cuda(x, w, bias, out)
    need(x.dim() == 2 and w.dim() == 2 and x.dtype == w.dtype and x.stride(1) == 1 and w.is_contiguous(),
         "gemm: x [M,K] and w [N,K] must share a dtype and be row-major")
    M, K = x.shape
    N = w.shape[0]
    need(w.shape[1] == K, f"gemm: inner sizes differ ({K} vs {w.shape[1]})")
    if bias is not None:
        need(bias.shape == (N,) and bias.dtype in (torch.float32, torch.bfloat16), "gemm: bias must be [N]")
    f = _f("gemm_simt", "rf_gemm_simt", c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
           c_int, c_int, c_int, c_int, c_int, c_void_p)
    if splits >= 1:
        need(not accumulate and out is None and bias is None, "gemm: partial sums take no bias and no output tensor")
        out = torch.empty((splits, M, N), dtype=torch.float32, device=x.device)
        check(f(dtype_code(x.dtype), ptr(x), ptr(w), ptr(None), 0, ptr(out), M, N, K, x.stride(0), N, 3, splits, stream()),
              f"gemm_simt ({M}x{N}x{K}, {splits} partial sums)")
        return out
    mode = 2 if accumulate else (1 if out_f32 else 0)
    odt = torch.float32 if mode else x.dtype
    if out is None:
        need(not accumulate, "gemm: accumulate needs an output tensor")
        out = torch.empty((M, N), dtype=odt, device=x.device)
    need(out.shape == (M, N) and out.dtype == odt and out.stride(1) == 1, "gemm: output has the wrong shape or dtype")
    check(f(dtype_code(x.dtype), ptr(x), ptr(w), ptr(bias), int(bias is not None and bias.dtype == torch.float32),
            ptr(out), M, N, K, x.stride(0), out.stride(0), mode, 1, stream()), f"gemm_simt ({M}x{N}x{K})")
    return out


def key_span(window: int | None, chunk: int | None = None) -> int:
    """The one number by which the attention kernels know which keys a query sees (rf_first_key in csrc/common.cuh):
    the last ``window`` positions (> 0), the positions of the query's own chunk of ``chunk`` positions, chunks counted
    from position 0 (< 0), or all (0)."""
    need(not (window and chunk), "attention: a window or chunks, not both")
    return -int(chunk) if chunk else int(window or 0)


def attention_generic(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                      tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None,
                      out: torch.Tensor | None = None, *, v_head_dim: int | None = None, softcap: float | None = None,
                      slopes: torch.Tensor | None = None, chunk: int | None = None, keep_first: int = 0,
                      sinks: torch.Tensor | None = None) -> torch.Tensor:
    """Attention of the T new tokens over the paged cache (their own keys included).  ``window`` / ``chunk``: see
    ``key_span``.  ``keep_first``: with a window, the first ``keep_first`` positions of a sequence stay visible to every
    later query as well (at their own positions).  ``sinks`` (float32 [heads]): exp(sinks[head]) is one more term of the
    softmax's denominator; it has no key and no value and is not scaled.

    ``v_head_dim``: size of a value head where it differs from a key head's (the output is [T, heads * v_head_dim]);
    ``softcap``: scores become softcap * tanh(score / softcap); ``slopes`` (float32 [heads]): after the cap, a score is
    lowered by slopes[head] * (query position - key position)."""
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table, slopes)
    T = q.shape[0]
    vd = head_dim if v_head_dim is None else int(v_head_dim)
    need(q.dim() == 2 and q.stride(1) == 1, "attention: q must be [T, >= heads*head_dim] with unit inner stride")
    need(k_pages.dtype == q.dtype and v_pages.dtype == q.dtype, "attention: cache dtype differs from q")
    need(tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim) and k_pages.is_contiguous()
         and tuple(v_pages.shape) == (k_pages.shape[0], n_kv_heads, PAGE, vd) and v_pages.is_contiguous(),
         "attention: bad cache page shape")
    if out is None:
        out = torch.empty((T, n_heads * vd), dtype=q.dtype, device=q.device)
    window = key_span(window, chunk)
    keep_first = int(keep_first or 0) if window > 0 else 0         # without a window every key is visible anyway
    if sinks is not None:
        need_cuda(sinks)
        need(sinks.dtype == torch.float32 and sinks.shape == (n_heads,) and sinks.is_contiguous()
             and (slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (n_heads,) and slopes.is_contiguous())),
             "attention: sinks (and slopes) must be float32 [heads]")
        f = _f("attention_generic", "rf_attention_generic_sink", c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
               c_void_p, c_int, c_int, c_void_p, c_int, c_void_p)
        check(f(dtype_code(q.dtype), ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages),
                ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads,
                n_kv_heads, head_dim, vd, float(scale), float(softcap or 0.0), ptr(slopes), window, keep_first, ptr(sinks), T,
                stream()),
              f"attention_generic (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim}, v_head_dim={vd}, sinks)")
        return out
    if vd != head_dim or softcap or slopes is not None or keep_first:
        need(slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (n_heads,) and slopes.is_contiguous()),
             "attention: slopes must be float32 [heads]")
        f = _f("attention_generic", "rf_attention_generic_ext", c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
               c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_float,
               c_void_p, c_int, c_int, c_int, c_void_p)
        check(f(dtype_code(q.dtype), ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages),
                ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads,
                n_kv_heads, head_dim, vd, float(scale), float(softcap or 0.0), ptr(slopes), window, keep_first, T, stream()),
              f"attention_generic (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim}, v_head_dim={vd})")
        return out
    f = _f("attention_generic", "rf_attention_generic", c_int, c_void_p, c_int, c_void_p, c_int, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int,
           c_void_p)
    check(f(dtype_code(q.dtype), ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages),
            ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads,
            n_kv_heads, head_dim, float(scale), window, T, stream()),
          f"attention_generic (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Row-wise argmax of float32 logits; of equal maxima the highest index."""
    need_cuda(logits)
    need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
         "argmax: logits must be [rows, vocab] float32")
    R, V = logits.shape
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _f("sampling", "rf_argmax", c_void_p, c_int, c_int, c_ll, c_void_p, c_void_p)
    check(f(ptr(logits), R, V, logits.stride(0), ptr(out), stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: float, top_p: float, top_k: int, seeds: torch.Tensor,
           draw_counter: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """One seeded draw per row after temperature, top-k and nucleus filtering.

    ``seeds`` [rows] int64 holds each row's 64-bit LCG seed; ``draw_counter`` (a device int32
    scalar) is added to every seed, so that a replayed step can advance its draws without the host.
    """
    need_cuda(logits, seeds, draw_counter)
    need(logits.dim() == 2 and logits.dtype == torch.float32 and logits.stride(1) == 1,
         "sample: logits must be [rows, vocab] float32")
    R, V = logits.shape
    need(seeds.dtype == torch.int64 and seeds.shape == (R,), "sample: seeds must be [rows] int64")
    need(temperature > 0.0, "sample: temperature must be positive (0 means argmax)")
    if out is None:
        out = torch.empty((R,), dtype=torch.int32, device=logits.device)
    f = _f("sampling", "rf_sample", c_void_p, c_int, c_int, c_ll, c_float, c_float, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p)
    check(f(ptr(logits), R, V, logits.stride(0), float(temperature), float(top_p), int(top_k), ptr(seeds),
            ptr(draw_counter), ptr(out), stream()), "sample")
    return out


def set_sample_cached(on: bool) -> None:
    """Which sampler ``sample`` launches where both can run: the one that keeps a CTA's slice of the row in shared
    memory (the default), or the one that walks the row in global memory (it also serves vocabularies whose slices do
    not fit).  Both give the same token."""
    check(_f("sampling", "rf_sample_set_cached", c_int)(1 if on else 0), "set_sample_cached")


def advance_decode(tokens, tok_pos, seq_start, sampled) -> None:
    """tokens <- sampled; positions and starts += 1 (one token per sequence), all on the device."""
    need_cuda(tokens, tok_pos, seq_start, sampled)
    B = tokens.shape[0]
    need(all(t.dtype == torch.int32 and t.shape == (B,) for t in (tokens, tok_pos, seq_start, sampled)),
         "advance_decode: four int32 arrays of one length")
    f = _f("sampling", "rf_advance_decode", c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p)
    check(f(ptr(tokens), ptr(tok_pos), ptr(seq_start), ptr(sampled), B, stream()), "advance_decode")


def gather_tokens(tokens, ids, row_map) -> None:
    """tokens[i] = ids[row_map[i]] on the device (all int32)."""
    need_cuda(tokens, ids, row_map)
    B = tokens.shape[0]
    need(all(t.dtype == torch.int32 and t.dim() == 1 for t in (tokens, ids, row_map)) and row_map.shape[0] == B,
         "gather_tokens: int32 vectors, one map entry per token")
    f = _f("sampling", "rf_gather_tokens", c_void_p, c_void_p, c_void_p, c_int, c_void_p)
    check(f(ptr(tokens), ptr(ids), ptr(row_map), B, stream()), "gather_tokens")


def attention_decode_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_decode", "rf_attention_decode_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


DECODE_CHUNK = 128


def attention_decode_scratch(B: int, n_heads: int, n_kv_heads: int, head_dim: int, max_chunks: int):
    """Element counts (partial outputs, partial max/sum, counters) the decode attention needs for B sequences."""
    return (B * n_heads * max_chunks * head_dim, B * n_heads * max_chunks * 2, B * n_kv_heads)


def attention_decode(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                     tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None, max_chunks: int,
                     part_o: torch.Tensor, part_ml: torch.Tensor, counters: torch.Tensor,
                     out: torch.Tensor | None = None, *, chunk: int | None = None) -> torch.Tensor:
    """One new token per sequence over the bfloat16 paged cache, keys in chunks of 128.

    ``max_chunks`` must cover the longest sequence (ceil(length / 128)); ``part_o``, ``part_ml`` (float32)
    and ``counters`` (int32, zero before the first call; the kernel leaves them zero) are scratch of at
    least ``attention_decode_scratch`` elements.
    """
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table, part_o, part_ml, counters)
    B = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_decode: q must be bfloat16 [B, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_decode: bad cache page shape or dtype")
    need(attention_decode_supported(n_heads, n_kv_heads, head_dim),
         f"attention_decode: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    n_o, n_ml, n_c = attention_decode_scratch(B, n_heads, n_kv_heads, head_dim, max_chunks)
    need(part_o.dtype == torch.float32 and part_o.numel() >= n_o and part_ml.dtype == torch.float32
         and part_ml.numel() >= n_ml and counters.dtype == torch.int32 and counters.numel() >= n_c,
         "attention_decode: scratch tensors are too small")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    f = _f("attention_decode", "rf_attention_decode", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p)
    from .tensor_core import status_word
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), ptr(tok_seq), ptr(tok_pos),
            ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale),
            key_span(window, chunk), B, max_chunks, ptr(part_o), ptr(part_ml), ptr(counters), ptr(status_word(q.device)),
            stream()),
          f"attention_decode (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


PREFILL_TILE = 64


def attention_prefill_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_prefill", "rf_attention_prefill_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


def attention_prefill(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                      q_tiles: torch.Tensor, seq_slot, seq_start, seq_nnew, cu_q, block_table, scale: float,
                      window: int | None, out: torch.Tensor | None = None, *, chunk: int | None = None) -> torch.Tensor:
    """Tiled causal attention of the new tokens over the bfloat16 paged cache (head_dim 64 or 128).

    ``q_tiles`` is an int32 array of (sequence index, first row within the sequence's new tokens) pairs,
    one per 64-row tile, built on the host.
    """
    need_cuda(q, k_pages, v_pages, q_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table)
    T = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_prefill: q must be bfloat16 [T, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_prefill: bad cache page shape or dtype")
    need(attention_prefill_supported(n_heads, n_kv_heads, head_dim),
         f"attention_prefill: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q_tiles.dtype == torch.int32 and q_tiles.numel() % 2 == 0, "attention_prefill: q_tiles must be int32 pairs")
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    f = _f("attention_prefill", "rf_attention_prefill", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_ll,
           c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int,
           c_void_p, c_void_p)
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(q_tiles),
            q_tiles.numel() // 2, ptr(seq_slot), ptr(seq_start), ptr(seq_nnew), ptr(cu_q), ptr(block_table),
            block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale), key_span(window, chunk),
            ptr(status_word(q.device)), stream()),
          f"attention_prefill (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


def decode_splits(B: int, n_kv_heads: int, longest: int | None = None, window: int | None = None) -> int:
    """CTAs that share one (sequence, kv head) in the clustered decode attention, from the batch and the
    longest context the launch may meet (a captured graph keeps its launch shape): about one CTA per SM,
    at most one CTA per page, and clusters of 8 only for very small batches, where nothing else fills the
    GPU.  Measured at 28 layers, 4 kv heads of 7 query heads, ms per decode step: batch 1 / 3,800 keys:
    1, 2, 4, 8 CTAs 3.45, 3.16, 2.92, 2.85; batch 8 / 1,900 keys: 3.21, 3.10, 3.01, 3.05; batch 32 / 512:
    3.54, 3.54, 3.72; batch 64 / 512: 3.76, 4.04."""
    pairs = max(1, B * n_kv_heads)
    s = 1
    while s < 8 and pairs * s * 2 <= device_sm_count() * 7 // 8:          # 128 on the 148 SMs these numbers were taken on
        s *= 2
    if s == 8 and pairs > 8:
        s = 4
    if longest is not None:
        pages = decode_pages(longest, window)
        # one sequence with a long context: clusters of 16 (beyond the portable size; four of them still find a
        # GPC each).  28 heads on 4 kv heads, 16,000 keys: 17.7 -> 11.8 us a layer; 8 such clusters were slower
        if s == 8 and pairs <= 4 and pages >= 32:
            s = 16
        while s > 1 and s > pages:
            s //= 2
    return s


def decode_pages(longest: int, window: int | None) -> int:
    """Most pages of 64 positions that a new token at context length ``longest`` reads (``window``: the most keys a
    query sees, be it a sliding window or a chunk)."""
    pages = (max(1, longest) + PAGE - 1) // PAGE
    if window:
        pages = min(pages, (window + PAGE - 2) // PAGE + 1)
    return pages


def attention_decode_warps(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                           tok_seq, tok_pos, seq_slot, block_table, scale: float, window: int | None,
                           splits: int | None = None, warps: int | None = None,
                           out: torch.Tensor | None = None, *, softcap: float | None = None,
                           slopes: torch.Tensor | None = None, chunk: int | None = None, keep_first: int = 0,
                           sinks: torch.Tensor | None = None) -> torch.Tensor:
    """One new token per sequence over the bfloat16 paged cache: a cluster of ``splits`` CTAs per (sequence,
    kv head), every warp on its own tiles of keys; merged through distributed shared memory.  ``warps``
    per CTA: 8 while one CTA per SM is enough for the batch, else 4 (three CTAs fit an SM).  ``softcap``, ``slopes``,
    ``keep_first`` and ``sinks`` as in ``attention_generic``."""
    need_cuda(q, k_pages, v_pages, tok_seq, tok_pos, seq_slot, block_table)
    B = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1, "attention_decode: q must be bfloat16 [B, ...]")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_decode: bad cache page shape or dtype")
    need(attention_decode_supported(n_heads, n_kv_heads, head_dim),
         f"attention_decode: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_decode: q rows must be 16-byte aligned")
    if splits is None:
        splits = decode_splits(B, n_kv_heads)
    if warps is None:
        warps = 8 if B * n_kv_heads * splits <= device_sm_count(q.device) else 4
    if out is None:
        out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    need(slopes is None or (slopes.is_cuda and slopes.dtype == torch.float32 and slopes.shape == (n_heads,) and slopes.is_contiguous()),
         "attention_decode: slopes must be float32 [heads]")
    need(sinks is None or (sinks.is_cuda and sinks.dtype == torch.float32 and sinks.shape == (n_heads,) and sinks.is_contiguous()),
         "attention_decode: sinks must be float32 [heads]")
    f = _f("attention_decode", "rf_attention_decode_warps_sink", c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p,
           c_ll, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float, c_int, c_int, c_int, c_int,
           c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p)
    span = key_span(window, chunk)
    check(f(ptr(q), q.stride(0), ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(tok_seq),
            ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1], n_heads, n_kv_heads, head_dim,
            float(scale), span, B, splits, warps, float(softcap or 0.0), ptr(slopes),
            int(keep_first or 0) if span > 0 else 0, ptr(sinks), ptr(status_word(q.device)), stream()),
          f"attention_decode_warps (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim}, splits={splits})")
    return out


PREFILL_TC_TILE = 128


def attention_prefill_tc_supported(n_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    f = _f("attention_prefill_tc", "rf_attention_prefill_tc_supported", c_int, c_int, c_int)
    return bool(f(n_heads, n_kv_heads, head_dim))


def attention_prefill_tc(q: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, k_pages, v_pages,
                         q_tiles: torch.Tensor, seq_slot, seq_start, seq_nnew, cu_q, block_table, scale: float,
                         window: int | None, out: torch.Tensor | None = None, *, softcap: float | None = None,
                         slopes: torch.Tensor | None = None, chunk: int | None = None, keep_first: int = 0,
                         sinks: torch.Tensor | None = None) -> torch.Tensor:
    """The same attention as ``attention_prefill`` with both products as tcgen05.mma (accumulators in tensor
    memory); ``q_tiles`` holds (sequence, first row) pairs of 128-row tiles.  ``softcap``, ``slopes``, ``keep_first`` and
    ``sinks`` as in ``attention_generic``."""
    need_cuda(q, k_pages, v_pages, q_tiles, seq_slot, seq_start, seq_nnew, cu_q, block_table, slopes, sinks)
    need(sinks is None or (sinks.dtype == torch.float32 and sinks.shape == (n_heads,) and sinks.is_contiguous()),
         "attention_prefill_tc: sinks must be float32 [heads]")
    need(slopes is None or (slopes.dtype == torch.float32 and slopes.shape == (n_heads,) and slopes.is_contiguous()),
         "attention_prefill_tc: slopes must be float32 [heads]")
    T = q.shape[0]
    need(q.dtype == torch.bfloat16 and q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= n_heads * head_dim,
         "attention_prefill_tc: q must be bfloat16 [T, >= heads*head_dim]")
    need(q.data_ptr() % 16 == 0 and (q.stride(0) * 2) % 16 == 0, "attention_prefill_tc: q rows must be 16-byte aligned")
    need(k_pages.dtype == torch.bfloat16 and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim)
         and k_pages.is_contiguous() and v_pages.shape == k_pages.shape and v_pages.is_contiguous(),
         "attention_prefill_tc: bad cache page shape or dtype")
    need(attention_prefill_tc_supported(n_heads, n_kv_heads, head_dim),
         f"attention_prefill_tc: heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim} is not supported")
    need(q_tiles.dtype == torch.int32 and q_tiles.numel() % 2 == 0, "attention_prefill_tc: q_tiles must be int32 pairs")
    if out is None:
        out = torch.empty((T, n_heads * head_dim), dtype=torch.bfloat16, device=q.device)
    from .tensor_core import status_word
    f = _f("attention_prefill_tc", "rf_attention_prefill_tc_sink", c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p,
           c_ll, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_float,
           c_int, c_float, c_void_p, c_int, c_void_p, c_void_p, c_void_p)
    span = key_span(window, chunk)
    check(f(ptr(q), q.stride(0), T, ptr(out), out.stride(0), ptr(k_pages), ptr(v_pages), k_pages.shape[0], ptr(q_tiles),
            q_tiles.numel() // 2, ptr(seq_slot), ptr(seq_start), ptr(seq_nnew), ptr(cu_q), ptr(block_table),
            block_table.shape[1], n_heads, n_kv_heads, head_dim, float(scale), span, float(softcap or 0.0),
            ptr(slopes), int(keep_first or 0) if span > 0 else 0, ptr(sinks), ptr(status_word(q.device)), stream()),
          f"attention_prefill_tc (heads={n_heads}, kv_heads={n_kv_heads}, head_dim={head_dim})")
    return out


def relu2(x: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """max(x, 0)^2 element by element (evaluated in 32-bit)."""
    need_cuda(x)
    need(x.is_contiguous(), "relu2: input must be contiguous")
    if out is None:
        out = torch.empty_like(x)
    f = _f("elementwise", "rf_relu2", c_int, c_void_p, c_void_p, c_ll, c_void_p)
    check(f(dtype_code(x.dtype), ptr(x), ptr(out), x.numel(), stream()), "relu2")
    return out


def add_row(h: torch.Tensor, vec: torch.Tensor) -> None:
    """h[t, :] += vec for every row of the float32 stream ``h``."""
    need_cuda(h, vec)
    need(h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous() and vec.shape == (h.shape[1],)
         and vec.is_contiguous(), "add_row: h must be [T, H] float32 and vec [H]")
    f = _f("elementwise", "rf_add_row", c_int, c_void_p, c_void_p, c_int, c_int, c_void_p)
    check(f(dtype_code(vec.dtype), ptr(h), ptr(vec), h.shape[0], h.shape[1], stream()), "add_row")


def branch_norm_add(h: torch.Tensor, branches, post_weight: torch.Tensor, eps: float, compute_dtype: torch.dtype, *,
                    extra: torch.Tensor | None = None, next_weight: torch.Tensor | None = None,
                    next_rounded: bool = False) -> torch.Tensor | None:
    """The residual update of a block that norms its sub-layers' outputs, in 32-bit and in one pass over the rows:

        m = a0                                    for branches == [(a0, None)]
        m = (rms(a0) * w0 + rms(a1) * w1) / 2     for branches == [(a0, w0), (a1, w1)]
        h += rms(m) * post_weight (+ extra)
        returns rms(h) * next_weight in the compute dtype if ``next_weight`` is given, h itself rounded to the compute
        dtype if ``next_rounded`` (the next sub-layer reads the stream itself), else None

    with rms(x) = x / sqrt(mean(x^2) + eps).  A branch is float32 [T, H], or a stack [S, T, H] of partial sums of a K-split
    product, which are added here in index order; all weight vectors share one dtype.
    """
    need(len(branches) in (1, 2), "branch_norm_add: one or two branches")
    a0, w0 = branches[0]
    a1, w1 = branches[1] if len(branches) == 2 else (None, None)
    need((len(branches) == 1) == (w0 is None), "branch_norm_add: two branches come with weights, one comes without")
    vecs = [v for v in (w0, w1, post_weight, extra, next_weight) if v is not None]
    need_cuda(h, a0, a1, *vecs)
    T, H = h.shape
    need(h.dtype == torch.float32 and h.is_contiguous(), "branch_norm_add: h must be contiguous float32 [T, H]")
    for a in (a0, a1):
        need(a is None or (a.dtype == torch.float32 and tuple(a.shape[-2:]) == (T, H) and a.dim() in (2, 3) and a.is_contiguous()),
             "branch_norm_add: a branch must be contiguous float32 [T, H] or [S, T, H]")
    n0 = a0.shape[0] if a0.dim() == 3 else 1
    n1 = (a1.shape[0] if a1.dim() == 3 else 1) if a1 is not None else 0
    need(all(v.shape == (H,) and v.dtype == vecs[0].dtype and v.is_contiguous() for v in vecs)
         and vecs[0].dtype in (torch.float32, torch.bfloat16), "branch_norm_add: weight vectors must be [H] of one dtype")
    need(not (next_rounded and next_weight is not None), "branch_norm_add: the next reader takes a norm or the stream itself")
    y = torch.empty((T, H), dtype=compute_dtype, device=h.device) if (next_weight is not None or next_rounded) else None
    f = _f("elementwise", "rf_branch_norm_add", c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_int, c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(a0), n0, ptr(w0), ptr(a1), n1, ptr(w1), ptr(post_weight), ptr(extra),
            ptr(next_weight), ptr(y), int(vecs[0].dtype == torch.float32), float(eps), T, H, stream()),
          f"branch_norm_add (H={H})")
    return y


def head_norm_kv_write(qkv: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, v_head_dim: int,
                       inv_freq: torch.Tensor | None, tok_seq, tok_pos, seq_slot, block_table: torch.Tensor,
                       k_pages: torch.Tensor | None, v_pages: torch.Tensor | None, write_kv: bool = True, *,
                       compute_dtype: torch.dtype | None = None, rot_dim: int = 0, interleaved: bool = False,
                       unit_norm_eps: float | None = None, q_norm_weight: torch.Tensor | None = None,
                       k_norm_weight: torch.Tensor | None = None, magnitude: float = 1.0, bias: torch.Tensor | None = None,
                       norm_after_rotation: bool = False, q_temperature=None, values_are_keys: bool = False) -> torch.Tensor:
    """q | k | v rows on their way into the cache, for heads that are normed and for values of another size than keys.

    More options: ``bias`` ([width] in float32 or bfloat16) is added to the columns read; ``norm_after_rotation``: the
    heads are divided by their root mean square as they are after the rotation (and then weighted), not before it;
    ``q_temperature`` = (coef, every): a query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1);
    ``values_are_keys``: the rows are q | k only, the keys are written and ``v_pages`` is not touched (the caller reads
    values from the key pages; ``v_head_dim`` must equal ``head_dim``).

    ``qkv`` is [T, heads*head_dim + kv_heads*head_dim + kv_heads*v_head_dim] in the compute dtype, or a float32 stack
    [S, T, ...] of partial sums.  With ``unit_norm_eps`` every query and key head is divided by its root mean square
    (x / sqrt(mean(x^2) + eps)) in 32-bit and multiplied by ``q_norm_weight`` / ``k_norm_weight`` ([head_dim], shared by
    the heads) where given; then the first ``rot_dim`` elements turn (0: no rotation), sine and cosine times ``magnitude``.  The rows may hold more columns
    than q | k | v (a gate's, say); without ``write_kv`` only the q heads are read.
    Returns q [T, heads*head_dim] in the compute dtype; k and v go to their pages.
    """
    need_cuda(qkv, inv_freq, tok_seq, tok_pos, seq_slot, block_table, k_pages, v_pages)
    need(not values_are_keys or v_head_dim == head_dim, "head_norm_kv_write: keys that are values have the keys' size")
    width = (n_heads + n_kv_heads) * head_dim + (0 if values_are_keys else n_kv_heads * v_head_dim)
    partials = qkv.dim() == 3
    if partials:
        need(qkv.dtype == torch.float32 and qkv.is_contiguous() and qkv.shape[2] >= (width if write_kv else n_heads * head_dim) and compute_dtype is not None,
             "head_norm_kv_write: partial sums must be a contiguous float32 [S, T, width] stack, with the compute dtype named")
        S, T, dt, row_stride, pstride = qkv.shape[0], qkv.shape[1], compute_dtype, qkv.shape[2], qkv.shape[1] * qkv.shape[2]
    else:
        need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= (width if write_kv else n_heads * head_dim),
             "head_norm_kv_write: qkv must be [T, >= width]")
        S, T, dt, row_stride, pstride = 0, qkv.shape[0], qkv.dtype, qkv.stride(0), 0
    need(rot_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2),
         "head_norm_kv_write: inv_freq must hold rot_dim/2 float32 frequencies")
    if write_kv:
        need(k_pages is not None and k_pages.dtype == dt and k_pages.is_contiguous()
             and tuple(k_pages.shape[1:]) == (n_kv_heads, PAGE, head_dim) and (values_are_keys or (v_pages is not None and v_pages.dtype == dt
             and v_pages.is_contiguous() and tuple(v_pages.shape[1:]) == (n_kv_heads, PAGE, v_head_dim))),
             "head_norm_kv_write: pages must be [n_pages, kv_heads, 64, head size] of the compute dtype")
    q_out = torch.empty((T, n_heads * head_dim), dtype=dt, device=qkv.device)
    nws = [w for w in (q_norm_weight, k_norm_weight) if w is not None]
    need_cuda(*nws)
    need(all(w.shape == (head_dim,) and w.is_contiguous() and w.dtype == nws[0].dtype for w in nws)
         and (not nws or (unit_norm_eps is not None and nws[0].dtype in (torch.float32, torch.bfloat16))),
         "head_norm_kv_write: norm weights are [head_dim] vectors of one dtype and go with unit_norm_eps")
    if bias is not None or norm_after_rotation or q_temperature is not None or values_are_keys:
        need_cuda(bias)
        need(bias is None or (bias.shape == (width,) and bias.is_contiguous() and bias.dtype in (torch.float32, torch.bfloat16)),
             "head_norm_kv_write: the bias must be [width] in float32 or bfloat16")
        coef, every = (float(q_temperature[0]), float(q_temperature[1])) if q_temperature is not None else (0.0, 0.0)
        need(q_temperature is None or every > 0, "head_norm_kv_write: the temperature's step must be a positive number of positions")
        f = _f("elementwise", "rf_head_norm_kv_write_x", c_int, c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_int, c_int,
               c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
               c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_int, c_float, c_float, c_int, c_void_p)
        check(f(dtype_code(dt), ptr(qkv), row_stride, S, pstride, ptr(q_out), q_out.stride(0), n_heads, n_kv_heads, head_dim,
                v_head_dim, ptr(inv_freq), ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1],
                ptr(k_pages), ptr(None if values_are_keys else v_pages), int(write_kv), T, int(rot_dim), int(interleaved),
                int(unit_norm_eps is not None), float(unit_norm_eps or 0.0), ptr(q_norm_weight), ptr(k_norm_weight),
                int(bool(nws) and nws[0].dtype == torch.float32), float(magnitude), ptr(bias),
                int(bias is not None and bias.dtype == torch.float32), int(bool(norm_after_rotation)), coef, every,
                int(bool(values_are_keys)), stream()), "head_norm_kv_write")
        return q_out
    f = _f("elementwise", "rf_head_norm_kv_write_w", c_int, c_void_p, c_int, c_int, c_ll, c_void_p, c_int, c_int, c_int,
           c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
           c_int, c_int, c_float, c_void_p, c_void_p, c_int, c_float, c_void_p)
    check(f(dtype_code(dt), ptr(qkv), row_stride, S, pstride, ptr(q_out), q_out.stride(0), n_heads, n_kv_heads, head_dim,
            v_head_dim, ptr(inv_freq), ptr(tok_seq), ptr(tok_pos), ptr(seq_slot), ptr(block_table), block_table.shape[1],
            ptr(k_pages), ptr(v_pages), int(write_kv), T, int(rot_dim), int(interleaved), int(unit_norm_eps is not None),
            float(unit_norm_eps or 0.0), ptr(q_norm_weight), ptr(k_norm_weight), int(bool(nws) and nws[0].dtype == torch.float32),
            float(magnitude), stream()), "head_norm_kv_write")
    return q_out


def gemm_simt_grouped(x: torch.Tensor, w: torch.Tensor, tiles: torch.Tensor, max_tiles: int, tile_rows: int,
                      n_rows: int, *, row_map: torch.Tensor | None = None, row_div: int = 1,
                      out_f32: bool = False) -> torch.Tensor:
    """One product for many weight matrices: y[r] = x[row_map[r] // row_div] @ w[group of r].T for the ``n_rows`` sorted
    rows that the tile table lists (``kernels.moe_sort``); ``w`` is [groups, N, K]; without ``row_map`` row r reads x[r]."""
    need_cuda(x, w, tiles, row_map)
    need(x.dim() == 2 and w.dim() == 3 and x.dtype == w.dtype and x.stride(1) == 1 and w.is_contiguous()
         and w.shape[2] == x.shape[1], "gemm_simt_grouped: x [M,K] and w [G,N,K] must share a dtype and K")
    need(tiles.dtype == torch.int32 and tiles.numel() >= 1 + 3 * max_tiles, "gemm_simt_grouped: tile table too small")
    need(row_map is None or (row_map.dtype == torch.int32 and row_map.numel() >= n_rows), "gemm_simt_grouped: bad row map")
    G, N, K = w.shape
    out = torch.empty((n_rows, N), dtype=torch.float32 if out_f32 else x.dtype, device=x.device)
    f = _f("gemm_simt", "rf_gemm_simt_grouped", c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
           c_int, c_int, c_void_p, c_void_p, c_int, c_ll, c_void_p)
    check(f(dtype_code(x.dtype), ptr(x), ptr(w), ptr(out), max_tiles, tile_rows, N, K, x.stride(0), N, int(out_f32),
            ptr(tiles), ptr(row_map), int(row_div), N * K, stream()), f"gemm_simt_grouped ({G} x {N}x{K})")
    return out


# ---------------------------------------------------------------- retention (csrc/retention.cu)

def retention_prepare(proj: torch.Tensor, q_col: int, k_col: int, heads: int, dim: int, rot_dim: int,
                      inv_freq: torch.Tensor | None, tok_pos: torch.Tensor, k_scale: float) -> torch.Tensor:
    """q and k of the projection's rows (columns q_col.. and k_col.., heads*dim each) rotated by position in 32-bit
    (first ``rot_dim`` elements of a head, pairs (i, i + rot_dim/2)), k times ``k_scale``: float32 [2, T, heads*dim]."""
    need_cuda(proj, inv_freq, tok_pos)
    need(proj.dim() == 2 and proj.stride(1) == 1, "retention_prepare: the projection must be [T, columns]")
    need(rot_dim == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dim // 2),
         "retention_prepare: inv_freq must hold rot_dim/2 float32 frequencies")
    T = proj.shape[0]
    qk = torch.empty((2, T, heads * dim), dtype=torch.float32, device=proj.device)
    f = _f("retention", "rf_retention_prepare", c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_int,
           c_void_p, c_void_p, c_float, c_int, c_void_p)
    check(f(dtype_code(proj.dtype), ptr(proj), proj.stride(0), q_col, k_col, ptr(qk), heads, dim, rot_dim, ptr(inv_freq),
            ptr(tok_pos), float(k_scale), T, stream()), "retention_prepare")
    return qk


def retention_scan(qk: torch.Tensor, v: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, cu_q: torch.Tensor,
                   seq_slot: torch.Tensor, heads: int, dim: int, vdim: int) -> torch.Tensor:
    """S <- decay_h S + k v^T, o = S^T q, token by token for every sequence of the step; ``state`` [slots, heads, vdim,
    dim] float32 (S transposed: a value dimension's column is contiguous) is read at the step's start and left as after
    its last token.  ``v`` is a [T, heads*vdim] view (rows
    may be strided).  Returns o float32 [T, heads*vdim]."""
    need_cuda(qk, v, state, decay, cu_q, seq_slot)
    T = qk.shape[1]
    need(qk.dtype == torch.float32 and qk.is_contiguous() and qk.shape == (2, T, heads * dim), "retention_scan: bad q/k")
    need(v.shape == (T, heads * vdim) and v.stride(1) == 1, "retention_scan: v must be [T, heads*vdim]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, dim),
         "retention_scan: state must be float32 [slots, heads, vdim, dim]")
    need(decay.dtype == torch.float32 and decay.shape == (heads,), "retention_scan: decay must be float32 [heads]")
    B = seq_slot.shape[0]
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=qk.device)
    f = _f("retention", "rf_retention_scan", c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(v.dtype), ptr(qk[0]), ptr(qk[1]), ptr(v), v.stride(0), ptr(state), ptr(decay), ptr(o), ptr(cu_q),
            ptr(seq_slot), B, heads, dim, vdim, stream()), f"retention_scan (heads={heads}, dim={dim}, vdim={vdim})")
    return o


RETENTION_CHUNK = 64


def retention_chunked(qk: torch.Tensor, v: torch.Tensor, state: torch.Tensor, decay: torch.Tensor, table: torch.Tensor,
                      cu_q: torch.Tensor, seq_slot: torch.Tensor, heads: int, dim: int, vdim: int) -> torch.Tensor:
    """What ``retention_scan`` computes, for prompts: the recurrence in chunks of 64 tokens that run side by side (per-chunk
    sums, then the states between the chunks one after the other, then every chunk's outputs from its start state), all
    in 32-bit.  ``table``: int32, first[B+1] (index of each sequence's first chunk) followed by (sequence, first row among
    the sequence's new tokens) of every chunk, in the order of the sequences.  Differs from the scan by rounding only."""
    need_cuda(qk, v, state, decay, table, cu_q, seq_slot)
    T = qk.shape[1]
    B = seq_slot.shape[0]
    need(qk.dtype == torch.float32 and qk.is_contiguous() and qk.shape == (2, T, heads * dim), "retention_chunked: bad q/k")
    need(v.shape == (T, heads * vdim) and v.stride(1) == 1, "retention_chunked: v must be [T, heads*vdim]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, vdim, dim),
         "retention_chunked: state must be float32 [slots, heads, vdim, dim]")
    need(decay.dtype == torch.float32 and decay.shape == (heads,), "retention_chunked: decay must be float32 [heads]")
    need(table.dtype == torch.int32 and (table.numel() - (B + 1)) % 2 == 0 and table.numel() > B + 1,
         "retention_chunked: the chunk table must hold first[B+1] and a pair per chunk")
    n_chunks = (table.numel() - (B + 1)) // 2
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=qk.device)
    scratch = torch.empty((n_chunks, heads, dim, vdim), dtype=torch.float32, device=qk.device)
    f = _f("retention", "rf_retention_chunked", c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
           c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(v.dtype), ptr(qk[0]), ptr(qk[1]), ptr(v), v.stride(0), ptr(state), ptr(decay), ptr(o), ptr(scratch),
            ptr(table), n_chunks, ptr(cu_q), ptr(seq_slot), B, heads, dim, vdim, stream()),
          f"retention_chunked (heads={heads}, dim={dim}, vdim={vdim})")
    return o


def retention_gate(o: torch.Tensor, gate: torch.Tensor, heads: int, vdim: int, eps: float,
                   weight: torch.Tensor | None = None, *, gate_fn: str = "silu", denominator=None) -> torch.Tensor:
    """o / sqrt(mean(o^2) + eps) per head, times ``weight`` if given ([vdim], one vector for all heads, or [heads*vdim]),
    times silu(gate) (``gate_fn`` "sigmoid": sigmoid(gate)), in the gate's dtype.  ``denominator`` = (qn, m), float32
    [T, heads] each: every head is first divided by max(|qn|, exp(-m)) + 1e-6."""
    need_cuda(o, gate, weight)
    need(gate_fn in ("silu", "sigmoid"), f"retention_gate: gate function {gate_fn!r} (silu, sigmoid)")
    need(weight is None or (weight.shape in ((vdim,), (heads * vdim,)) and weight.is_contiguous()
                            and weight.dtype in (torch.float32, torch.bfloat16)),
         "retention_gate: the norm's weight must be [vdim] or [heads*vdim]")
    T = o.shape[0]
    need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, heads * vdim), "retention_gate: bad o")
    need(gate.shape == (T, heads * vdim) and gate.stride(1) == 1, "retention_gate: gate must be [T, heads*vdim]")
    qn, mt = denominator if denominator is not None else (None, None)
    for d in (qn, mt):
        need(d is None or (d.is_cuda and d.dtype == torch.float32 and d.shape == (T, heads) and d.is_contiguous()),
             "retention_gate: the denominator's parts must be float32 [T, heads]")
    out = torch.empty((T, heads * vdim), dtype=gate.dtype, device=o.device)
    per_head = weight is not None and heads > 1 and weight.shape == (heads * vdim,)
    f = _f("retention", "rf_retention_gate_x", c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_float, c_int,
           c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p)
    check(f(dtype_code(gate.dtype), ptr(o), ptr(gate), gate.stride(0), ptr(out), heads, vdim, float(eps), T, ptr(weight),
            int(weight is not None and weight.dtype == torch.float32), int(per_head), int(gate_fn == "sigmoid"), ptr(qn),
            ptr(mt), stream()), "retention_gate")
    return out


# ---------------------------------------------------------------- gated linear attention (csrc/gla.cu)

def gla_prepare(proj: torch.Tensor, q_col: int, k_col: int, z: torch.Tensor, heads: int, dim: int, q_scale: float,
                tau: float) -> torch.Tensor:
    """float32 [3, T, heads*dim]: q of the projection's rows (columns q_col..) times ``q_scale``, k (columns k_col..), and
    the decay alpha = sigmoid(z)^(1/tau) = exp(log sigmoid(z) / tau) per key channel, from z float32 [T, heads*dim]."""
    need_cuda(proj, z)
    T, width = proj.shape[0], heads * dim
    need(proj.dim() == 2 and proj.stride(1) == 1 and max(q_col, k_col) + width <= proj.shape[1],
         "gla_prepare: the projection must be [T, columns] and hold q and k")
    need(z.dtype == torch.float32 and z.shape == (T, width) and z.is_contiguous(), "gla_prepare: z must be float32 [T, heads*dim]")
    qka = torch.empty((3, T, width), dtype=torch.float32, device=proj.device)
    f = _f("gla", "rf_gla_prepare", c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_float, c_float, c_int,
           c_void_p)
    check(f(dtype_code(proj.dtype), ptr(proj), proj.stride(0), q_col, k_col, ptr(z), ptr(qka), width, float(q_scale), float(tau),
            T, stream()), "gla_prepare")
    return qka


def gla_scan(qka: torch.Tensor, v: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor, seq_slot: torch.Tensor,
             heads: int, dim: int, vdim: int, one_token: bool = False) -> torch.Tensor:
    """S <- diag(alpha_t) S + k_t v_t^T, o_t = S^T q_t, token by token for every sequence of the step; ``qka`` as
    ``gla_prepare`` leaves it; ``state`` [slots, heads, dim, vdim] float32 is read at the step's start and
    left as after its last token; ``v`` a [T, heads*vdim] view (rows may be strided).  ``one_token``: every sequence brings
    exactly one token (a kernel without staging runs; the same bits).  Returns o float32 [T, heads*vdim]."""
    need_cuda(qka, v, state, cu_q, seq_slot)
    T = qka.shape[1]
    need(qka.dtype == torch.float32 and qka.is_contiguous() and qka.shape == (3, T, heads * dim), "gla_scan: bad q/k/alpha")
    need(v.shape == (T, heads * vdim) and v.stride(1) == 1, "gla_scan: v must be [T, heads*vdim]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
         "gla_scan: state must be float32 [slots, heads, dim, vdim]")
    B = seq_slot.shape[0]
    need(not one_token or T == B, "gla_scan: one_token means one token for every sequence")
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=qka.device)
    f = _f("gla", "rf_gla_scan", c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
           c_int, c_int, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(v.dtype), ptr(qka[0]), ptr(qka[1]), ptr(qka[2]), ptr(v), v.stride(0), ptr(state), ptr(o), ptr(cu_q),
            ptr(seq_slot), B, heads, dim, vdim, int(one_token), device_sm_count(qka.device), stream()),
          f"gla_scan (heads={heads}, dim={dim}, vdim={vdim})")
    return o


# ---------------------------------------------------------------- routing of experts (csrc/moe.cu)

MOE_TILE_SMALL, MOE_TILE_LARGE = 16, 64
MOE_TILE_TC = 128          # rows of a tile of the grouped tensor-core product


def moe_gather(x: torch.Tensor, perm: torch.Tensor, top: int) -> torch.Tensor:
    """out[r] = x[perm[r] // top]: the tokens' activations in the order the sort left their (token, choice) pairs in."""
    need_cuda(x, perm)
    need(x.dim() == 2 and x.stride(1) == 1 and perm.dtype == torch.int32, "moe_gather: x [T, K] and an int32 permutation")
    n, K = perm.numel(), x.shape[1]
    out = torch.empty((n, K), dtype=x.dtype, device=x.device)
    f = _f("moe", "rf_moe_gather", c_void_p, c_ll, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p)
    check(f(ptr(x), x.stride(0) * x.element_size(), ptr(perm), top, ptr(out), K * x.element_size(), n, stream()), "moe_gather")
    return out


MOE_SCORINGS = {"softmax_of_chosen": 0, "sigmoid": 1, "softmax_of_all": 2}


def moe_route(logits: torch.Tensor, top: int, scoring: str = "softmax_of_chosen"):
    """(experts int32 [T, top], weights float32 [T, top]): the ``top`` largest router logits of every token (of equal
    logits the lower index) and their weights: the softmax over those alone, or (``scoring`` "sigmoid") each one's
    own sigmoid, not renormalised, or ("softmax_of_all") each one's share of the softmax over all E logits, not
    renormalised."""
    need(scoring in MOE_SCORINGS, f"moe_route: scoring {scoring!r} is not one of {sorted(MOE_SCORINGS)}")
    need_cuda(logits)
    need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.is_contiguous(), "moe_route: logits must be float32 [T, E]")
    T, E = logits.shape
    idx = torch.empty((T, top), dtype=torch.int32, device=logits.device)
    w = torch.empty((T, top), dtype=torch.float32, device=logits.device)
    f = _f("moe", "rf_moe_route_scored", c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p)
    check(f(ptr(logits), E, top, ptr(idx), ptr(w), T, MOE_SCORINGS[scoring], stream()), f"moe_route (E={E}, top={top})")
    return idx, w


def moe_sort(idx: torch.Tensor, n_experts: int, tile_rows: int, weights: torch.Tensor | None = None):
    """The (token, choice) pairs sorted by expert, on the device: (perm [n], inv [n], tiles, max_tiles); the tile table
    lists (expert, first sorted row, end row) for row tiles of at most ``tile_rows`` rows that never span two experts.
    With ``weights`` (float32, one per pair) a fifth result: the weights in the order of the sorted rows, float32 [n]."""
    need_cuda(idx, weights)
    n = idx.numel()
    max_tiles = (n + tile_rows - 1) // tile_rows + n_experts
    dev = idx.device
    perm = torch.empty((n,), dtype=torch.int32, device=dev)
    inv = torch.empty((n,), dtype=torch.int32, device=dev)
    offsets = torch.empty((n_experts + 1,), dtype=torch.int32, device=dev)
    tiles = torch.empty((1 + 3 * max_tiles,), dtype=torch.int32, device=dev)
    if weights is not None:
        need(weights.dtype == torch.float32 and weights.is_contiguous() and weights.numel() == n, "moe_sort: one float32 weight per pair")
        ws = torch.empty((n,), dtype=torch.float32, device=dev)
        f = _f("moe", "rf_moe_sort_w", c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
               c_void_p, c_void_p)
        check(f(ptr(idx), n, n_experts, tile_rows, ptr(perm), ptr(inv), ptr(offsets), ptr(tiles), max_tiles, ptr(weights), ptr(ws),
                stream()), f"moe_sort (E={n_experts})")
        return perm, inv, tiles, max_tiles, ws
    f = _f("moe", "rf_moe_sort", c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p)
    check(f(ptr(idx), n, n_experts, tile_rows, ptr(perm), ptr(inv), ptr(offsets), ptr(tiles), max_tiles, stream()),
          f"moe_sort (E={n_experts})")
    return perm, inv, tiles, max_tiles


def moe_combine(y: torch.Tensor, inv: torch.Tensor, w: torch.Tensor | None, top: int | None = None) -> torch.Tensor:
    """out[t] = sum_k w[t, k] * y[inv[t*top + k]] in the order of k; y float32 [T*top, H] in sorted order.  Without ``w``
    (``top`` must then be given) the plain sum."""
    need_cuda(y, inv, w)
    if w is None:
        need(top is not None and top >= 1 and inv.numel() % top == 0, "moe_combine: without weights, top must be given")
        T = inv.numel() // top
    else:
        T, top = w.shape
    need(y.dtype == torch.float32 and y.is_contiguous() and y.shape[0] == T * top, "moe_combine: y must be float32 [T*top, H]")
    H = y.shape[1]
    out = torch.empty((T, H), dtype=torch.float32, device=y.device)
    f = _f("moe", "rf_moe_combine", c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p)
    check(f(ptr(y), ptr(inv), ptr(w), ptr(out), top, H, T, stream()), "moe_combine")
    return out


# ---------------------------------------------------------------- Dynamic Tanh and the scaled residual update (csrc/elementwise.cu)

def dyt_rows(h: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, compute_dtype: torch.dtype,
             rows: torch.Tensor | None = None) -> torch.Tensor:
    """y = tanh(alpha h) * weight + bias in the compute dtype, of all rows of the float32 stream ``h`` [T, H] or of those
    that ``rows`` (int32) lists; alpha (one number), weight and bias [H] are float32."""
    need_cuda(h, alpha, weight, bias, rows)
    need(h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous(), "dyt_rows: h must be contiguous float32 [T, H]")
    T, H = h.shape
    need(all(v.dtype == torch.float32 and v.is_contiguous() for v in (alpha, weight, bias)) and alpha.numel() == 1
         and weight.shape == (H,) and bias.shape == (H,), "dyt_rows: alpha [1], weight [H] and bias [H] must be float32")
    need(rows is None or rows.dtype == torch.int32, "dyt_rows: rows must be int32")
    R = T if rows is None else rows.numel()
    y = torch.empty((R, H), dtype=compute_dtype, device=h.device)
    f = _f("elementwise", "rf_dyt_rows", c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
           c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(rows), ptr(alpha), ptr(weight), ptr(bias), ptr(y), R, H, stream()),
          f"dyt_rows (H={H})")
    return y


def scaled_add(h: torch.Tensor, addends, mult: float, compute_dtype: torch.dtype, *, eps: float = 0.0,
               next_dyt=None) -> torch.Tensor | None:
    """The residual update of a block that scales its sub-layers' outputs, in 32-bit and one pass over the rows:

        m = a0 (+ a1)                             for addends == [(a0, None)] or [(a0, None), (a1, None)]
        m = (rms(a0) * w0 + rms(a1) * w1) / 2     for addends == [(a0, w0), (a1, w1)], rms(x) = x / sqrt(mean(x^2) + eps)
        h += mult * m
        returns tanh(alpha h) * w + b in the compute dtype if ``next_dyt`` = (alpha, w, b) (float32) is given, else None

    An addend is float32 [T, H] or a stack [S, T, H] of a K-split product's partial sums, added here in index order.
    """
    need(len(addends) in (1, 2), "scaled_add: one or two addends")
    a0, w0 = addends[0]
    a1, w1 = addends[1] if len(addends) == 2 else (None, None)
    need((w0 is None) == (w1 is None) or a1 is None, "scaled_add: both addends are normed with a weight, or neither")
    need(not (a1 is None and w0 is not None), "scaled_add: one addend comes without a weight")
    vecs = [v for v in (w0, w1) if v is not None]
    nd = list(next_dyt) if next_dyt is not None else []
    need_cuda(h, a0, a1, *vecs, *nd)
    T, H = h.shape
    need(h.dtype == torch.float32 and h.is_contiguous(), "scaled_add: h must be contiguous float32 [T, H]")
    for a in (a0, a1):
        need(a is None or (a.dtype == torch.float32 and tuple(a.shape[-2:]) == (T, H) and a.dim() in (2, 3) and a.is_contiguous()),
             "scaled_add: an addend must be contiguous float32 [T, H] or [S, T, H]")
    need(all(v.shape == (H,) and v.is_contiguous() and v.dtype == vecs[0].dtype for v in vecs)
         and (not vecs or vecs[0].dtype in (torch.float32, torch.bfloat16)), "scaled_add: the weights must be [H] of one dtype")
    if nd:
        need(len(nd) == 3 and all(v.dtype == torch.float32 and v.is_contiguous() for v in nd) and nd[0].numel() == 1
             and nd[1].shape == (H,) and nd[2].shape == (H,), "scaled_add: the next norm is (alpha [1], weight [H], bias [H]) in float32")
    n0 = a0.shape[0] if a0.dim() == 3 else 1
    n1 = (a1.shape[0] if a1.dim() == 3 else 1) if a1 is not None else 0
    y = torch.empty((T, H), dtype=compute_dtype, device=h.device) if nd else None
    f = _f("elementwise", "rf_scaled_add", c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p, c_int,
           c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(a0), n0, ptr(w0), ptr(a1), n1, ptr(w1),
            int(bool(vecs) and vecs[0].dtype == torch.float32), float(eps), float(mult), ptr(nd[0] if nd else None),
            ptr(nd[1] if nd else None), ptr(nd[2] if nd else None), ptr(y), T, H, stream()), f"scaled_add (H={H})")
    return y


def softcap_(x: torch.Tensor, cap: float) -> torch.Tensor:
    """x <- cap * tanh(x / cap), in place, float32."""
    need_cuda(x)
    need(x.dtype == torch.float32 and x.is_contiguous(), "softcap: a contiguous float32 tensor")
    f = _f("elementwise", "rf_softcap", c_void_p, c_ll, c_float, c_void_p)
    check(f(ptr(x), x.numel(), float(cap), stream()), "softcap")
    return x


# ---------------------------------------------------------------- recurrences with one decay per head and token (csrc/gla.cu)

def gated_scan(q: torch.Tensor, k: torch.Tensor, ab: torch.Tensor, v: torch.Tensor, state: torch.Tensor, cu_q: torch.Tensor,
               seq_slot: torch.Tensor, heads: int, dim: int, vdim: int, *, qk_heads: int | None = None,
               nstate: torch.Tensor | None = None, one_token: bool = False):
    """S_t = a_t S_(t-1) + b_t k_t v_t^T, o_t = S_t^T q_t per head, token by token for every sequence of the step.

    ``q``, ``k``: float32 [T, >= qk_heads*dim] views (rows may be strided; both with the same row stride) that hold
    ``qk_heads`` heads of ``dim``; head h reads head h // (heads / qk_heads).  ``ab`` float32 [T, heads, 2] = (a_t, b_t).
    ``v`` [T, heads*vdim] view of float32 or bfloat16.  ``state`` float32 [slots, heads, dim, vdim], read at the step's
    start and left as after its last token.  With ``nstate`` (float32 [slots, heads, dim]) the normaliser
    n_t = a_t n_(t-1) + b_t k_t is carried along and the second result is n_t . q_t, float32 [T, heads].
    Returns (o float32 [T, heads*vdim], qn or None)."""
    need_cuda(q, k, ab, v, state, cu_q, seq_slot, nstate)
    T = ab.shape[0]
    qk_heads = heads if qk_heads is None else int(qk_heads)
    need(heads % qk_heads == 0, "gated_scan: the heads must share q and k heads evenly")
    for x in (q, k):
        need(x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] == T and x.shape[1] >= qk_heads * dim and x.stride(1) == 1
             and x.stride(0) == q.stride(0), "gated_scan: q and k must be float32 [T, >= qk_heads*dim] with one row stride")
    need(ab.dtype == torch.float32 and ab.is_contiguous() and ab.shape == (T, heads, 2), "gated_scan: ab must be float32 [T, heads, 2]")
    need(v.shape == (T, heads * vdim) and v.stride(1) == 1, "gated_scan: v must be [T, heads*vdim]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
         "gated_scan: state must be float32 [slots, heads, dim, vdim]")
    need(nstate is None or (nstate.dtype == torch.float32 and nstate.is_contiguous() and tuple(nstate.shape[1:]) == (heads, dim)),
         "gated_scan: the normaliser's state must be float32 [slots, heads, dim]")
    B = seq_slot.shape[0]
    need(not one_token or T == B, "gated_scan: one_token means one token for every sequence")
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=ab.device)
    qn = torch.empty((T, heads), dtype=torch.float32, device=ab.device) if nstate is not None else None
    f = _f("gla", "rf_gated_scan", c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(v.dtype), ptr(q), ptr(k), qk_heads, q.stride(0), ptr(ab), ptr(v), v.stride(0), ptr(state), ptr(nstate),
            ptr(o), ptr(qn), ptr(cu_q), ptr(seq_slot), B, heads, dim, vdim, int(one_token), device_sm_count(ab.device), stream()),
          f"gated_scan (heads={heads}, dim={dim}, vdim={vdim})")
    return o, qn


def gated_chunked(q: torch.Tensor, k: torch.Tensor, ab: torch.Tensor, v: torch.Tensor, state: torch.Tensor, table: torch.Tensor,
                  cu_q: torch.Tensor, seq_slot: torch.Tensor, heads: int, dim: int, vdim: int, *, qk_heads: int | None = None,
                  nstate: torch.Tensor | None = None):
    """What ``gated_scan`` computes, for prompts: the recurrence in chunks of 64 tokens that run side by side (per-chunk
    sums weighted by running products of the decays, then the states between the chunks one after the other, then every
    chunk's outputs from its start state), all in 32-bit.  ``table``: the chunk table of ``retention_chunked``.  The other
    arguments and the results are ``gated_scan``'s.  Differs from the scan by rounding only."""
    need_cuda(q, k, ab, v, state, table, cu_q, seq_slot, nstate)
    T = ab.shape[0]
    B = seq_slot.shape[0]
    qk_heads = heads if qk_heads is None else int(qk_heads)
    need(heads % qk_heads == 0, "gated_chunked: the heads must share q and k heads evenly")
    for x in (q, k):
        need(x.dtype == torch.float32 and x.dim() == 2 and x.shape[0] == T and x.shape[1] >= qk_heads * dim and x.stride(1) == 1
             and x.stride(0) == q.stride(0), "gated_chunked: q and k must be float32 [T, >= qk_heads*dim] with one row stride")
    need(ab.dtype == torch.float32 and ab.is_contiguous() and ab.shape == (T, heads, 2), "gated_chunked: ab must be float32 [T, heads, 2]")
    need(v.shape == (T, heads * vdim) and v.stride(1) == 1, "gated_chunked: v must be [T, heads*vdim]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
         "gated_chunked: state must be float32 [slots, heads, dim, vdim]")
    need(nstate is None or (nstate.dtype == torch.float32 and nstate.is_contiguous() and tuple(nstate.shape[1:]) == (heads, dim)),
         "gated_chunked: the normaliser's state must be float32 [slots, heads, dim]")
    need(table.dtype == torch.int32 and (table.numel() - (B + 1)) % 2 == 0 and table.numel() > B + 1,
         "gated_chunked: the chunk table must hold first[B+1] and a pair per chunk")
    n_chunks = (table.numel() - (B + 1)) // 2
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=ab.device)
    qn = torch.empty((T, heads), dtype=torch.float32, device=ab.device) if nstate is not None else None
    scratch = torch.empty((n_chunks * heads * (dim * vdim + 1 + (dim if nstate is not None else 0)),), dtype=torch.float32,
                          device=ab.device)
    f = _f("gla", "rf_gated_chunked", c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(v.dtype), ptr(q), ptr(k), qk_heads, q.stride(0), ptr(ab), ptr(v), v.stride(0), ptr(state), ptr(nstate),
            ptr(o), ptr(qn), ptr(scratch), ptr(table), n_chunks, ptr(cu_q), ptr(seq_slot), B, heads, dim, vdim, stream()),
          f"gated_chunked (heads={heads}, dim={dim}, vdim={vdim})")
    return o, qn


# ---------------------------------------------------------------- matrix memory (csrc/mlstm.cu)

def mlstm_prepare(proj: torch.Tensor, q_col: int, k_col: int, width: int, q_scale: float) -> torch.Tensor:
    """float32 [2, T, width]: q of the projection's rows (columns q_col..) times ``q_scale``, and k (columns k_col..)."""
    need_cuda(proj)
    need(proj.dim() == 2 and proj.stride(1) == 1 and max(q_col, k_col) + width <= proj.shape[1],
         "mlstm_prepare: the projection must be [T, columns] and hold q and k")
    T = proj.shape[0]
    qk = torch.empty((2, T, width), dtype=torch.float32, device=proj.device)
    f = _f("mlstm", "rf_mlstm_prepare", c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_float, c_int, c_void_p)
    check(f(dtype_code(proj.dtype), ptr(proj), proj.stride(0), q_col, k_col, ptr(qk), width, float(q_scale), T, stream()),
          "mlstm_prepare")
    return qk


def mlstm_gates(z: torch.Tensor, mstate: torch.Tensor, cu_q: torch.Tensor, seq_slot: torch.Tensor, heads: int, cap: float,
                max_new: int):
    """The gates' chain of the matrix memory.  ``z`` float32 [T, 2*heads]: the input gate's pre-activations (bias added),
    then the forget gate's.  li = cap tanh(zi / cap), lf = log sigmoid(cap tanh(zf / cap)) (cap <= 0: not capped),
    m_t = max(lf + m_(t-1), li) from ``mstate`` float32 [slots, heads] (updated), a_t = exp(lf + m_(t-1) - m_t),
    b_t = exp(li - m_t).  Returns (ab float32 [T, heads, 2], m float32 [T, heads])."""
    need_cuda(z, mstate, cu_q, seq_slot)
    T = z.shape[0]
    need(z.dtype == torch.float32 and z.is_contiguous() and z.shape == (T, 2 * heads), "mlstm_gates: z must be float32 [T, 2*heads]")
    need(mstate.dtype == torch.float32 and mstate.is_contiguous() and tuple(mstate.shape[1:]) == (heads,),
         "mlstm_gates: the maximum's state must be float32 [slots, heads]")
    ab = torch.empty((T, heads, 2), dtype=torch.float32, device=z.device)
    mt = torch.empty((T, heads), dtype=torch.float32, device=z.device)
    f = _f("mlstm", "rf_mlstm_gates", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int,
           c_void_p)
    check(f(ptr(z), ptr(ab), ptr(mt), ptr(mstate), ptr(cu_q), ptr(seq_slot), seq_slot.shape[0], heads, float(cap or 0.0),
            int(max_new), stream()), "mlstm_gates")
    return ab, mt


# ---------------------------------------------------------------- state-space mixer (csrc/mamba2.cu)

def conv_silu(src: torch.Tensor, col0: int, channels: int, state: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor,
              tok_seq: torch.Tensor, cu_q: torch.Tensor, seq_slot: torch.Tensor) -> torch.Tensor:
    """silu of a causal convolution per channel over the last ``taps`` inputs: ``src`` [T, columns], the channels from
    column ``col0`` on; ``weight`` [channels, taps] (the last column weighs the current token) and ``bias`` [channels] of
    one dtype; ``state`` float32 [slots, taps-1, channels] holds every sequence's inputs before the step (zeros at its
    start) and is replaced by the step's last inputs.  Returns float32 [T, channels]."""
    need_cuda(src, state, weight, bias, tok_seq, cu_q, seq_slot)
    T = src.shape[0]
    need(src.dim() == 2 and src.stride(1) == 1 and col0 + channels <= src.shape[1], "conv_silu: src must be [T, >= col0 + channels]")
    taps = weight.shape[1]
    need(weight.shape == (channels, taps) and bias.shape == (channels,) and weight.dtype == bias.dtype and weight.is_contiguous()
         and bias.is_contiguous() and weight.dtype in (torch.float32, torch.bfloat16), "conv_silu: weight [channels, taps], bias [channels]")
    need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (taps - 1, channels),
         "conv_silu: state must be float32 [slots, taps-1, channels]")
    out = torch.empty((T, channels), dtype=torch.float32, device=src.device)
    f = _f("mamba2", "rf_conv_silu", c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p)
    check(f(dtype_code(src.dtype), ptr(src), src.stride(0), col0, ptr(state), ptr(weight), ptr(bias),
            int(weight.dtype == torch.float32), ptr(out), ptr(tok_seq), ptr(cu_q), ptr(seq_slot), T, seq_slot.shape[0], channels,
            taps, stream()), f"conv_silu (channels={channels}, taps={taps})")
    return out


def mamba_gates(z: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor) -> torch.Tensor:
    """float32 [T, heads, 2] = (exp(-exp(a_log) dt), dt) with dt = softplus(z + dt_bias); z float32 [T, heads]."""
    need_cuda(z, dt_bias, a_log)
    T, heads = z.shape
    need(z.dtype == torch.float32 and z.is_contiguous(), "mamba_gates: z must be contiguous float32 [T, heads]")
    need(dt_bias.shape == (heads,) and a_log.shape == (heads,) and dt_bias.dtype == a_log.dtype and dt_bias.is_contiguous()
         and a_log.is_contiguous() and a_log.dtype in (torch.float32, torch.bfloat16), "mamba_gates: dt_bias and a_log are [heads] of one dtype")
    ab = torch.empty((T, heads, 2), dtype=torch.float32, device=z.device)
    f = _f("mamba2", "rf_mamba_gates", c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p)
    check(f(ptr(z), ptr(dt_bias), ptr(a_log), int(a_log.dtype == torch.float32), ptr(ab), T, heads, stream()), "mamba_gates")
    return ab


def mamba_finish(y: torch.Tensor, x: torch.Tensor, gate: torch.Tensor, skip: torch.Tensor, norm_w: torch.Tensor, parts: int,
                 vdim: int, eps: float) -> torch.Tensor:
    """(y + skip[head] x) * silu(gate), each of the ``parts`` equal parts of a row divided by its own root mean square,
    times ``norm_w``; y float32 [T, inner], x a float32 [T, inner] view, gate a [T, inner] view of the compute dtype (the
    result's), skip [inner / vdim] and norm_w [inner] of one dtype."""
    need_cuda(y, x, gate, skip, norm_w)
    T, inner = y.shape
    need(y.dtype == torch.float32 and y.is_contiguous() and x.dtype == torch.float32 and x.shape == (T, inner) and x.stride(1) == 1
         and gate.shape == (T, inner) and gate.stride(1) == 1, "mamba_finish: y, x float32 [T, inner], gate [T, inner]")
    need(inner % parts == 0 and inner % vdim == 0 and skip.shape == (inner // vdim,) and norm_w.shape == (inner,)
         and skip.dtype == norm_w.dtype and skip.is_contiguous() and norm_w.is_contiguous()
         and skip.dtype in (torch.float32, torch.bfloat16), "mamba_finish: skip [heads] and norm_w [inner] of one dtype")
    out = torch.empty((T, inner), dtype=gate.dtype, device=y.device)
    f = _f("mamba2", "rf_mamba_finish", c_int, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, c_void_p, c_int, c_void_p,
           c_int, c_int, c_int, c_int, c_float, c_void_p)
    check(f(dtype_code(gate.dtype), ptr(y), ptr(x), x.stride(0), ptr(gate), gate.stride(0), ptr(skip), ptr(norm_w),
            int(skip.dtype == torch.float32), ptr(out), T, inner, parts, vdim, float(eps), stream()), "mamba_finish")
    return out


# ---------------------------------------------------------------- two results side by side, each with a factor

def weighted_add(h: torch.Tensor, addends, compute_dtype: torch.dtype, *, next_norm=None) -> torch.Tensor | None:
    """h += s0 a0 (+ s1 a1) for ``addends`` = [(a0, s0)] or [(a0, s0), (a1, s1)], in 32-bit and one pass over the rows; an
    addend is float32 [T, H] or a stack [S, T, H] of a K-split product's partial sums, added here in index order.  With
    ``next_norm`` = (weight [H], eps) returns rms(h) * weight of the new rows in the compute dtype, else None."""
    need(len(addends) in (1, 2), "weighted_add: one or two addends")
    (a0, s0), (a1, s1) = addends[0], (addends[1] if len(addends) == 2 else (None, 0.0))
    w, eps = next_norm if next_norm is not None else (None, 0.0)
    need_cuda(h, a0, a1, w)
    T, H = h.shape
    need(h.dtype == torch.float32 and h.is_contiguous(), "weighted_add: h must be contiguous float32 [T, H]")
    for a in (a0, a1):
        need(a is None or (a.dtype == torch.float32 and tuple(a.shape[-2:]) == (T, H) and a.dim() in (2, 3) and a.is_contiguous()),
             "weighted_add: an addend must be contiguous float32 [T, H] or [S, T, H]")
    need(w is None or (w.shape == (H,) and w.is_contiguous() and w.dtype in (torch.float32, torch.bfloat16)),
         "weighted_add: the next norm's weight must be [H] in float32 or bfloat16")
    n0 = a0.shape[0] if a0.dim() == 3 else 1
    n1 = (a1.shape[0] if a1.dim() == 3 else 1) if a1 is not None else 0
    y = torch.empty((T, H), dtype=compute_dtype, device=h.device) if w is not None else None
    f = _f("elementwise", "rf_weighted_add", c_int, c_void_p, c_void_p, c_int, c_float, c_void_p, c_int, c_float, c_void_p, c_int,
           c_float, c_void_p, c_int, c_int, c_void_p)
    check(f(dtype_code(compute_dtype), ptr(h), ptr(a0), n0, float(s0), ptr(a1), n1, float(s1), ptr(w),
            int(w is not None and w.dtype == torch.float32), float(eps), ptr(y), T, H, stream()), f"weighted_add (H={H})")
    return y


def stretch_norm(src: torch.Tensor, stretches, eps: float):
    """RMS norms of stretches of the rows of ``src`` [T, columns]: for every (col, n, weight) of ``stretches`` (one or two;
    weight [n] or None) a tensor [T, n] of src's dtype, x / sqrt(mean(x^2) + eps) * weight over columns col .. col + n,
    sums in 32-bit; one launch."""
    need(len(stretches) in (1, 2), "stretch_norm: one or two stretches")
    ws = [w for _, _, w in stretches if w is not None]
    need_cuda(src, *ws)
    need(src.dim() == 2 and src.stride(1) == 1, "stretch_norm: src must be [T, columns] with unit inner stride")
    need(all(0 <= c and n >= 1 and c + n <= src.shape[1] for c, n, _ in stretches), "stretch_norm: a stretch leaves the row")
    need(all(w.shape == (n,) and w.is_contiguous() for _, n, w in stretches if w is not None)
         and all(w.dtype == ws[0].dtype for w in ws) and (not ws or ws[0].dtype in (torch.float32, torch.bfloat16)),
         "stretch_norm: weights are [n] vectors of one dtype, float32 or bfloat16")
    T = src.shape[0]
    outs = [torch.empty((T, n), dtype=src.dtype, device=src.device) for _, n, _ in stretches]
    (c0, n0, w0), o0 = stretches[0], outs[0]
    (c1, n1, w1), o1 = (stretches[1], outs[1]) if len(stretches) == 2 else ((0, 0, None), None)
    f = _f("elementwise", "rf_stretch_norm", c_int, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_int, c_int,
           c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p)
    check(f(dtype_code(src.dtype), ptr(src), src.stride(0), int(c0), int(n0), ptr(w0), ptr(o0), n0, int(c1), int(n1), ptr(w1),
            ptr(o1), n1, int(bool(ws) and ws[0].dtype == torch.float32), float(eps), T, stream()), "stretch_norm")
    return outs


# ---------------------------------------------------------------- gated delta rule (csrc/delta.cu)

def delta_prepare(qkv: torch.Tensor, a: torch.Tensor, dt_bias: torch.Tensor, a_log: torch.Tensor, beta_src: torch.Tensor,
                  heads: int, qk_heads: int, dim: int, q_scale: float, unit_eps: float):
    """What the gated delta rule's recurrence reads, all float32: (qn, kn, kq, decay, beta).

    ``qkv`` float32 [T, >= 2 qk_heads dim]: q heads, then k heads (the values that follow are left alone); qn = q / sqrt(sum
    q^2 + unit_eps) * q_scale and kn likewise without the scale, per head, [T, qk_heads*dim]; kq [T, qk_heads] = kn . qn;
    decay [T, heads*dim] = exp(-exp(a_log[head]) softplus(a + dt_bias)) with ``a`` float32 [T, heads*dim]; beta [T, heads] =
    sigmoid(beta_src), ``beta_src`` a [T, heads] view of the projection's output."""
    need_cuda(qkv, a, dt_bias, a_log, beta_src)
    T = qkv.shape[0]
    need(qkv.dtype == torch.float32 and qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= 2 * qk_heads * dim,
         "delta_prepare: qkv must be float32 [T, >= 2 qk_heads dim]")
    need(a.dtype == torch.float32 and a.shape == (T, heads * dim) and a.is_contiguous(), "delta_prepare: a must be float32 [T, heads*dim]")
    need(dt_bias.shape == (heads * dim,) and a_log.shape == (heads,) and dt_bias.dtype == a_log.dtype and dt_bias.is_contiguous()
         and a_log.is_contiguous() and a_log.dtype in (torch.float32, torch.bfloat16),
         "delta_prepare: dt_bias [heads*dim] and a_log [heads] of one dtype")
    need(beta_src.shape == (T, heads) and beta_src.stride(1) == 1 and beta_src.dtype in (torch.float32, torch.bfloat16),
         "delta_prepare: beta_src must be a [T, heads] view")
    need(heads % qk_heads == 0, "delta_prepare: the q/k heads must divide the heads")
    dev = qkv.device
    qn = torch.empty((T, qk_heads * dim), dtype=torch.float32, device=dev)
    kn = torch.empty_like(qn)
    kq = torch.empty((T, qk_heads), dtype=torch.float32, device=dev)
    decay = torch.empty((T, heads * dim), dtype=torch.float32, device=dev)
    beta = torch.empty((T, heads), dtype=torch.float32, device=dev)
    f = _f("delta", "rf_delta_prepare", c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p,
           c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_float, c_int, c_void_p)
    check(f(dtype_code(beta_src.dtype), ptr(qkv), qkv.stride(0), ptr(a), ptr(dt_bias), ptr(a_log), int(a_log.dtype == torch.float32),
            ptr(beta_src), beta_src.stride(0), ptr(qn), ptr(kn), ptr(kq), ptr(decay), ptr(beta), heads, qk_heads, dim,
            float(q_scale), float(unit_eps), T, stream()), "delta_prepare")
    return qn, kn, kq, decay, beta


def delta_scan(qn: torch.Tensor, kn: torch.Tensor, kq: torch.Tensor, decay: torch.Tensor, beta: torch.Tensor, v: torch.Tensor,
               state: torch.Tensor, cu_q: torch.Tensor, seq_slot: torch.Tensor, heads: int, qk_heads: int, dim: int,
               vdim: int, one_token: bool = False, lanes: int = 0) -> torch.Tensor:
    """The gated delta rule, token by token for every sequence of the step, per head (head h reads q/k head h // (heads /
    qk_heads)):  S <- diag(decay_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t.

    ``state`` float32 [slots, heads, dim, vdim] is read and replaced; ``v`` float32 [T, >= heads*vdim] view; returns o float32
    [T, heads*vdim].  The sums' order depends on (dim, position) alone.  ``one_token``: every sequence of the
    step brings exactly one token (the kernel form for decoding: four lanes a value column instead of eight, which adds a
    column's products in another order; ``lanes`` 4 or 8 forces a form, for measurements)."""
    need_cuda(qn, kn, kq, decay, beta, v, state, cu_q, seq_slot)
    T = qn.shape[0]
    B = seq_slot.shape[0]
    need(all(x.dtype == torch.float32 and x.is_contiguous() for x in (qn, kn, kq, decay, beta, state)), "delta_scan: float32 inputs")
    need(qn.shape == (T, qk_heads * dim) and kn.shape == qn.shape and kq.shape == (T, qk_heads) and decay.shape == (T, heads * dim)
         and beta.shape == (T, heads), "delta_scan: shapes of qn, kn, kq, decay, beta")
    need(v.dtype == torch.float32 and v.dim() == 2 and v.stride(1) == 1 and v.shape == (T, heads * vdim), "delta_scan: v must be float32 [T, heads*vdim]")
    need(tuple(state.shape[1:]) == (heads, dim, vdim), "delta_scan: state must be [slots, heads, dim, vdim]")
    need(dim <= 256, "delta_scan: at most 256 key channels a head")
    o = torch.empty((T, heads * vdim), dtype=torch.float32, device=qn.device)
    f = _f("delta", "rf_delta_scan", c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
           c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p)
    check(f(ptr(qn), ptr(kn), ptr(kq), ptr(decay), ptr(beta), ptr(v), v.stride(0), ptr(state), ptr(o), ptr(cu_q), ptr(seq_slot),
            B, heads, qk_heads, dim, vdim, int(bool(one_token)), int(lanes), stream()), f"delta_scan (heads={heads}, dim={dim}, vdim={vdim})")
    return o
