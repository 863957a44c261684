"""Plain, slow implementation of the Ludusun decoder, used as the test oracle.

One function per mechanism, whole sequences only, no cache, no batching; everything in ``dtype`` (float64 by
default).  It shares no code with ``rocmforge_b200``: tensors come in as a plain {name: tensor} dict and the
configuration as the dict that config.json holds.

Notation: W[name] is stored [out, in] and applied as x @ W.T; rms(x) = x / sqrt(mean(x^2) + eps).
"""
from __future__ import annotations

import math

import torch


def silu(z):
    return z * torch.sigmoid(z)


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def zero_centred_norm(x, w, eps):
    """RMS norm whose weight is stored around zero: rms(x) * (1 + w)."""
    return unit_rms(x, eps) * (1.0 + w)


# --------------------------------------------------------------------------- rotation

def ramped_frequencies(dims: int, base: float, scaling):
    """(f [dims/2], magnitude): f_i = base^(-2i/dims); with ``scaling`` (factor, original, fast, slow) a ramp over the pair
    index blends f_i towards f_i / factor, and sine and cosine grow by 0.1 ln(factor) + 1."""
    f = [float(base) ** (-2.0 * i / dims) for i in range(dims // 2)]
    if not scaling:
        return torch.tensor(f, dtype=torch.float64), 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=torch.float64), 0.1 * math.log(factor) + 1.0


def turn_pairs(x, positions, freqs, magnitude, dims):
    """x [T, heads, dim]: element i < dims/2 of a head is paired with element i + dims/2; the rest pass."""
    if dims == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :]
    c, s = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    u, v, rest = x[..., : dims // 2], x[..., dims // 2: dims], x[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


# --------------------------------------------------------------------------- attention, three ways

def softmax_attention(q, k, v, scale, window=None, sinks=None):
    """q [T, H, D], k [T, G, D], v [T, G, V] -> [T, H, V].  Position i sees j <= i (with ``window``: i - j < window).
    ``sinks`` [H]: exp(sink_h) is one more term of the denominator, without key, value or scale."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    out = []
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        top = s.max(dim=-1, keepdim=True).values
        if sinks is not None:
            top = torch.maximum(top, sinks[h].expand_as(top))
        e = torch.exp(s - top)
        den = e.sum(dim=-1, keepdim=True)
        if sinks is not None:
            den = den + torch.exp(sinks[h] - top)
        out.append((e / den) @ v[:, g])
    return torch.stack(out, dim=1)


def sink_attention(h, W, pre, m, eps, borrowed):
    """Grouped-query attention over all earlier positions: rotation, then q and k heads divided by their root mean square,
    a sink per head.  ``borrowed``: (k, v) of the layer named by kv_from, else None.  Returns (out, (k, v))."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    pos = torch.arange(T)
    freqs, mag = ramped_frequencies(dims, rot["base"], rot.get("scaling")) if dims else (None, 1.0)
    q = unit_rms(turn_pairs((h @ W[pre + "q"].T).view(T, H, D), pos, freqs, mag, dims), eps)
    if borrowed is None:
        k = unit_rms(turn_pairs((h @ W[pre + "k"].T).view(T, G, D), pos, freqs, mag, dims), eps)
        v = (h @ W[pre + "v"].T).view(T, G, V)
    else:
        k, v = borrowed
    o = softmax_attention(q, k, v, m["scale"], sinks=W[pre + "sink"])
    return o.reshape(T, H * V) @ W[pre + "o"].T, (k, v)


def latent_attention(h, W, pre, m, eps):
    """Queries, keys and values expanded from RMS-normed latents; a window; one sigmoid gate per head."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    cq = unit_rms(h @ W[pre + "dq"].T, eps) * W[pre + "dq.norm"]
    c = unit_rms(h @ W[pre + "dkv"].T, eps) * W[pre + "dkv.norm"]
    q = (cq @ W[pre + "uq"].T).view(T, H, D)
    k = (c @ W[pre + "uk"].T).view(T, H, D)
    v = (c @ W[pre + "uv"].T).view(T, H, V)
    o = softmax_attention(q, k, v, m["scale"], window=(m.get("mask") or {}).get("size"))
    o = o * torch.sigmoid(h @ W[pre + "g"].T)[:, :, None]
    return o.reshape(T, H * V) @ W[pre + "o"].T


def key_value_attention(h, W, pre, m):
    """Causal attention whose values are its keys; q and k biases; a query temperature; an element-wise sigmoid gate."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[pre + "q"].T + W[pre + "q.b"]).view(T, H, D)
    k = (h @ W[pre + "k"].T + W[pre + "k.b"]).view(T, G, D)
    qt = m.get("q_temp")
    if qt:
        p = torch.arange(T, dtype=h.dtype)
        q = q * (1.0 + qt["coef"] * torch.log(torch.floor((p + 1) / qt["every"]) + 1.0))[:, None, None]
    o = softmax_attention(q, k, k, m["scale"]).reshape(T, H * D)
    return (o * torch.sigmoid(h @ W[pre + "g"].T)) @ W[pre + "o"].T


# --------------------------------------------------------------------------- the gated delta rule

def causal_taps(x, w):
    """silu of y_t = sum_j w[:, taps-1-j] x_(t-j): the last column weighs the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([x.new_zeros((taps - 1, C)), x], dim=0)
    y = sum(padded[j: j + T] * w[:, j][None, :] for j in range(taps))
    return silu(y)


def delta_recurrence(q, k, v, beta, g, S=None):
    """q, k [T, D], v [T, V], beta [T], g [T, D]: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    T, D = q.shape
    S = q.new_zeros((D, v.shape[1])) if S is None else S.clone()
    out = []
    for t in range(T):
        S = g[t][:, None] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out), S


def gated_delta(h, W, pre, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_taps(h @ W[pre + "q"].T, W[pre + "q.conv"]).view(T, G, D)
    k = causal_taps(h @ W[pre + "k"].T, W[pre + "k.conv"]).view(T, G, D)
    v = causal_taps(h @ W[pre + "v"].T, W[pre + "v.conv"]).view(T, H, V)
    q = q / torch.sqrt((q * q).sum(dim=-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(dim=-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[pre + "b"].T)
    a = ((h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]).view(T, H, D)
    g = torch.exp(-torch.exp(W[pre + "A_log"])[None, :, None] * torch.nn.functional.softplus(a))
    o = torch.stack([delta_recurrence(q[:, n // (H // G)], k[:, n // (H // G)], v[:, n], beta[:, n], g[:, n])[0]
                     for n in range(H)], dim=1)
    o = unit_rms(o, eps) * W[pre + "norm"]
    o = o * torch.sigmoid((h @ W[pre + "g1"].T) @ W[pre + "g2"].T).view(T, H, V)
    return o.reshape(T, H * V) @ W[pre + "o"].T


def side_by_side(h, W, pre, m, eps):
    return (m["left_scale"] * key_value_attention(h, W, pre + "left.", m["left"])
            + m["right_scale"] * gated_delta(h, W, pre + "right.", m["right"], eps))


# --------------------------------------------------------------------------- the model

def gated_unit(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def forward(cfg: dict, W: dict, tokens, dtype=torch.float64, trace=None):
    """Logits [T, vocab] of one sequence; ``trace`` (a list) receives the residual stream after every layer."""
    W = {k: v.to(dtype) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = zero_centred_norm(x, W[pre + "norm1"], eps)
        m = L["mixer"]
        if L["type"] == "attention":
            src = m.get("kv_from")
            y, kv = sink_attention(h, W, pre + "mix.", m, eps, None if src is None else kept[src])
            if src is None:
                kept[i] = kv
        elif L["type"] == "latent_attention":
            y = latent_attention(h, W, pre + "mix.", m, eps)
        else:
            y = side_by_side(h, W, pre + "mix.", m, eps)
        x = x + y
        if L.get("mlp") is not None:
            x = x + gated_unit(zero_centred_norm(x, W[pre + "norm2"], eps), W, pre + "mlp.")
        if trace is not None:
            trace.append(x.clone())
    logits = zero_centred_norm(x, W["final.norm"], eps) @ W["embed"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(logits / cap) if cap else logits


class PlainLudusun:
    def __init__(self, cfg: dict, tensors: dict):
        self.cfg, self.W = cfg, tensors

    def logits(self, tokens, trace=None):
        return forward(self.cfg, self.W, list(tokens), trace=trace)
