"""Plain, slow implementation of the Figalix decoder, used as the test oracle.

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


def dynamic_tanh(x, W, name):
    """tanh(alpha x) * w + b: a norm without statistics."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


# --------------------------------------------------------------------------- rotation

def stretched_frequencies(dims: int, base: float, scaling):
    """(f [dims/2], magnitude).  f_i = base^(-2i/dims); with ``scaling`` (factor, original, fast, slow) the pairs whose
    index lies beyond the ramp turn ``factor`` times slower, those before it as they were, and sine and cosine are
    multiplied by 0.1 ln(factor) + 1."""
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


def rotate_half(x, positions, freqs, magnitude, dims):
    """x [T, heads, dim]: element i < dims/2 of a head is paired with element i + dims/2; the rest pass."""
    if dims == 0:
        return x
    ang = positions.to(x.dtype)[:, None] * freqs.to(x.dtype)[None, :]
    c, s = (torch.cos(ang) * magnitude)[:, None, :], (torch.sin(ang) * magnitude)[:, None, :]
    u, v, rest = x[..., : dims // 2], x[..., dims // 2: dims], x[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


# --------------------------------------------------------------------------- left mixer: windowed attention

def visible(T: int, size, keep_first: int):
    """[T, T] mask: i sees j <= i with i - j < size, and the first ``keep_first`` positions always."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    near = (i - j < size) if size else torch.ones((T, T), dtype=torch.bool)
    return (j <= i) & (near | (j < keep_first))


def window_attention(h, W, pre, m):
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[pre + "q"].T).reshape(T, H, D)
    k = (h @ W[pre + "k"].T).reshape(T, G, D)
    v = (h @ W[pre + "v"].T).reshape(T, G, DV)
    rot = m.get("rot") or {}
    dims = int(rot.get("dims", 0))
    if dims:
        freqs, mag = stretched_frequencies(dims, rot["base"], rot.get("scaling"))
        pos = torch.arange(T)
        q, k = rotate_half(q, pos, freqs, mag, dims), rotate_half(k, pos, freqs, mag, dims)
    mask = m.get("mask") or {}
    see = visible(T, mask.get("size"), int(mask.get("keep_first", 0)))
    out = torch.zeros((T, H, DV), dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~see, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    gate = torch.sigmoid(h @ W[pre + "g"].T)                  # [T, H]: one number per head
    return (out * gate[:, :, None]).reshape(T, H * DV) @ W[pre + "o"].T


# --------------------------------------------------------------------------- right mixer: matrix memory

def capped(z, cap):
    return z if cap is None else cap * torch.tanh(z / cap)


def memory_recurrence(q, k, v, li, lf, S=None, n=None, mx=None):
    """q, k [T, H, D], v [T, H, DV], log gates li, lf [T, H]; state (S [H, D, DV], n [H, D], m [H]), zeros if not given.
    Returns (o [T, H, DV], S, n, m)."""
    T, H, D = q.shape
    DV = v.shape[2]
    S = torch.zeros((H, D, DV), dtype=q.dtype) if S is None else S.clone()
    n = torch.zeros((H, D), dtype=q.dtype) if n is None else n.clone()
    mx = torch.zeros((H,), dtype=q.dtype) if mx is None else mx.clone()
    o = torch.zeros((T, H, DV), dtype=q.dtype)
    for t in range(T):
        new = torch.maximum(lf[t] + mx, li[t])
        keep, take = torch.exp(lf[t] + mx - new), torch.exp(li[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
    return o, S, n, mx


def matrix_memory(h, W, pre, m, eps):
    """S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T with the running maximum m_t = max(f + m_(t-1), i)
    (m starts at 0), n likewise with k alone, o = S^T q / (max(|n . q|, exp(-m_t)) + 1e-6)."""
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    cap = float(m["gate_cap"]) if m.get("gate_cap") is not None else None
    q = (h @ W[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ W[pre + "k"].T).reshape(T, H, D)
    v = (h @ W[pre + "v"].T).reshape(T, H, DV)
    li = capped(h @ W[pre + "i"].T + W[pre + "i.b"], cap)
    lf = torch.nn.functional.logsigmoid(capped(h @ W[pre + "f"].T + W[pre + "f.b"], cap))
    o = memory_recurrence(q, k, v, li, lf)[0]
    o = unit_rms(o, eps).reshape(T, H * DV) * W[pre + "norm"]
    return (o * torch.sigmoid(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def parallel_mixer(h, W, pre, m, eps):
    left = unit_rms(window_attention(h, W, pre + "left.", m["left"]), eps) * W[pre + "left.out"]
    right = unit_rms(matrix_memory(h, W, pre + "right.", m["right"], eps), eps) * W[pre + "right.out"]
    return 0.5 * (left + right)


# --------------------------------------------------------------------------- mixer 'mamba2'

def short_convolution(x, w, b):
    """x [T, C], w [C, taps] (last column weighs the current token), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, x.shape[1]), dtype=x.dtype), x], dim=0)
    out = b.expand(T, -1).clone()
    for j in range(taps):
        out = out + padded[j: j + T] * w[:, j]
    return out


def duality_recurrence(x, B, C, dt, decay, skip, S=None):
    """x [T, H, DV], B, C [T, G, N], dt, decay [T, H], skip [H]; state S [H, N, DV], zeros if not given.
    S_t = decay_t S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + skip x_t.  Returns (y [T, H, DV], S)."""
    T, H, DV = x.shape
    G, N = B.shape[1], B.shape[2]
    S = torch.zeros((H, N, DV), dtype=x.dtype) if S is None else S.clone()
    y = torch.zeros((T, H, DV), dtype=x.dtype)
    group = torch.arange(H) // (H // G)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnv,hn->hv", S, C[t][group]) + skip[:, None] * x[t]
    return y, S


def state_space(h, W, pre, m, eps):
    T = h.shape[0]
    H, DV, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * DV
    p = h @ W[pre + "in"].T
    z, xbc, dt = p[:, :inner], p[:, inner: 2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, W[pre + "conv"], W[pre + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, DV)
    B = xbc[:, inner: inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = torch.nn.functional.softplus(dt + W[pre + "dt_bias"], threshold=1e9)
    decay = torch.exp(-torch.exp(W[pre + "A_log"]) * dt)                       # [T, H]
    y = duality_recurrence(x, B, C, dt, decay, W[pre + "D"])[0]
    y = y.reshape(T, inner) * silu(z)
    parts = int(m["norm_groups"])
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W[pre + "norm"]
    return y @ W[pre + "o"].T


# --------------------------------------------------------------------------- feed-forward

def gated_unit(h, W, pre):
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def expert_scores(h, W, pre):
    return torch.softmax(h @ W[pre + "router"].T, dim=-1)


def mixture(h, W, pre, mlp, forced=None):
    """``top`` experts by the largest softmax score over all experts, weighted by that score as it is; plus the shared
    expert.  ``forced`` [T, top]: take these experts instead of the largest (the weights stay their own scores)."""
    s = expert_scores(h, W, pre)
    top = int(mlp["router"]["top"])
    chosen = torch.topk(s, top, dim=-1).indices if forced is None else torch.as_tensor(forced, dtype=torch.long)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += s[t, e] * gated_unit(h[t: t + 1], W, f"{pre}e{e}.")[0]
    if mlp.get("shared"):
        out = out + gated_unit(h, W, pre + "shared.")
    return out, s, chosen


# --------------------------------------------------------------------------- the model

def forward(cfg: dict, W: dict, tokens, dtype=torch.float64, forced=None, trace=None):
    """Logits [T, vocab] of one sequence.  ``forced``: {layer: [T, top]} expert choices; ``trace``: a list that
    receives the residual stream after every layer."""
    W = {k: v.to(dtype) if v.is_floating_point() else v for k, v in W.items()}
    eps, mult = float(cfg["norm"]["eps"]), float(cfg["residual_mult"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    choices = {}
    for i, L in enumerate(cfg["layers"]):
        pre = f"l{i}."
        h = dynamic_tanh(x, W, pre + "norm1")
        if L["type"] == "parallel":
            mixed = parallel_mixer(h, W, pre + "mix.", L["mixer"], eps)
        elif L["type"] == "mamba2":
            mixed = state_space(h, W, pre + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + mult * mixed
        mlp = L.get("mlp")
        if mlp is not None:
            h = dynamic_tanh(x, W, pre + "norm2")
            if mlp["kind"] == "dense":
                x = x + mult * gated_unit(h, W, pre + "mlp.")
            else:
                out, s, chosen = mixture(h, W, pre + "mlp.", mlp, None if forced is None else forced.get(i))
                choices[i] = (s, chosen)
                x = x + mult * out
        if trace is not None:
            trace.append(x.clone())
    y = dynamic_tanh(x, W, "final.norm")
    logits = y @ W["embed"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return logits, choices


class PlainFigalix:
    """The plain model of a folder's config.json and tensors."""

    def __init__(self, cfg: dict, tensors: dict):
        self.cfg, self.W = cfg, tensors

    def logits(self, tokens, forced=None, chosen=None, trace=None):
        """float64 logits [T, vocab].  ``chosen``: a dict that receives, per layer with experts, for every token the
        plain model's own experts and the margin between the last one taken and the first one left out, as a share of
        the router logits' spread (infinite where every expert is taken)."""
        out, choices = forward(self.cfg, self.W, list(tokens), forced=forced, trace=trace)
        if chosen is not None:
            for layer, (s, _) in choices.items():
                top = int(self.cfg["layers"][layer]["mlp"]["router"]["top"])
                z = torch.log(s)
                ranked = torch.sort(z, dim=-1, descending=True)
                rows = []
                for t in range(z.shape[0]):
                    own = ranked.indices[t, :top].tolist()
                    if top == z.shape[1]:
                        rows.append((own, float("inf")))
                    else:
                        spread = float(ranked.values[t, 0] - ranked.values[t, -1])
                        rows.append((own, float(ranked.values[t, top - 1] - ranked.values[t, top]) / max(spread, 1e-30)))
                chosen[layer] = rows
        return out
