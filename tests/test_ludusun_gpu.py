"""The Ludusun decoder in the engine against the plain implementation (needs a GPU): whole prompts, token-by-token
decoding, portions, ragged batches, slots and pages used again, long decoding over a window's edge, generation through the
public entry point and the command line, the replay program; then each mechanism's kernels alone against the plain
functions, with inputs made so that a key one place off, a sink left out, a lost state or a missing gate shows."""
import json
import math
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import LUDUSUN_CONFIGS, ROOT, TraceRun, random_tokens
from plain import ludusun_plain as P

pytestmark = pytest.mark.gpu

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
NAMES = ["LA", "LB", "LC", "LD"]
_models, _plains, _refs = {}, {}, {}


def engine(folders, name, dtype):
    import rocmforge_b200 as rf
    if (name, dtype) not in _models:
        _models[(name, dtype)] = rf.Model.from_folder(folders(name, dtype), dtype=TORCH[dtype])
    return _models[(name, dtype)]


def plain_model(folders, name, dtype):
    from safetensors.torch import load_file
    if (name, dtype) not in _plains:
        folder = folders(name, dtype)
        _plains[(name, dtype)] = P.PlainLudusun(json.load(open(os.path.join(folder, "config.json"))),
                                                load_file(os.path.join(folder, "model.safetensors")))
    return _plains[(name, dtype)]


def plain_logits(folders, name, dtype, tokens):
    """Logits of the plain model on the folder's stored (rounded) weights, every position."""
    key = (name, dtype, tuple(tokens))
    if key not in _refs:
        _refs[key] = plain_model(folders, name, dtype).logits(list(tokens))
    return _refs[key]


def row_errors(got, ref):
    """Per row: root mean square of the difference (mean taken off) over the root mean square of the reference logits."""
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    assert got.shape == ref.shape and torch.isfinite(got).all()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / (ref - ref.mean(dim=-1, keepdim=True)).pow(2).mean().sqrt()


def close(got, ref, dtype, what):
    """Rows compared by the root mean square of their difference as a share of the logits' spread: 32-bit within 3e-4 (the
    sums' order differs from the float64 model's), bfloat16 2 % on average and none beyond 8 %."""
    err = row_errors(got, ref)
    if dtype == "float32":
        assert float(err.max()) < 3e-4, f"{what}: row errors up to {float(err.max()):.2e} (row {int(err.argmax())})"
        return
    assert float(err.mean()) < 0.02 and float(err.max()) < 0.08, \
        f"{what}: row errors up to {float(err.max()):.3f} (row {int(err.argmax())}), mean {float(err.mean()):.3f}"


def vocab(name):
    return LUDUSUN_CONFIGS[name]["vocab"]


def poison_free_pages(cache):
    for g in cache.groups:
        free = [p for p in range(g.n_pages) if not g.pool.is_held(p)]
        if free:
            idx = torch.tensor(free, device=g.storage.device)
            g.storage[:, :, idx] = float("nan")
            if g.value_storage is not None:
                g.value_storage[:, :, idx] = float("nan")


# --------------------------------------------------------------------------- the model in the engine

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompt(folders, name, dtype):
    """Every position of a prompt that crosses four page borders and leaves every window of the configuration behind."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    toks = random_tokens(vocab(name), 270, 3)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got = m.step(cache, [StepRequest(s, toks, range(len(toks)))]).cpu()
    close(got, plain_logits(folders, name, dtype, toks), dtype, f"{name} {dtype} whole prompt")


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(folders, name, monkeypatch):
    """The 32-bit residual stream after each layer against the plain model's, so that a fault names its layer."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, "float32")
    toks = random_tokens(vocab(name), 90, 4)
    want = []
    plain_model(folders, name, "float32").logits(toks, trace=want)
    cache = m.new_cache(max_tokens=256, max_slots=1)
    s = cache.alloc_slot()
    got = []
    for block in m.spec.blocks:
        def recording(ctx, stream, view, inner=block.forward):
            inner(ctx, stream, view)
            stream.flush()
            got.append(stream.h.detach().cpu().clone())
        monkeypatch.setattr(block, "forward", recording)
    m.step(cache, [StepRequest(s, toks, range(len(toks)))])
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert float((g.double() - w).abs().max()) < 2e-5 * max(1.0, float(w.abs().max())), f"{name}: the stream differs after layer {i}"


@pytest.mark.parametrize("name", ["LA", "LB", "LD"])
def test_token_by_token_from_the_first_token(folders, name):
    """One token a step from an empty cache and zero states: the first tokens (fewer than the convolution's taps, the
    temperature's first steps), a page border, a window's edge; and the same logits as the prompt in one step."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, "float32")
    toks = random_tokens(vocab(name), 150, 5)
    ref = plain_logits(folders, name, "float32", toks)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    s = cache.alloc_slot()
    got = torch.cat([m.step(cache, [StepRequest(s, [t], [0])]).cpu() for t in toks])
    close(got, ref, "float32", f"{name} token by token")
    s2 = cache.alloc_slot()
    whole = m.step(cache, [StepRequest(s2, toks, range(len(toks)))]).cpu()
    assert float(row_errors(got, whole).max()) < 1e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_portions_of_many_sizes(folders, name, dtype):
    """A prompt cut into portions of 1 to 70 tokens: the delta rule's state and the convolution's last inputs are carried
    from step to step (portions shorter than the taps among them); positions count from the sequence's start, not a
    portion's (the temperature, the rotation, the windows)."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    sizes = [2, 3, 64, 1, 5, 17, 2, 70, 33, 2, 1, 8, 40]
    toks = random_tokens(vocab(name), sum(sizes), 7)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    got, at = [], 0
    for n in sizes:
        got.append(m.step(cache, [StepRequest(s, toks[at:at + n], range(n))]).cpu())
        at += n
    close(torch.cat(got), plain_logits(folders, name, dtype, toks), dtype, f"{name} {dtype} portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_ragged_batch_then_decoding_with_slots_used_again(folders, name, dtype):
    """Unequal prompts in one step (one of a single token, one shorter than the convolution's taps), decoded together;
    requests end at different steps, their slots (a state and a convolution's inputs) and pages go to new requests; every
    request must equal the plain model's logits for it alone."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    V = vocab(name)
    lens = [(1, 30), (70, 12), (131, 25), (2, 6)]
    seqs = [random_tokens(V, a + b, 20 + i) for i, (a, b) in enumerate(lens)]
    refs = [plain_logits(folders, name, dtype, t) for t in seqs]
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    poison_free_pages(cache)
    slots = [cache.alloc_slot() for _ in lens]
    got = m.step(cache, [StepRequest(sl, t[:a], [0, a - 1]) for sl, t, (a, _) in zip(slots, seqs, lens)]).cpu()
    want = torch.stack([r[i] for r, (a, _) in zip(refs, lens) for i in (0, a - 1)])
    close(got, want, dtype, f"{name} {dtype} ragged prompts")
    live = list(range(len(lens)))
    for step in range(30):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        poison_free_pages(cache)
        got = m.step(cache, [StepRequest(slots[i], [seqs[i][lens[i][0] + step]], [0]) for i in live]).cpu()
        close(got, torch.stack([refs[i][lens[i][0] + step] for i in live]), dtype, f"{name} {dtype} batch decode step {step}")
    for i in live:
        cache.free_slot(slots[i])
    # the freed slots again: a state or a convolution's inputs that were not zeroed, or a page that kept old keys, would show
    again = [random_tokens(V, n, 40 + n) for n in (45, 9)]
    slots = [cache.alloc_slot() for _ in again]
    got = m.step(cache, [StepRequest(sl, t, [0, len(t) - 1]) for sl, t in zip(slots, again)]).cpu()
    want = torch.cat([plain_logits(folders, name, dtype, t)[[0, len(t) - 1]] for t in again])
    close(got, want, dtype, f"{name} {dtype} reused slots")


def test_a_batch_changes_nothing_beyond_rounding(folders):
    """A request's logits in a batch of unequal requests equal its logits alone up to the order of 32-bit sums (products of
    few tokens cut K into partial sums, products of many do not), in the prompt step and in decoding."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "LB", "float32")
    V = vocab("LB")
    seqs = [random_tokens(V, n, 80 + n) for n in (150, 3, 77)]
    cache = m.new_cache(max_tokens=64 * 12, max_slots=6)
    alone_rows = []
    for t in seqs:
        s = cache.alloc_slot()
        a = [m.step(cache, [StepRequest(s, t[:-2], [len(t) - 3])]).cpu()]
        a += [m.step(cache, [StepRequest(s, [x], [0])]).cpu() for x in t[-2:]]
        alone_rows.append(torch.cat(a))
        cache.free_slot(s)
    slots = [cache.alloc_slot() for _ in seqs]
    tog = [m.step(cache, [StepRequest(sl, t[:-2], [len(t) - 3]) for sl, t in zip(slots, seqs)]).cpu()]
    tog += [m.step(cache, [StepRequest(sl, [t[k]], [0]) for sl, t in zip(slots, seqs)]).cpu() for k in (-2, -1)]
    for i in range(len(seqs)):
        assert float(row_errors(torch.stack([x[i] for x in tog]), alone_rows[i]).max()) < 1e-4, f"request {i} depends on its batch"


@pytest.mark.parametrize("name,dtype", [("LB", "float32"), ("LC", "float32"), ("LC", "bfloat16")])
def test_long_decoding_past_the_windows(folders, name, dtype):
    """Three hundred single-token steps after a short prompt, two sequences side by side: windows of 33 to 130 pass over
    decoded tokens and the pages that left them are handed back, the attention without a window reaches back to the first
    token, the temperature steps several times, the state runs on."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    a, b = random_tokens(vocab(name), 330, 9), random_tokens(vocab(name), 330, 10)
    cache = m.new_cache(max_tokens=64 * 13, max_slots=2)
    sa, sb = cache.alloc_slot(), cache.alloc_slot()
    got = [m.step(cache, [StepRequest(sa, a[:30], [29]), StepRequest(sb, b[:30], [29])]).cpu()]
    for x, y in zip(a[30:], b[30:]):
        poison_free_pages(cache)
        got.append(m.step(cache, [StepRequest(sa, [x], [0]), StepRequest(sb, [y], [0])]).cpu())
    got = torch.stack(got)
    close(got[:, 0], plain_logits(folders, name, dtype, a)[29:], dtype, f"{name} long decoding, first sequence")
    close(got[:, 1], plain_logits(folders, name, dtype, b)[29:], dtype, f"{name} long decoding, second sequence")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(folders, dtype):
    """LLM.generate: the scheduler admits unequal prompts, decode steps replay from graphs (the warm-up run before a
    capture must leave the state and the convolution's inputs as they were), requests end at different lengths."""
    import rocmforge_b200 as rf
    name = "LC"
    llm = rf.LLM(folders(name, dtype), dtype=dtype)
    prompts = [random_tokens(vocab(name), n, 60 + n) for n in (3, 140, 11)]
    out = llm.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 12
        seq = list(p)
        for k, tok in enumerate(r.tokens):
            row = plain_logits(folders, name, dtype, seq)[-1]
            best = int(torch.argmax(row))
            slack = (1e-5 if dtype == "float32" else 2e-2) * float(row.abs().max())
            assert tok == best or float(row[best] - row[tok]) <= slack, \
                f"request of {len(p)} tokens, generated token {k}: {tok}, plain {best}"
            seq.append(tok)


def test_command_line(folders):
    """bin/rocmforge on a Ludusun folder: greedy tokens equal the plain model's."""
    folder = folders("LA", "float32")
    prompt = random_tokens(vocab("LA"), 9, 91)
    out = subprocess.run([os.path.join(ROOT, "bin", "rocmforge"), "--model", folder, "--dtype", "float32", "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--stop-ids", "", "--debug"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [int(l.split("token_id=")[1]) for l in out.stderr.splitlines() if l.startswith("[Generated]")]
    seq = list(prompt)
    for tok in ids:
        row = plain_logits(folders, "LA", "float32", seq)[-1]
        assert tok == int(torch.argmax(row)) or float(row.max() - row[tok]) <= 1e-5 * float(row.abs().max())
        seq.append(tok)
    assert len(ids) == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    """bin/trace_run on a Ludusun folder: whole prompts, a prompt and its last tokens one by one, and a batch."""
    name = "LB"
    V = vocab(name)
    a, b, c = random_tokens(V, 180, 71), random_tokens(V, 37, 72), random_tokens(V, 5, 73)
    ra, rb, rc = (plain_logits(folders, name, dtype, t) for t in (a, b, c))
    tr = TraceRun(folders(name, dtype), dtype, str(tmp_path / "out"), max_tokens=512)
    got = tr.step([("a", a, [0, 6, 7, 99, 100, 179])], end=["a"])
    close(got, ra[[0, 6, 7, 99, 100, 179]], dtype, "replay: whole")
    got = tr.step([("b", b[:30], [29])])
    close(got, rb[[29]], dtype, "replay: prompt")
    for i in range(30, 37):
        got = tr.step([("b", [b[i]], [0])], end=["b"] if i == 36 else [])
        close(got, rb[[i]], dtype, f"replay: decoded {i}")
    got = tr.step([("x", a[:160], [159]), ("y", c[:3], []), ("z", b[:20], [0, 19])])
    close(got, torch.stack([ra[159], rb[0], rb[19]]), dtype, "replay: batch")
    got = tr.step([("x", [a[160]], [0]), ("y", [c[3]], [0]), ("z", [b[20]], [0])], end=["y"])
    close(got, torch.stack([ra[160], rc[3], rb[20]]), dtype, "replay: batch decoded")
    assert tr.step([("x", [a[161]], []), ("z", [b[21]], [])], end=["x", "z"]) is None
    assert tr.close() == 0


# --------------------------------------------------------------------------- the kernels alone

def _paged(k, v, n_pages_extra=2):
    """One sequence's keys [T, nkv, d] and values [T, nkv, dv] as pages in a shuffled order, with its block table."""
    T, nkv, d = k.shape
    dv = v.shape[2]
    n = (T + 63) // 64
    order = torch.randperm(n + n_pages_extra)[:n]
    kp = torch.full((n + n_pages_extra, nkv, 64, d), float("nan"), device=k.device, dtype=k.dtype)
    vp = torch.full((n + n_pages_extra, nkv, 64, dv), float("nan"), device=k.device, dtype=k.dtype)
    for p in range(n):
        rows = slice(64 * p, min(T, 64 * p + 64))
        kp[order[p], :, : rows.stop - rows.start] = k[rows].transpose(0, 1)
        vp[order[p], :, : rows.stop - rows.start] = v[rows].transpose(0, 1)
    return kp, vp, order.to(torch.int32).to(k.device).reshape(1, n)


def _standing_out(T, i, j, dev, dtype, nh, nkv, d, dv, hidden=()):
    """Queries, keys and values in which the query at position i scores key j far above all others, and the keys in
    ``hidden`` (which the mask must not let through) higher still, with huge values."""
    torch.manual_seed(1000 * i + j)
    q = torch.randn(T, nh, d, device=dev) * 0.05
    k = torch.randn(T, nkv, d, device=dev) * 0.05
    v = torch.randn(T, nkv, dv, device=dev)
    q[i] = 0.0
    q[i, :, 0] = 40.0
    k[j, :, 0] = 1.0
    for x in hidden:
        k[x, :, 0] = 2.0
        v[x] = 1000.0
    return q.to(dtype), k.to(dtype), v.to(dtype)


def _generic(q, k, v, rows, scale, window=None, sinks=None):
    from rocmforge_b200 import kernels
    T, nh, d = q.shape
    nkv, dv = k.shape[1], v.shape[2]
    kp, vp, bt = _paged(k, v)
    dev = q.device
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.tensor(list(rows), dtype=torch.int32, device=dev)
    seq = torch.zeros(len(pos), dtype=torch.int32, device=dev)
    return kernels.attention_generic(q[list(rows)].reshape(len(pos), nh * d).contiguous(), nh, nkv, d, kp, vp, seq, pos, zero,
                                     bt, scale, window, v_head_dim=dv, sinks=sinks).reshape(len(pos), nh, dv)


@pytest.mark.parametrize("i,j", [(299, 0), (299, 63), (299, 64), (130, 1), (255, 128), (256, 127), (64, 0), (63, 63)])
def test_a_far_key_among_hundreds_with_sinks(i, j):
    """Full causal attention with a sink per head: one key far back (the first token, a page's last and first position)
    stands out among hundreds and is found, in a prompt and as a step of its own; then every row against the softmax
    written out; and a sink that stands out swallows the output while one far below changes nothing."""
    dev, T, nh, nkv, d, dv = "cuda", 300, 6, 2, 24, 40
    q, k, v = _standing_out(T, i, j, dev, torch.float32, nh, nkv, d, dv)
    sinks = torch.linspace(-2.0, 2.0, nh, device=dev)
    for rows in (range(i + 1), [i]):
        out = _generic(q, k, v, rows, 1.0, sinks=sinks)
        assert (out[-1] - v[j][[0, 0, 0, 1, 1, 1]]).abs().max() < 1e-3, f"query {i} does not find key {j}"
    out = _generic(q, k, v, range(T), 0.5, sinks=sinks)
    want = P.softmax_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), 0.5, sinks=sinks.double().cpu())
    assert (out.double().cpu() - want).abs().max() < 1e-4 * max(1.0, float(want.abs().max()))
    big = torch.tensor([60.0, -60.0, 60.0, -60.0, 60.0, -60.0], device=dev)
    out = _generic(q, k, v, [i], 1.0, sinks=big)[0]
    assert out[[0, 2, 4]].abs().max() < 1e-6 and (out[[1, 3, 5]] - v[j][[0, 1, 1]]).abs().max() < 1e-3


@pytest.mark.parametrize("window,i", [(7, 299), (7, 6), (7, 7), (64, 64), (64, 63), (64, 200), (70, 133), (130, 129), (130, 130),
                                      (1, 150), (100, 299), (33, 64)])
def test_keys_just_inside_and_just_outside_a_window(window, i):
    """The oldest key of the window stands out and is found; the key just before it stands out more, with a huge value,
    and leaves no trace; window edges on and off page borders, windows longer than the sequence so far; the query in a
    prompt and as a step of its own."""
    dev, T, nh, nkv, d, dv = "cuda", 300, 4, 4, 16, 16
    lo = max(0, i - window + 1)
    q, k, v = _standing_out(T, i, lo, dev, torch.float32, nh, nkv, d, dv, hidden=[lo - 1] if lo > 0 else [])
    for rows in (range(i + 1), [i]):
        out = _generic(q, k, v, rows, 1.0, window=window)
        assert (out[-1] - v[lo]).abs().max() < 1e-3, f"window {window}, query {i}: the wrong keys are seen"
    out = _generic(q, k, v, range(T), 0.5, window=window)
    want = P.softmax_attention(q.double().cpu(), k.double().cpu(), v.double().cpu(), 0.5, window=window)
    assert (out.double().cpu() - want).abs().max() < 1e-3 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("hd,nh,nkv", [(64, 4, 2), (128, 8, 1), (64, 6, 6)])
def test_tensor_core_attention_with_sinks(hd, nh, nkv):
    """The bfloat16 kernels with a sink per head: the tcgen05 prompt attention (whole prompt and a second portion) and the
    clustered decode attention with one to eight CTAs a sequence, against the generic kernel on every row, with sinks from
    far below to far above the scores."""
    from rocmforge_b200 import kernels
    dev, T = "cuda", 450
    q, k, v = _standing_out(T, 449, 3, dev, torch.bfloat16, nh, nkv, hd, hd)
    q = (q.float() * 8).to(torch.bfloat16)
    sinks = torch.linspace(-6.0, 6.0, nh, device=dev)
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    q2 = q.reshape(T, nh * hd).contiguous()
    ref = kernels.attention_generic(q2, nh, nkv, hd, kp, vp, seq, pos, zero, bt, 0.3, None, sinks=sinks).float()
    plain = kernels.attention_generic(q2, nh, nkv, hd, kp, vp, seq, pos, zero, bt, 0.3, None).float()
    assert (ref - plain).abs().max() > 0.05                                  # the sinks matter in this case
    tiles = torch.tensor([[0, r] for r in range(0, T, 128)], dtype=torch.int32, device=dev).flip(0).reshape(-1).contiguous()
    nnew = torch.tensor([T], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    got = kernels.attention_prefill_tc(q2, nh, nkv, hd, kp, vp, tiles, zero, zero, nnew, cu, bt, 0.3, None, sinks=sinks).float()
    assert (got - ref).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0), "prompt kernel"
    for j in (0, 1, 70, 200, T - 1):
        for splits in (1, 2, 8):
            one = kernels.attention_decode_warps(q2[j:j + 1].contiguous(), nh, nkv, hd, kp, vp, zero, pos[j:j + 1].contiguous(),
                                                 zero, bt, 0.3, None, splits=splits, sinks=sinks).float()
            assert (one[0] - ref[j]).abs().max() <= 2e-2 * ref[j].abs().max().clamp(min=1.0), f"decode kernel, query {j}, {splits} CTAs"
    half = 201
    tiles2 = torch.tensor([[0, r] for r in range(0, T - half, 128)], dtype=torch.int32, device=dev).reshape(-1).contiguous()
    got2 = kernels.attention_prefill_tc(q2[half:].contiguous(), nh, nkv, hd, kp, vp, tiles2, zero,
                                        torch.tensor([half], dtype=torch.int32, device=dev),
                                        torch.tensor([T - half], dtype=torch.int32, device=dev),
                                        torch.tensor([0, T - half], dtype=torch.int32, device=dev), bt, 0.3, None, sinks=sinks).float()
    assert (got2 - ref[half:]).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0)


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window,i", [(64, 448), (64, 63), (64, 64), (100, 449), (33, 395), (130, 129), (130, 130), (200, 449), (500, 449)])
def test_tensor_core_attention_at_a_window_edge_with_a_kv_head_per_head(window, i, hd):
    """The window of the latent attention on the bfloat16 kernels, as many kv heads as heads: the oldest key of the window
    stands out and is found, the key just before it stands out more and leaves no trace; the tcgen05 prompt attention
    (whole prompt, and a second portion whose tiles start in the middle of the sequence) and the clustered decode attention
    with one to eight CTAs a sequence, against the generic kernel on every row."""
    from rocmforge_b200 import kernels
    dev, T, nh = "cuda", 450, 4
    lo = max(0, i - window + 1)
    q, k, v = _standing_out(T, i, lo, dev, torch.bfloat16, nh, nh, hd, hd, hidden=[lo - 1] if lo > 0 else [])
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    q2 = q.reshape(T, nh * hd).contiguous()
    ref = kernels.attention_generic(q2, nh, nh, hd, kp, vp, seq, pos, zero, bt, 1.0, window).float()
    assert (ref[i].reshape(nh, hd) - v[lo].float()).abs().max() < 0.05
    tiles = torch.tensor([[0, r] for r in range(0, T, 128)], dtype=torch.int32, device=dev).flip(0).reshape(-1).contiguous()
    nnew = torch.tensor([T], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    got = kernels.attention_prefill_tc(q2, nh, nh, hd, kp, vp, tiles, zero, zero, nnew, cu, bt, 1.0, window).float()
    assert (got - ref).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0), f"prompt kernel, window {window}"
    assert (got[i].reshape(nh, hd) - v[lo].float()).abs().max() < 0.05
    for j in sorted({i, 70, 200, T - 1}):
        for splits in (1, 2, 8):
            one = kernels.attention_decode_warps(q2[j:j + 1].contiguous(), nh, nh, hd, kp, vp, zero, pos[j:j + 1].contiguous(),
                                                 zero, bt, 1.0, window, splits=splits).float()
            assert (one[0] - ref[j]).abs().max() <= 2e-2 * ref[j].abs().max().clamp(min=1.0), \
                f"decode kernel, window {window}, query {j}, {splits} CTAs"
    half = 201
    tiles2 = torch.tensor([[0, r] for r in range(0, T - half, 128)], dtype=torch.int32, device=dev).reshape(-1).contiguous()
    got2 = kernels.attention_prefill_tc(q2[half:].contiguous(), nh, nh, hd, kp, vp, tiles2, zero,
                                        torch.tensor([half], dtype=torch.int32, device=dev),
                                        torch.tensor([T - half], dtype=torch.int32, device=dev),
                                        torch.tensor([0, T - half], dtype=torch.int32, device=dev), bt, 1.0, window).float()
    assert (got2 - ref[half:]).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0)


@pytest.mark.parametrize("nh,nkv,hd,rot,after,temp,same,bias", [
    (4, 2, 16, 8, True, None, False, False), (9, 1, 20, 6, True, None, False, False), (4, 1, 128, 128, True, None, False, False),
    (4, 2, 16, 0, False, (0.3, 5), True, True), (3, 3, 40, 0, False, None, True, True), (16, 1, 64, 0, False, (1.0, 1), True, True),
    (2, 2, 64, 32, False, (0.5, 64), False, True), (2, 1, 24, 0, False, (0.7, 2.5), True, False)])
def test_heads_on_their_way_into_the_cache(nh, nkv, hd, rot, after, temp, same, bias):
    """The per-head writer's options, alone and together: heads divided by their root mean square after the rotation (with
    lengthened pairs the order matters), a bias, a query temperature at positions around its steps, rows whose keys are
    their values; from one tensor and from a stack of partial sums; positions across a page border."""
    from rocmforge_b200 import kernels
    dev = "cuda"
    torch.manual_seed(nh * 100 + hd)
    T, hdv, eps, mag = 140, hd if same else 24, 1e-5, 1.3
    width = (nh + nkv) * hd + (0 if same else nkv * hdv)
    x = torch.randn(T, width + 8, device=dev)
    b = torch.randn(width, device=dev) if bias else None
    pos = torch.arange(3, 3 + T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    n_pages = 4
    bt = torch.tensor([[2, 0, 3, 1]], dtype=torch.int32, device=dev)
    inv = (torch.rand(rot // 2, device=dev) * 0.5).float() if rot else None
    # the plain way
    xb = x[:, :width].double() + (b.double() if bias else 0.0)
    qh = xb[:, : nh * hd].view(T, nh, hd)
    kh = xb[:, nh * hd: (nh + nkv) * hd].view(T, nkv, hd)
    if rot:
        qh = P.turn_pairs(qh, pos.cpu().to(x.device), inv.double(), mag, rot)
        kh = P.turn_pairs(kh, pos.cpu().to(x.device), inv.double(), mag, rot)
    if after:
        qh, kh = P.unit_rms(qh, eps), P.unit_rms(kh, eps)
    if temp:
        p = pos.double()
        qh = qh * (1.0 + temp[0] * torch.log(torch.floor((p + 1) / temp[1]) + 1.0))[:, None, None]
    for form in ("tensor", "partials"):
        kp = torch.zeros(n_pages, nkv, 64, hd, device=dev)
        vp = None if same else torch.zeros(n_pages, nkv, 64, hdv, device=dev)
        src = x if form == "tensor" else torch.stack([x * 0.25, x * 0.5, x * 0.25]).contiguous()
        q = kernels.head_norm_kv_write(src, nh, nkv, hd, hdv, inv, seq, pos, zero, bt, kp, vp, True, compute_dtype=torch.float32,
                                       rot_dim=rot, unit_norm_eps=eps if after else None, magnitude=mag if rot else 1.0, bias=b,
                                       norm_after_rotation=after, q_temperature=temp, values_are_keys=same)
        assert (q.double().view(T, nh, hd) - qh).abs().max() < 2e-5 * max(1.0, float(qh.abs().max())), form
        for t in (0, 60, 61, 139):
            pg, off = bt[0, (3 + t) // 64], (3 + t) % 64
            assert (kp[pg, :, off].double() - kh[t]).abs().max() < 2e-5 * max(1.0, float(kh.abs().max())), (form, t)
            if not same:
                want_v = xb[t, (nh + nkv) * hd:].view(nkv, hdv)
                assert (vp[pg, :, off].double() - want_v).abs().max() < 1e-5, (form, t)


def _steps(lengths_per_step):
    """[(slot, tokens)] per step -> per step (cu_q, seq_slot) on the device and the rows of each sequence."""
    out = []
    for step in lengths_per_step:
        cu = [0]
        for _, n in step:
            cu.append(cu[-1] + n)
        out.append((torch.tensor(cu, dtype=torch.int32, device="cuda"),
                    torch.tensor([s for s, _ in step], dtype=torch.int32, device="cuda"), step))
    return out


@pytest.mark.parametrize("heads,qk_heads,dim,vdim", [(2, 1, 24, 12), (4, 2, 64, 32), (1, 1, 256, 8), (3, 3, 16, 70), (4, 4, 128, 128),
                                                     (2, 2, 33, 40)])
def test_delta_rule_kernels(heads, qk_heads, dim, vdim):
    """The prepared inputs (unit vectors, k . q, decays, beta) and the recurrence against the plain functions: two sequences
    in slots 2 and 0 over four steps (a long portion, a short one, single tokens), a slot zeroed and used again, decays of
    exactly 1 (a channel that never forgets) and of 0 (one that forgets at once), beta of 0 and 1; the same bits however
    the tokens are cut into steps; and the form for steps of one token a sequence against the general one."""
    from rocmforge_b200 import kernels
    dev = "cuda"
    torch.manual_seed(heads * 1000 + dim)
    plan = [[(2, 37), (0, 5)], [(2, 2), (0, 70)], [(2, 1), (0, 1)], [(2, 1), (0, 1)]]
    total = {2: 41, 0: 77}
    G, H, D, V = qk_heads, heads, dim, vdim
    data = {}
    for slot, n in total.items():
        qkv = torch.randn(n, 2 * G * D + H * V, device=dev)
        a = torch.randn(n, H * D, device=dev) * 2
        a[:, 0] = -200.0                                  # softplus -> 0: decay exactly 1
        a[:, 1] = 200.0                                   # a large step: the channel forgets (decay exp(-200 e^A))
        bsrc = torch.randn(n, H, device=dev) * 2
        bsrc[3] = -200.0                                  # beta 0: the token writes nothing
        bsrc[5] = 200.0                                   # beta 1: the token's value replaces what its key read
        data[slot] = (qkv, a, bsrc)
    dt_bias = torch.randn(H * D, device=dev) * 0.5
    a_log = torch.tensor([-1.0, 0.5, 2.0, 0.0][:H], device=dev)
    q_scale = D ** -0.5

    def plain(slot):
        qkv, a, bsrc = (x.double().cpu() for x in data[slot])
        n = qkv.shape[0]
        q = qkv[:, : G * D].view(n, G, D)
        k = qkv[:, G * D: 2 * G * D].view(n, G, D)
        v = qkv[:, 2 * G * D:].view(n, H, V)
        q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * q_scale
        k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
        g = torch.exp(-torch.exp(a_log.double().cpu())[None, :, None]
                      * torch.nn.functional.softplus(a.view(n, H, D) + dt_bias.double().cpu().view(H, D)))
        beta = torch.sigmoid(bsrc)
        outs, states = [], []
        for h in range(H):
            o, S = P.delta_recurrence(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], beta[:, h], g[:, h])
            outs.append(o); states.append(S)
        return torch.stack(outs, dim=1), torch.stack(states)

    def run(plan, one_token=False):
        state = torch.full((3, H, D, V), float("nan"), device=dev)
        state[[0, 2]] = 0.0
        at = {s: 0 for s in total}
        outs = {s: [] for s in total}
        for cu, slots, step in _steps(plan):
            parts = [tuple(x[at[s]: at[s] + n] for x in data[s]) for s, n in step]
            qkv, a, bsrc = (torch.cat([p[i] for p in parts]).contiguous() for i in range(3))
            qn, kn, kq, decay, beta = kernels.delta_prepare(qkv, a, dt_bias, a_log, bsrc, H, G, D, q_scale, 1e-6)
            o = kernels.delta_scan(qn, kn, kq, decay, beta, qkv[:, 2 * G * D:], state, cu, slots, H, G, D, V, one_token=one_token)
            row = 0
            for s, n in step:
                outs[s].append(o[row: row + n]); row += n; at[s] += n
        return {s: torch.cat(v) for s, v in outs.items()}, state
    got, state = run(plan)
    for slot, n in total.items():
        want_o, want_S = plain(slot)
        scale = max(1.0, float(want_o.abs().max()))
        assert (got[slot].double().cpu().view(n, H, V) - want_o).abs().max() < 2e-4 * scale, f"slot {slot}: outputs"
        assert (state[slot].double().cpu() - want_S).abs().max() < 2e-4 * max(1.0, float(want_S.abs().max())), f"slot {slot}: state"
    assert torch.isnan(state[1]).all()                    # a slot that no sequence of the step holds is left alone
    # other cuts, the same bits: token by token, and all at once
    single = [[(2, 1), (0, 1)]] * 41 + [[(0, 1)]] * 36
    got1, state1 = run(single)
    got2, state2 = run([[(0, 77), (2, 41)]])
    for slot in total:
        assert torch.equal(got[slot], got1[slot]) and torch.equal(got[slot], got2[slot]), "the cut changes the outputs' bits"
        assert torch.equal(state[slot], state1[slot]) and torch.equal(state[slot], state2[slot])
    # the kernel form of decoding (one token a sequence) adds a column's products in another order: equal up to rounding
    got3, state3 = run(single, one_token=True)
    for slot in total:
        assert (got3[slot] - got[slot]).abs().max() < 1e-5 * max(1.0, float(got[slot].abs().max()))
        assert (state3[slot] - state[slot]).abs().max() < 1e-5 * max(1.0, float(state[slot].abs().max()))


def test_the_sum_of_two_branches_and_the_norm_after_it():
    """stream += s0 a0 + s1 a1 with stacks of partial sums, and the next norm (weight stored around zero) in the same pass;
    RMS norms of two stretches of a row; the scaled embedding."""
    from rocmforge_b200 import kernels
    dev = "cuda"
    torch.manual_seed(5)
    for T, H in ((3, 100), (300, 256), (1, 64)):
        h = torch.randn(T, H, device=dev)
        a0 = torch.randn(3, T, H, device=dev)
        a1 = torch.randn(T, H, device=dev)
        w = torch.randn(H, device=dev) * 0.1 + 1.0
        want_h = h.double() + 0.8 * a0.double().sum(0) + 0.5 * a1.double()
        want_y = P.unit_rms(want_h, 1e-5) * w.double()
        for dt in (torch.float32, torch.bfloat16):
            hh = h.clone()
            y = kernels.weighted_add(hh, [(a0, 0.8), (a1, 0.5)], dt, next_norm=(w, 1e-5))
            assert (hh.double() - want_h).abs().max() < 1e-5
            assert (y.double() - want_y).abs().max() < (1e-5 if dt == torch.float32 else 3e-2)
        hh = h.clone()
        assert kernels.weighted_add(hh, [(a1, -2.0)], torch.float32) is None
        assert (hh.double() - (h.double() - 2.0 * a1.double())).abs().max() < 1e-5
    x = torch.randn(50, 61, device=dev)
    w0, w1 = torch.randn(12, device=dev), torch.randn(20, device=dev)
    y0, y1 = kernels.stretch_norm(x, [(8, 12, w0), (32, 20, w1)], 1e-6)
    assert (y0.double() - P.unit_rms(x[:, 8:20].double(), 1e-6) * w0.double()).abs().max() < 1e-5
    assert (y1.double() - P.unit_rms(x[:, 32:52].double(), 1e-6) * w1.double()).abs().max() < 1e-5
    table = torch.randn(30, 40, device=dev).to(torch.bfloat16)
    ids = torch.tensor([3, 29, 0], dtype=torch.int32, device=dev)
    assert torch.equal(kernels.embed(table, ids, scale=3.0), table[ids.long()].float() * 3.0)
    assert torch.equal(kernels.embed(table, ids), table[ids.long()].float())
