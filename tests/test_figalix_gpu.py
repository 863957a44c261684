"""The Figalix decoder in the engine against the plain implementation (needs a GPU): whole prompts, token-by-token
decoding, portions, ragged batches, slots and pages used again, long decoding over a window's edge with kept first
positions, generation through the public entry point and the command line, the replay program; then each mechanism's
kernels alone against the plain functions, with inputs made so that a key one place off, a dropped kept position, a
lost state or a missing gate shows."""
import json
import os
import subprocess

import numpy as np
import pytest
import torch

from helpers import FIGALIX_CONFIGS, ROOT, TraceRun, random_tokens
from plain import figalix_plain as P

pytestmark = pytest.mark.gpu

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
NAMES = ["FA", "FB", "FC", "FD"]
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
        _plains[(name, dtype)] = P.PlainFigalix(json.load(open(os.path.join(folder, "config.json"))),
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
    """Rows compared by the root mean square of their difference as a share of the logits' spread: 32-bit within 3e-4
    (the sums' order differs from the float64 model's; the logits of these random models are small numbers, so an absolute
    bound would say little); bfloat16, with the experts' choice agreed (``routed_like_the_engine``), 2.5 % on average and
    none beyond 15 %: the merge of the two mixers norms both outputs to unit size, which carries their rounding at full
    size into the stream."""
    err = row_errors(got, ref)
    if dtype == "float32":
        assert float(err.max()) < 3e-4, f"{what}: row errors up to {float(err.max()):.2e} (row {int(err.argmax())})"
        return
    assert float(err.mean()) < 0.025 and float(err.max()) < 0.15, \
        f"{what}: row errors up to {float(err.max()):.3f} (row {int(err.argmax())}), mean {float(err.mean()):.3f}"


class routed_like_the_engine:
    """With random weights a token's best experts are now and then nearly tied, and the bfloat16 engine, whose router
    sees rounded activations, takes another one than the plain model: that row is then off by its whole size, and through
    the recurrent states so are, a little, all rows after it.  So the comparison is done in two halves.  Inside this
    context every choice of the engine's router is recorded (``kernels.moe_route`` is wrapped); ``logits`` then runs the
    plain model with those choices forced on it (the weights stay its own scores) and checks that the engine's choices are
    the plain model's own wherever the plain model's margin (2 % of the router logits' spread) is not small."""

    def __init__(self, monkeypatch):
        from rocmforge_b200 import kernels
        self.calls = []
        real = kernels.moe_route

        def recording(z, top, scoring="softmax_of_chosen"):
            idx, w = real(z, top, scoring)
            self.calls.append(idx)
            return idx, w
        monkeypatch.setattr(kernels, "moe_route", recording)

    def logits(self, plain, tokens, steps=1):
        moe_layers = [i for i, L in enumerate(plain.cfg["layers"]) if (L.get("mlp") or {}).get("kind") == "moe"]
        assert len(self.calls) == steps * len(moe_layers)
        forced = {layer: torch.cat([self.calls[s * len(moe_layers) + n] for s in range(steps)]).cpu()
                  for n, layer in enumerate(moe_layers)}
        chosen = {}
        out = plain.logits(list(tokens), forced=forced, chosen=chosen)
        clear = agree = 0
        for layer in moe_layers:
            for t, (own, margin) in enumerate(chosen[layer]):
                if margin > 0.02:
                    clear += 1
                    agree += set(own) == set(int(e) for e in forced[layer][t])
        assert clear == 0 or agree >= 0.995 * clear, f"the engine's router differs from the plain one on {clear - agree} of {clear} clear calls"
        self.calls.clear()
        return out


def vocab(name):
    return FIGALIX_CONFIGS[name]["vocab"]


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
def test_whole_prompt(folders, name, dtype, monkeypatch):
    """Every position of a prompt that crosses four page borders, leaves every window of the configuration and every
    stretch of kept first positions behind."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    toks = random_tokens(vocab(name), 270, 3)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    routes = routed_like_the_engine(monkeypatch)
    got = m.step(cache, [StepRequest(s, toks, range(len(toks)))]).cpu()
    ref = plain_logits(folders, name, dtype, toks) if dtype == "float32" else routes.logits(plain_model(folders, name, dtype), toks)
    close(got, ref, dtype, f"{name} {dtype} whole prompt")


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


@pytest.mark.parametrize("name", ["FA", "FB"])
def test_token_by_token_from_the_first_token(folders, name):
    """One token a step from an empty cache and zero states: the first tokens (fewer than the convolution's taps, fewer
    than the kept positions), a page border, a window's edge; and the same logits as the prompt in one step."""
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
def test_portions_of_many_sizes(folders, name, dtype, monkeypatch):
    """A prompt cut into portions of 1 to 70 tokens: the states, the gates' running maximum and the convolution's last
    inputs are carried from step to step (portions shorter than the taps among them), and the kept positions are the
    sequence's first, not a portion's."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    sizes = [2, 3, 64, 1, 5, 17, 2, 70, 33, 2, 1, 8, 40]
    toks = random_tokens(vocab(name), sum(sizes), 7)
    cache = m.new_cache(max_tokens=512, max_slots=2)
    poison_free_pages(cache)
    s = cache.alloc_slot()
    routes = routed_like_the_engine(monkeypatch)
    got, at = [], 0
    for n in sizes:
        got.append(m.step(cache, [StepRequest(s, toks[at:at + n], range(n))]).cpu())
        at += n
    ref = (plain_logits(folders, name, dtype, toks) if dtype == "float32"
           else routes.logits(plain_model(folders, name, dtype), toks, steps=len(sizes)))
    close(torch.cat(got), ref, dtype, f"{name} {dtype} portions")


def alone(m, tokens, n_prompt):
    """A request through the engine by itself: its prompt in one step, the rest token by token; logits of every position
    from the prompt's last on, and of the prompt's first."""
    from rocmforge_b200 import StepRequest
    cache = m.new_cache(max_tokens=512, max_slots=1)
    s = cache.alloc_slot()
    rows = {}
    first = m.step(cache, [StepRequest(s, tokens[:n_prompt], [0, n_prompt - 1])]).cpu()
    rows[0], rows[n_prompt - 1] = first[0], first[-1]
    for i in range(n_prompt, len(tokens)):
        rows[i] = m.step(cache, [StepRequest(s, [tokens[i]], [0])]).cpu()[0]
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", NAMES)
def test_ragged_batch_then_decoding_with_slots_used_again(folders, name, dtype):
    """Unequal prompts in one step (one of a single token, one shorter than the convolution's taps), decoded together;
    requests end at different steps, their slots (three kinds of state!) and pages go to new requests; every request must
    equal itself alone: the plain model's logits on the 32-bit path; on the bfloat16 path the engine's own for the
    request by itself (nearly tied experts make single rows of the bfloat16 engine differ from the plain model, see
    ``routed_like_the_engine``; between two schedules of the same engine that is rare, so nine rows in ten must agree to
    2 % and the rest may differ)."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    V = vocab(name)
    lens = [(1, 30), (70, 12), (131, 25), (2, 6)]
    seqs = [random_tokens(V, a + b, 20 + i) for i, (a, b) in enumerate(lens)]
    if dtype == "float32":
        refs = [plain_logits(folders, name, dtype, t) for t in seqs]
    else:
        refs = [alone(m, t, a) for t, (a, _) in zip(seqs, lens)]
    errs = []

    def compare(got, want, what):
        if dtype == "float32":
            close(got, want, dtype, what)
        else:
            errs.extend(row_errors(got, want).tolist())
    cache = m.new_cache(max_tokens=64 * 8, max_slots=4)
    poison_free_pages(cache)
    slots = [cache.alloc_slot() for _ in lens]
    got = m.step(cache, [StepRequest(sl, t[:a], [0, a - 1]) for sl, t, (a, _) in zip(slots, seqs, lens)]).cpu()
    want = torch.stack([r[i] for r, (a, _) in zip(refs, lens) for i in (0, a - 1)])
    compare(got, want, f"{name} {dtype} ragged prompts")
    live = list(range(len(lens)))
    for step in range(30):
        for i in [i for i in live if lens[i][1] <= step]:
            cache.free_slot(slots[i]); live.remove(i)
        poison_free_pages(cache)
        got = m.step(cache, [StepRequest(slots[i], [seqs[i][lens[i][0] + step]], [0]) for i in live]).cpu()
        compare(got, torch.stack([refs[i][lens[i][0] + step] for i in live]), f"{name} {dtype} batch decode step {step}")
    for i in live:
        cache.free_slot(slots[i])
    # the freed slots again: a state, a running maximum or a convolution's inputs that were not zeroed, or a page that
    # kept old keys, would show here
    again = [random_tokens(V, n, 40 + n) for n in (45, 9)]
    slots = [cache.alloc_slot() for _ in again]
    got = m.step(cache, [StepRequest(sl, t, [0, len(t) - 1]) for sl, t in zip(slots, again)]).cpu()
    if dtype == "float32":
        want = torch.cat([plain_logits(folders, name, dtype, t)[[0, len(t) - 1]] for t in again])
    else:
        want = torch.stack([r[i] for t in again for r in [alone(m, t, len(t))] for i in (0, len(t) - 1)])
    compare(got, want, f"{name} {dtype} reused slots")
    if errs:
        errs = torch.tensor(errs)
        assert float((errs < 0.02).double().mean()) >= 0.9 and float(errs.median()) < 0.01, \
            f"{name} bfloat16: batch against alone, median row error {float(errs.median()):.4f}, {int((errs >= 0.02).sum())} of {errs.numel()} rows over 2 %"


def test_a_batch_changes_nothing_beyond_rounding(folders):
    """A request's logits in a batch of unequal requests equal its logits alone up to the order of 32-bit sums (products of
    few tokens cut K into partial sums, products of many do not), in the prompt step and in decoding."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, "FB", "float32")
    V = vocab("FB")
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


@pytest.mark.parametrize("name,dtype", [("FB", "float32"), ("FC", "float32"), ("FC", "bfloat16")])
def test_long_decoding_past_the_window_with_kept_first_positions(folders, name, dtype):
    """Three hundred single-token steps after a short prompt, two sequences side by side: windows of 33 to 130 pass over
    decoded tokens, the pages that left every window are handed back while those of the kept first positions (5, 70 and
    100 of them: less than a page and more) stay; the two sequences have twelve pages' worth of tokens and the cache
    eleven pages; the states run on.  On the bfloat16 path this is the clustered decode kernel."""
    from rocmforge_b200 import StepRequest
    m = engine(folders, name, dtype)
    a, b = random_tokens(vocab(name), 330, 9), random_tokens(vocab(name), 330, 10)
    cache = m.new_cache(max_tokens=64 * 11, max_slots=2)
    sa, sb = cache.alloc_slot(), cache.alloc_slot()
    got = [m.step(cache, [StepRequest(sa, a[:30], [29]), StepRequest(sb, b[:30], [29])]).cpu()]
    for x, y in zip(a[30:], b[30:]):
        poison_free_pages(cache)
        got.append(m.step(cache, [StepRequest(sa, [x], [0]), StepRequest(sb, [y], [0])]).cpu())
    got = torch.stack(got)
    if dtype == "float32":
        close(got[:, 0], plain_logits(folders, name, dtype, a)[29:], dtype, f"{name} long decoding, first sequence")
        close(got[:, 1], plain_logits(folders, name, dtype, b)[29:], dtype, f"{name} long decoding, second sequence")
        return
    # bfloat16: against the same engine on the whole sequence in one step (the tcgen05 prompt kernel)
    for seq, col in ((a, 0), (b, 1)):
        c2 = m.new_cache(max_tokens=512, max_slots=1)
        whole = m.step(c2, [StepRequest(c2.alloc_slot(), seq, range(29, len(seq)))]).cpu()
        errs = row_errors(got[:, col], whole)
        assert float((errs < 0.03).double().mean()) >= 0.9 and float(errs.median()) < 0.015, \
            f"{name} bfloat16 long decoding: median row error {float(errs.median()):.4f}, worst {float(errs.max()):.3f}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_public_entry_point(folders, dtype):
    """LLM.generate: the scheduler admits unequal prompts, decode steps replay from graphs (the warm-up run before a
    capture must leave the three kinds of state as they were), requests end at different lengths."""
    import rocmforge_b200 as rf
    name = "FC"
    llm = rf.LLM(folders(name, dtype), dtype=dtype)
    prompts = [random_tokens(vocab(name), n, 60 + n) for n in (3, 140, 11)]
    out = llm.generate(prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    for p, r in zip(prompts, out):
        assert len(r.tokens) == 12
        if dtype == "float32":
            seq = list(p)
            for k, tok in enumerate(r.tokens):
                row = plain_logits(folders, name, dtype, seq)[-1]
                best = int(torch.argmax(row))
                assert tok == best or float(row[best] - row[tok]) <= 1e-5 * float(row.abs().max()), \
                    f"request of {len(p)} tokens, generated token {k}: {tok}, plain {best}"
                seq.append(tok)
        else:
            # bfloat16: against the engine's own step function, token by token without graphs (the plain model may take
            # another expert on a nearly tied token): the generated token is the best one there, or next to it
            from rocmforge_b200 import StepRequest
            cache = llm.model.new_cache(max_tokens=512, max_slots=1)
            s = cache.alloc_slot()
            row = llm.model.step(cache, [StepRequest(s, list(p), [len(p) - 1])]).cpu()[0]
            for tok in r.tokens:
                assert float(row.max() - row[tok]) <= 2e-2 * float(row.abs().max())
                row = llm.model.step(cache, [StepRequest(s, [tok], [0])]).cpu()[0]


def test_command_line(folders):
    """bin/rocmforge on a Figalix folder: greedy tokens equal the plain model's."""
    folder = folders("FA", "float32")
    prompt = random_tokens(vocab("FA"), 9, 91)
    out = subprocess.run([os.path.join(ROOT, "bin", "rocmforge"), "--model", folder, "--dtype", "float32", "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--stop-ids", "", "--debug"],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    ids = [int(l.split("token_id=")[1]) for l in out.stderr.splitlines() if l.startswith("[Generated]")]
    seq = list(prompt)
    for tok in ids:
        row = plain_logits(folders, "FA", "float32", seq)[-1]
        assert tok == int(torch.argmax(row)) or float(row.max() - row[tok]) <= 1e-5 * float(row.abs().max())
        seq.append(tok)
    assert len(ids) == 5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_program(folders, tmp_path, dtype):
    """bin/trace_run on a Figalix folder: whole prompts, a prompt and its last tokens one by one, and a batch."""
    name = "FB"
    V = vocab(name)
    a, b, c = random_tokens(V, 180, 71), random_tokens(V, 37, 72), random_tokens(V, 5, 73)
    ra, rb, rc = (plain_logits(folders, name, dtype, t) for t in (a, b, c))
    tr = TraceRun(folders(name, dtype), dtype, str(tmp_path / "out"), max_tokens=512)

    def ok(got, want, what):
        if dtype == "float32":
            close(got, want, dtype, what)
        else:                                    # rows of a nearly tied expert apart (one expert a token in this model)
            assert float(row_errors(got, want).median()) < 0.03, what
    got = tr.step([("a", a, [0, 6, 7, 99, 100, 179])], end=["a"])
    ok(got, ra[[0, 6, 7, 99, 100, 179]], "replay: whole")
    got = tr.step([("b", b[:30], [29])])
    ok(got, rb[[29]], "replay: prompt")
    for i in range(30, 37):
        got = tr.step([("b", [b[i]], [0])], end=["b"] if i == 36 else [])
        ok(got, rb[[i]], f"replay: decoded {i}")
    got = tr.step([("x", a[:160], [159]), ("y", c[:3], []), ("z", b[:20], [0, 19])])
    ok(got, torch.stack([ra[159], rb[0], rb[19]]), "replay: batch")
    got = tr.step([("x", [a[160]], [0]), ("y", [c[3]], [0]), ("z", [b[20]], [0])], end=["y"])
    ok(got, torch.stack([ra[160], rc[3], rb[20]]), "replay: batch decoded")
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


def _kept_case(window, keep, T, i, dev, dtype, nh, nkv, d, dv, target):
    """Queries, keys and values in which, for the query at position i, one visible key stands out (``target``: "kept" the
    last kept first position, "edge" the oldest key of the window) and the two hidden keys next to the visible stretches
    (the first position that is not kept, the key just before the window) stand out more, with huge values: the output
    is the visible key's value, and not a trace of a hidden key's."""
    torch.manual_seed(window * 1000 + keep * 10 + i)
    q = torch.randn(T, nh, d, device=dev) * 0.05
    k = torch.randn(T, nkv, d, device=dev) * 0.05
    v = torch.randn(T, nkv, dv, device=dev)
    lo = max(0, i - window + 1)
    q[i] = 0.0
    q[i, :, 0] = 40.0
    hidden = [j for j in (keep, lo - 1) if keep <= j < lo]
    for j in hidden:
        k[j, :, 0] = 2.0                          # would win if it were seen
        v[j] = 1000.0
    seen = keep - 1 if target == "kept" and 0 < keep <= lo else lo
    k[seen, :, 0] = 1.0
    return q.to(dtype), k.to(dtype), v.to(dtype), seen


KEPT_CASES = [(7, 3, 299, "kept"), (7, 3, 299, "edge"), (1, 2, 150, "kept"), (70, 100, 299, "kept"), (70, 100, 171, "edge"),
              (64, 1, 64, "kept"), (64, 1, 65, "kept"), (64, 64, 191, "kept"), (64, 65, 192, "kept"), (130, 5, 134, "kept"),
              (130, 5, 135, "kept"), (130, 0, 299, "edge"), (33, 70, 299, "kept"), (33, 70, 102, "edge"), (200, 4, 203, "edge")]


@pytest.mark.parametrize("window,keep,i,target", KEPT_CASES)
def test_attention_sees_its_window_and_the_kept_first_positions(window, keep, i, target):
    """Queries just before and just after the first unkept position leaves the window, kept stretches shorter and longer
    than a page and than the window, window edges on and off page borders; the query in a prompt and as a step of its own;
    heads of 24 with values of 40 on the generic kernel (32-bit)."""
    from rocmforge_b200 import kernels
    dev, T, nh, nkv, d, dv = "cuda", 300, 4, 2, 24, 40
    q, k, v, seen = _kept_case(window, keep, T, i, dev, torch.float32, nh, nkv, d, dv, target)
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    for rows in (range(i + 1), [i]):
        pos = torch.tensor(list(rows), dtype=torch.int32, device=dev)
        seq = torch.zeros(len(pos), dtype=torch.int32, device=dev)
        out = kernels.attention_generic(q[list(rows)].reshape(len(pos), nh * d).contiguous(), nh, nkv, d, kp, vp, seq, pos,
                                        zero, bt, 1.0, window, v_head_dim=dv, keep_first=keep).reshape(len(pos), nh, dv)
        assert (out[-1] - v[seen][[0, 0, 1, 1]]).abs().max() < 1e-3, f"window {window}, kept {keep}, query {i}: the wrong keys are seen"
    # every row against the mask written out
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    out = kernels.attention_generic(q.reshape(T, nh * d).contiguous(), nh, nkv, d, kp, vp, seq, pos, zero, bt, 0.5, window,
                                    v_head_dim=dv, keep_first=keep).reshape(T, nh, dv)
    see = P.visible(T, window, keep).to(dev)
    for h in range(nh):
        s = (q[:, h].double() @ k[:, h // 2].double().T * 0.5).masked_fill(~see, float("-inf"))
        want = torch.softmax(s, dim=-1) @ v[:, h // 2].double()
        assert (out[:, h].double() - want).abs().max() < 1e-3 * max(1.0, float(want.abs().max())), f"head {h}"


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("window,keep,i,target", [(64, 1, 448, "kept"), (64, 64, 449, "kept"), (64, 65, 449, "kept"),
                                                  (120, 5, 359, "kept"), (120, 5, 360, "edge"), (130, 100, 389, "kept"),
                                                  (33, 70, 395, "kept"), (33, 130, 449, "kept"), (200, 4, 449, "edge"),
                                                  (500, 3, 449, "edge"), (70, 200, 449, "kept")])
def test_tensor_core_attention_sees_its_window_and_the_kept_first_positions(window, keep, i, target, hd):
    """The same on the bfloat16 kernels: the tcgen05 prompt attention (tiles of 128 queries of which some still hold the
    kept positions in their window and others no longer do) and the clustered decode attention with one to eight CTAs
    a sequence, against the generic kernel on every row."""
    from rocmforge_b200 import kernels
    dev, T, nh, nkv = "cuda", 450, 4, 2
    q, k, v, seen = _kept_case(window, keep, T, i, dev, torch.bfloat16, nh, nkv, hd, hd, target)
    kp, vp, bt = _paged(k, v)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    seq = torch.zeros(T, dtype=torch.int32, device=dev)
    q2 = q.reshape(T, nh * hd).contiguous()
    ref = kernels.attention_generic(q2, nh, nkv, hd, kp, vp, seq, pos, zero, bt, 0.3, window, keep_first=keep).float()
    tiles = torch.tensor([[0, r] for r in range(0, T, 128)], dtype=torch.int32, device=dev).flip(0).reshape(-1).contiguous()
    start, nnew = zero, torch.tensor([T], dtype=torch.int32, device=dev)
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    got = kernels.attention_prefill_tc(q2, nh, nkv, hd, kp, vp, tiles, zero, start, nnew, cu, bt, 0.3, window, keep_first=keep).float()
    assert (got - ref).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0), f"prompt kernel, window {window}, kept {keep}"
    assert (got[i].reshape(nh, hd) - v[seen][[0, 0, 1, 1]].float()).abs().max() < 0.1
    for j in sorted({i, 70, 200, T - 1}):
        for splits in (1, 2, 8):
            one = kernels.attention_decode_warps(q2[j:j + 1].contiguous(), nh, nkv, hd, kp, vp, zero, pos[j:j + 1].contiguous(),
                                                 zero, bt, 0.3, window, splits=splits, keep_first=keep).float()
            assert (one[0] - ref[j]).abs().max() <= 2e-2 * ref[j].abs().max().clamp(min=1.0), \
                f"decode kernel, window {window}, kept {keep}, query {j}, {splits} CTAs"
    # a prompt's second portion: the tiles start in the middle of the sequence
    half = 201
    tiles2 = torch.tensor([[0, r] for r in range(0, T - half, 128)], dtype=torch.int32, device=dev).reshape(-1).contiguous()
    got2 = kernels.attention_prefill_tc(q2[half:].contiguous(), nh, nkv, hd, kp, vp, tiles2, zero,
                                        torch.tensor([half], dtype=torch.int32, device=dev),
                                        torch.tensor([T - half], dtype=torch.int32, device=dev),
                                        torch.tensor([0, T - half], dtype=torch.int32, device=dev), bt, 0.3, window,
                                        keep_first=keep).float()
    assert (got2 - ref[half:]).abs().max() <= 2e-2 * ref.abs().max().clamp(min=1.0)


def _steps(lengths_per_step):
    """For each step its (cu_q, seq_slot, tok_seq) on the device: ``lengths_per_step`` is a list of steps, each a list of
    (slot, tokens of that sequence in the step)."""
    out = []
    for step in lengths_per_step:
        cu = [0]
        for _, n in step:
            cu.append(cu[-1] + n)
        seq = [i for i, (_, n) in enumerate(step) for _ in range(n)]
        out.append((torch.tensor(cu, dtype=torch.int32, device="cuda"),
                    torch.tensor([s for s, _ in step], dtype=torch.int32, device="cuda"),
                    torch.tensor(seq, dtype=torch.int32, device="cuda")))
    return out


def _chunk_table(step):
    """first[B+1], then (sequence, first row) of every chunk of 64 of a step's new tokens."""
    first, pairs = [0], []
    for b, (_, n) in enumerate(step):
        first.append(first[-1] + (n + 63) // 64)
        pairs += [(b, r) for r in range(0, n, 64)]
    return torch.tensor(first + [x for pair in pairs for x in pair], dtype=torch.int32, device="cuda")


def _recurrence(form, step, q, k, ab, v, S, cu, slots, heads, dim, vdim, **kw):
    """The scalar recurrence by the kernel that runs token by token, or (``form`` "chunks", steps with a portion of more
    than one token) by the chunked kernels."""
    from rocmforge_b200 import kernels
    if form == "chunks" and any(c > 1 for _, c in step):
        return kernels.gated_chunked(q, k, ab, v, S, _chunk_table(step), cu, slots, heads, dim, vdim, **kw)
    return kernels.gated_scan(q, k, ab, v, S, cu, slots, heads, dim, vdim, one_token=all(c == 1 for _, c in step), **kw)


# two sequences in slots 2 and 0 of 3: a prompt step of unequal portions, a second portion (one of them of 2 tokens),
# then two single-token steps
MEMORY_STEPS = [[(2, 37), (0, 5)], [(2, 2), (0, 70)], [(2, 1), (0, 1)], [(2, 1), (0, 1)]]


@pytest.mark.parametrize("heads,dim,vdim,cap", [(2, 24, 12, 3.0), (1, 40, 20, None), (3, 64, 32, 15.0), (2, 128, 128, 1.0),
                                                 (1, 256, 8, 30.0), (2, 16, 200, 15.0)])
@pytest.mark.parametrize("form", ["scan", "chunks"])
def test_matrix_memory_kernels(heads, dim, vdim, cap, form):
    """The gates' chain, the recurrence with its normaliser and the division, against the plain recurrence: states carried
    over steps in slots of their own, sizes that are no multiple of a warp's rows, capped and uncapped gates.  The first
    sequence's input gates are all far below zero, so that its running maximum is what the forget gates leave of the
    starting value 0: a maximum that started anywhere else would change every denominator."""
    from rocmforge_b200 import kernels
    torch.manual_seed(heads * 1000 + dim)
    totals = {2: 41, 0: 77}
    data = {}
    for slot, T in totals.items():
        zi = torch.randn(T, heads) * 2.0 - (12.0 if slot == 2 else 0.0)
        zf = torch.randn(T, heads) * 2.0 + 2.0
        data[slot] = dict(q=torch.randn(T, heads, dim) * dim ** -0.5, k=torch.randn(T, heads, dim), v=torch.randn(T, heads, vdim),
                          zi=zi, zf=zf)
    want = {}
    for slot, d in data.items():
        li = P.capped(d["zi"].double(), cap)
        lf = torch.nn.functional.logsigmoid(P.capped(d["zf"].double(), cap))
        want[slot] = P.memory_recurrence(d["q"].double(), d["k"].double(), d["v"].double(), li, lf)
    S = torch.full((3, heads, dim, vdim), float("nan"), device="cuda")
    n = torch.full((3, heads, dim), float("nan"), device="cuda")
    m = torch.full((3, heads), float("nan"), device="cuda")
    for t in (S, n, m):
        t[[0, 2]] = 0.0
    at = {2: 0, 0: 0}
    got = {2: [], 0: []}
    for (cu, slots, _), step in zip(_steps(MEMORY_STEPS), MEMORY_STEPS):
        rows = {k: torch.cat([data[s][k][at[s]: at[s] + c] for s, c in step]).cuda() for k in ("q", "k", "v", "zi", "zf")}
        T = rows["q"].shape[0]
        z = torch.cat([rows["zi"], rows["zf"]], dim=1).contiguous()
        ab, mt = kernels.mlstm_gates(z, m, cu, slots, heads, cap or 0.0, max(c for _, c in step))
        o, qn = _recurrence(form, step, rows["q"].reshape(T, -1).contiguous(), rows["k"].reshape(T, -1).contiguous(), ab,
                            rows["v"].reshape(T, -1).contiguous(), S, cu, slots, heads, dim, vdim, nstate=n)
        den = torch.maximum(qn.abs(), torch.exp(-mt)) + 1e-6
        o = (o.reshape(T, heads, vdim) / den[:, :, None]).cpu()
        r = 0
        for s, c in step:
            got[s].append(o[r: r + c]); r += c; at[s] += c
    for slot in totals:
        o_want, S_want, n_want, m_want = want[slot]
        g = torch.cat(got[slot]).double()
        assert (g - o_want).abs().max() < 2e-4 * max(1.0, float(o_want.abs().max())), f"slot {slot}: outputs differ"
        assert (S[slot].cpu().double() - S_want).abs().max() < 2e-4 * max(1.0, float(S_want.abs().max()))
        assert (n[slot].cpu().double() - n_want).abs().max() < 2e-4 * max(1.0, float(n_want.abs().max()))
        assert (m[slot].cpu().double() - m_want).abs().max() < 1e-5
    assert torch.isnan(S[1]).all() and torch.isnan(m[1]).all()      # the slot of no sequence was not touched


@pytest.mark.parametrize("dim,vdim,qk_heads", [(16, 8, 2), (128, 128, 1), (40, 70, 2)])
def test_chunked_recurrence_at_its_edges(dim, vdim, qk_heads):
    """The chunked kernels against the recurrence written out, where random gates would hide a fault.  Head 0 never forgets
    (decay exactly 1) and takes in one early token only, so every later output is that token's value times q . k, across
    every chunk border and the border between two steps.  Head 1 forgets everything (decay exactly 0) at the first and at
    the last token of a chunk and in the middle of one, so nothing older may show after these.  The sequences' lengths
    leave chunks of one token, of 63, 64 and 65 tokens."""
    from rocmforge_b200 import kernels
    torch.manual_seed(dim)
    heads = 2
    steps = [[(1, 193), (0, 63)], [(1, 65), (0, 64)], [(1, 1), (0, 1)]]
    totals = {1: 259, 0: 128}
    data = {}
    for slot, T in totals.items():
        a = torch.rand(T, heads) * 0.5 + 0.5
        b = torch.rand(T, heads)
        a[:, 0] = 1.0
        b[:, 0] = 0.0
        b[3, 0] = 1.0
        for t in (64, 127, 100, 192, 193):
            if t < T:
                a[t, 1] = 0.0
        data[slot] = dict(q=torch.randn(T, qk_heads, dim) * dim ** -0.5, k=torch.randn(T, qk_heads, dim), v=torch.randn(T, heads, vdim),
                          ab=torch.stack([a, b], dim=2))
    want = {}
    for slot, d in data.items():
        T = totals[slot]
        S = torch.zeros(heads, dim, vdim, dtype=torch.float64)
        nn_ = torch.zeros(heads, dim, dtype=torch.float64)
        o = torch.zeros(T, heads, vdim, dtype=torch.float64)
        qn = torch.zeros(T, heads, dtype=torch.float64)
        for t in range(T):
            for h in range(heads):
                g = h // (heads // qk_heads)
                a, b = d["ab"][t, h].double()
                S[h] = a * S[h] + b * torch.outer(d["k"][t, g].double(), d["v"][t, h].double())
                nn_[h] = a * nn_[h] + b * d["k"][t, g].double()
                o[t, h] = S[h].T @ d["q"][t, g].double()
                qn[t, h] = nn_[h] @ d["q"][t, g].double()
        want[slot] = (o, qn, S.clone(), nn_.clone())
        o3 = torch.einsum("td,d->t", d["q"][:, 0].double(), d["k"][3, 0].double())[:, None] * d["v"][3, 0].double()
        assert (o[3:, 0] - o3[3:]).abs().max() < 1e-9          # the plain loop itself keeps the early token for ever
    S = torch.full((2, heads, dim, vdim), 0.0, device="cuda")
    n = torch.full((2, heads, dim), 0.0, device="cuda")
    at = {1: 0, 0: 0}
    got_o, got_n = {1: [], 0: []}, {1: [], 0: []}
    for (cu, slots, _), step in zip(_steps(steps), steps):
        rows = {k: torch.cat([data[s][k][at[s]: at[s] + c] for s, c in step]).cuda() for k in ("q", "k", "v", "ab")}
        T = rows["q"].shape[0]
        o, qn = _recurrence("chunks", step, rows["q"].reshape(T, -1).contiguous(), rows["k"].reshape(T, -1).contiguous(),
                            rows["ab"].contiguous(), rows["v"].reshape(T, -1).contiguous(), S, cu, slots, heads, dim, vdim,
                            qk_heads=qk_heads, nstate=n)
        r = 0
        for s, c in step:
            got_o[s].append(o[r: r + c].cpu().reshape(c, heads, vdim)); got_n[s].append(qn[r: r + c].cpu()); r += c; at[s] += c
    for slot in totals:
        o_want, qn_want, S_want, n_want = want[slot]
        assert (torch.cat(got_o[slot]).double() - o_want).abs().max() < 1e-4 * max(1.0, float(o_want.abs().max())), f"slot {slot}"
        assert (torch.cat(got_n[slot]).double() - qn_want).abs().max() < 1e-4 * max(1.0, float(qn_want.abs().max()))
        assert (S[slot].cpu().double() - S_want).abs().max() < 1e-4 * max(1.0, float(S_want.abs().max()))
        assert (n[slot].cpu().double() - n_want).abs().max() < 1e-4 * max(1.0, float(n_want.abs().max()))


def test_matrix_memory_norm_and_gate():
    """Each head divided by its denominator and by its root mean square, times a weight of all heads' size, times the
    sigmoid of the gate."""
    from rocmforge_b200 import kernels
    torch.manual_seed(5)
    T, heads, vdim, eps = 9, 3, 20, 1e-5
    o = torch.randn(T, heads * vdim, device="cuda") * 3.0
    gate = torch.randn(T, heads * vdim, device="cuda")
    w = torch.randn(heads * vdim, device="cuda")
    qn = torch.randn(T, heads, device="cuda") * 2.0
    mt = torch.randn(T, heads, device="cuda")
    got = kernels.retention_gate(o, gate, heads, vdim, eps, weight=w, gate_fn="sigmoid", denominator=(qn, mt)).cpu().double()
    den = torch.maximum(qn.abs(), torch.exp(-mt)).double().cpu() + 1e-6
    x = o.cpu().double().reshape(T, heads, vdim) / den[:, :, None]
    want = P.unit_rms(x, eps).reshape(T, -1) * w.cpu().double() * torch.sigmoid(gate.cpu().double())
    assert (got - want).abs().max() < 1e-5 * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("heads,vdim,state,groups,taps,parts", [(4, 8, 12, 2, 3, 4), (3, 20, 7, 3, 1, 1), (6, 16, 64, 1, 4, 2),
                                                                 (2, 100, 256, 1, 7, 5), (8, 64, 128, 2, 4, 1)])
@pytest.mark.parametrize("form", ["scan", "chunks"])
def test_state_space_kernels(heads, vdim, state, groups, taps, parts, form):
    """The short convolution with its carried inputs (a portion shorter than the taps among the steps), the step sizes
    without a clamp (pre-activations up to 40), the recurrence with heads that share a group's B and C, the skip, the
    gate before the norm and the norm in parts, against the plain functions."""
    from rocmforge_b200 import kernels
    torch.manual_seed(heads * 100 + taps)
    inner, bc = heads * vdim, groups * state
    C = inner + 2 * bc
    totals = {2: 41, 0: 77}
    data, want = {}, {}
    w = torch.randn(C, taps) * 0.4
    bias = torch.randn(C) * 0.1
    dt_bias, a_log, skip = torch.randn(heads), torch.randn(heads) - 1.0, torch.randn(heads)
    norm_w = torch.randn(inner)
    eps = 1e-5
    for slot, T in totals.items():
        d = dict(xbc=torch.randn(T, C), zdt=torch.randn(T, heads) * 3.0, gate=torch.randn(T, inner))
        d["zdt"][T // 2] = 40.0
        data[slot] = d
        u = P.silu(P.short_convolution(d["xbc"].double(), w.double(), bias.double()))
        dt = torch.nn.functional.softplus(d["zdt"].double() + dt_bias.double(), threshold=1e9)
        decay = torch.exp(-torch.exp(a_log.double()) * dt)
        y, S = P.duality_recurrence(u[:, :inner].reshape(T, heads, vdim), u[:, inner: inner + bc].reshape(T, groups, state),
                                    u[:, inner + bc:].reshape(T, groups, state), dt, decay, skip.double())
        y = y.reshape(T, inner) * P.silu(d["gate"].double())
        y = P.unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * norm_w.double()
        want[slot] = (u, y, S)
    S = torch.full((3, heads, state, vdim), float("nan"), device="cuda")
    conv = torch.full((3, taps - 1, C), float("nan"), device="cuda") if taps > 1 else torch.empty((0, 0, C), device="cuda")
    S[[0, 2]] = 0.0
    if taps > 1:
        conv[[0, 2]] = 0.0
    dev = {k: v.cuda() for k, v in dict(w=w, bias=bias, dt_bias=dt_bias, a_log=a_log, skip=skip, norm_w=norm_w).items()}
    at = {2: 0, 0: 0}
    got_u, got_y = {2: [], 0: []}, {2: [], 0: []}
    for (cu, slots, tok_seq), step in zip(_steps(MEMORY_STEPS), MEMORY_STEPS):
        rows = {k: torch.cat([data[s][k][at[s]: at[s] + c] for s, c in step]).cuda().contiguous() for k in ("xbc", "zdt", "gate")}
        u = kernels.conv_silu(rows["xbc"], 0, C, conv, dev["w"], dev["bias"], tok_seq, cu, slots)
        ab = kernels.mamba_gates(rows["zdt"], dev["dt_bias"], dev["a_log"])
        y, _ = _recurrence(form, step, u[:, inner + bc:], u[:, inner: inner + bc], ab, u[:, :inner], S, cu, slots, heads, state,
                           vdim, qk_heads=groups)
        out = kernels.mamba_finish(y, u[:, :inner], rows["gate"], dev["skip"], dev["norm_w"], parts, vdim, eps)
        r = 0
        for s, c in step:
            got_u[s].append(u[r: r + c].cpu()); got_y[s].append(out[r: r + c].cpu()); r += c; at[s] += c
    for slot in totals:
        u_want, y_want, S_want = want[slot]
        assert (torch.cat(got_u[slot]).double() - u_want).abs().max() < 1e-5 * max(1.0, float(u_want.abs().max())), "convolution"
        assert (torch.cat(got_y[slot]).double() - y_want).abs().max() < 2e-4 * max(1.0, float(y_want.abs().max())), "mixer output"
        assert (S[slot].cpu().double() - S_want).abs().max() < 2e-4 * max(1.0, float(S_want.abs().max())), "state"
    assert torch.isnan(S[1]).all()


@pytest.mark.parametrize("experts,top", [(5, 2), (8, 1), (3, 3), (16, 2), (9, 4), (64, 6)])
def test_router_weights_are_shares_of_all_experts(experts, top):
    """The chosen experts are those of the largest scores, and their weights are their shares of the softmax over all
    experts as they are: they do not add up to one (unless every expert is taken)."""
    from rocmforge_b200 import kernels
    torch.manual_seed(experts)
    z = torch.randn(50, experts, device="cuda") * 2.0
    idx, w = kernels.moe_route(z, top, "softmax_of_all")
    s = torch.softmax(z.double(), dim=-1)
    best = torch.topk(s, top, dim=-1)
    assert (idx.long().sort(dim=-1).values == best.indices.sort(dim=-1).values).all()
    assert (w.double() - s.gather(1, idx.long())).abs().max() < 1e-6
    if top < experts:
        assert float(w.sum(-1).max()) < 1.0 - 1e-4


def test_dynamic_tanh_and_the_scaled_update():
    """tanh(alpha x) w + b of chosen rows; and the stream's update by a multiple of one output, of two, and of half the sum
    of two outputs that are each normed over the width with a weight, with the next layer's Dynamic Tanh in the same pass."""
    from rocmforge_b200 import kernels
    torch.manual_seed(3)
    T, H, eps, mult = 7, 100, 1e-5, 0.3
    h = torch.randn(T, H, device="cuda") * 2.0
    alpha, w, b = torch.tensor([0.7], device="cuda"), torch.randn(H, device="cuda"), torch.randn(H, device="cuda")
    rows = torch.tensor([5, 0, 3], dtype=torch.int32, device="cuda")
    want = torch.tanh(0.7 * h.double()) * w.double() + b.double()
    assert (kernels.dyt_rows(h, alpha, w, b, torch.float32).double() - want).abs().max() < 1e-5
    assert (kernels.dyt_rows(h, alpha, w, b, torch.float32, rows=rows).double() - want[rows.long()]).abs().max() < 1e-5
    a0, a1 = torch.randn(T, H, device="cuda") * 5.0, torch.randn(2, T, H, device="cuda") * 0.01
    w0, w1 = torch.randn(H, device="cuda"), torch.randn(H, device="cuda")
    h1 = h.clone()
    y = kernels.scaled_add(h1, [(a0, w0), (a1, w1)], mult, torch.float32, eps=eps, next_dyt=(alpha, w, b))
    merged = 0.5 * (P.unit_rms(a0.double(), eps) * w0.double() + P.unit_rms(a1.double().sum(0), eps) * w1.double())
    h_want = h.double() + mult * merged
    assert (h1.double() - h_want).abs().max() < 1e-5
    assert (y.double() - (torch.tanh(0.7 * h_want) * w.double() + b.double())).abs().max() < 1e-5
    h2 = h.clone()
    assert kernels.scaled_add(h2, [(a0, None)], mult, torch.float32) is None
    assert (h2.double() - (h.double() + mult * a0.double())).abs().max() < 1e-5
    x = torch.randn(5, 300, device="cuda") * 20.0
    assert (kernels.softcap_(x.clone(), 8.0).double() - 8.0 * torch.tanh(x.double() / 8.0)).abs().max() < 1e-5


@pytest.mark.parametrize("dims,base,scaling", [(8, 100.0, (4.0, 16, 4.0, 1.0)), (40, 1e4, (8.0, 64, 8.0, 2.0)),
                                               (32, 1e6, (4.0, 256, 16.0, 2.0)), (64, 1e4, (16.0, 32, 2.0, 0.5)),
                                               (64, 1e6, (8.0, 8192, 32.0, 1.0)), (6, 50.0, (2.0, 4, 1.0, 1.0))])
def test_stretched_frequencies(dims, base, scaling):
    """The position encoding's table against the plain one: ramps that start below pair 0, end beyond the last pair, and
    have no length at all; the size by which sine and cosine grow."""
    from rocmforge_b200.parts.rope import YarnRope
    named = dict(zip(("factor", "original", "fast", "slow"), scaling))
    rope = YarnRope(dims, base, dims, **named)
    f, magnitude = P.stretched_frequencies(dims, base, named)
    assert (rope.inv_freq_host.double() - f).abs().max() <= 1e-7 * float(f.max())
    assert abs(rope.magnitude - magnitude) < 1e-12
