"""Figalix without a GPU: its configuration (keys, defaults, faults), the parts and tensor names its builder picks, what
the cache keeps for a window with kept first positions and for the recurrent layers, the stretched rotary frequencies, and
the plain implementation's mechanisms against the same sums written another way."""
import copy
import json
import math

import pytest
import torch

from helpers import FIGALIX_CONFIGS, figalix_config, random_tokens, write_figalix
from plain import figalix_plain as P


def test_the_design_is_chosen_by_its_name(tmp_path):
    from rocmforge_b200.config import load_config
    write_figalix(FIGALIX_CONFIGS["FA"], str(tmp_path))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Figalix" and cfg.width == 64 and cfg.vocab == 96 and cfg.eps == 1e-5
    assert cfg.residual_mult == 0.5 and cfg.logit_softcap == 8.0
    assert [L.type for L in cfg.layers] == ["mamba2", "parallel", "parallel", "mamba2"]
    ssm, par = cfg.layers[0].mixer, cfg.layers[1].mixer
    assert (ssm.heads, ssm.vdim, ssm.state, ssm.groups, ssm.taps, ssm.norm_groups) == (4, 8, 12, 2, 3, 4)
    assert (par.left.heads, par.left.kv_heads, par.left.dim, par.left.vdim) == (4, 2, 16, 24)
    assert (par.left.window, par.left.keep_first, par.left.rot_dims, par.left.scale) == (7, 3, 8, 0.4)
    assert par.left.rot_scaling == dict(factor=4.0, original=16.0, fast=4.0, slow=1.0)
    assert (par.right.heads, par.right.dim, par.right.vdim, par.right.gate_cap) == (2, 24, 12, 3.0)
    assert cfg.layers[1].mlp is None and cfg.layers[2].mlp.kind == "dense" and cfg.layers[2].mlp.ff == 40
    moe = cfg.layers[0].mlp
    assert (moe.kind, moe.ff, moe.experts, moe.top, moe.shared_ff) == ("moe", 20, 5, 2, 24)
    assert cfg.to_dict() == json.load(open(tmp_path / "config.json"))


def test_what_a_configuration_may_leave_out():
    cfg, _ = figalix_config(FIGALIX_CONFIGS["FB"])
    assert cfg.logit_softcap is None and cfg.layers[2].mixer.right.gate_cap is None
    assert cfg.layers[2].mixer.left.rot_scaling is None and cfg.layers[2].mlp.shared_ff is None
    cfg, _ = figalix_config(FIGALIX_CONFIGS["FD"])
    left = cfg.layers[2].mixer.left
    assert left.window is None and left.keep_first == 0 and left.rot_dims == 0 and left.rot_base is None
    assert figalix_config(FIGALIX_CONFIGS["FC"])[0].layers[3].mixer.left.keep_first == 0


@pytest.mark.parametrize("path,value,error", [
    ("width", None, "MissingKey"), ("vocab", 0, "InvalidValue"), ("norm.eps", None, "MissingKey"), ("layers", [], "InvalidValue"),
    ("layers.0.type", "attention", "InvalidValue"), ("layers.0.mixer.groups", 3, "InvalidValue"),
    ("layers.0.mixer.norm_groups", 5, "InvalidValue"), ("layers.0.mixer.conv", 17, "InvalidValue"),
    ("layers.0.mixer.state", None, "MissingKey"), ("layers.0.mixer.state", 257, "InvalidValue"),
    ("layers.0.mlp.router.top", 6, "InvalidValue"), ("layers.0.mlp.kind", "glu", "InvalidValue"), ("layers.0.mlp.expert.ff", None, "MissingKey"),
    ("layers.1.mixer.left.kv_heads", 3, "InvalidValue"), ("layers.1.mixer.left.scale", None, "MissingKey"),
    ("layers.1.mixer.left.rot.dims", 7, "InvalidValue"), ("layers.1.mixer.left.rot.dims", 18, "InvalidValue"),
    ("layers.1.mixer.left.rot.base", 1.0, "InvalidValue"), ("layers.1.mixer.left.rot.scaling.factor", None, "MissingKey"),
    ("layers.1.mixer.left.mask.size", 0, "InvalidValue"), ("layers.1.mixer.right.dim", 257, "InvalidValue"),
    ("layers.1.mixer.right.gate_cap", 0.0, "InvalidValue"), ("layers.1.mixer.right.vdim", None, "MissingKey"),
    ("layers.2.mlp.ff", None, "MissingKey"),
])
def test_faults_of_a_configuration_name_their_key(path, value, error):
    from rocmforge_b200.config import architecture_for, errors
    raw = copy.deepcopy(figalix_config(FIGALIX_CONFIGS["FA"])[1])
    cur = raw
    parts = path.split(".")
    for p in parts[:-1]:
        cur = cur[int(p)] if p.isdigit() else cur[p]
    if value is None:
        del cur[parts[-1]]
    else:
        cur[parts[-1]] = value
    with pytest.raises(getattr(errors, error)) as e:
        architecture_for("Figalix").config_cls.from_dict(raw)
    assert parts[-1] in str(e.value)


def test_the_builder_picks_parts_and_names_by_the_configuration():
    from rocmforge_b200.config import architecture_for
    from rocmforge_b200.cache.requests import KVRequest, StateRequest
    for name, c in FIGALIX_CONFIGS.items():
        cfg, _ = figalix_config(c)
        spec = architecture_for("Figalix").build(cfg)
        specs = spec.param_specs()
        W = c["width"]
        assert specs["embed"].shape == (c["vocab"], W) and specs["head"].tied_to == "embed"        # the table is the head
        assert specs["final.norm"].shape == (W,) and specs["final.norm.alpha"].shape == () and specs["final.norm.b"].shape == (W,)
        requests = spec.cache_requests()
        for i, L in enumerate(c["layers"]):
            m, mlp, p = L["mixer"], L["mlp"], f"l{i}."
            assert specs[p + "norm1"].shape == (W,) and specs[p + "norm1.alpha"].shape == () and specs[p + "norm1.b"].shape == (W,)
            if mlp is None:
                assert p + "norm2" not in specs or specs[p + "norm2"].optional
            else:
                assert specs[p + "norm2.alpha"].shape == () and not specs[p + "norm2"].optional
            if L["type"] == "parallel":
                a, r = m["left"], m["right"]
                assert specs[p + "mix.left.q"].shape == (a["heads"] * a["dim"], W)
                assert specs[p + "mix.left.k"].shape == (a["kv_heads"] * a["dim"], W)
                assert specs[p + "mix.left.v"].shape == (a["kv_heads"] * a["vdim"], W)
                assert specs[p + "mix.left.g"].shape == (a["heads"], W) and specs[p + "mix.left.o"].shape == (W, a["heads"] * a["vdim"])
                assert specs[p + "mix.left.out"].shape == (W,) and specs[p + "mix.right.out"].shape == (W,)
                assert specs[p + "mix.right.q"].shape == specs[p + "mix.right.k"].shape == (r["heads"] * r["dim"], W)
                assert specs[p + "mix.right.v"].shape == specs[p + "mix.right.g"].shape == (r["heads"] * r["vdim"], W)
                assert specs[p + "mix.right.i"].shape == specs[p + "mix.right.f"].shape == (r["heads"], W)
                assert specs[p + "mix.right.i.b"].shape == specs[p + "mix.right.f.b"].shape == (r["heads"],)
                assert specs[p + "mix.right.norm"].shape == (r["heads"] * r["vdim"],)
                assert specs[p + "mix.right.o"].shape == (W, r["heads"] * r["vdim"])
                kv, state = requests[i]["left"], requests[i]["right"]
                mask = a.get("mask") or {}
                assert (kv.n_kv_heads, kv.head_dim, kv.window, kv.chunk, kv.keep_first) == (
                    a["kv_heads"], a["dim"], mask.get("size"), None, mask.get("keep_first") or 0)
                assert (kv.v_head_dim or kv.head_dim) == a["vdim"]
                assert isinstance(state, StateRequest)
                assert {n: (s, d) for n, s, d in state.tensors} == {"S": ((r["heads"], r["dim"], r["vdim"]), torch.float32),
                                                                    "n": ((r["heads"], r["dim"]), torch.float32),
                                                                    "m": ((r["heads"],), torch.float32)}
            else:
                inner, ch = m["heads"] * m["vdim"], m["heads"] * m["vdim"] + 2 * m["groups"] * m["state"]
                assert specs[p + "mix.in"].shape == (inner + ch + m["heads"], W) and specs[p + "mix.o"].shape == (W, inner)
                assert specs[p + "mix.conv"].shape == (ch, m["conv"]) and specs[p + "mix.conv.b"].shape == (ch,)
                assert specs[p + "mix.dt_bias"].shape == specs[p + "mix.A_log"].shape == specs[p + "mix.D"].shape == (m["heads"],)
                assert specs[p + "mix.norm"].shape == (inner,)
                want = {"S": ((m["heads"], m["state"], m["vdim"]), torch.float32)}
                if m["conv"] > 1:
                    want["conv"] = ((m["conv"] - 1, ch), torch.float32)
                assert {n: (s, d) for n, s, d in requests[i].tensors} == want
            if mlp is None:
                assert not any(k.startswith(p + "mlp.") for k in specs)
            elif mlp["kind"] == "dense":
                assert specs[p + "mlp.gate"].shape == specs[p + "mlp.up"].shape == (mlp["ff"], W) and specs[p + "mlp.down"].shape == (W, mlp["ff"])
            else:
                E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
                assert specs[p + "mlp.router"].shape == (E, W) and p + f"mlp.e{E}.gate" not in specs
                assert specs[p + f"mlp.e{E - 1}.gate"].shape == (ff, W) and specs[p + "mlp.e0.down"].shape == (W, ff)
                assert (p + "mlp.shared.up" in specs) == ("shared" in mlp)
                if "shared" in mlp:
                    assert specs[p + "mlp.shared.down"].shape == (W, mlp["shared"]["ff"])
        assert not spec.stop_token_ids


def test_the_cache_keeps_the_first_positions_beside_the_window():
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.cache.requests import KVRequest
    kept, bare = KVRequest(2, 8, 70, None, None, 100), KVRequest(2, 8, 70)
    assert kept.group_key() != bare.group_key()
    cache = SequenceCache({0: kept, 1: bare, 2: KVRequest(2, 8, 70, None, None, 3)}, max_tokens=64 * 12, max_slots=2,
                          dtype=torch.float32, device="cpu")
    g_kept, g_bare, g_few = cache._group_of[0], cache._group_of[1], cache._group_of[2]

    def held(g, s):
        return [int(p) for p in (g.table[s] >= 0).nonzero()[0]]
    s = cache.alloc_slot()
    cache.prepare([s], [130]); cache.commit([s], [130])           # the next query (130) sees 61.. and the first positions
    assert held(g_bare, s) == [0, 1, 2] and held(g_kept, s) == [0, 1, 2] and held(g_few, s) == [0, 1, 2]
    cache.prepare([s], [200]); cache.commit([s], [200])           # length 330: the window starts at 261, in page 4
    assert held(g_bare, s) == [4, 5]
    assert held(g_kept, s) == [0, 1, 4, 5]                        # positions 0..99 lie in pages 0 and 1
    assert held(g_few, s) == [0, 4, 5]
    for _ in range(60):                                            # decoding: the window's page changes, the first ones stay
        cache.prepare([s], [1]); cache.commit([s], [1])
    assert held(g_bare, s) == [5, 6] and held(g_kept, s) == [0, 1, 5, 6] and held(g_few, s) == [0, 5, 6]
    assert g_kept.pages_missing(s, 390, 460) == 1                 # page 7 alone: the kept pages are held
    cache.free_slot(s)
    for g in (g_kept, g_bare, g_few):
        assert g.pool.n_free == g.n_pages
    s2 = cache.alloc_slot()                                       # a slot that is used again starts with no pages at all
    assert held(g_kept, s2) == []
    with pytest.raises(ValueError):
        KVRequest(2, 8, None, None, None, 4)                      # first positions are kept beside a window only


@pytest.mark.parametrize("dims,base,scaling", [(32, 1e6, (4.0, 256, 16.0, 2.0)), (40, 1e4, (8.0, 64, 8.0, 2.0)), (8, 100.0, (4.0, 16, 4.0, 1.0)),
                                                (64, 1e4, (16.0, 32, 2.0, 0.5)), (128, 5e5, (32.0, 8192, 32.0, 1.0)), (6, 1e6, None)])
def test_stretched_frequencies(dims, base, scaling):
    """The part's table against the plain rule, and the rule against what it means: pairs that turn more than ``fast``
    times in ``original`` positions keep their frequency, those that turn fewer than ``slow`` times turn ``factor`` times
    slower, the ones between lie between."""
    from rocmforge_b200.parts import POSITIONS
    sc = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    want, mag = P.stretched_frequencies(dims, base, sc)
    if sc is None:
        rope = POSITIONS.build("rope_neox", head_dim=dims + 8, theta=base, rotary_dim=dims)
        assert mag == 1.0
    else:
        rope = POSITIONS.build("rope_yarn", head_dim=dims + 8, theta=base, rotary_dim=dims, **sc)
        assert math.isclose(mag, 0.1 * math.log(sc["factor"]) + 1.0)
    assert torch.allclose(rope.inv_freq_host.double(), want, rtol=1e-6, atol=0)
    plain = base ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
    if sc is not None:
        turns = sc["original"] * plain / (2 * math.pi)
        i = torch.arange(dims // 2)
        # one index of slack on either side: the ramp's ends are a floor and a ceiling of fractional indices
        fast, slow = turns > sc["fast"], turns < sc["slow"]
        fast[1:] &= fast[:-1].clone() & (turns[1:] > sc["fast"]); slow[:-1] &= (turns[1:] < sc["slow"])
        inner_fast = fast & torch.cat([fast[1:], fast[-1:]])
        assert torch.equal(want[inner_fast], plain[inner_fast])
        assert torch.allclose(want[slow], plain[slow] / sc["factor"])
        assert ((want <= plain) & (want >= plain / sc["factor"] * (1 - 1e-12))).all()
        assert (want[1:] < want[:-1]).all() or dims <= 8


def test_plain_matrix_memory_against_its_closed_form():
    """The state without its stabiliser is U_t = sum_(s<=t) exp(li_s + sum_(s<r<=t) lf_r) k_s v_s^T (a double loop here), and
    the stabilised one is S_t = exp(-m_t) U_t; so o_t = exp(-m_t) U_t^T q_t / (max(exp(-m_t) |u_t . q_t|, exp(-m_t)) + 1e-6)
    with u_t the same sum over k_s alone."""
    torch.manual_seed(0)
    T, H, D, DV = 11, 2, 5, 3
    q, k = torch.randn(T, H, D, dtype=torch.float64), torch.randn(T, H, D, dtype=torch.float64)
    v = torch.randn(T, H, DV, dtype=torch.float64)
    li = torch.randn(T, H, dtype=torch.float64) * 3
    lf = torch.nn.functional.logsigmoid(torch.randn(T, H, dtype=torch.float64) * 3)
    o, S, n, mx = P.memory_recurrence(q, k, v, li, lf)
    m = torch.zeros(H, dtype=torch.float64)
    for t in range(T):
        m = torch.maximum(lf[t] + m, li[t])
        Su = torch.zeros(H, D, DV, dtype=torch.float64)
        nu = torch.zeros(H, D, dtype=torch.float64)
        for s in range(t + 1):
            w = torch.exp(li[s] + lf[s + 1: t + 1].sum(0))
            Su += w[:, None, None] * k[s][:, :, None] * v[s][:, None, :]
            nu += w[:, None] * k[s]
        # the stabilised state is the plain one times exp(-m_t)
        den = torch.maximum((nu * q[t]).sum(-1).abs() * torch.exp(-m), torch.exp(-m)) + 1e-6
        want = torch.einsum("hdv,hd->hv", Su, q[t]) * torch.exp(-m)[:, None] / den[:, None]
        assert torch.allclose(o[t], want, rtol=1e-9, atol=1e-12)
    assert torch.allclose(S, Su * torch.exp(-m)[:, None, None], rtol=1e-9) and torch.allclose(mx, m)
    # a state handed on: two halves give what the whole gives
    o1, S1, n1, m1 = P.memory_recurrence(q[:4], k[:4], v[:4], li[:4], lf[:4])
    o2 = P.memory_recurrence(q[4:], k[4:], v[4:], li[4:], lf[4:], S1, n1, m1)[0]
    assert torch.allclose(torch.cat([o1, o2]), o, rtol=1e-12, atol=1e-14)


def test_plain_state_space_recurrence_against_its_closed_form():
    """y_t = sum_(s<=t) (C_t . B_s) dt_s prod_(s<r<=t) a_r x_s + D x_t."""
    torch.manual_seed(1)
    T, H, DV, N = 10, 3, 4, 6
    x = torch.randn(T, H, DV, dtype=torch.float64)
    B, C = torch.randn(T, H, N, dtype=torch.float64), torch.randn(T, H, N, dtype=torch.float64)
    dt = torch.rand(T, H, dtype=torch.float64) + 0.1
    decay = torch.exp(-torch.rand(T, H, dtype=torch.float64) * dt)
    skip = torch.randn(H, dtype=torch.float64)
    y, S = P.duality_recurrence(x, B, C, dt, decay, skip)
    for t in range(T):
        want = skip[:, None] * x[t]
        for s in range(t + 1):
            want = want + ((C[t] * B[s]).sum(-1) * dt[s] * decay[s + 1: t + 1].prod(0))[:, None] * x[s]
        assert torch.allclose(y[t], want, rtol=1e-9, atol=1e-12)
    y1, S1 = P.duality_recurrence(x[:3], B[:3], C[:3], dt[:3], decay[:3], skip)
    y2, S2 = P.duality_recurrence(x[3:], B[3:], C[3:], dt[3:], decay[3:], skip, S1)
    assert torch.allclose(torch.cat([y1, y2]), y, rtol=1e-12, atol=1e-14) and torch.allclose(S2, S, rtol=1e-12)


def test_plain_convolution_starts_from_zeros_and_ends_on_the_current_token():
    x = torch.arange(1.0, 7.0, dtype=torch.float64)[:, None].repeat(1, 2)
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 10.0, 100.0]], dtype=torch.float64)
    y = P.short_convolution(x, w, torch.tensor([0.5, 0.0], dtype=torch.float64))
    assert torch.equal(y[:, 0], x[:, 0] + 0.5)                                    # the last column is the current token's
    assert torch.equal(y[:, 1], torch.tensor([100.0, 210.0, 321.0, 432.0, 543.0, 654.0], dtype=torch.float64))


def test_plain_mask_and_shares():
    see = P.visible(9, 3, 2)
    assert see[8].tolist() == [True, True, False, False, False, False, True, True, True]
    assert see[2].tolist() == [True, True, True] + [False] * 6 and see[0].tolist() == [True] + [False] * 8
    assert P.visible(5, None, 0).tolist() == torch.ones(5, 5).tril().bool().tolist()
    W = {"r.router": torch.tensor([[1.0, 0.0], [0.0, 1.0], [-1.0, 0.0], [0.5, 0.5]], dtype=torch.float64)}
    s = P.expert_scores(torch.tensor([[2.0, 0.0]], dtype=torch.float64), W, "r.")
    assert torch.allclose(s.sum(-1), torch.ones(1, dtype=torch.float64)) and s[0].argmax() == 0 and s[0, 0] < 1


def test_plain_model_window_and_kept_positions():
    """With the recurrent halves and the experts left out, a changed token is felt by later logits only while it lies in the
    window of every layer, or for good when it is one of the kept first positions."""
    from safetensors.torch import load_file
    import tempfile
    base = copy.deepcopy(FIGALIX_CONFIGS["FA"])
    layer = copy.deepcopy(base["layers"][1])
    layer["mlp"] = None
    base["layers"] = [layer]
    with tempfile.TemporaryDirectory() as d:
        write_figalix(base, d)
        W = load_file(d + "/model.safetensors")
        raw = json.load(open(d + "/config.json"))
    for name in list(W):
        if ".mix.right.o" in name:
            W[name] = torch.zeros_like(W[name])                    # the matrix memory carries everything forward: silence it
    model = P.PlainFigalix(raw, W)
    toks = random_tokens(base["vocab"], 40, 5)

    def changed(at):
        other = list(toks)
        other[at] = (other[at] + 1) % base["vocab"]
        return (model.logits(toks) - model.logits(other)).abs().amax(-1)
    d = changed(10)                                                # window 7: positions 10..16 see it, 17 does not
    assert (d[:10] == 0).all() and (d[10:17] > 1e-9).all() and (d[17:] == 0).all()
    d = changed(2)                                                 # one of the first three: seen for good
    assert (d[:2] == 0).all() and (d[2:] > 1e-9).all()
    d = changed(3)                                                 # the first one that is not kept
    assert (d[3:10] > 1e-9).all() and (d[10:] == 0).all()
