"""Ludusun without a GPU: its configuration (keys, defaults, faults, the ranks that are tensor shapes), the parts and
tensor names its builder picks, what the cache keeps for its four kinds of mixer, and the plain implementation's
mechanisms against the same sums written another way."""
import copy
import json
import math

import pytest
import torch

from helpers import LUDUSUN_CONFIGS, ludusun_config, random_tokens, write_ludusun
from plain import ludusun_plain as P


def test_the_design_is_chosen_by_its_name(tmp_path):
    from rocmforge_b200.config import load_config
    write_ludusun(LUDUSUN_CONFIGS["LA"], str(tmp_path))
    arch, cfg = load_config(str(tmp_path))
    assert arch.name == "Ludusun" and cfg.width == 64 and cfg.vocab == 96 and cfg.eps == 1e-5
    assert cfg.embedding_scale == 2.0 and cfg.logit_softcap == 8.0
    assert [L.type for L in cfg.layers] == ["parallel", "attention", "latent_attention", "attention"]
    par, att, lat, bor = (L.mixer for L in cfg.layers)
    assert (par.left.heads, par.left.kv_heads, par.left.dim, par.left.scale, par.left.q_temp) == (4, 2, 16, 0.25, (0.3, 5))
    assert (par.right.heads, par.right.kv_heads, par.right.dim, par.right.vdim, par.right.taps) == (2, 1, 24, 12, 3)
    assert (par.right.decay_rank, par.right.gate_rank) == (5, 3)          # the shapes of the folder's a1 and g1
    assert (par.left_scale, par.right_scale) == (1.0, 0.7)
    assert (att.heads, att.kv_heads, att.dim, att.vdim, att.rot_dims, att.kv_from) == (4, 2, 16, 24, 8, None)
    assert att.rot_scaling == dict(factor=4.0, original=16.0, fast=4.0, slow=1.0)
    assert (lat.heads, lat.dim, lat.vdim, lat.q_rank, lat.kv_rank, lat.window) == (3, 8, 16, 12, 20, 7)
    assert bor.kv_from == 1 and bor.scale == 0.5
    assert [L.ff for L in cfg.layers] == [40, None, 48, 24]
    assert {k: v for k, v in cfg.to_dict().items() if k != "ranks"} == json.load(open(tmp_path / "config.json"))


def test_what_a_configuration_may_leave_out():
    cfg, _ = ludusun_config(LUDUSUN_CONFIGS["LB"])
    assert cfg.logit_softcap is None and cfg.embedding_scale == 1.0
    assert cfg.layers[0].mixer.rot_scaling is None and cfg.layers[2].mixer.left.q_temp is None
    cfg, _ = ludusun_config(LUDUSUN_CONFIGS["LD"])
    assert cfg.layers[1].mixer.rot_dims == 0 and cfg.layers[1].mixer.rot_base is None and cfg.layers[2].mixer.window is None
    raw = copy.deepcopy(ludusun_config(LUDUSUN_CONFIGS["LA"])[1])
    del raw["embedding"]
    from rocmforge_b200.config import architecture_for
    c = architecture_for("Ludusun").config_cls.from_dict(raw)             # no tensor shapes at hand: the default ranks
    assert c.embedding_scale == 1.0 and c.layers[0].mixer.right.decay_rank == c.DEFAULT_RANK


@pytest.mark.parametrize("path,value,error", [
    ("width", None, "MissingKey"), ("vocab", 0, "InvalidValue"), ("norm.eps", None, "MissingKey"), ("layers", [], "InvalidValue"),
    ("layers.0.type", "mamba2", "InvalidValue"), ("layers.0.mixer.left.kv_heads", 3, "InvalidValue"),
    ("layers.0.mixer.left.vdim", 24, "InvalidValue"), ("layers.0.mixer.left.q_temp.every", 0, "InvalidValue"),
    ("layers.0.mixer.right.kv_heads", 3, "InvalidValue"), ("layers.0.mixer.right.dim", 257, "InvalidValue"),
    ("layers.0.mixer.right.conv", 17, "InvalidValue"), ("layers.0.mixer.right.vdim", None, "MissingKey"),
    ("layers.0.mixer.left_scale", None, "MissingKey"), ("layers.0.mlp.kind", "moe", "InvalidValue"), ("layers.0.mlp.ff", None, "MissingKey"),
    ("layers.1.mixer.kv_heads", 3, "InvalidValue"), ("layers.1.mixer.scale", None, "MissingKey"),
    ("layers.1.mixer.rot.dims", 7, "InvalidValue"), ("layers.1.mixer.rot.dims", 18, "InvalidValue"),
    ("layers.1.mixer.rot.base", 1.0, "InvalidValue"), ("layers.1.mixer.rot.scaling.factor", None, "MissingKey"),
    ("layers.2.mixer.mask.size", 0, "InvalidValue"), ("layers.2.mixer.kv_rank", None, "MissingKey"), ("layers.2.mixer.q_rank", 0, "InvalidValue"),
    ("layers.3.mixer.kv_from", 3, "InvalidValue"), ("layers.3.mixer.kv_from", 2, "InvalidValue"), ("layers.3.mixer.vdim", 16, "InvalidValue"),
])
def test_faults_of_a_configuration_name_their_key(path, value, error):
    from rocmforge_b200.config import architecture_for, errors
    raw = copy.deepcopy(ludusun_config(LUDUSUN_CONFIGS["LA"])[1])
    cur = raw
    parts = path.split(".")
    for p in parts[:-1]:
        cur = cur[int(p)] if p.isdigit() else cur[p]
    if value is None:
        del cur[parts[-1]]
    else:
        cur[parts[-1]] = value
    with pytest.raises(getattr(errors, error)) as e:
        architecture_for("Ludusun").config_cls.from_dict(raw)
    assert parts[-1] in str(e.value) or "kv_from" in str(e.value)


def test_the_builder_picks_parts_and_names_by_the_configuration():
    from rocmforge_b200.cache.requests import KVRequest, StateRequest
    from rocmforge_b200.config import architecture_for
    for name, c in LUDUSUN_CONFIGS.items():
        cfg, _ = ludusun_config(c)
        spec = architecture_for("Ludusun").build(cfg)
        specs = spec.param_specs()
        W = c["width"]
        assert specs["embed"].shape == (c["vocab"], W) and specs["head"].tied_to == "embed" and specs["final.norm"].shape == (W,)
        requests = spec.cache_requests()
        for i, L in enumerate(c["layers"]):
            pre, m = f"l{i}.", L["mixer"]
            assert (pre + "mlp.gate" in specs) == (L["mlp"] is not None)
            if L["mlp"] is None:
                assert specs[pre + "norm2"].optional                      # a folder may hold the unused norm
            if L["type"] == "attention":
                borrowed = m.get("kv_from") is not None
                assert specs[pre + "mix.q"].shape == (m["heads"] * m["dim"], W) and specs[pre + "mix.sink"].shape == (m["heads"],)
                assert specs[pre + "mix.o"].shape == (W, m["heads"] * m["vdim"])
                assert (pre + "mix.k" in specs) == (not borrowed) and (pre + "mix.v" in specs) == (not borrowed)
                assert (i in requests) == (not borrowed) and spec.schedule[i].kv_from == m.get("kv_from")
                if not borrowed:
                    assert requests[i] == KVRequest(m["kv_heads"], m["dim"], None, None if m["vdim"] == m["dim"] else m["vdim"])
            elif L["type"] == "latent_attention":
                assert specs[pre + "mix.dq"].shape == (m["q_rank"], W) and specs[pre + "mix.dq.norm"].shape == (m["q_rank"],)
                assert specs[pre + "mix.uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
                assert specs[pre + "mix.uv"].shape == (m["heads"] * m["vdim"], m["kv_rank"]) and specs[pre + "mix.g"].shape == (m["heads"], W)
                assert requests[i].window == (m.get("mask") or {}).get("size") and requests[i].n_kv_heads == m["heads"]
            else:
                left, right = m["left"], m["right"]
                assert pre + "mix.left.v" not in specs and specs[pre + "mix.left.q.b"].shape == (left["heads"] * left["dim"],)
                assert specs[pre + "mix.left.g"].shape == (left["heads"] * left["dim"], W)
                assert specs[pre + "mix.right.a1"].shape == (c["ranks"][pre + "mix.right.a1"], W)
                assert specs[pre + "mix.right.g2"].shape == (right["heads"] * right["vdim"], c["ranks"][pre + "mix.right.g1"])
                assert specs[pre + "mix.right.q.conv"].shape == (right["kv_heads"] * right["dim"], right["conv"])
                assert specs[pre + "mix.right.dt_bias"].shape == (right["heads"] * right["dim"],)
                req = requests[i]
                assert req["left"] == KVRequest(left["kv_heads"], left["dim"], values_are_keys=True)
                assert isinstance(req["right"], StateRequest)
                shapes = {n: s for n, s, _ in req["right"].tensors}
                assert shapes["S"] == (right["heads"], right["dim"], right["vdim"])
                channels = 2 * right["kv_heads"] * right["dim"] + right["heads"] * right["vdim"]
                assert shapes.get("conv") == ((right["conv"] - 1, channels) if right["conv"] > 1 else None)


def test_keys_that_serve_as_values_are_stored_once():
    from rocmforge_b200.cache import SequenceCache
    from rocmforge_b200.cache.requests import KVRequest
    cache = SequenceCache({0: KVRequest(2, 16, values_are_keys=True), 1: KVRequest(2, 16)}, max_tokens=256, max_slots=2,
                          dtype=torch.float32)
    shared, plain = cache.view(0), cache.view(1)
    assert shared.k_pages.data_ptr() == shared.v_pages.data_ptr() and plain.k_pages.data_ptr() != plain.v_pages.data_ptr()
    assert sum(g.storage.numel() for g in cache.groups) == 3 * plain.k_pages.numel()
    with pytest.raises(ValueError):
        KVRequest(2, 16, v_head_dim=8, values_are_keys=True)


def test_the_norm_adds_its_offset_once_in_32_bits():
    from rocmforge_b200.parts import NORMS
    n = NORMS.build("rmsnorm", size=4, eps=1e-5, param_name="", weight_offset=1.0)
    w = torch.tensor([0.25, -0.5, 0.0078125, 0.0], dtype=torch.bfloat16)
    n.bind({"": w}, torch.bfloat16)
    assert n.weight.dtype == torch.float32 and torch.equal(n.weight, torch.tensor([1.25, 0.5, 1.0078125, 1.0]))
    plain = NORMS.build("rmsnorm", size=4, eps=1e-5, param_name="")
    plain.bind({"": w}, torch.bfloat16)
    assert plain.weight is w


# --------------------------------------------------------------------------- the plain implementation against closed forms

def test_plain_delta_rule_against_its_closed_form():
    """With decays of 1 and beta of 1 the state after writing orthonormal keys reads every stored value back exactly, and
    writing a key a second time replaces its value; with a decay g < 1 on every channel what was stored fades by g a step."""
    torch.manual_seed(0)
    D, V = 6, 4
    keys = torch.linalg.qr(torch.randn(D, D, dtype=torch.float64))[0][:3]
    vals = torch.randn(4, V, dtype=torch.float64)
    k = torch.stack([keys[0], keys[1], keys[2], keys[0]])
    ones = torch.ones(4, D, dtype=torch.float64)
    o, S = P.delta_recurrence(k, k, vals, torch.ones(4, dtype=torch.float64), ones)
    assert (o - vals).abs().max() < 1e-12                                   # the read-out sees the token's own write
    assert (S.T @ keys[0] - vals[3]).abs().max() < 1e-12 and (S.T @ keys[1] - vals[1]).abs().max() < 1e-12
    o, S = P.delta_recurrence(k[:2], k[:2], vals[:2], torch.ones(2, dtype=torch.float64), 0.5 * ones[:2])
    assert (S.T @ keys[0] - 0.5 * vals[0]).abs().max() < 1e-12 and (S.T @ keys[1] - vals[1]).abs().max() < 1e-12
    o, S = P.delta_recurrence(k[:1], k[:1], vals[:1], torch.tensor([0.25], dtype=torch.float64), ones[:1])
    assert (S - 0.25 * torch.outer(keys[0], vals[0])).abs().max() < 1e-12


def test_plain_convolution_starts_from_zeros_and_ends_on_the_current_token():
    x = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None].repeat(1, 2)
    w = torch.tensor([[0.0, 0.0, 1.0], [1.0, 10.0, 100.0]], dtype=torch.float64)
    y = P.causal_taps(x, w)
    assert torch.allclose(y[:, 0], P.silu(x[:, 0]))                          # the last column weighs the current token
    want = torch.tensor([100.0, 210.0, 321.0, 432.0, 543.0], dtype=torch.float64)
    assert torch.allclose(y[:, 1], P.silu(want))


def test_plain_attention_mask_sink_and_temperature():
    torch.manual_seed(1)
    T, H, G, D = 9, 4, 2, 5
    q, k, v = (torch.randn(T, n, D, dtype=torch.float64) for n in (H, G, G))
    out = P.softmax_attention(q, k, v, 0.7, window=3, sinks=torch.tensor([0.5, -1.0, 2.0, 0.0], dtype=torch.float64))
    for i in (0, 2, 8):
        for h in range(H):
            js = [j for j in range(T) if 0 <= i - j < 3]
            e = torch.tensor([math.exp(0.7 * float(q[i, h] @ k[j, h // 2])) for j in js], dtype=torch.float64)
            sink = math.exp([0.5, -1.0, 2.0, 0.0][h])
            want = sum(e[n] * v[j, h // 2] for n, j in enumerate(js)) / (e.sum() + sink)
            assert (out[i, h] - want).abs().max() < 1e-12
    # the temperature: 1 up to position every - 2, then 1 + coef ln 2, ...
    W = {"q": torch.eye(2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64), "q.b": torch.zeros(2, dtype=torch.float64),
         "k.b": torch.zeros(2, dtype=torch.float64), "g": torch.zeros(2, 2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64)}
    h = torch.randn(7, 2, dtype=torch.float64)
    m = dict(heads=1, kv_heads=1, dim=2, scale=1.0, q_temp=dict(coef=0.5, every=3))
    got = P.key_value_attention(h, W, "", m)
    for i in (1, 2, 6):
        temp = 1.0 + 0.5 * math.log((i + 1) // 3 + 1)
        s = torch.tensor([temp * float(h[i] @ h[j]) for j in range(i + 1)], dtype=torch.float64)
        want = 0.5 * (torch.softmax(s, 0)[:, None] * h[: i + 1]).sum(0)       # sigmoid(0) = 1/2; the values are the keys
        assert (got[i] - want).abs().max() < 1e-12


def test_plain_frequencies_follow_the_ramp():
    f, mag = P.ramped_frequencies(8, 100.0, dict(factor=4.0, original=16, fast=4.0, slow=1.0))
    base = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    idx = lambda t: 8 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(100.0))
    lo, hi = max(math.floor(idx(4.0)), 0), min(math.ceil(idx(1.0)), 7)
    for i in range(4):
        r = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        assert abs(float(f[i]) - (base[i] / 4.0 * r + base[i] * (1 - r))) < 1e-15
    assert abs(mag - (0.1 * math.log(4.0) + 1.0)) < 1e-15
    f, mag = P.ramped_frequencies(6, 1e6, None)
    assert mag == 1.0 and abs(float(f[2]) - 1e6 ** (-4.0 / 6)) < 1e-18


def test_plain_model_runs_every_configuration_and_borrowed_keys_matter():
    from safetensors.torch import load_file
    import os
    import tempfile
    for name, c in LUDUSUN_CONFIGS.items():
        with tempfile.TemporaryDirectory() as d:
            write_ludusun(c, d)
            cfg = json.load(open(os.path.join(d, "config.json")))
            W = load_file(os.path.join(d, "model.safetensors"))
        toks = random_tokens(c["vocab"], 20, 1)
        trace = []
        lg = P.PlainLudusun(cfg, W).logits(toks, trace=trace)
        assert lg.shape == (20, c["vocab"]) and torch.isfinite(lg).all() and len(trace) == len(c["layers"])
        # causal: a later token changes no earlier row
        lg2 = P.PlainLudusun(cfg, W).logits(toks[:12])
        assert (lg[:12] - lg2).abs().max() < 1e-9


def test_a_folder_may_hold_the_second_norm_of_a_layer_without_feed_forward(tmp_path):
    import os
    from safetensors.torch import load_file, save_file
    from rocmforge_b200.config import load_config
    from rocmforge_b200.weights import WeightError, load_folder
    write_ludusun(LUDUSUN_CONFIGS["LA"], str(tmp_path), "bfloat16")
    path = os.path.join(str(tmp_path), "model.safetensors")
    W = load_file(path)
    assert "l1.norm2" not in W                                              # layer 1 has no feed-forward
    W["l1.norm2"] = torch.zeros(64, dtype=torch.bfloat16)
    save_file(W, path)
    arch, cfg = load_config(str(tmp_path))
    specs = arch.build(cfg).param_specs()
    assert "l1.norm2" in load_folder(str(tmp_path), specs, torch.bfloat16, "cpu")
    W["l1.mix.v"] = torch.zeros(3, dtype=torch.bfloat16)                    # any other unknown or misshapen tensor is a fault
    save_file(W, path)
    with pytest.raises(WeightError):
        load_folder(str(tmp_path), specs, torch.bfloat16, "cpu")
