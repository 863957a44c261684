"""Tiny configurations, folders with random weights, and comparison helpers for the tests."""
from __future__ import annotations

import json
import os
import subprocess
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# Three tiny configurations that differ in every size and option.
TINY_A = dict(   # grouped queries (4 heads on 2 kv heads), tied head, no window
    seed=0, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=64, num_attention_heads=4,
    num_key_value_heads=2, head_dim=16, intermediate_size=176, vocab_size=256, rope_theta=10000.0,
    rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128, use_sliding_window=False,
    sliding_window=None, max_window_layers=2, eos_token_id=7)
TINY_B = dict(   # one kv head for 3 heads, untied head, other eps/theta, longer context
    seed=1, architectures=["Qwen2ForCausalLM"], num_hidden_layers=3, hidden_size=96, num_attention_heads=3,
    num_key_value_heads=1, head_dim=32, intermediate_size=240, vocab_size=384, rope_theta=1e6,
    rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256, use_sliding_window=False,
    sliding_window=4096, max_window_layers=3)
TINY_C = dict(   # as many kv heads as heads, head_dim given and != hidden/heads, a window from layer 2 on
    seed=2, architectures=["Qwen2ForCausalLM"], num_hidden_layers=4, hidden_size=80, num_attention_heads=5,
    num_key_value_heads=5, head_dim=48, intermediate_size=112, vocab_size=300, rope_theta=50000.0,
    rms_norm_eps=3e-6, tie_word_embeddings=True, max_position_embeddings=512, use_sliding_window=True,
    sliding_window=24, max_window_layers=2, eos_token_id=[3, 5])
# Two more whose head sizes (64, 128) and widths let the bfloat16 engine take its tuned kernels (tcgen05 products
# of every orientation, tiled prefill attention, chunked decode attention) instead of the generic ones.
TINY_D = dict(   # head_dim 64, 2 query heads per kv head
    seed=3, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=256, num_attention_heads=4,
    num_key_value_heads=2, head_dim=64, intermediate_size=328, vocab_size=520, rope_theta=1e6,
    rms_norm_eps=1e-6, tie_word_embeddings=False, max_position_embeddings=1024, use_sliding_window=False)
TINY_E = dict(   # head_dim 128, 8 query heads on one kv head, a window of 200 from layer 1 on
    seed=4, architectures=["Qwen2ForCausalLM"], num_hidden_layers=2, hidden_size=320, num_attention_heads=8,
    num_key_value_heads=1, head_dim=128, intermediate_size=264, vocab_size=300, rope_theta=1e4,
    rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=1024, use_sliding_window=True,
    sliding_window=200, max_window_layers=1)
CONFIGS = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E}

F32_ATOL, F32_RTOL = 2e-5, 1e-4          # maeddesg/ROCmForge compares at 1e-4 (tests/gpu_test_utils.rs:12)
BF16_REL_TO_MAX = 2e-2                   # bfloat16 path against the plain model on the same weights


def config_dict(cfg: dict) -> dict:
    return {k: v for k, v in cfg.items() if k != "seed"}


def write_tiny(cfg: dict, folder: str, dtype: str = "float32", device: str = "cpu") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import Qwen2Config, architecture_for
    c = Qwen2Config.from_dict(config_dict(cfg))
    spec = architecture_for(c.architecture).build(c)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, c.to_dict(), spec.param_specs(), cfg["seed"], dt, device=device)


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def assert_logits_close(got, ref, dtype: str, what: str = ""):
    got = torch.as_tensor(np.asarray(got), dtype=torch.float64)
    ref = torch.as_tensor(np.asarray(ref), dtype=torch.float64)
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    diff = (got - ref).abs()
    if dtype == "float32":
        bound = F32_ATOL + F32_RTOL * ref.abs()
    else:
        bound = torch.full_like(ref, BF16_REL_TO_MAX * float(ref.abs().max()))
    bad = diff > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.numel()} logits differ; first at {idx}: "
                             f"got {got[tuple(idx)].item():.6g}, plain {ref[tuple(idx)].item():.6g}, "
                             f"max diff {diff.max().item():.3g}")


class TraceRun:
    """Drives bin/trace_run as a child process, one step at a time."""

    def __init__(self, folder: str, dtype: str, out_dir: str, max_tokens: int, env=None):
        self.out_dir = out_dir
        cfg = json.load(open(os.path.join(folder, "config.json")))
        self.vocab = cfg["vocab_size"] if "vocab_size" in cfg else cfg["vocab"]
        self.proc = subprocess.Popen(
            [os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
             "--max-tokens", str(max_tokens)], stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env)
        self.n = 0

    def step(self, entries, end=()):
        """entries: [(id, tokens, want)] -> float32 array [wanted, vocab] or None."""
        msg = {"step": self.n, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(msg) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        assert line == f"done {self.n}", f"trace_run answered {line!r} (exit code {self.proc.poll()})"
        path = os.path.join(self.out_dir, f"{self.n}.f32")
        self.n += 1
        if any(len(w) for _, _, w in entries):
            return np.fromfile(path, dtype="<f4").reshape(-1, self.vocab)
        assert not os.path.exists(path)
        return None

    def close(self) -> int:
        self.proc.stdin.close()
        return self.proc.wait(timeout=120)


# --------------------------------------------------------------------------- Rifizen

def rifizen_layer(*, heads, kv_heads, dim, vdim, window, scale, softcap, r_heads, r_dim, r_vdim, decay, rot_dims,
                  rot_base, mlp):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
                               "scale": scale, "softcap": softcap},
                      "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay),
                                "rot": {"dims": rot_dims, "base": rot_base}}},
            "mlp": mlp}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


# Sizes that differ from each other in every respect: values of another size than keys, value columns that do not
# fill a group of eight, a partly rotated head, decays of exactly 1 and far below, a layer without feed-forward, a
# loop that starts at the first layer / in the middle / is absent, one expert per token and several, windows below
# and above a page, as many kv heads as heads and one for all.
RIFIZEN_A = dict(seed=11, architecture="Rifizen", vocab=96, width=64, norm={"eps": 1e-5},
                 loop={"start": 0, "stop": 2, "times": 2},
                 layers=[rifizen_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=7, scale=0.3, softcap=5.0, r_heads=2,
                                       r_dim=24, r_vdim=12, decay=[0.9, 1.0], rot_dims=8, rot_base=100.0, mlp=_dense(40)),
                         rifizen_layer(heads=4, kv_heads=2, dim=16, vdim=24, window=3, scale=0.3, softcap=5.0, r_heads=2,
                                       r_dim=24, r_vdim=12, decay=[0.5, 0.99], rot_dims=8, rot_base=100.0, mlp=_moe(20, 5, 2)),
                         rifizen_layer(heads=2, kv_heads=1, dim=8, vdim=8, window=1, scale=1.0, softcap=2.0, r_heads=1,
                                       r_dim=40, r_vdim=20, decay=[0.97], rot_dims=40, rot_base=50.0, mlp=None)])
RIFIZEN_B = dict(seed=12, architecture="Rifizen", vocab=200, width=128, norm={"eps": 1e-6},
                 layers=[rifizen_layer(heads=3, kv_heads=3, dim=40, vdim=40, window=70, scale=0.05, softcap=50.0, r_heads=3,
                                       r_dim=64, r_vdim=32, decay=[0.8, 0.999, 0.99], rot_dims=32, rot_base=1e4,
                                       mlp=_moe(48, 8, 1)),
                         rifizen_layer(heads=9, kv_heads=1, dim=20, vdim=12, window=130, scale=0.2, softcap=8.0, r_heads=2,
                                       r_dim=96, r_vdim=64, decay=[0.95, 0.9999], rot_dims=96, rot_base=1e6,
                                       mlp=_dense(100))])
RIFIZEN_C = dict(seed=13, architecture="Rifizen", vocab=300, width=256, norm={"eps": 1e-6},
                 loop={"start": 1, "stop": 2, "times": 3},
                 layers=[rifizen_layer(heads=8, kv_heads=2, dim=64, vdim=64, window=100, scale=0.125, softcap=20.0, r_heads=4,
                                       r_dim=64, r_vdim=64, decay=[0.9, 0.99, 0.999, 0.9999], rot_dims=64, rot_base=1e5,
                                       mlp=_moe(64, 4, 2)),
                         rifizen_layer(heads=4, kv_heads=4, dim=32, vdim=48, window=33, scale=0.18, softcap=30.0, r_heads=8,
                                       r_dim=32, r_vdim=16, decay=[0.5, 0.75, 0.9, 0.95, 0.97, 0.98, 0.99, 0.995],
                                       rot_dims=16, rot_base=1e4, mlp=_dense(320)),
                         rifizen_layer(heads=4, kv_heads=1, dim=128, vdim=128, window=64, scale=0.09, softcap=15.0, r_heads=2,
                                       r_dim=128, r_vdim=128, decay=[0.98, 0.999], rot_dims=64, rot_base=1e4,
                                       mlp=_moe(96, 6, 3))])
RIFIZEN_CONFIGS = {"RA": RIFIZEN_A, "RB": RIFIZEN_B, "RC": RIFIZEN_C}


def write_rifizen(cfg: dict, folder: str, dtype: str = "float32") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import architecture_for
    arch = architecture_for("Rifizen")
    c = arch.config_cls.from_dict(config_dict(cfg))
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, c.to_dict(), arch.build(c).param_specs(), cfg["seed"], dt)


# --------------------------------------------------------------------------- Vilulorn

def _gla(*, heads, dim, vdim, tau, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def _chunk_attention(*, heads, kv_heads, dim, vdim, chunk, scale, rot_dims, rot_base, scaling=None, kv_from=None, mlp):
    rot = {"dims": rot_dims, "base": rot_base}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "scale": scale, "rot": rot}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _scored(ff, experts, top, limit):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


# Sizes that differ from each other in every respect: the order of the two kinds of layer, values of another size than
# keys, value columns that do not fill a warp's share, key sizes that are no multiple of 32, decay ranks that are no
# multiple of 8, tau of 1 and large, chunks below a page, of a page, and above one, a wholly rotated and a partly rotated
# head with and without stretched frequencies, one kv head for all and as many as heads, layers that borrow keys with
# the lender's chunk size and with another, a layer without feed-forward, one expert a token and several, limits that
# bite.  ``ranks``: rows of each gla layer's first decay matrix (a tensor's shape, not a key of config.json).
VILULORN_A = dict(seed=21, architecture="Vilulorn", vocab=96, width=64, max_positions=400, norm={"eps": 1e-5}, ranks={1: 5, 3: 8},
                  layers=[_chunk_attention(heads=4, kv_heads=2, dim=16, vdim=24, chunk=7, scale=0.4, rot_dims=8, rot_base=100.0,
                                           mlp=_scored(20, 5, 2, 0.5)),
                          _gla(heads=2, dim=24, vdim=12, tau=1.0, mlp=None),
                          _chunk_attention(heads=4, kv_heads=2, dim=16, vdim=24, chunk=64, scale=0.25, rot_dims=8, rot_base=100.0,
                                           kv_from=0, mlp=_scored(24, 3, 3, 4.0)),
                          _gla(heads=1, dim=40, vdim=20, tau=4.0, mlp=_scored(16, 4, 1, 1.0))])
VILULORN_B = dict(seed=22, architecture="Vilulorn", vocab=200, width=128, max_positions=512, norm={"eps": 1e-6}, ranks={0: 16, 3: 3},
                  layers=[_gla(heads=3, dim=64, vdim=32, tau=16.0, mlp=_scored(48, 8, 1, 2.0)),
                          _chunk_attention(heads=3, kv_heads=3, dim=40, vdim=40, chunk=100, scale=0.16, rot_dims=40, rot_base=1e4,
                                           scaling=(8.0, 1.0, 4.0, 64), mlp=None),
                          _chunk_attention(heads=3, kv_heads=3, dim=40, vdim=40, chunk=100, scale=0.3, rot_dims=40, rot_base=1e4,
                                           scaling=(8.0, 1.0, 4.0, 64), kv_from=1, mlp=_scored(40, 6, 2, 1.5)),
                          _gla(heads=2, dim=96, vdim=72, tau=7.0, mlp=_scored(32, 2, 2, 3.0))])
VILULORN_C = dict(seed=23, architecture="Vilulorn", vocab=300, width=256, max_positions=1024, norm={"eps": 1e-6}, ranks={0: 32, 2: 16},
                  layers=[_gla(heads=2, dim=128, vdim=128, tau=10.0, mlp=_scored(96, 6, 3, 2.5)),
                          _chunk_attention(heads=8, kv_heads=2, dim=64, vdim=64, chunk=130, scale=0.125, rot_dims=32, rot_base=1e6,
                                           scaling=(4.0, 1.0, 4.0, 256), mlp=_scored(64, 4, 2, 2.0)),
                          _gla(heads=4, dim=32, vdim=64, tau=2.0, mlp=_scored(64, 16, 1, 6.0)),
                          _chunk_attention(heads=4, kv_heads=1, dim=128, vdim=128, chunk=33, scale=0.09, rot_dims=64, rot_base=1e4,
                                           mlp=_scored(128, 3, 1, 1.0)),
                          _chunk_attention(heads=8, kv_heads=2, dim=64, vdim=64, chunk=130, scale=0.2, rot_dims=32, rot_base=1e6,
                                           scaling=(4.0, 1.0, 4.0, 256), kv_from=1, mlp=_scored(64, 4, 4, 2.0))])
# Two more at the edges of what the kernels take: a width that is no multiple of 8 (no operand of a product is aligned for
# the tensor-core kernels), sixteen query heads on one kv head (more than the clustered decode attention serves), a state
# of 256 key channels by 8 value columns and one of 16 by 200, a decay projection of rank 1, 64-element keys with
# 128-element values, chunks of 2.
VILULORN_D = dict(seed=24, architecture="Vilulorn", vocab=130, width=100, max_positions=300, norm={"eps": 1e-6}, ranks={1: 1},
                  layers=[_chunk_attention(heads=16, kv_heads=1, dim=64, vdim=64, chunk=50, scale=0.125, rot_dims=64, rot_base=1e4,
                                           mlp=_scored(24, 2, 1, 3.0)),
                          _gla(heads=1, dim=256, vdim=8, tau=32.0, mlp=None),
                          _chunk_attention(heads=16, kv_heads=1, dim=64, vdim=64, chunk=50, scale=0.2, rot_dims=64, rot_base=1e4,
                                           kv_from=0, mlp=_scored(16, 3, 2, 1.0))])
VILULORN_E = dict(seed=25, architecture="Vilulorn", vocab=150, width=128, max_positions=300, norm={"eps": 1e-5}, ranks={2: 24},
                  layers=[_chunk_attention(heads=16, kv_heads=1, dim=64, vdim=64, chunk=70, scale=0.125, rot_dims=2, rot_base=10.0,
                                           mlp=_scored(32, 4, 2, 2.0)),
                          _chunk_attention(heads=2, kv_heads=2, dim=64, vdim=128, chunk=2, scale=0.3, rot_dims=16, rot_base=1e3,
                                           scaling=(2.0, 1.0, 2.0, 16), mlp=None),
                          _gla(heads=2, dim=16, vdim=200, tau=0.5, mlp=_scored(8, 9, 4, 0.25))])
VILULORN_CONFIGS = {"VA": VILULORN_A, "VB": VILULORN_B, "VC": VILULORN_C, "VD": VILULORN_D, "VE": VILULORN_E}


def vilulorn_config(cfg: dict):
    """(typed configuration, the dict that goes into config.json)."""
    from rocmforge_b200.config import architecture_for
    raw = {k: v for k, v in cfg.items() if k not in ("seed", "ranks")}
    shapes = {f"l{i}.mix.a1": (r, cfg["width"]) for i, r in cfg.get("ranks", {}).items()}
    return architecture_for("Vilulorn").config_cls.from_dict(raw, shapes=shapes), raw


def write_vilulorn(cfg: dict, folder: str, dtype: str = "float32") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import architecture_for
    c, raw = vilulorn_config(cfg)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, raw, architecture_for("Vilulorn").build(c).param_specs(), cfg["seed"], dt)


# --------------------------------------------------------------------------- Figalix

def _kept_window(*, heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot_dims=0, rot_base=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None or keep_first is not None:
        m["mask"] = {}
        if window is not None:
            m["mask"]["size"] = window
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": rot_base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return m


def _side_by_side(left, *, heads, dim, vdim, gate_cap, mlp):
    right = {"heads": heads, "dim": dim, "vdim": vdim}
    if gate_cap is not None:
        right["gate_cap"] = gate_cap
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def _ssd(*, heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def _shares(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


# Sizes that differ from each other in every respect: which kind of layer comes first, values of another size than keys,
# as many kv heads as heads and one for all, heads rotated wholly, partly (with and without stretched frequencies) and not
# at all, windows of 1, below a page, above one and absent, first positions kept: none, fewer than the window, more than
# the window, more than a page; a matrix memory of 256 x 8 and of 16 x 200, gates capped tightly, loosely and not at all;
# state-space layers with one group, as many groups as heads and in between, one to seven taps, a norm in one part and in
# several, states that are no multiple of eight; layers without feed-forward, dense ones, one expert a token and all of
# them, with and without the shared expert; multipliers of 1 and others; logits capped and not; a width that no
# tensor-core kernel takes.
FIGALIX_A = dict(seed=31, architecture="Figalix", vocab=96, width=64, norm={"eps": 1e-5}, residual_mult=0.5, logit_softcap=8.0,
                 layers=[_ssd(heads=4, vdim=8, state=12, groups=2, conv=3, norm_groups=4, mlp=_shares(20, 5, 2, 24)),
                         _side_by_side(_kept_window(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.4, window=7, keep_first=3,
                                                    rot_dims=8, rot_base=100.0, scaling=(4.0, 16, 4.0, 1.0)),
                                       heads=2, dim=24, vdim=12, gate_cap=3.0, mlp=None),
                         _side_by_side(_kept_window(heads=2, kv_heads=1, dim=8, vdim=8, scale=1.0, window=1, keep_first=2,
                                                    rot_dims=8, rot_base=50.0),
                                       heads=1, dim=40, vdim=20, gate_cap=30.0, mlp=_dense(40)),
                         _ssd(heads=3, vdim=20, state=7, groups=3, conv=1, norm_groups=1, mlp=None)])
FIGALIX_B = dict(seed=32, architecture="Figalix", vocab=200, width=128, norm={"eps": 1e-6}, residual_mult=1.0,
                 layers=[_side_by_side(_kept_window(heads=3, kv_heads=3, dim=40, vdim=40, scale=0.16, window=70, keep_first=100,
                                                    rot_dims=40, rot_base=1e4, scaling=(8.0, 64, 8.0, 2.0)),
                                       heads=3, dim=64, vdim=32, gate_cap=15.0, mlp=_shares(48, 8, 1, 16)),
                         _ssd(heads=6, vdim=16, state=64, groups=1, conv=4, norm_groups=2, mlp=_dense(100)),
                         _side_by_side(_kept_window(heads=9, kv_heads=1, dim=20, vdim=12, scale=0.2, window=130, keep_first=0,
                                                    rot_dims=6, rot_base=1e6),
                                       heads=2, dim=96, vdim=72, gate_cap=None, mlp=_shares(40, 3, 3))])
FIGALIX_C = dict(seed=33, architecture="Figalix", vocab=300, width=256, norm={"eps": 1e-6}, residual_mult=0.8, logit_softcap=50.0,
                 layers=[_side_by_side(_kept_window(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, window=100, keep_first=5,
                                                    rot_dims=32, rot_base=1e6, scaling=(4.0, 256, 16.0, 2.0)),
                                       heads=2, dim=128, vdim=128, gate_cap=10.0, mlp=_shares(64, 4, 2, 96)),
                         _ssd(heads=8, vdim=64, state=128, groups=2, conv=4, norm_groups=1, mlp=_shares(64, 16, 1, 32)),
                         _side_by_side(_kept_window(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, window=33, keep_first=70,
                                                    rot_dims=128, rot_base=1e4),
                                       heads=4, dim=32, vdim=64, gate_cap=15.0, mlp=_dense(320)),
                         _side_by_side(_kept_window(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, window=64, keep_first=None,
                                                    rot_dims=64, rot_base=1e5, scaling=(2.0, 128, 4.0, 1.0)),
                                       heads=2, dim=64, vdim=64, gate_cap=20.0, mlp=_shares(96, 6, 3, 64)),
                         _ssd(heads=4, vdim=32, state=16, groups=4, conv=2, norm_groups=4, mlp=_dense(128))])
FIGALIX_D = dict(seed=34, architecture="Figalix", vocab=130, width=100, norm={"eps": 1e-6}, residual_mult=0.3, logit_softcap=2.0,
                 layers=[_side_by_side(_kept_window(heads=16, kv_heads=1, dim=64, vdim=64, scale=0.125, window=50, keep_first=1,
                                                    rot_dims=64, rot_base=1e4, scaling=(16.0, 32, 2.0, 0.5)),
                                       heads=1, dim=256, vdim=8, gate_cap=1.0, mlp=_shares(24, 2, 2, 8)),
                         _ssd(heads=2, vdim=100, state=256, groups=1, conv=7, norm_groups=5, mlp=None),
                         _side_by_side(_kept_window(heads=2, kv_heads=2, dim=64, vdim=128, scale=0.3, rot_dims=0),
                                       heads=2, dim=16, vdim=200, gate_cap=15.0, mlp=_shares(8, 9, 4))])
FIGALIX_CONFIGS = {"FA": FIGALIX_A, "FB": FIGALIX_B, "FC": FIGALIX_C, "FD": FIGALIX_D}


def figalix_config(cfg: dict):
    """(typed configuration, the dict that goes into config.json)."""
    from rocmforge_b200.config import architecture_for
    raw = config_dict(cfg)
    return architecture_for("Figalix").config_cls.from_dict(raw), raw


def write_figalix(cfg: dict, folder: str, dtype: str = "float32") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import architecture_for
    c, raw = figalix_config(cfg)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, raw, architecture_for("Figalix").build(c).param_specs(), cfg["seed"], dt)


# --------------------------------------------------------------------------- Ludusun

def _sink_attention(*, heads, kv_heads, dim, vdim, scale, rot_dims=0, rot_base=None, scaling=None, kv_from=None, mlp):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot_dims:
        m["rot"] = {"dims": rot_dims, "base": rot_base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _latent(*, heads, dim, vdim, q_rank, kv_rank, scale, window=None, mlp):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _summed(*, heads, kv_heads, dim, scale, q_temp=None, r_heads, r_kv_heads, r_dim, r_vdim, conv, left_scale, right_scale, mlp):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if q_temp is not None:
        left["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    right = {"heads": r_heads, "kv_heads": r_kv_heads, "dim": r_dim, "vdim": r_vdim, "conv": conv}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


# Sizes that differ from each other in every respect: which kind of layer comes first, values of another size than keys,
# one kv head for nine and for sixteen heads and as many as heads, heads rotated wholly, partly (with and without the ramp
# of stretched frequencies) and not at all, layers that read an earlier layer's keys, latents narrower and wider than the
# heads they expand to, windows of 7, 33, 70, 100, 130 and none, a query temperature that steps every position, every 5 and
# every 64 positions and none, delta-rule heads that share q and k and heads with their own, 1 to 7 taps, low ranks of 1 to
# 24 (no multiple of 8 among them), a state of 256 x 8, layers without feed-forward, an embedding scale of 1 and others,
# branch factors of 1 and others, logits capped and not, a width that no tensor-core kernel takes.  ``ranks``: rows of the
# delta rule's two narrow matrices (a tensor's shape, not a key of the design).
LUDUSUN_A = dict(seed=41, architecture="Ludusun", vocab=96, width=64, norm={"eps": 1e-5}, embedding={"scale": 2.0},
                 logit_softcap=8.0, ranks={"l0.mix.right.a1": 5, "l0.mix.right.g1": 3},
                 layers=[_summed(heads=4, kv_heads=2, dim=16, scale=0.25, q_temp=(0.3, 5), r_heads=2, r_kv_heads=1, r_dim=24,
                                 r_vdim=12, conv=3, left_scale=1.0, right_scale=0.7, mlp=_dense(40)),
                         _sink_attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.3, rot_dims=8, rot_base=100.0,
                                         scaling=(4.0, 16, 4.0, 1.0), mlp=None),
                         _latent(heads=3, dim=8, vdim=16, q_rank=12, kv_rank=20, scale=0.35, window=7, mlp=_dense(48)),
                         _sink_attention(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.5, rot_dims=8, rot_base=100.0,
                                         scaling=(4.0, 16, 4.0, 1.0), kv_from=1, mlp=_dense(24))])
LUDUSUN_B = dict(seed=42, architecture="Ludusun", vocab=200, width=128, norm={"eps": 1e-6}, embedding={"scale": 1.0},
                 ranks={"l2.mix.right.a1": 16, "l2.mix.right.g1": 9},
                 layers=[_sink_attention(heads=9, kv_heads=1, dim=20, vdim=12, scale=0.2, rot_dims=6, rot_base=1e6, mlp=_dense(100)),
                         _latent(heads=2, dim=40, vdim=40, q_rank=8, kv_rank=64, scale=0.16, window=70, mlp=None),
                         _summed(heads=3, kv_heads=3, dim=40, scale=0.16, r_heads=4, r_kv_heads=2, r_dim=64, r_vdim=32, conv=1,
                                 left_scale=0.5, right_scale=1.0, mlp=_dense(64)),
                         _sink_attention(heads=9, kv_heads=1, dim=20, vdim=12, scale=0.3, rot_dims=6, rot_base=1e6, kv_from=0,
                                         mlp=_dense(40)),
                         _latent(heads=1, dim=24, vdim=8, q_rank=30, kv_rank=16, scale=0.2, window=130, mlp=_dense(32))])
LUDUSUN_C = dict(seed=43, architecture="Ludusun", vocab=300, width=256, norm={"eps": 1e-6}, embedding={"scale": 4.0},
                 logit_softcap=30.0, ranks={"l2.mix.right.a1": 24, "l2.mix.right.g1": 12},
                 layers=[_latent(heads=4, dim=64, vdim=64, q_rank=96, kv_rank=136, scale=0.125, window=100, mlp=_dense(320)),
                         _sink_attention(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, rot_dims=32, rot_base=1e6,
                                         scaling=(4.0, 256, 16.0, 2.0), mlp=_dense(128)),
                         _summed(heads=8, kv_heads=2, dim=64, scale=0.125, q_temp=(0.5, 64), r_heads=4, r_kv_heads=2, r_dim=32,
                                 r_vdim=48, conv=2, left_scale=0.8, right_scale=0.5, mlp=_dense(96)),
                         _sink_attention(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.2, rot_dims=32, rot_base=1e6,
                                         scaling=(4.0, 256, 16.0, 2.0), kv_from=1, mlp=None),
                         _sink_attention(heads=4, kv_heads=1, dim=128, vdim=128, scale=0.09, rot_dims=128, rot_base=1e4,
                                         mlp=_dense(64)),
                         _latent(heads=2, dim=128, vdim=128, q_rank=64, kv_rank=32, scale=0.09, window=33, mlp=_dense(64))])
LUDUSUN_D = dict(seed=44, architecture="Ludusun", vocab=130, width=100, norm={"eps": 1e-6}, embedding={"scale": 0.5},
                 logit_softcap=2.0, ranks={"l0.mix.right.a1": 1, "l0.mix.right.g1": 2},
                 layers=[_summed(heads=16, kv_heads=1, dim=64, scale=0.125, q_temp=(1.0, 1), r_heads=1, r_kv_heads=1, r_dim=256,
                                 r_vdim=8, conv=7, left_scale=0.3, right_scale=2.0, mlp=None),
                         _sink_attention(heads=2, kv_heads=2, dim=64, vdim=128, scale=0.3, mlp=_dense(24)),
                         _latent(heads=16, dim=16, vdim=24, q_rank=7, kv_rank=9, scale=0.25, mlp=_dense(16))])
LUDUSUN_CONFIGS = {"LA": LUDUSUN_A, "LB": LUDUSUN_B, "LC": LUDUSUN_C, "LD": LUDUSUN_D}


def ludusun_config(cfg: dict):
    """(typed configuration, the dict that goes into config.json)."""
    from rocmforge_b200.config import architecture_for
    raw = {k: v for k, v in cfg.items() if k not in ("seed", "ranks")}
    shapes = {name: (r, cfg["width"]) for name, r in cfg.get("ranks", {}).items()}
    return architecture_for("Ludusun").config_cls.from_dict(raw, shapes=shapes), raw


def write_ludusun(cfg: dict, folder: str, dtype: str = "float32") -> None:
    import rocmforge_b200 as rf
    from rocmforge_b200.config import architecture_for
    c, raw = ludusun_config(cfg)
    dt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    rf.write_model_folder(folder, raw, architecture_for("Ludusun").build(c).param_specs(), cfg["seed"], dt)
