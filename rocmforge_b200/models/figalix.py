"""The Figalix decoder as a list of parts.

x = embed[token].  A layer is pre-norm with one multiplier m for both sub-layers: x += m mixer(norm1(x));
x += m ff(norm2(x)) (the ``scaled_prenorm`` block); every norm is a Dynamic Tanh.  The mixer is, layer by layer,

  "parallel"  two mixers side by side on the same input, merged as the mean of their RMS-normed outputs (``parallel``):
              grouped-query softmax attention over a sliding window that also keeps a sequence's first positions, with a
              partly rotated head (rotate-half pairs, YaRN-stretched frequencies) and one sigmoid gate per head
              (``gqa_attention``), beside the matrix memory of xLSTM (``mlstm``);
  "mamba2"    the Mamba-2 state-space mixer (``mamba2``).

The feed-forward is a gated silu unit (``gated_mlp``), or a mixture of such units chosen by the largest shares of a
softmax over all experts and weighted by those shares as they are, plus a shared unit that every token uses
(``sum`` of ``routed_experts`` and ``gated_mlp``); a layer may have none.  Final Dynamic Tanh, then the embedding
matrix as the head, and a tanh cap on the logits.

Tensor names: ``embed``; ``l<i>.norm1|norm2`` with ``.alpha`` and ``.b``; parallel: ``l<i>.mix.left.q|k|v|g|o|out``,
``l<i>.mix.right.q|k|v|g|o|norm|i|i.b|f|f.b|out``; mamba2: ``l<i>.mix.in|conv|conv.b|dt_bias|A_log|D|norm|o``;
``l<i>.mlp.gate|up|down`` or ``l<i>.mlp.router``, ``.e<j>.gate|up|down``, ``.shared.gate|up|down``; ``final.norm``.
"""
from __future__ import annotations

from ..config.figalix import FigalixConfig
from ..config.registry import register_architecture
from ..engine.model import ModelSpec, ScheduleEntry
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..parts.embedding import OutputHead, TokenEmbedding

NO_POSITION_LIMIT = 1 << 20      # the design has no longest sequence; the cache's size is the only limit
UNIT_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def build_figalix(cfg: FigalixConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps

    def norm():
        return NORMS.build("dyt", size=W, param_name="")

    def left_mixer(a):
        position = None
        if a.rot_dims > 0 and a.rot_scaling is not None:
            position = POSITIONS.build("rope_yarn", head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims, **a.rot_scaling)
        elif a.rot_dims > 0:
            position = POSITIONS.build("rope_neox", head_dim=a.dim, theta=a.rot_base, rotary_dim=a.rot_dims)
        return MIXERS.build("gqa_attention", hidden=W, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim,
                            v_head_dim=a.vdim, qkv_bias=False, window=a.window, keep_first=a.keep_first, position=position,
                            scale=a.scale, gate="sigmoid_head", names={"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"})

    def right_mixer(r):
        return MIXERS.build("mlstm", hidden=W, n_heads=r.heads, dim=r.dim, vdim=r.vdim, eps=eps, gate_cap=r.gate_cap,
                            names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "i": "i", "i_bias": "i.b", "f": "f",
                                   "f_bias": "f.b", "norm": "norm"})

    blocks, prefixes = [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "parallel":
            mixer = MIXERS.build("parallel", hidden=W, eps=eps,
                                 branches={"left": left_mixer(m.left), "right": right_mixer(m.right)})
        else:
            mixer = MIXERS.build("mamba2", hidden=W, n_heads=m.heads, vdim=m.vdim, state=m.state, groups=m.groups,
                                 taps=m.taps, norm_groups=m.norm_groups, eps=eps,
                                 names={"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias",
                                        "a_log": "A_log", "d": "D", "norm": "norm", "o": "o"})
        ffn = None
        if L.mlp is not None and L.mlp.kind == "dense":
            ffn = FEED_FORWARDS.build("gated_mlp", hidden=W, intermediate=L.mlp.ff, names=UNIT_NAMES)
        elif L.mlp is not None:
            ffn = FEED_FORWARDS.build("routed_experts", hidden=W, intermediate=L.mlp.ff, n_experts=L.mlp.experts,
                                      top=L.mlp.top, router_bias=False, scoring="softmax_of_all")
            if L.mlp.shared_ff is not None:
                shared = FEED_FORWARDS.build("gated_mlp", hidden=W, intermediate=L.mlp.shared_ff, names=UNIT_NAMES)
                ffn = FEED_FORWARDS.build("sum", branches={"": ffn, "shared.": shared})
        blocks.append(BLOCKS.build("scaled_prenorm", norm1=norm(), mixer=mixer, norm2=norm() if ffn is not None else None,
                                   ffn=ffn, mult=cfg.residual_mult,
                                   names={"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp."}))
        prefixes.append(f"l{i}.")
    return ModelSpec(
        config=cfg, embedding=TokenEmbedding(cfg.vocab, W, param_name=""), embedding_prefix="embed",
        blocks=blocks, block_prefixes=prefixes, final_norm=norm(), final_norm_prefix="final.norm",
        head=OutputHead(cfg.vocab, W, tied_to="embed", param_name="", softcap=cfg.logit_softcap), head_prefix="head",
        schedule=[ScheduleEntry(layer=i) for i in range(len(cfg.layers))], vocab_size=cfg.vocab, hidden_size=W,
        max_position=NO_POSITION_LIMIT, stop_token_ids=[])


register_architecture(FigalixConfig.ARCHITECTURE, FigalixConfig, build_figalix)
