"""The Ludusun decoder as a list of parts.

x = embed[token] * embedding.scale.  A layer is pre-norm, x += mixer(norm1(x)); x += ff(norm2(x)) (the ``prenorm`` block; a
layer may have no feed-forward), every norm an RMS norm whose weight is stored around zero (``rmsnorm`` with
``weight_offset`` 1).  The mixer is, layer by layer,

  "attention"         grouped-query softmax attention over all earlier positions (``gqa_attention``): rotate-half pairs on
                      the first ``rot.dims`` elements of a head with YaRN-stretched frequencies, q and k heads divided by
                      their root mean square AFTER the rotation, values of a size of their own, and a learned sink per head
                      in the softmax's denominator; a layer with ``kv_from`` has no key and value tensors and reads the
                      named layer's cache;
  "latent_attention"  attention without positions over a sliding window whose queries, keys and values are expanded from
                      RMS-normed latents, with one sigmoid gate per head (``latent_attention``);
  "parallel"          two mixers on the same input, summed with a factor each (``parallel`` with ``scales``): causal
                      attention without rotation whose values are its keys, with q and k biases, a query temperature that
                      grows with the logarithm of the position and an element-wise sigmoid gate (``gqa_attention``), beside
                      the gated delta rule (``gated_delta``).

The feed-forward is a gated silu unit (``gated_mlp``).  Final norm, then the embedding matrix itself (unscaled) as the
head, and a tanh cap on the logits.

Tensor names: ``embed``; ``l<i>.norm1|norm2``; attention: ``l<i>.mix.q|k|v|sink|o``; latent_attention:
``l<i>.mix.dq|dq.norm|uq|dkv|dkv.norm|uk|uv|g|o``; parallel: ``l<i>.mix.left.q|q.b|k|k.b|g|o`` and
``l<i>.mix.right.q|q.conv|k|k.conv|v|v.conv|b|A_log|norm|a1|a2|dt_bias|g1|g2|o``; ``l<i>.mlp.gate|up|down``; ``final.norm``.
"""
from __future__ import annotations

from ..config.ludusun import LudusunConfig
from ..config.registry import register_architecture
from ..engine.model import ModelSpec, ScheduleEntry
from ..parts import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, POSITIONS
from ..parts.embedding import OutputHead, TokenEmbedding

NO_POSITION_LIMIT = 1 << 20      # the design has no longest sequence; the cache's size is the only limit
UNIT_VECTOR_EPS = 1e-6           # inside the root that makes the delta rule's q and k unit vectors: fixed by the design
NORM_WEIGHT_OFFSET = 1.0         # the layers' and the final norm's weights are stored around zero


def build_ludusun(cfg: LudusunConfig) -> ModelSpec:
    W, eps = cfg.width, cfg.eps

    def norm():
        return NORMS.build("rmsnorm", size=W, eps=eps, param_name="", weight_offset=NORM_WEIGHT_OFFSET)

    def sink_attention(m):
        position = None
        if m.rot_dims > 0 and m.rot_scaling is not None:
            position = POSITIONS.build("rope_yarn", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims, **m.rot_scaling)
        elif m.rot_dims > 0:
            position = POSITIONS.build("rope_neox", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims)
        return MIXERS.build("gqa_attention", hidden=W, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                            v_head_dim=m.vdim, qkv_bias=False, position=position, scale=m.scale, qk_norm_eps=eps,
                            qk_norm_after_rotation=True, sink=True, shares_kv=m.kv_from is not None,
                            names={"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink"})

    def side_by_side(m):
        left = MIXERS.build("gqa_attention", hidden=W, n_heads=m.left.heads, n_kv_heads=m.left.kv_heads, head_dim=m.left.dim,
                            qkv_bias=True, position=None, scale=m.left.scale, values_are_keys=True, gate="sigmoid",
                            q_temperature=m.left.q_temp,
                            names={"q": "q", "k": "k", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b"})
        r = m.right
        right = MIXERS.build("gated_delta", hidden=W, n_heads=r.heads, qk_heads=r.kv_heads, dim=r.dim, vdim=r.vdim,
                             taps=r.taps, decay_rank=r.decay_rank, gate_rank=r.gate_rank, eps=eps, unit_eps=UNIT_VECTOR_EPS,
                             names={"q": "q", "k": "k", "v": "v", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv",
                                    "b": "b", "a_log": "A_log", "dt_bias": "dt_bias", "a1": "a1", "a2": "a2", "g1": "g1",
                                    "g2": "g2", "norm": "norm", "o": "o"})
        return MIXERS.build("parallel", hidden=W, branches={"left": left, "right": right},
                            scales={"left": m.left_scale, "right": m.right_scale})

    blocks, prefixes, schedule = [], [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        if L.type == "attention":
            mixer = sink_attention(m)
        elif L.type == "latent_attention":
            mixer = MIXERS.build("latent_attention", hidden=W, n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim,
                                 q_rank=m.q_rank, kv_rank=m.kv_rank, eps=eps, scale=m.scale, window=m.window,
                                 names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm",
                                        "uk": "uk", "uv": "uv", "g": "g", "o": "o"})
        else:
            mixer = side_by_side(m)
        ffn = (FEED_FORWARDS.build("gated_mlp", hidden=W, intermediate=L.ff, names={"gate": "gate", "up": "up", "down": "down"})
               if L.ff is not None else None)
        blocks.append(BLOCKS.build("prenorm", norm1=norm(), mixer=mixer, norm2=norm() if ffn is not None else None, ffn=ffn,
                                   names={"norm1": "norm1", "mixer": "mix.", "norm2": "norm2", "ffn": "mlp."}))
        prefixes.append(f"l{i}.")
        schedule.append(ScheduleEntry(layer=i, kv_from=m.kv_from if L.type == "attention" else None))
    return ModelSpec(
        config=cfg, embedding=TokenEmbedding(cfg.vocab, W, param_name="", scale=cfg.embedding_scale), embedding_prefix="embed",
        blocks=blocks, block_prefixes=prefixes, final_norm=norm(), final_norm_prefix="final.norm",
        head=OutputHead(cfg.vocab, W, tied_to="embed", param_name="", softcap=cfg.logit_softcap), head_prefix="head",
        schedule=schedule, vocab_size=cfg.vocab, hidden_size=W, max_position=NO_POSITION_LIMIT, stop_token_ids=[])


register_architecture(LudusunConfig.ARCHITECTURE, LudusunConfig, build_ludusun)
