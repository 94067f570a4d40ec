"""Kafepel, assembled from parts.

Every layer is a `PreNormBlock` (RMS norms with plain weights) around a `PairMixer` and a feed-forward, or the mixer
alone.  The pair's left branch is a `GQAAttention` on its route with 32-bit scores and sigmoid weights (q and k
normalised over the whole projection, rotary positions in the half-split pairing with the frequency bands
optionally rescaled, capped scores, a number per head in front of the sigmoid, the heads' weights mixed by a square
matrix); its right branch is a `RetentionMixer` (one fixed decay per head, a gated read-out normalised per head).
The feed-forward is a `SwiGLU` or a `PlainRoutedExperts` (squared-relu experts chosen by score + correction, a
gated shared expert).  The embedding is multiplied by a constant.  Tensor names: `embed`, `l<i>.norm1|norm2`,
`l<i>.mix.left.q|k|v|o|q.norm|k.norm|talk|pb|out`, `l<i>.mix.right.q|k|v|g|o|out`, `l<i>.mlp.gate|up|down` or
`l<i>.mlp.router|correction|e<j>.up|e<j>.down|shared.up|shared.down|shared.sg`, `final.norm`, `head`; matrices are
stored [out, in] under their bare names.
"""
from __future__ import annotations

from .. import registry
from ..config.kafepel import KafepelConfig
from ..parts import (Embedding, GQAAttention, LMHead, MixerOnly, Model, NoPositionEncoding, PairMixer, PlainRoutedExperts, PreNormBlock,
                     RetentionMixer, RMSNorm, RotaryEmbedding, Run, SwiGLU)


def build_kafepel(cfg: KafepelConfig) -> Model:
    d, eps = cfg.width, cfg.norm_eps
    embed = Embedding(cfg.vocab, d, "embed", suffix="", scale=cfg.embedding_scale)
    layers, schedule, drop = [], [], []
    for i, spec in enumerate(cfg.layers):
        p = f"l{i}"
        a, r = spec.mixer.left, spec.mixer.right
        pos = RotaryEmbedding(a.dim, a.rot.base, scaling=a.rot.scaling, rotary_dim=a.rot.dims) if a.rot.dims \
            else NoPositionEncoding()
        left = GQAAttention(d, a.heads, a.kv_heads, a.dim, pos, f"{p}.mix.left", scale=a.scale, proj_names=("q", "k", "v", "o"),
                            v_head_dim=a.vdim, softcap=a.softcap, qk_norm_eps=eps, qk_norm_weights=("q.norm", "k.norm"),
                            qk_norm_first=True, qk_norm_whole=True, weights="sigmoid", head_bias="pb", head_mix="talk",
                            weight_suffix="")
        right = RetentionMixer(d, r.heads, r.dim, r.vdim, r.decay, eps, f"{p}.mix.right", rot_dims=r.rot.dims,
                               rot_base=r.rot.base, rot_scaling=r.rot.scaling)
        mixer = PairMixer(d, left, right, eps, f"{p}.mix")
        norm1 = RMSNorm(d, eps, f"{p}.norm1", suffix="")
        if spec.mlp is None:
            drop.append(f"{p}.norm2")                 # a layer without a feed-forward uses no second norm
            layers.append(MixerOnly(mixer, norm1))
        else:
            if spec.mlp.kind == "dense":
                ffn = SwiGLU(d, spec.mlp.ff, f"{p}.mlp", proj_names=("gate", "up", "down"), weight_suffix="")
            else:
                m = spec.mlp
                ffn = PlainRoutedExperts(d, m.experts, m.top, m.ff, f"{p}.mlp", scale=m.router_scale, shared_ff=m.shared_ff)
            layers.append(PreNormBlock(mixer, ffn, norm1, RMSNorm(d, eps, f"{p}.norm2", suffix="")))
        schedule.append(Run(i))
    head = LMHead(cfg.vocab, d, "head", suffix="")
    return Model(embed, layers, RMSNorm(d, eps, "final.norm", suffix=""), head, schedule=schedule, vocab_size=cfg.vocab, drop=drop)


registry.register(["kafepel", "Kafepel"], KafepelConfig.from_dict, build_kafepel, replace=True)
