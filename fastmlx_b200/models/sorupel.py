"""Sorupel, assembled from parts.

Every layer is a `PreNormBlock` (RMS norms with plain weights) around one of three mixers and a gated feed-forward
of tanh-gelu, or none: a `GQAAttention` on its route with 32-bit scores whose values are the keys as projected
(q and k normalised over the whole projection, partial rotary positions in the half-split pairing, capped scores,
a mask of runs of positions, one more term of score 0 in the denominator, one gate value per head); a
`LatentAttention` with direct queries, a rotated key part beside the cached latent, a learned term per head in
the denominator and a gate per output element, which may read the cache of an earlier layer (`kv_from`: the
schedule's `cache_from`); or a `StateSpaceMixer`.  The embedding is a `BigramEmbedding` where the configuration
names a bigram table.  Tensor names: `embed`, `bigram`, `l<i>.norm1|norm2`, `l<i>.mix.<name>` (norm weights
`<name>.norm`, the convolution's bias `conv.b`), `l<i>.mlp.gate|up|down`, `final.norm`, `head`; matrices are stored
[out, in] under their bare names.
"""
from __future__ import annotations

from .. import registry
from ..config.sorupel import SorupelConfig
from ..parts import (BigramEmbedding, Embedding, GQAAttention, LatentAttention, LMHead, MixerOnly, Model, NoPositionEncoding,
                     PreNormBlock, RMSNorm, RotaryEmbedding, Run, StateSpaceMixer, SwiGLU)


def build_sorupel(cfg: SorupelConfig) -> Model:
    d = cfg.width
    if cfg.bigram is not None:
        b = cfg.bigram
        embed = BigramEmbedding(cfg.vocab, d, "embed", "bigram", b.buckets, b.mul_prev, b.mul_cur, suffix="")
    else:
        embed = Embedding(cfg.vocab, d, "embed", suffix="")
    layers, schedule, drop = [], [], []
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}", spec.mixer
        src = None
        if spec.type == "attention":
            pos = RotaryEmbedding(m.dim, m.rot_base, rotary_dim=m.rot_dims) if m.rot_dims else NoPositionEncoding()
            mixer = GQAAttention(d, m.heads, m.kv_heads, m.dim, pos, f"{p}.mix", scale=m.scale, proj_names=("q", "k", "v", "o"),
                                 softcap=m.softcap, qk_norm_eps=cfg.norm_eps, qk_norm_weights=("q.norm", "k.norm"),
                                 qk_norm_first=True, qk_norm_whole=True, values_from_keys=True, chunk=m.chunk, sink=0.0,
                                 gate="g", gate_per_head=True, weight_suffix="")
        elif spec.type == "latent_attention":
            src = m.kv_from
            mixer = LatentAttention(d, m.heads, m.dim, m.vdim, 0, m.kv_rank, cfg.norm_eps, f"{p}.mix", scale=m.scale,
                                    gate="element", rot_dim=m.rot_dim, rot_base=m.rot_base, sink="sink",
                                    share_kv=src is not None)
        else:
            mixer = StateSpaceMixer(d, m.heads, m.vdim, m.state, m.groups, m.norm_groups, m.conv, cfg.norm_eps, f"{p}.mix")
        norm1 = RMSNorm(d, cfg.norm_eps, f"{p}.norm1", suffix="")
        if spec.mlp is not None:
            ffn = SwiGLU(d, spec.mlp.ff, f"{p}.mlp", proj_names=("gate", "up", "down"), activation="gelu_tanh",
                         weight_suffix="")
            layers.append(PreNormBlock(mixer, ffn, norm1, RMSNorm(d, cfg.norm_eps, f"{p}.norm2", suffix="")))
        else:
            drop.append(f"{p}.norm2")                 # a layer without a feed-forward uses no second norm
            layers.append(MixerOnly(mixer, norm1))
        schedule.append(Run(i, cache_from=src))       # layers run once each, in order: layer j is schedule entry j
    head = LMHead(cfg.vocab, d, "head", suffix="")
    return Model(embed, layers, RMSNorm(d, cfg.norm_eps, "final.norm", suffix=""), head, schedule=schedule,
                 vocab_size=cfg.vocab, drop=drop)


registry.register(["sorupel", "Sorupel"], SorupelConfig.from_dict, build_sorupel, replace=True)
