"""Typed configuration of the Sorupel design, read from config.json.

A Sorupel model is a list of pre-norm layers (x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x))),
each with a mixer of its own kind and sizes:

* `attention`: grouped queries whose values are the keys as projected; q and k normalised over the
  whole projection; partial rotary positions; capped scores; a mask of chunks counted from position
  0; one more term of score 0 in the softmax's denominator; one gate value per head;
* `latent_attention`: a cached latent per token from which every head's keys and values are read,
  beside a rotated key part shared by the heads; a learned term per head in the denominator; a gate
  per output element; `kv_from` names an earlier layer whose cache the layer reads instead of
  projecting its own;
* `mamba2`: a state-space recurrence with a matrix of 32-bit state per head, a short causal
  convolution in front of it and a gated norm in groups behind it.

The feed-forward is dense and gated (tanh form of gelu) or absent.  The token embedding may have a
hashed bigram table added to it.  Every size and constant stands in config.json; what it does not
name does not exist (no mask: every earlier key is seen; no softcap: scores are not capped; no rot:
nothing is rotated).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ModelConfig


def _int(d: Mapping, key: str, where: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"sorupel: {where}.{key} must be an integer >= {low}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"sorupel: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


def _rot(d: Mapping, where: str, limit: int) -> tuple[int, float]:
    rot = d.get("rot") or {}
    dims = _int(rot, "dims", where + ".rot", 0) if rot else 0
    base = _float(rot, "base", where + ".rot") if dims else 1.0
    if dims % 2 or dims > limit:
        raise ConfigError(f"sorupel: {where}.rot.dims must be even and at most {limit}, got {dims}")
    if dims and base <= 0:
        raise ConfigError(f"sorupel: {where}.rot.base must be positive, got {base}")
    return dims, base


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                # 0: scores are not capped
    chunk: int                    # 0: every earlier token is seen
    rot_dims: int                 # 0: no rotation
    rot_base: float

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "ChunkedAttentionConfig":
        mask = d.get("mask") or {}
        dim = _int(d, "dim", where)
        rot_dims, rot_base = _rot(d, where, dim)
        c = ChunkedAttentionConfig(
            _int(d, "heads", where), _int(d, "kv_heads", where), dim, _int(d, "vdim", where) if d.get("vdim") is not None else dim,
            _float(d, "scale", where), _float(d, "softcap", where) if d.get("softcap") is not None else 0.0,
            _int(mask, "size", where + ".mask") if mask else 0, rot_dims, rot_base)
        if c.heads % c.kv_heads:
            raise ConfigError(f"sorupel: {where}: {c.heads} heads are no multiple of {c.kv_heads} kv_heads")
        if c.vdim != c.dim:
            raise ConfigError(f"sorupel: {where}: the values are the keys, so vdim must equal dim, got {c.vdim} and {c.dim}")
        if c.softcap < 0 or c.dim > 256:
            raise ConfigError(f"sorupel: {where}: softcap >= 0 and a head size up to 256")
        return c


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                      # unrotated query/key dimensions per head
    rot_dim: int                  # rotated ones: the key's are shared by the heads
    vdim: int
    kv_rank: int
    scale: float
    rot_base: float
    kv_from: int | None           # the layer whose cached latent and rotated key part this layer reads

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "LatentAttentionConfig":
        rot_dim = _int(d, "rot_dim", where, 0) if d.get("rot_dim") is not None else 0
        dims, base = _rot(d, where, max(rot_dim, 0))
        if dims != rot_dim:
            raise ConfigError(f"sorupel: {where}: the rotated part is rot_dim wide, so rot.dims must equal it, got "
                              f"{dims} and {rot_dim}")
        src = d.get("kv_from")
        c = LatentAttentionConfig(_int(d, "heads", where), _int(d, "dim", where), rot_dim, _int(d, "vdim", where),
                                  _int(d, "kv_rank", where), _float(d, "scale", where), base,
                                  None if src is None else _int(d, "kv_from", where, 0))
        if c.kv_rank + c.rot_dim > 512:
            raise ConfigError(f"sorupel: {where}: kv_rank + rot_dim up to 512, got {c.kv_rank + c.rot_dim}")
        return c


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    norm_groups: int
    conv: int                     # taps of the short convolution

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "StateSpaceConfig":
        c = StateSpaceConfig(_int(d, "heads", where), _int(d, "vdim", where), _int(d, "state", where),
                             _int(d, "groups", where), _int(d, "norm_groups", where), _int(d, "conv", where))
        if c.heads % c.groups:
            raise ConfigError(f"sorupel: {where}: {c.heads} heads are no multiple of {c.groups} groups")
        if (c.heads * c.vdim) % c.norm_groups:
            raise ConfigError(f"sorupel: {where}: {c.heads * c.vdim} inner channels are no multiple of {c.norm_groups} norm_groups")
        if c.conv > 16 or c.state > 1024:
            raise ConfigError(f"sorupel: {where}: at most 16 taps and a state of 1,024, got conv={c.conv}, state={c.state}")
        return c


@dataclass(frozen=True)
class GatedMlpConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class BigramConfig:
    buckets: int
    mul_prev: int
    mul_cur: int


@dataclass(frozen=True)
class LayerConfig:
    type: str                     # "attention" | "latent_attention" | "mamba2"
    mixer: ChunkedAttentionConfig | LatentAttentionConfig | StateSpaceConfig
    mlp: GatedMlpConfig | None


_MIXERS = {"attention": ChunkedAttentionConfig, "latent_attention": LatentAttentionConfig, "mamba2": StateSpaceConfig}


@dataclass(frozen=True)
class SorupelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    layers: tuple[LayerConfig, ...] = ()
    bigram: BigramConfig | None = None
    norm_eps: float = 0.0
    raw: tuple = ()               # the config.json items as read, for to_dict

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> int:
        return -1

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "SorupelConfig":
        layers = c.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("sorupel: `layers` must be a list with at least one layer")
        out = []
        for i, spec in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(spec, Mapping) or not isinstance(spec.get("mixer"), Mapping):
                raise ConfigError(f"sorupel: {where} must be an object with a `mixer`")
            kind = spec.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"sorupel: {where}.type must be one of {sorted(_MIXERS)}, got {kind!r}")
            mixer = _MIXERS[kind].from_dict(spec["mixer"], where + ".mixer")
            mlp = spec.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind", "dense") != "dense":
                    raise ConfigError(f"sorupel: {where}.mlp.kind must be 'dense', got {mlp!r}")
                mlp = GatedMlpConfig(_int(mlp, "ff", where + ".mlp"))
            out.append(LayerConfig(kind, mixer, mlp))
        for i, layer in enumerate(out):
            m = layer.mixer
            if layer.type != "latent_attention" or m.kv_from is None:
                continue
            where = f"layers[{i}].mixer"
            src = out[m.kv_from] if m.kv_from < i else None
            if src is None or src.type != "latent_attention" or src.mixer.kv_from is not None:
                raise ConfigError(f"sorupel: {where}.kv_from must name an earlier latent_attention layer with a cache of its own")
            s = src.mixer
            if (s.kv_rank, s.rot_dim, s.rot_base) != (m.kv_rank, m.rot_dim, m.rot_base):
                raise ConfigError(f"sorupel: {where}: kv_rank, rot_dim and the rotation must equal those of layer {m.kv_from}")
        norm = c.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("sorupel: `norm` must be an object with `eps`")
        eps = _float(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"sorupel: norm.eps must not be negative, got {eps}")
        bigram = (c.get("embedding") or {}).get("bigram") if isinstance(c.get("embedding"), Mapping) else None
        if bigram is not None:
            if not isinstance(bigram, Mapping):
                raise ConfigError("sorupel: embedding.bigram must be an object")
            bigram = BigramConfig(_int(bigram, "buckets", "embedding.bigram"), _int(bigram, "mul_prev", "embedding.bigram", 0),
                                  _int(bigram, "mul_cur", "embedding.bigram", 0))
        return SorupelConfig(vocab=_int(c, "vocab", "config"), width=_int(c, "width", "config"), layers=tuple(out),
                             bigram=bigram, norm_eps=eps, raw=tuple(sorted(c.items(), key=lambda kv: kv[0])))

    def to_dict(self) -> dict:
        return dict(self.raw)
