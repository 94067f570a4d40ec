"""Typed configuration of the Kafepel design, read from config.json.

A Kafepel model is a list of pre-norm layers (x <- x + mixer(norm1(x)), then x <- x + ff(norm2(x))).  The mixer
of a `parallel` layer runs two branches on the same input and returns half the sum of their RMS-normed outputs:

* `left`: grouped-query attention without a softmax: q and k normalised over the whole projection, rotary
  positions (optionally with the frequency bands rescaled), scaled and capped scores, a visible key's weight
  sigmoid(score + a number per head), and the heads' weights mixed by a square matrix before they meet the values;
* `right`: a retention: per head a matrix of 32-bit state with one fixed decay, S <- decay S + k v^T, o = S^T q,
  the read-out divided by its root mean square and gated.

The feed-forward is dense and gated (SiLU), a routed mixture of small squared-relu experts with an optional
gated shared expert, or absent.  The embedding is multiplied by a constant.  Every size and constant stands in
config.json; what it does not name does not exist (no softcap: scores are not capped; no rot: nothing is rotated;
no scaling: the frequencies stand as they are; no shared: no shared expert).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping

from .base import ConfigError, ModelConfig
from .llama import RopeScaling


def _int(d: Mapping, key: str, where: str, low: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v or int(v) < low:
        raise ConfigError(f"kafepel: {where}.{key} must be an integer >= {low}, got {v!r}")
    return int(v)


def _float(d: Mapping, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"kafepel: {where}.{key} must be a finite number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotaryConfig:
    dims: int                     # 0: no rotation
    base: float
    scaling: RopeScaling | None   # the frequency-band rescaling, or None

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str, limit: int) -> "RotaryConfig":
        rot = d.get("rot") or {}
        if not isinstance(rot, Mapping):
            raise ConfigError(f"kafepel: {where}.rot must be an object")
        dims = _int(rot, "dims", where + ".rot", 0) if rot else 0
        if dims % 2 or dims > limit:
            raise ConfigError(f"kafepel: {where}.rot.dims must be even and at most {limit}, got {dims}")
        if not dims:
            return RotaryConfig(0, 1.0, None)
        base = _float(rot, "base", where + ".rot")
        if base <= 0:
            raise ConfigError(f"kafepel: {where}.rot.base must be positive, got {base}")
        sc = rot.get("scaling")
        scaling = None
        if sc is not None:
            if not isinstance(sc, Mapping):
                raise ConfigError(f"kafepel: {where}.rot.scaling must be an object")
            w = where + ".rot.scaling"
            scaling = RopeScaling("llama3", _float(sc, "factor", w), _float(sc, "low", w), _float(sc, "high", w),
                                  _int(sc, "original", w))
            if scaling.factor <= 0 or scaling.low_freq_factor <= 0 or scaling.high_freq_factor <= 0:
                raise ConfigError(f"kafepel: {w}: factor, low and high must be positive")
        return RotaryConfig(dims, base, scaling)


@dataclass(frozen=True)
class SigmoidAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float                # 0: scores are not capped
    rot: RotaryConfig

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "SigmoidAttentionConfig":
        dim = _int(d, "dim", where)
        c = SigmoidAttentionConfig(
            _int(d, "heads", where), _int(d, "kv_heads", where), dim, _int(d, "vdim", where) if d.get("vdim") is not None else dim,
            _float(d, "scale", where), _float(d, "softcap", where) if d.get("softcap") is not None else 0.0,
            RotaryConfig.from_dict(d, where, dim))
        if c.heads % c.kv_heads:
            raise ConfigError(f"kafepel: {where}: {c.heads} heads are no multiple of {c.kv_heads} kv_heads")
        if c.softcap < 0 or c.dim > 256 or c.vdim > 512:
            raise ConfigError(f"kafepel: {where}: softcap >= 0, keys up to 256 and values up to 512 wide")
        return c


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]      # one per head
    rot: RotaryConfig

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "RetentionConfig":
        heads, dim = _int(d, "heads", where), _int(d, "dim", where)
        decay = d.get("decay")
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"kafepel: {where}.decay must list one decay per head ({heads})")
        vals = []
        for v in decay:
            if isinstance(v, bool) or not isinstance(v, (int, float)) or not 0.0 <= float(v) <= 1.0:
                raise ConfigError(f"kafepel: {where}.decay holds numbers between 0 and 1, got {v!r}")
            vals.append(float(v))
        c = RetentionConfig(heads, dim, _int(d, "vdim", where) if d.get("vdim") is not None else dim, tuple(vals),
                            RotaryConfig.from_dict(d, where, dim))
        if c.dim > 1024:
            raise ConfigError(f"kafepel: {where}: the recurrence keeps up to 1,024 rows of state per column, got dim={c.dim}")
        return c


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SigmoidAttentionConfig
    right: RetentionConfig

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "ParallelMixerConfig":
        for side in ("left", "right"):
            if not isinstance(d.get(side), Mapping):
                raise ConfigError(f"kafepel: {where}.{side} must be an object")
        return ParallelMixerConfig(SigmoidAttentionConfig.from_dict(d["left"], where + ".left"),
                                   RetentionConfig.from_dict(d["right"], where + ".right"))


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"


@dataclass(frozen=True)
class MoeMlpConfig:
    experts: int
    top: int
    router_scale: float
    ff: int
    shared_ff: int                # 0: no shared expert
    kind: str = "moe"

    @staticmethod
    def from_dict(d: Mapping[str, Any], where: str) -> "MoeMlpConfig":
        router, expert, shared = d.get("router"), d.get("expert"), d.get("shared")
        if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
            raise ConfigError(f"kafepel: {where} needs `router` and `expert` objects")
        if shared is not None and not isinstance(shared, Mapping):
            raise ConfigError(f"kafepel: {where}.shared must be an object or null")
        c = MoeMlpConfig(_int(router, "experts", where + ".router"), _int(router, "top", where + ".router"),
                         _float(router, "scale", where + ".router") if router.get("scale") is not None else 1.0,
                         _int(expert, "ff", where + ".expert"), _int(shared, "ff", where + ".shared") if shared else 0)
        if c.top > c.experts:
            raise ConfigError(f"kafepel: {where}: top={c.top} of {c.experts} experts")
        return c


@dataclass(frozen=True)
class LayerConfig:
    type: str                     # "parallel"
    mixer: ParallelMixerConfig
    mlp: DenseMlpConfig | MoeMlpConfig | None


_MIXERS = {"parallel": ParallelMixerConfig}


@dataclass(frozen=True)
class KafepelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    layers: tuple[LayerConfig, ...] = ()
    embedding_scale: float = 1.0
    norm_eps: float = 0.0
    raw: tuple = ()               # the config.json items as read, for to_dict

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def eos_token_id(self) -> int:
        return -1

    @staticmethod
    def from_dict(c: Mapping[str, Any]) -> "KafepelConfig":
        layers = c.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("kafepel: `layers` must be a list with at least one layer")
        out = []
        for i, spec in enumerate(layers):
            where = f"layers[{i}]"
            if not isinstance(spec, Mapping) or not isinstance(spec.get("mixer"), Mapping):
                raise ConfigError(f"kafepel: {where} must be an object with a `mixer`")
            kind = spec.get("type")
            if kind not in _MIXERS:
                raise ConfigError(f"kafepel: {where}.type must be one of {sorted(_MIXERS)}, got {kind!r}")
            mixer = _MIXERS[kind].from_dict(spec["mixer"], where + ".mixer")
            mlp = spec.get("mlp")
            if mlp is not None:
                if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"kafepel: {where}.mlp.kind must be 'dense' or 'moe', got {mlp!r}")
                mlp = DenseMlpConfig(_int(mlp, "ff", where + ".mlp")) if mlp["kind"] == "dense" \
                    else MoeMlpConfig.from_dict(mlp, where + ".mlp")
            out.append(LayerConfig(kind, mixer, mlp))
        norm = c.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError("kafepel: `norm` must be an object with `eps`")
        eps = _float(norm, "eps", "norm")
        if eps < 0:
            raise ConfigError(f"kafepel: norm.eps must not be negative, got {eps}")
        emb = c.get("embedding")
        scale = 1.0
        if emb is not None:
            if not isinstance(emb, Mapping):
                raise ConfigError("kafepel: `embedding` must be an object")
            if emb.get("scale") is not None:
                scale = _float(emb, "scale", "embedding")
        return KafepelConfig(vocab=_int(c, "vocab", "config"), width=_int(c, "width", "config"), layers=tuple(out),
                             embedding_scale=scale, norm_eps=eps, raw=tuple(sorted(c.items(), key=lambda kv: kv[0])))

    def to_dict(self) -> dict:
        return dict(self.raw)
