"""The arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

import torch

from .base import FeedForward, Mixer, Norm, Part, WeightSpec, to_f32_vector
from .linear import JoinedLinear, Linear
from .norm import Pending


class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += ffn(norm2(h)) (tamnd/fastmlx compute/models/llama.go:402-429).
    The stream is carried as (delta, residual): each norm first adds the delta to the
    residual in 32-bit, then normalises the sum, so the add costs no pass of its own."""

    def __init__(self, mixer: Mixer, ffn: FeedForward, norm1: Norm, norm2: Norm):
        self.mixer, self.ffn, self.norm1, self.norm2 = mixer, ffn, norm1, norm2

    def children(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        delta, residual = self.mixer.forward_in_block(delta, residual, self.norm1, ctx, cache)
        return self.ffn.forward_in_block(delta, residual, self.norm2, ctx)

    def emit(self, b, delta, stream, pos):
        """Native program: (delta register, stream register or None) -> (delta', stream)."""
        x, stream = self.norm1.emit(b, delta, stream)
        y = self.mixer.emit(b, x, pos)
        b.release(x)
        x, stream = self.norm2.emit(b, y, stream)
        z = self.ffn.emit(b, x)
        b.release(x)
        return z, stream


class MixerOnly(PreNormBlock):
    """A pre-norm layer without a feed-forward: x <- x + mixer(norm1(x))."""

    def __init__(self, mixer, norm1):
        self.mixer, self.ffn, self.norm1, self.norm2 = mixer, None, norm1, None

    def children(self):
        return (self.norm1, self.mixer)

    def forward(self, delta, residual, ctx, cache):
        return self.mixer.forward_in_block(delta, residual, self.norm1, ctx, cache)


class ParallelBlock(Part):
    """h = norm(x); x <- x + (mixer(h) + ffn(h)): one norm, and both sublayers read its output.

    Mixer and feed-forward are built with `output=False`: their output projections are joined
    into one product over [mixer's heads | feed-forward's hidden layer], so that the two
    sublayers' outputs are added inside the product's 32-bit accumulators, and the block's
    output is rounded once before the 32-bit residual sum takes it.  `ffn` may be None."""

    def __init__(self, mixer: Mixer, ffn: FeedForward | None, norm: Norm, width: int):
        self.mixer, self.ffn, self.norm = mixer, ffn, norm
        pieces = [mixer.out_piece] + ([ffn.out_piece] if ffn is not None else [])
        self.out = JoinedLinear(width, pieces)

    def children(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn, self.out) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        h, residual = self.norm.forward(delta, residual)
        joined = torch.empty((h.shape[0], self.out.in_features), dtype=self.rt.dtype, device=h.device)
        m = self.mixer.inner_features
        self.mixer.forward_inner(h, ctx, cache, out=joined[:, :m] if self.ffn is not None else joined)
        if self.ffn is not None:
            self.ffn.forward_inner(h, ctx, out=joined[:, m:])
        return self.out.forward(joined), residual


class SandwichBlock(Part):
    """x <- x + r * norm1b(mixer(norm1(x))); x <- x + r * norm2b(ffn(norm2(x))): a norm in front of and behind each
    sublayer, and a multiplier r on what enters the stream.  `ffn` (with its two norms) may be None.

    The block hands its last sublayer's output on as a `Pending` sum, so that the norm behind a sublayer, the
    scaled sum into the 32-bit stream and the norm in front of the next sublayer are one kernel; its norms must
    take a `Pending` (`DynamicTanh` does)."""

    def __init__(self, mixer: Mixer, ffn: FeedForward | None, norm1: Norm, norm1b: Norm, norm2: Norm | None,
                 norm2b: Norm | None, mult: float = 1.0):
        self.mixer, self.ffn, self.mult = mixer, ffn, float(mult)
        self.norm1, self.norm1b, self.norm2, self.norm2b = norm1, norm1b, norm2, norm2b
        if ffn is not None and (norm2 is None or norm2b is None):
            raise ValueError("a feed-forward needs the norms around it")

    def children(self):
        parts = [self.norm1, self.mixer, self.norm1b]
        if self.ffn is not None:
            parts += [self.norm2, self.ffn, self.norm2b]
        return tuple(parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        h, residual = self.norm1.forward(delta, residual)
        pending = Pending(self.mixer.forward(h, ctx, cache), self.norm1b, self.mult)
        if self.ffn is None:
            return pending, residual
        h, residual = self.norm2.forward(pending, residual)
        return Pending(self.ffn.forward(h, ctx), self.norm2b, self.mult), residual


class PairMixer(Mixer):
    """Two mixers side by side on the same input: mixer(x) = (N_l(left(x)) + N_r(right(x))) / 2, each branch's output
    divided by its root mean square over the model width and multiplied by a plain weight of its own (`norm_names`:
    the two tensors, under `name`) before the two are averaged, in 32-bit.

    The branches' input projections run as one product over x (their matrices are stacked at bind time and each
    branch is handed its slice, in 32-bit); either branch may keep pages and either a state slot, which the layer's
    cache entry holds together.  A branch offers `forward_inner(x, ctx, cache, <projection>=slice)` and an output
    projection `o`; `left` takes its slice as `qkv` (a `GQAAttention`), `right` as `proj` (a `RetentionMixer`)."""

    def __init__(self, width: int, left: Mixer, right: Mixer, norm_eps: float, name: str,
                 norm_names=("left.out", "right.out"), weight_suffix: str = ""):
        self.width, self.left, self.right, self.eps = int(width), left, right, float(norm_eps)
        self.norm_tensors = tuple(f"{name}.{n}" for n in norm_names)
        if left.cache_spec() is not None and right.cache_spec() is not None:
            raise ValueError("at most one branch keeps pages")
        if left.state_spec() is not None and right.state_spec() is not None:
            raise ValueError("at most one branch keeps a state slot")
        # one product for both branches' projections; the branches give theirs up
        self.split = left.qkv.out_features
        self.proj = Linear(width, list(left.qkv.names) + list(right.proj.names), weight_suffix=weight_suffix)
        left.qkv = right.proj = None
        self.w_left = self.w_right = None

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.left, "supports_cuda_graph", False)) and bool(getattr(self.right, "supports_cuda_graph", False))

    def children(self):
        return (self.proj, self.left, self.right)

    def own_weight_specs(self):
        return [WeightSpec(n, (self.width,), "norm") for n in self.norm_tensors]

    def bind_own(self, tensors, rt):
        self.w_left, self.w_right = (to_f32_vector(tensors[n], rt) for n in self.norm_tensors)

    def weight_bytes(self):
        return super().weight_bytes() + 8 * self.width

    def cache_spec(self):
        return self.left.cache_spec() or self.right.cache_spec()

    def state_spec(self):
        return self.left.state_spec() or self.right.state_spec()

    def forward(self, x, ctx, cache):
        proj = self.proj.forward(x, out_dtype=torch.float32)
        a = self.left.forward_inner(x, ctx, cache, qkv=proj[:, :self.split])
        b = self.right.forward_inner(x, ctx, cache, proj=proj[:, self.split:])
        a = self.left.o.forward(a, out_dtype=torch.float32)
        b = self.right.o.forward(b, out_dtype=torch.float32)
        return self.rt.k.rmsnorm_pair_mean(a, b, self.w_left, self.w_right, self.eps, self.rt.dtype)
