"""Token embedding and output head."""
from __future__ import annotations

import torch

from .base import Part, Runtime, StateSpec, WeightSpec, to_compute


class Embedding(Part):
    """h[t] = E[id_t], no scaling (tamnd/fastmlx compute/models/llama.go:385-390); or, with `scale` s != 1,
    h[t] = s E[id_t], multiplied in 32-bit: the product is then the 32-bit stream's first value (`starts_stream`)."""

    starts_stream = False

    def __init__(self, vocab: int, width: int, name: str, suffix: str = ".weight", scale: float = 1.0):
        self.vocab, self.width, self.name = int(vocab), int(width), name
        self.tensor = name + suffix
        self.scale = float(scale)
        if self.scale != 1.0:
            self.starts_stream = True
        self.weight = None

    def own_weight_specs(self):
        return [WeightSpec(self.tensor, (self.vocab, self.width), "embedding")]

    def bind_own(self, tensors, rt: Runtime):
        self.weight = to_compute(tensors[self.tensor], rt)

    def weight_bytes(self):
        return 0          # a step reads T rows, not the table

    def state_spec(self):
        """Per-request state of the embedding itself (none here); a part that has some gets a state slot from the
        cache manager and is called with it, `forward(ids, ctx, cache)`."""
        return None

    def forward(self, ids, ctx, cache=None):
        if self.scale != 1.0:
            return self.rt.k.embed_scaled(ids, self.weight, self.scale, ctx.status)
        if self.weight.dtype != self.rt.dtype:          # a table stored in 32-bit under bfloat16 activations
            return self.rt.k.embedding(ids, self.weight, ctx.status, self.rt.dtype)
        return self.rt.k.embedding(ids, self.weight, ctx.status)


    def emit(self, b) -> int:
        from ..engine.native import NotNative, OP_EMBED, _dt
        if self.scale != 1.0:
            raise NotNative("a scaled embedding runs in Python only")
        out = b.reg(self.width)
        b.op(OP_EMBED, out0=out, w=b.ptr(self.weight), w_dtype=_dt(self.weight.dtype), n=self.width, table_rows=self.vocab)
        return out


class BigramEmbedding(Embedding):
    """h[t] = E[id_t] + B[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets]: a second table addressed by a hash
    of the token and the one before it; a sequence's first token takes the table's last row (row `buckets`).

    The token before a step's first one is part of the request's state: one integer per request slot, read by
    the first token of each row of the step and replaced by the row's last token.  The two rows are summed in
    32-bit and the sum is the stream's first value, so beside bfloat16 activations the part hands on a 32-bit
    stream (`starts_stream`)."""

    starts_stream = True
    supports_cuda_graph = True

    def __init__(self, vocab: int, width: int, name: str, bigram: str, buckets: int, mul_prev: int, mul_cur: int,
                 suffix: str = ".weight"):
        super().__init__(vocab, width, name, suffix)
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.bigram_tensor = bigram + suffix
        self.bigram = None

    def own_weight_specs(self):
        return super().own_weight_specs() + [WeightSpec(self.bigram_tensor, (self.buckets + 1, self.width), "embedding")]

    def bind_own(self, tensors, rt: Runtime):
        super().bind_own(tensors, rt)
        self.bigram = to_compute(tensors[self.bigram_tensor], rt)

    def state_spec(self):
        return StateSpec((1,), torch.int32)

    def forward(self, ids, ctx, cache=None):
        return self.rt.k.embed_bigram(ids, self.weight, self.bigram, ctx, cache.state, self.buckets, self.mul_prev,
                                      self.mul_cur)


class LMHead(Part):
    """logits = x W^T in 32-bit, no bias, cap or scale; W is the embedding table when the
    model ties them (tamnd/fastmlx compute/models/llama.go:433-437).  Only the rows whose
    logits are wanted reach it."""

    def __init__(self, vocab: int, width: int, name: str | None, tied: Embedding | None = None,
                 suffix: str = ".weight", scale: float = 1.0):
        """`scale`: a constant the logits are multiplied by (in 32-bit, after the product)."""
        if (name is None) == (tied is None):
            raise ValueError("LMHead takes either a tensor name or an embedding to tie to")
        self.vocab, self.width, self.name, self.tied = int(vocab), int(width), name, tied
        self.tensor = None if name is None else name + suffix
        self.scale = float(scale)
        self.weight = None

    def own_weight_specs(self):
        return [] if self.tied is not None else [WeightSpec(self.tensor, (self.vocab, self.width), "matrix")]

    def bind_own(self, tensors, rt: Runtime):
        if self.tied is None:
            self.weight = to_compute(tensors[self.tensor], rt)

    def weight_bytes(self):
        w = self.tied.weight if self.tied is not None else self.weight
        return w.numel() * w.element_size()

    def forward(self, x):
        w = self.tied.weight if self.tied is not None else self.weight
        logits = self.rt.k.linear(x, w, None, torch.float32)
        if self.scale != 1.0:
            logits.mul_(self.scale)
        return logits

    def forward_after(self, delta, residual, norm, greedy: bool = False):
        """Final norm, then logits; `greedy`: the index of each row's largest logit instead
        (int32), chosen inside the head's product where its kernel can (no logits written)."""
        x, _ = norm.forward(delta, residual)
        if not greedy:
            return self.forward(x)
        k = self.rt.k
        w = self.tied.weight if self.tied is not None else self.weight
        if self.scale > 0 and hasattr(k, "can_greedy_head") and k.can_greedy_head(x, w):
            return k.greedy_head(x, w)                # a positive scale does not change the choice
        return k.argmax(self.forward(x))

    def emit_after(self, b, delta, stream, norm) -> None:
        """Native program: final norm, then the step's logits."""
        from ..engine.native import F32, LOGITS, NotNative, OP_LINEAR, _dt
        if self.scale != 1.0:
            raise NotNative("the native executor's head does not scale its logits")
        x, _ = norm.emit(b, delta, stream)
        w = self.tied.weight if self.tied is not None else self.weight
        b.op(OP_LINEAR, in0=x, out0=LOGITS, w=b.ptr(w), w_dtype=_dt(w.dtype), ldw=w.stride(0), n=self.vocab, k=self.width,
             out_dtype=F32)
        # the greedy choice inside the product takes bfloat16 operands in 16-byte rows
        b.greedy_head_ok = bool(w.dtype == torch.bfloat16 and b.act == _dt(torch.bfloat16) and self.width % 8 == 0
                                and w.stride(0) % 8 == 0 and w.data_ptr() % 16 == 0)
