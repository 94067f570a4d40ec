"""Dense feed-forwards: gated (SwiGLU) and plain (one hidden layer and an activation)."""
from __future__ import annotations

import torch

from .base import FeedForward
from .linear import Linear


class SwiGLU(FeedForward):
    """down(act(gate(x)) * up(x)) with act = silu, silu(g) = g * sigmoid(g) in 32-bit (tamnd/fastmlx
    compute/models/llama.go:426-428, compute/models/qwen3_forward.go:229-239), or, with
    `activation="gelu_tanh"`, the tanh form of gelu.  gate and up run as one product whose output is [gate | up].
    The suffixes complete the tensors' names."""

    BLOCK = 128          # gate and up rows alternate in blocks of this many when the width allows

    def __init__(self, width: int, intermediate: int, name: str, bias: bool = False,
                 proj_names=("gate_proj", "up_proj", "down_proj"), activation: str = "silu",
                 weight_suffix: str = ".weight", bias_suffix: str = ".bias"):
        if activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"unknown gate activation {activation!r}")
        self.width, self.intermediate, self.activation = int(width), int(intermediate), activation
        g, u, d = (f"{name}.{p}" for p in proj_names)
        # In blocks, a 256-wide tile of the product holds 128 gates and their 128 ups: the
        # tensor-core kernel then applies the activation and the multiplication in its epilogue and the [T, 2I]
        # intermediate is never written.
        self.block = self.BLOCK if intermediate % self.BLOCK == 0 else 0
        self.gate_up = Linear(width, [(g, intermediate), (u, intermediate)], bias, interleave=self.block,
                              weight_suffix=weight_suffix, bias_suffix=bias_suffix)
        self.down = Linear(intermediate, [(d, width)], bias, weight_suffix=weight_suffix, bias_suffix=bias_suffix)

    def children(self):
        return (self.gate_up, self.down)

    def forward(self, x, ctx):
        k, w = self.rt.k, self.gate_up.weight
        fused = self.block and self.gate_up.bias is None and hasattr(k, "can_tc")
        if self.activation != "silu":
            epi = getattr(k, "EPI_GELU_MUL", None)
            if fused and epi is not None and k.can_tc(x, w, None, x.dtype, epi):
                act = k.gemm_tcgen05(x, w, ctx.status if ctx is not None else None, epilogue=epi)
            elif fused and epi is not None and self.block % 16 == 0 and k.can_gemv(x, w):
                act = k.gemv(x, w, block=self.block, act=self.activation)
            else:
                act = k.act_mul(self.gate_up.forward(x), self.activation, self.block or None)
            return self.down.forward(act)
        if fused and k.can_tc(x, w, None, x.dtype, k.EPI_SILU_MUL):
            # prompt portions: a 256-wide tile holds 128 gates and their ups, SiLU-mul in the epilogue
            act = k.gemm_tcgen05(x, w, ctx.status if ctx is not None else None, epilogue=k.EPI_SILU_MUL)
        elif fused and self.block % 16 == 0 and k.can_gemv(x, w):
            # decode steps: a block owns some gate rows and their up rows, SiLU-mul in its epilogue
            act = k.gemv(x, w, block=self.block)
        else:
            act = k.silu_mul(self.gate_up.forward(x), self.block or None)
        return self.down.forward(act)

    def emit(self, b, x):
        from ..engine.native import NotNative, OP_GATE_UP, _dt
        if self.activation != "silu":
            raise NotNative("the native executor's gate/up operation applies SiLU")
        act = b.reg(self.intermediate)
        both = b.reg(2 * self.intermediate)              # gate and up side by side, where no kernel fuses SiLU-mul in
        w = self.gate_up.weight
        b.op(OP_GATE_UP, in0=x, out0=act, out1=both, w=b.ptr(w), bias=b.ptr(self.gate_up.bias), w_dtype=_dt(w.dtype),
             ldw=w.stride(0), n=2 * self.intermediate, k=self.width, block=self.block, out_dtype=b.act)
        b.release(both)
        out = self.down.emit(b, act)
        b.release(act)
        return out


class DenseMLP(FeedForward):
    """down(act(up(x))) with act one of relu2 (the square of relu), gelu_tanh, silu, computed in
    32-bit.  `output=False` leaves the down projection to the block (`out_piece` names its tensor),
    which may join it with the mixer's output projection."""

    def __init__(self, width: int, intermediate: int, name: str, activation: str = "relu2", bias: bool = False,
                 proj_names=("up", "down"), output: bool = True, weight_suffix: str = ".weight",
                 bias_suffix: str = ".bias"):
        if activation not in ("relu2", "gelu_tanh", "silu"):
            raise ValueError(f"unknown activation {activation!r}")
        self.width, self.intermediate, self.activation = int(width), int(intermediate), activation
        u, d = (f"{name}.{p}" for p in proj_names)
        self.up = Linear(width, [(u, intermediate)], bias, weight_suffix=weight_suffix, bias_suffix=bias_suffix)
        self.inner_features = self.intermediate
        self.out_piece = (d + weight_suffix, self.intermediate, d + bias_suffix if bias else None)
        self.down = Linear(intermediate, [(d, width)], bias, weight_suffix=weight_suffix,
                           bias_suffix=bias_suffix) if output else None

    def children(self):
        return tuple(p for p in (self.up, self.down) if p is not None)

    def forward_inner(self, x, ctx, out=None):
        """The hidden layer after its activation, [T, intermediate]; into `out` where one is given."""
        k, w, b = self.rt.k, self.up.weight, self.up.bias
        if hasattr(k, "can_gemv") and k.can_gemv(x, w) and (out is None or out.dtype == torch.bfloat16):
            # decode steps: the activation in the product's epilogue
            return k.gemv(x, w, b, act=self.activation, out=out)
        if self.activation == "relu2" and b is None and hasattr(k, "can_tc") and k.can_tc(x, w, None, x.dtype, k.EPI_RELU2):
            # prompt portions: the same on the tensor-memory kernel
            return k.gemm_tcgen05(x, w, ctx.status if ctx is not None else None, epilogue=k.EPI_RELU2, out=out)
        return k.activation(self.up.forward(x), self.activation, out=out)

    def forward(self, x, ctx):
        return self.down.forward(self.forward_inner(x, ctx))
