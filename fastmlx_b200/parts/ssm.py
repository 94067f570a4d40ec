"""A state-space recurrence with a matrix of state per head (the scalar-decay form), as a mixer."""
from __future__ import annotations

import torch

from .base import Mixer, Runtime, StateSpec, WeightSpec, to_f32_vector
from .linear import Linear


class StateSpaceMixer(Mixer):
    """One input projection laid out as [z: inner | x: inner | B: groups*N | C: groups*N | dt: heads], inner =
    heads * vdim.  x, B and C pass a causal convolution per channel (`taps` taps with a bias, the last tap the current
    token's, zeros before the start) and SiLU.  Per head h (reading B and C of group h // (heads / groups)), with
    S [N, vdim] carried from token to token in 32-bit and starting at zero,

        dt = softplus(dt + dt_bias);   S <- exp(-exp(A_log) dt) S + dt B x^T;   y = S^T C + D x

    then y (heads side by side) is multiplied by SiLU(z), divided by its root mean square in `norm_groups` equal
    parts of the row (each part by its own), multiplied by a weight, and goes through the output projection.

    Per request the part keeps, in one state slot of 32-bit floats, S^T of every head ([heads, vdim, N]) and the
    last taps-1 inputs of the convolution; a step runs each request's tokens in order from what the steps before
    left there.  Everything behind the convolution's activation is 32-bit: step sizes, decays, the recurrence,
    the gate and the norm.  `names`: the tensors of (in, conv, conv bias, dt_bias, A_log, D, norm, o)."""

    supports_cuda_graph = True

    def __init__(self, width: int, heads: int, vdim: int, state: int, groups: int, norm_groups: int, taps: int,
                 norm_eps: float, name: str, names=("in", "conv", "conv.b", "dt_bias", "A_log", "D", "norm", "o"),
                 weight_suffix: str = ""):
        if heads % groups:
            raise ValueError(f"{heads} heads are no multiple of {groups} groups")
        if (heads * vdim) % norm_groups:
            raise ValueError(f"{heads * vdim} channels are no multiple of {norm_groups} parts")
        if not 1 <= taps <= 16:
            raise ValueError(f"a short convolution has 1 to 16 taps, not {taps}")
        if state > 1024:
            raise ValueError(f"the recurrence keeps up to 1,024 rows of state per column, not {state}")
        self.H, self.P, self.N, self.G = int(heads), int(vdim), int(state), int(groups)
        self.norm_groups, self.taps, self.eps = int(norm_groups), int(taps), float(norm_eps)
        self.inner = self.H * self.P
        self.channels = self.inner + 2 * self.G * self.N           # what the convolution runs over
        w_in, conv, conv_b, dtb, alog, d, norm, o = (f"{name}.{n}" for n in names)
        self.proj = Linear(width, [(w_in, 2 * self.inner + 2 * self.G * self.N + self.H)], weight_suffix=weight_suffix)
        self.conv_name, self.conv_bias_name = conv, conv_b
        self.vec_names = (dtb, alog, d)
        self.norm_name = norm
        self.o = Linear(self.inner, [(o, width)], weight_suffix=weight_suffix)
        self.s_floats = self.H * self.P * self.N

    def children(self):
        return (self.proj, self.o)

    def own_weight_specs(self):
        dtb, alog, d = self.vec_names
        return [WeightSpec(self.conv_name, (self.channels, self.taps), "conv"),
                WeightSpec(self.conv_bias_name, (self.channels,), "bias"),
                WeightSpec(dtb, (self.H,), "rate_bias"), WeightSpec(alog, (self.H,), "log_rate"),
                WeightSpec(d, (self.H,), "norm"), WeightSpec(self.norm_name, (self.inner,), "norm")]

    def bind_own(self, tensors, rt: Runtime):
        self.conv_w = to_f32_vector(tensors[self.conv_name], rt)
        self.conv_b = to_f32_vector(tensors[self.conv_bias_name], rt)
        self.dt_bias, self.a_log, self.d_skip = (to_f32_vector(tensors[n], rt) for n in self.vec_names)
        self.norm_w = to_f32_vector(tensors[self.norm_name], rt)

    def weight_bytes(self):
        return super().weight_bytes() + 4 * (self.conv_w.numel() + self.conv_b.numel() + 3 * self.H + self.inner)

    def state_spec(self):
        # a multiple of four floats, so that every slot starts on 16 bytes
        n = self.s_floats + (self.taps - 1) * self.channels
        return StateSpec((-(-n // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache):
        k = self.rt.k
        proj = self.proj.forward(x)
        # convolution, SiLU, step sizes and decays: x | B | C in 32-bit, (dt | decay) per head
        xbc, dd = k.ssm_prepare(proj, self.conv_w, self.conv_b, self.a_log, self.dt_bias, ctx, cache.state, self.s_floats,
                                self.H, self.G, self.N, self.P, self.taps)
        y = k.ssm_scan(xbc, dd, self.d_skip, ctx, cache.state, self.H, self.G, self.N, self.P)
        y = k.gated_group_rmsnorm(y, proj[:, :self.inner], self.norm_w, self.eps, self.norm_groups, self.rt.dtype)
        return self.o.forward(y)
