"""Retention: linear attention with one fixed decay per head, as a mixer."""
from __future__ import annotations

import torch

from .base import Mixer, Runtime, StateSpec
from .linear import Linear
from .rope import inverse_frequencies


class RetentionMixer(Mixer):
    """q = W_q x and k = W_k x (heads x dim), v = W_v x (heads x vdim), no biases; q and k are rotated over their first
    `rot_dims` dimensions (dimension i paired with i + rot_dims/2, angle position * base^(-2i/rot_dims), optionally with
    the frequency bands rescaled), k is multiplied by dim^-1/2 after the rotation.  Per head h, with S [dim, vdim] carried
    from token to token in 32-bit and starting at zero,

        S <- decay_h S + k v^T;   o = S^T q

    with one fixed decay per head and neither a softmax nor a denominator.  Each head's o is divided by its root mean
    square (no weight), the heads side by side are multiplied by silu(W_g x), and go through the output projection.

    The recurrence is the state-space scan (`ssm_scan`) with a step size of 1, as many groups as heads and no skip
    term; per request the part keeps S^T of every head ([heads, vdim, dim]) in one state slot of 32-bit floats.
    Everything between the projections and the gated read-out is 32-bit.  `names`: the tensors of (q, k, v, g, o).
    `output=False` leaves the output projection out (`o` is None)."""

    supports_cuda_graph = True

    def __init__(self, width: int, heads: int, dim: int, vdim: int, decay, norm_eps: float, name: str, rot_dims: int = 0,
                 rot_base: float = 10000.0, rot_scaling=None, names=("q", "k", "v", "g", "o"), weight_suffix: str = ""):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if dim > 1024:
            raise ValueError(f"the recurrence keeps up to 1,024 rows of state per column, not {dim}")
        if rot_dims % 2 or not 0 <= rot_dims <= dim:
            raise ValueError(f"rot_dims {rot_dims} must be even and at most dim {dim}")
        self.H, self.D, self.P, self.eps = int(heads), int(dim), int(vdim), float(norm_eps)
        self.decay_values = tuple(float(d) for d in decay)
        self.rot_dims, self.rot_base, self.rot_scaling = int(rot_dims), float(rot_base), rot_scaling
        self.inner = self.H * self.P
        q, k, v, g, o = (f"{name}.{n}" for n in names)
        # one product: q | k | v | g
        self.proj = Linear(width, [(q, self.H * self.D), (k, self.H * self.D), (v, self.inner), (g, self.inner)],
                           weight_suffix=weight_suffix)
        self.proj_features = 2 * self.H * self.D + 2 * self.inner
        self.o = Linear(self.inner, [(o, width)], weight_suffix=weight_suffix)
        self.s_floats = self.H * self.P * self.D
        self.decay = self.inv_freq = self.no_skip = None

    def children(self):
        return tuple(p for p in (self.proj, self.o) if p is not None)

    def bind_own(self, tensors, rt: Runtime):
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=rt.device)
        self.no_skip = torch.zeros(self.H, dtype=torch.float32, device=rt.device)
        self.inv_freq = None
        if self.rot_dims:
            self.inv_freq = inverse_frequencies(self.rot_dims, self.rot_base, self.rot_scaling) \
                .to(torch.float32).to(rt.device).contiguous()

    def weight_bytes(self):
        return super().weight_bytes() + 8 * self.H

    def state_spec(self):
        # a multiple of four floats, so that every slot starts on 16 bytes
        return StateSpec((-(-self.s_floats // 4) * 4,), torch.float32)

    def forward(self, x, ctx, cache, out_dtype=None):
        return self.o.forward(self.forward_inner(x, ctx, cache), out_dtype=out_dtype)

    def forward_inner(self, x, ctx, cache, proj=None):
        """The gated read-out, [T, heads * vdim], in front of the output projection.  `proj`: the part's projection
        q | k | v | g where the caller has computed it already (a slice of a product shared with another part)."""
        k = self.rt.k
        if proj is None:
            proj = self.proj.forward(x, out_dtype=torch.float32)
        qkv, dd = k.retention_prepare(proj, ctx.positions, self.inv_freq, self.decay, self.H, self.D, self.P, self.rot_dims,
                                      self.D ** -0.5)
        o = k.ssm_scan(qkv, dd, self.no_skip, ctx, cache.state, self.H, self.H, self.D, self.P)
        gate = proj[:, 2 * self.H * self.D + self.inner:self.proj_features]
        return k.retention_gate_norm(o, gate, self.eps, self.H, self.P, self.rt.dtype)
