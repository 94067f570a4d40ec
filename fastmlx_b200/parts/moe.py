"""A routed feed-forward: a router that chooses a few small experts per token, and an optional expert for all."""
from __future__ import annotations

import torch

from .base import FeedForward, Part, Runtime, WeightSpec, to_compute, to_f32_vector


class RoutedExperts(FeedForward):
    """y = sum over the token's chosen experts of s_e expert_e(x) (+ shared(x)).

    Router: logits z = W_r x and scores s = softmax(z) over all experts, in 32-bit; the experts form `groups`
    equal groups of neighbours, a group scores as its best member, and only experts of the `keep` best groups may
    be chosen; the `top` best of those are, with their scores as weights (not renormalised).

    Expert (no biases): g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1)).
    The shared expert has the same form with a width and a limit of its own and weight 1.

    Two ways to compute it, chosen once by size (`sparse`), neither of which loops on the host or makes a token's
    result depend on what else is in the batch, so that a decode step can be captured:

    * all experts side by side (small experts, and the 32-bit path): all gate and up matrices are stacked into one
      matrix and the down matrices laid side by side; a step runs the stacked product for every token, the activation
      kernel zeroes the columns of experts a token did not choose and scales the others by the token's weight, and one
      product with the down matrices gives the weighted sum inside the product's 32-bit accumulators.  It reads every
      expert's weights and multiplies experts / top times more than needed: right for experts as small as a tile of
      the product, wrong for large ones.
    * grouped products (bfloat16, large experts): the (token, expert) pairs are sorted expert by expert on the device,
      a tiled kernel multiplies each tile of pairs with its expert's gate and up rows and applies the activation and
      the pair's weight in its epilogue, a second one multiplies with the expert's down matrix, and a last kernel adds
      a token's pair outputs in the order of its choices to the shared expert's output, in 32-bit.  Only chosen experts'
      weights are read.

    Tensors, under `name`: router; e<i>.gate, e<i>.up, e<i>.down; shared.gate, shared.up, shared.down."""

    supports_cuda_graph = True

    def __init__(self, width: int, experts: int, top: int, ff: int, limit: float, name: str, groups: int = 1,
                 keep: int = 1, shared_ff: int = 0, shared_limit: float = 0.0, weight_suffix: str = "",
                 expert_prefix: str = "e", shared_name: str = "shared", router_name: str = "router",
                 proj_names=("gate", "up", "down"), sparse: bool | None = None):
        """`sparse`: grouped products (True), all experts side by side (False), or by size (None): grouped where the
        experts' matrices together pass SPARSE_MIN_BYTES and more than twice as many experts exist as a token uses."""
        self.width, self.E, self.top, self.ff, self.limit = int(width), int(experts), int(top), int(ff), float(limit)
        self.groups, self.keep = max(1, int(groups)), max(1, int(keep))
        if self.E % self.groups or not 0 < self.top <= self.E:
            raise ValueError(f"{experts} experts do not form {groups} equal groups, or top={top} is out of range")
        if self.top > (self.E // self.groups) * min(self.keep, self.groups):
            raise ValueError(f"top={top} experts cannot come from {keep} groups of {self.E // self.groups}")
        self.shared_ff, self.shared_limit = int(shared_ff), float(shared_limit)
        self.F = self.E * self.ff + self.shared_ff
        g, u, d = proj_names
        pre = [f"{name}.{expert_prefix}{i}" for i in range(self.E)] + ([f"{name}.{shared_name}"] if self.shared_ff else [])
        widths = [self.ff] * self.E + ([self.shared_ff] if self.shared_ff else [])
        self.gate_names = [(f"{p}.{g}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.up_names = [(f"{p}.{u}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.down_names = [(f"{p}.{d}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.router_name = f"{name}.{router_name}{weight_suffix}"
        self.want_sparse = sparse
        self.sparse = False

    def own_weight_specs(self):
        specs = [WeightSpec(self.router_name, (self.E, self.width), "matrix")]
        specs += [WeightSpec(n, (w, self.width), "matrix") for n, w in self.gate_names + self.up_names]
        specs += [WeightSpec(n, (self.width, w), "matrix") for n, w in self.down_names]
        return specs

    SPARSE_MIN_BYTES = 8 << 20

    def bind_own(self, tensors, rt: Runtime):
        self.router = to_compute(tensors[self.router_name], rt)
        mats = [to_compute(tensors[n], rt) for n, _ in self.gate_names + self.up_names + self.down_names]
        can = (rt.dtype == torch.bfloat16 and all(m.dtype == torch.bfloat16 for m in mats) and self.width % 8 == 0
               and self.ff % 8 == 0 and rt.device.type == "cuda" and hasattr(rt.k, "moe_sort"))
        big = 3 * self.E * self.ff * self.width * 2 >= self.SPARSE_MIN_BYTES and self.E > 2 * self.top
        self.sparse = can and (big if self.want_sparse is None else bool(self.want_sparse))
        n = len(self.gate_names)
        gates, ups, downs = mats[:n], mats[n:2 * n], mats[2 * n:]
        self.shared_gate_up = self.shared_down = None
        self.shared_block = 0
        if self.sparse and self.shared_ff:        # the shared expert is an ordinary gated feed-forward beside the routed ones
            g, u = gates.pop(), ups.pop()
            sb = int(getattr(rt.k, "GATE_UP_BLOCK", 0) or 0)
            if sb and self.shared_ff % sb == 0 and hasattr(rt.k, "expert_gate_up_tc"):
                # gate and up rows in blocks, as the tcgen05 product's epilogue takes them (the activation rides there)
                self.shared_block = sb
                self.shared_gate_up = torch.stack([g.view(-1, sb, self.width), u.view(-1, sb, self.width)], 1) \
                    .reshape(-1, self.width).contiguous()
            else:
                self.shared_gate_up = torch.cat([g, u], 0).contiguous()
            self.shared_down = downs.pop().contiguous()
        # grouped products of wide experts: expert after expert, gate and up rows in alternating blocks (a tile of the
        # tcgen05 product then holds gates and their ups), down matrices one under the other (rows of ff for its TMA)
        mb = int(getattr(rt.k, "MOE_BLOCK", 0) or 0)
        self.block = mb if self.sparse and mb and self.ff % mb == 0 else 0
        if self.block:
            b = self.block
            per = [torch.stack([g.view(-1, b, self.width), u.view(-1, b, self.width)], 1).reshape(-1, self.width)
                   for g, u in zip(gates, ups)]
            self.gate_up = torch.cat(per, 0).contiguous()
            self.down = torch.cat(downs, 0).contiguous()
        else:
            self.gate_up = torch.cat(gates + ups, 0).contiguous()
            self.down = torch.cat(downs, 1).contiguous()

    def weight_bytes(self):
        """Bytes a step reads when every expert is used (a decode step of a few tokens reads fewer with grouped products)."""
        return sum(t.numel() * t.element_size() for t in (self.router, self.gate_up, self.down, self.shared_gate_up,
                                                           self.shared_down) if t is not None)

    def active_weight_bytes(self, tokens: int) -> int:
        """Bytes of weights a step of `tokens` tokens reads at most: all with the experts side by side; with grouped
        products the router, the shared expert and at most tokens * top experts."""
        if not self.sparse:
            return self.weight_bytes()
        e = self.router.element_size()
        used = min(self.E, tokens * self.top)
        return e * (self.router.numel() + 3 * used * self.ff * self.width + 3 * self.shared_ff * self.width)

    def route(self, x):
        """-> the tokens' weights over the experts, 32-bit [T, E], zero where an expert is not chosen."""
        k = self.rt.k
        return k.moe_route(k.linear(x, self.router, None, torch.float32), self.top, self.groups, self.keep)

    def forward(self, x, ctx):
        k = self.rt.k
        if self.sparse:
            return self.forward_grouped(x)
        w = self.route(x)
        gu = k.linear(x, self.gate_up, None, self.rt.dtype)
        act = k.moe_expert_act(gu, w, self.E, self.ff, self.limit, self.shared_limit)
        return k.linear(act, self.down, None, self.rt.dtype)

    def forward_grouped(self, x):
        k, T = self.rt.k, x.shape[0]
        w, chosen = k.moe_route(k.linear(x, self.router, None, torch.float32), self.top, self.groups, self.keep, want_chosen=True)
        plan = k.moe_sort(chosen, w)
        y = k.moe_grouped_gate_up(x, plan, self.gate_up, self.E, self.ff, self.limit, self.block)
        pairs = k.moe_grouped_down(y, plan, self.down, self.E, self.ff, stacked=bool(self.block), tokens=T)
        shared = None
        if self.shared_gate_up is not None:
            if self.shared_block and k.can_expert_tc(x, self.shared_gate_up):
                act = k.expert_gate_up_tc(x, self.shared_gate_up, self.shared_limit)
            else:
                gu = k.linear(x, self.shared_gate_up, None, self.rt.dtype)
                none = torch.empty((T, 0), dtype=torch.float32, device=x.device)
                act = k.moe_expert_act(gu, none, 0, 8, 0.0, self.shared_limit, block=self.shared_block)
            shared = k.linear(act, self.shared_down, None, self.rt.dtype)
        return k.moe_combine(pairs, plan, shared, T, self.top, self.rt.dtype)


class PlainRoutedExperts(FeedForward):
    """y = sum over the token's chosen experts of w_e expert_e(x) (+ sigmoid(g . x) shared(x)), experts without a gate:
    expert(x) = W_down act(W_up x), act the square of relu (or gelu_tanh, silu), no biases.

    Router: logits z = W_r x and scores s = softmax(z) over all experts, in 32-bit.  The `top` experts with the largest
    s + correction are chosen (a vector of one number per expert that bears on the choice only; the lower index on a
    tie); a chosen expert weighs w_e = s_e * scale, not renormalised.  A shared expert of the same form and a width of
    its own runs for every token and is added times sigmoid(g . x), one number per token.

    All experts run side by side: the up matrices are stacked into one matrix and the down matrices laid side by side;
    the activation kernel zeroes the columns of experts a token did not choose and multiplies the others by the token's
    weight (the shared columns by the token's gate), and one product with the down matrices gives the weighted sum inside
    the product's 32-bit accumulators.  The router's matrix and the shared gate's vector are stacked too, so that one
    32-bit product gives a token's logits and its gate.  Nothing loops on the host and no token's result depends on what
    else is in the batch, so a decode step can be captured.

    Tensors, under `name`: router, correction; e<i>.up, e<i>.down; shared.up, shared.down, shared.sg."""

    supports_cuda_graph = True

    def __init__(self, width: int, experts: int, top: int, ff: int, name: str, scale: float = 1.0, shared_ff: int = 0,
                 activation: str = "relu2", correction: str | None = "correction", shared_gate: str | None = "sg",
                 weight_suffix: str = "", expert_prefix: str = "e", shared_name: str = "shared", router_name: str = "router",
                 proj_names=("up", "down")):
        if activation not in ("relu2", "gelu_tanh", "silu"):
            raise ValueError(f"unknown activation {activation!r}")
        if not 0 < top <= experts:
            raise ValueError(f"top={top} of {experts} experts")
        self.width, self.E, self.top, self.ff, self.scale = int(width), int(experts), int(top), int(ff), float(scale)
        self.shared_ff, self.activation = int(shared_ff), activation
        self.F = self.E * self.ff + self.shared_ff
        u, d = proj_names
        pre = [f"{name}.{expert_prefix}{i}" for i in range(self.E)] + ([f"{name}.{shared_name}"] if self.shared_ff else [])
        widths = [self.ff] * self.E + ([self.shared_ff] if self.shared_ff else [])
        self.up_names = [(f"{p}.{u}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.down_names = [(f"{p}.{d}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.router_name = f"{name}.{router_name}{weight_suffix}"
        self.correction_name = f"{name}.{correction}" if correction else None
        self.gate_name = f"{name}.{shared_name}.{shared_gate}{weight_suffix}" if self.shared_ff and shared_gate else None

    def own_weight_specs(self):
        specs = [WeightSpec(self.router_name, (self.E, self.width), "matrix")]
        if self.correction_name:
            specs.append(WeightSpec(self.correction_name, (self.E,), "bias"))
        specs += [WeightSpec(n, (w, self.width), "matrix") for n, w in self.up_names]
        specs += [WeightSpec(n, (self.width, w), "matrix") for n, w in self.down_names]
        if self.gate_name:
            specs.append(WeightSpec(self.gate_name, (1, self.width), "matrix"))
        return specs

    def bind_own(self, tensors, rt: Runtime):
        rows = [to_compute(tensors[self.router_name], rt)]
        if self.gate_name:
            rows.append(to_compute(tensors[self.gate_name], rt).reshape(1, self.width))
        if len({r.dtype for r in rows}) > 1:
            rows = [r.float() for r in rows]
        self.router = torch.cat(rows, 0).contiguous()             # [E (+1), width]: the experts' logits, then the shared gate's
        self.correction = to_f32_vector(tensors[self.correction_name], rt) if self.correction_name else None
        ups = [to_compute(tensors[n], rt) for n, _ in self.up_names]
        downs = [to_compute(tensors[n], rt) for n, _ in self.down_names]
        if len({m.dtype for m in ups + downs}) > 1:
            ups, downs = [m.float() for m in ups], [m.float() for m in downs]
        self.up = torch.cat(ups, 0).contiguous()                  # [F, width]
        self.down = torch.cat(downs, 1).contiguous()              # [width, F]

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.router, self.up, self.down))

    def forward(self, x, ctx):
        k = self.rt.k
        z = k.linear(x, self.router, None, torch.float32)
        w = k.moe_route(z, self.top, experts=self.E, correction=self.correction, scale=self.scale)
        hidden = k.linear(x, self.up, None, self.rt.dtype)
        act = k.moe_plain_act(hidden, w, self.E, self.ff, self.activation, shared_gate=z[:, self.E:] if self.gate_name else None)
        return k.linear(act, self.down, None, self.rt.dtype)
