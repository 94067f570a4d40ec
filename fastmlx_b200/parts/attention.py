"""Grouped-query attention over a paged cache."""
from __future__ import annotations

import torch

from .base import Mixer, PagedKVSpec, PositionEncoding, Runtime, WeightSpec, to_f32_vector
from .linear import Linear


class GQAAttention(Mixer):
    """softmax(scale * q k^T + causal mask) v with nh query heads sharing nkv key/value
    heads: query head h reads kv head h // (nh / nkv) (tamnd/fastmlx
    compute/models/llama.go:403-422; the grouping happens inside its fused call,
    mlxgo/binding_cgo.go:619-634).  Every query token sees the keys of its own request at
    positions <= its own (compute/models/batch_mask.go:33-41), or only the last `window`.

    The step writes this step's k and v into the pages first and then attends from the
    pages alone, so a token's result does not depend on how the tokens were cut into steps.
    With `share_kv=True` the part has no k/v projections and reads the cache of the
    schedule entry it is pointed at.

    Three further choices put a layer on the route with 32-bit scores and weights (`qk_prepare`
    and `paged_attention_general`): `softcap` c > 0 caps the scaled scores, s <- c tanh(s / c);
    `qk_norm_eps` divides q and k, after their rotation, by their root mean square over the head
    (no weight); `v_head_dim` gives values another width than keys.  There the queries stay in
    32-bit from the rotation to the scores.  `output=False` leaves the output projection to the
    block (`out_piece` names its tensors), which may join it with the feed-forward's.

    Further choices of that route.  `qk_norm_weights` = (name, name): the normalised q and k heads are multiplied
    by a weight of head_dim values each, shared by the heads; `qk_norm_first`: q and k are normalised before the
    rotation instead of after it.  `keep_first` k > 0 beside a window: a request's first k tokens stay visible to
    every later query, at their true positions (the cache keeps their pages).  `gate` = a projection's name: the
    heads' outputs are multiplied element by element with sigmoid(W_g x), W_g of the output's width, before the
    output projection; it rides in the q/k/v product.  `late_bias`: the q/k/v product leaves in 32-bit and the
    biases are added, in 32-bit, by the kernel that normalises and rotates (a gate has no bias).

    And these.  `values_from_keys`: there is no value projection; a token's values are its keys as projected, before
    norm and rotation (values as wide as keys).  `qk_norm_whole` (with `qk_norm_first` and weights): q and k are
    divided by the root mean square of the whole projection, all heads at once, and the weights have the
    projection's width.  `chunk` c > 0 (instead of a window): position i sees j <= i only where i // c == j // c,
    runs counted from position 0 of the request whatever the cut of its prompt; the cache gives earlier runs' pages
    back.  `sink` s: the softmax's denominator has one more term exp(s) that has no value (s = 0 adds one).
    `gate_per_head`: the gate has one value per head, not one per output element.

    And a form without a softmax.  `weights="sigmoid"`: a visible key weighs sigmoid(score + b_h) with one number per
    head (`head_bias`: its tensor's name, or None for no number); nothing is normalised over the keys.  `head_mix` (a
    tensor's name, [heads, heads]): the heads' weights are mixed, w'_h = sum_g M[h, g] w_g, before head h applies them to
    the values of its own key/value head.  Scores, weights and their sums over the keys are 32-bit.
    """

    supports_cuda_graph = True

    def __init__(self, width: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 pos: PositionEncoding, name: str, bias: bool = False, scale: float | None = None,
                 window: int = 0, share_kv: bool = False,
                 proj_names=("q_proj", "k_proj", "v_proj", "o_proj"), v_head_dim: int | None = None,
                 softcap: float = 0.0, qk_norm_eps: float | None = None, output: bool = True,
                 weight_suffix: str = ".weight", bias_suffix: str = ".bias", qk_norm_weights=None,
                 qk_norm_first: bool = False, keep_first: int = 0, gate: str | None = None, late_bias: bool = False,
                 out_bias: bool | None = None, values_from_keys: bool = False, qk_norm_whole: bool = False,
                 chunk: int = 0, sink: float | None = None, gate_per_head: bool = False, weights: str = "softmax",
                 head_bias: str | None = None, head_mix: str | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are no multiple of {num_kv_heads} kv heads")
        self.nh, self.nkv, self.hd = int(num_heads), int(num_kv_heads), int(head_dim)
        self.vd = int(v_head_dim) if v_head_dim else self.hd
        self.softcap = float(softcap or 0.0)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.qk_norm_weights = tuple(f"{name}.{n}" for n in qk_norm_weights) if qk_norm_weights else None
        self.qk_norm_first, self.keep_first = bool(qk_norm_first), int(keep_first)
        self.gate_name = f"{name}.{gate}" if gate else None
        self.late_bias = bool(late_bias) and bool(bias)
        self.values_from_keys, self.qk_norm_whole = bool(values_from_keys), bool(qk_norm_whole)
        self.chunk, self.sink, self.gate_per_head = int(chunk or 0), None if sink is None else float(sink), bool(gate_per_head)
        if weights not in ("softmax", "sigmoid"):
            raise ValueError(f"attention weights are a softmax or sigmoids, not {weights!r}")
        self.sigmoid = weights == "sigmoid"
        self.head_bias_name = f"{name}.{head_bias}" if head_bias else None
        self.head_mix_name = f"{name}.{head_mix}" if head_mix else None
        if not self.sigmoid and (head_bias or head_mix):
            raise ValueError("a number per head and a mix of the heads' weights belong to sigmoid weights")
        if self.sigmoid and (chunk or sink is not None or gate or keep_first or share_kv):
            raise ValueError("sigmoid weights come without runs of positions, extra terms, gates, kept tokens or a shared cache")
        self.head_bias = self.head_mix = None
        if self.chunk and window:
            raise ValueError("a layer masks by a window or by runs of positions, not both")
        if self.values_from_keys and (self.vd != self.hd or share_kv):
            raise ValueError("values that are the keys have the keys' width and a cache of their own")
        if self.qk_norm_whole and not (self.qk_norm_weights and qk_norm_first):
            raise ValueError("the norm over the whole projection comes before the rotation and has weights")
        self.sinks = None
        if self.keep_first and not window:
            self.keep_first = 0                         # without a window every token is seen anyway
        if (self.qk_norm_weights or self.qk_norm_first) and self.qk_norm_eps is None:
            raise ValueError("a weight or an order for the q/k norm needs its eps")
        self.general = (self.softcap > 0 or self.qk_norm_eps is not None or self.vd != self.hd or self.keep_first > 0
                        or self.gate_name is not None or self.late_bias or self.values_from_keys or self.chunk > 0
                        or self.sink is not None or self.sigmoid)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.window = int(window)
        self.share_kv = bool(share_kv)
        self.pos = pos
        qn, kn, vn, on = (f"{name}.{p}" for p in proj_names)
        outs = [(qn, self.nh * self.hd)]
        if not share_kv:
            outs += [(kn, self.nkv * self.hd)] + ([] if self.values_from_keys else [(vn, self.nkv * self.vd)])
        self.qkv_features = sum(o for _, o in outs)
        self.bias_names = [(n + bias_suffix, o) for n, o in outs] if self.late_bias else []
        self.inner_features = self.nh * self.vd
        if self.gate_name:
            outs = outs + [(self.gate_name, self.nh if self.gate_per_head else self.inner_features)]
        self.qkv = Linear(width, outs, bias and not self.late_bias, weight_suffix=weight_suffix, bias_suffix=bias_suffix)
        out_bias = bool(bias) if out_bias is None else bool(out_bias)
        self.out_piece = (on + weight_suffix, self.inner_features, on + bias_suffix if out_bias else None)
        self.o = Linear(self.inner_features, [(on, width)], out_bias, weight_suffix=weight_suffix,
                        bias_suffix=bias_suffix) if output else None
        self.row_bias = self.q_weight = self.k_weight = None

    def children(self):
        return tuple(p for p in (self.qkv, self.o, self.pos) if p is not None)

    def own_weight_specs(self):
        specs = [WeightSpec(n, (o,), "bias") for n, o in self.bias_names]
        if self.qk_norm_weights:
            widths = (self.nh * self.hd, self.nkv * self.hd) if self.qk_norm_whole else (self.hd, self.hd)
            specs += [WeightSpec(n, (w,), "norm") for n, w in zip(self.qk_norm_weights, widths)]
        if self.head_mix_name:
            specs.append(WeightSpec(self.head_mix_name, (self.nh, self.nh), "head_mix"))
        if self.head_bias_name:
            specs.append(WeightSpec(self.head_bias_name, (self.nh,), "head_bias"))
        return specs

    def bind_own(self, tensors, rt: Runtime):
        if self.bias_names:
            self.row_bias = torch.cat([to_f32_vector(tensors[n], rt) for n, _ in self.bias_names]).contiguous()
        if self.qk_norm_weights:
            self.q_weight, self.k_weight = (to_f32_vector(tensors[n], rt) for n in self.qk_norm_weights)
        if self.sink is not None:
            self.sinks = torch.full((self.nh,), self.sink, dtype=torch.float32, device=rt.device)
        if self.sigmoid:
            self.head_mix = to_f32_vector(tensors[self.head_mix_name], rt) if self.head_mix_name else \
                torch.eye(self.nh, dtype=torch.float32, device=rt.device)
            self.head_bias = to_f32_vector(tensors[self.head_bias_name], rt) if self.head_bias_name else None

    def weight_bytes(self):
        return super().weight_bytes() + 4 * (len(self.bias_names) and self.qkv_features)

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.hd, self.window, 0 if self.vd == self.hd else self.vd, self.keep_first,
                           False, self.chunk)

    def forward(self, x, ctx, cache):
        return self.o.forward(self.forward_inner(x, ctx, cache))

    def forward_inner(self, x, ctx, cache, out=None, qkv=None):
        """The heads' outputs side by side, [T, nh * v width], before the output projection; into
        `out` (a slice of a wider buffer) where one is given.  `qkv`: the part's projection where the caller has
        computed it already (as a slice of a product that it shares with another part)."""
        extended = self.late_bias or self.gate_name is not None
        if qkv is None:
            qkv = self.qkv.forward(x, out_dtype=torch.float32 if extended or self.sigmoid else None)
        if not self.general:
            res = self._attend(qkv, ctx, cache)
            if out is None:
                return res
            out.copy_(res)
            return out
        k = self.rt.k
        inv_freq, rot, trad = self.pos.native_args()
        g = ctx.groups[cache.group]
        store = cache.writable and not self.share_kv
        more = dict(whole=True, values_from_keys=self.values_from_keys) if self.qk_norm_whole or self.values_from_keys else {}
        q = k.qk_prepare(qkv, ctx.positions, inv_freq, rot, trad, self.qk_norm_eps, g.slot_mapping if store else None,
                         cache.kv if store else None, self.nh, self.nkv, self.hd, self.vd, ctx.status,
                         **(dict(bias=self.row_bias, q_weight=self.q_weight, k_weight=self.k_weight,
                                 norm_first=self.qk_norm_first) if extended or self.q_weight is not None or self.qk_norm_first
                            else {}), **more)
        gate = qkv[:, self.qkv_features:] if self.gate_name else None
        if self.sigmoid:
            return k.sigmoid_attention(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.vd, self.scale, self.softcap,
                                       self.window, g.page_size, self.head_bias, self.head_mix, out=out, out_dtype=self.rt.dtype)
        if self.chunk or self.sinks is not None or self.gate_per_head:
            # runs of positions, a term without a value in the denominator, one gate value per head
            opts = dict(chunk=self.chunk, sinks=self.sinks, gate=gate, gate_group=self.vd if self.gate_per_head else 1)
            wide_ex = getattr(k, "wide_attention_takes", None) if getattr(k, "WIDE_HAS_SINKS", False) else None
            if wide_ex is not None and wide_ex(q, cache.kv, self.hd, self.vd, out):
                return k.paged_attention_wide(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.scale, self.softcap,
                                              self.window, out=out, keep_first=self.keep_first, **opts)
            return k.paged_attention_general(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.vd, self.scale,
                                             self.softcap, self.window, g.page_size, out=out, keep_first=self.keep_first,
                                             **opts)
        if extended or self.keep_first:
            wide_ex = getattr(k, "wide_attention_takes", None)
            if wide_ex is not None and wide_ex(q, cache.kv, self.hd, self.vd, out):
                return k.paged_attention_wide(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.scale, self.softcap,
                                              self.window, out=out, keep_first=self.keep_first, gate=gate)
            return k.paged_attention_general(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.vd, self.scale,
                                             self.softcap, self.window, g.page_size, out=out, keep_first=self.keep_first,
                                             gate=gate)
        wide = getattr(k, "wide_attention_ok", None)
        if wide is not None and wide(q, cache.kv, self.hd, self.vd) and (out is None or (out.stride(0) % 2 == 0
                                                                                         and out.data_ptr() % 4 == 0)):
            # bfloat16 pages: the tiled tensor-core kernel, queries and weights as two bfloat16 terms each
            return k.paged_attention_wide(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.scale, self.softcap,
                                          self.window, out=out)
        return k.paged_attention_general(q, cache.kv, ctx, g, self.nh, self.nkv, self.hd, self.vd, self.scale,
                                         self.softcap, self.window, g.page_size, out=out)

    def _attend(self, qkv, ctx, cache):
        k = self.rt.k
        fuses = getattr(k, "decode_attention_fuses_rope", None)
        rope = None
        if fuses is not None and fuses(qkv, cache.kv, ctx, self.nh, self.nkv, self.hd):
            rope = self.pos.fused_args(cache)
        if rope is not None:
            # decode steps: the attention kernel rotates q and the new k and stores k and v itself
            if self.share_kv:
                rope = rope[:3] + (False,)
            return k.paged_attention(qkv, cache.kv, ctx, ctx.groups[cache.group], self.nh, self.nkv, self.hd,
                                     self.scale, self.window, rope=rope)
        self.pos.apply_and_store(qkv, ctx, cache, self.nh, 0 if self.share_kv else self.nkv, self.hd)
        return self.rt.k.paged_attention(qkv, cache.kv, ctx, ctx.groups[cache.group],
                                         self.nh, self.nkv, self.hd, self.scale, self.window)

    def emit(self, b, x, pos):
        from ..engine.native import BF16, NotNative, OP_ATTENTION, _fn
        from ..kernels import lib as klib
        if self.general or self.o is None:
            raise NotNative("capped scores, normalised q and k, values of another width and a joined output "
                            "projection run in Python only")
        cache = b.manager.entries[pos]
        if cache.kv is None:
            raise NotNative("an attention layer without pages")
        inv_freq, rot, trad = self.pos.native_args()
        qkv = self.qkv.emit(b, x)
        out = b.reg(self.nh * self.hd)
        kv = cache.kv
        num_pages, page_size = kv.shape[0], kv.shape[3]
        fns = {}
        tc_ok = 0
        if b.act == BF16 and kv.dtype == self.rt.dtype and self.hd % 16 == 0 and self.hd <= 256:
            lib = klib.load(f"attn_hd{self.hd}")
            fns = dict(fn_attn_decode=_fn(lib, "fmx_attn_decode"), fn_attn_prefill=_fn(lib, "fmx_attn_prefill"),
                       fn_attn_prefill_tc=_fn(lib, "fmx_attn_prefill_tc"), fn_attn_plan=_fn(lib, "fmx_attn_decode_plan"),
                       fn_attn_prefill_tc_plan=_fn(lib, "fmx_attn_prefill_tc_plan_splits"))
            tc_ok = int(bool(lib.fmx_attn_prefill_tc_available())
                        and self.rt.k.tc_attention_ok(self.nh, self.nkv, self.hd, page_size, self.window))
        b.op(OP_ATTENTION, in0=qkv, out0=out, vec=b.ptr(inv_freq), nh=self.nh, nkv=self.nkv, hd=self.hd, window=self.window,
             rot=int(rot), trad=int(bool(trad)), store=int(bool(cache.writable and not self.share_kv)),
             share_kv=int(self.share_kv), group=cache.group, kv=b.ptr(kv), page_size=page_size, num_pages=num_pages,
             scale=self.scale, tc_attention_ok=tc_ok, **fns)
        b.release(qkv)
        o = self.o.emit(b, out)
        b.release(out)
        return o
