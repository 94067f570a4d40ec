"""Attention whose keys and values are read out of one cached latent per token."""
from __future__ import annotations

import torch

from .base import Mixer, PagedKVSpec, Runtime, WeightSpec, to_compute, to_f32_vector
from .linear import Linear


class LatentAttention(Mixer):
    """Per token one latent c = rmsnorm(W_dkv x) w of `kv_rank` values is cached; head h has keys k = W_uk,h c and
    values v = W_uv,h c.  The queries pass a latent of their own, q = W_uq (rmsnorm(W_dq x) w).  No positions
    enter.  A query sees itself and the window - 1 tokens before it (window 0: every earlier token).  Head h's
    output is multiplied by sigmoid(W_g x)_h where a gate is named, and the heads go through W_o.

    Only c lies in the pages (one "kv head" of size kv_rank, whose keys are its values too), and neither k nor
    v is ever formed: since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, each query is carried into the latent's space
    (one small product per head), attention runs over the latents with all heads sharing them, and the heads'
    outputs, weighted sums of latents, are read out through W_uv,h afterwards.  Scores and weights are 32-bit
    (the queries stay in 32-bit from their product to the scores).

    That form reads kv_rank values per key and head, which suits single tokens (the cache is what a decode step
    reads).  A long portion of a prompt multiplies kv_rank / dim times more than it must, so steps with a portion of
    LONG_PORTION tokens or more (bfloat16, head sizes the tiled kernel takes) read the keys and values of the tokens in
    sight out of the latents once per step, into pages of their own that live for the step, and attend over those
    with the heads' own sizes.  The cache holds latents either way.

    Tensors, under `name`: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g (optional), o.

    A second form, chosen by its parameters.  `q_rank` = 0: the queries are one projection `q` of the input, no latent
    of their own.  `rot_dim` R > 0: a query head is [dim unrotated | R rotated] values; the down-projection `dkv` has R
    more rows, which are not normalised, are rotated by the token's position (pairs (i, i + R/2), angles
    position * rot_base^(-2i/R), 32-bit) and are one key part shared by all heads, so that a score is
    (q_unrotated . W_uk,h c + q_rotated . k_rotated) * scale.  The cache row of a token is then [c | rotated part], and
    a query is carried to [W_uk,h^T q_unrotated | q_rotated]; the values are read out of the row's first kv_rank
    entries.  `sink`: a tensor of one learned number per head whose exponential is one more term of the softmax's
    denominator (it has no key and no value and is not scaled).  `gate` = "element": the gate has one value per
    output element (`True`: one per head).  `share_kv`: the layer has no `dkv` and reads the rows that the schedule
    entry it is pointed at has cached."""

    supports_cuda_graph = True
    LONG_PORTION = 128

    def __init__(self, width: int, num_heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int,
                 eps: float, name: str, scale: float | None = None, window: int = 0, gate: bool | str = True,
                 weight_suffix: str = "", norm_suffix: str = ".norm", rot_dim: int = 0, rot_base: float = 10000.0,
                 sink: str | None = None, share_kv: bool = False):
        self.width, self.nh, self.hd, self.vd = int(width), int(num_heads), int(head_dim), int(v_head_dim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.window = int(window)
        self.name, self.wsfx = name, weight_suffix
        self.rot, self.rot_base, self.share_kv = int(rot_dim), float(rot_base), bool(share_kv)
        if self.rot % 2:
            raise ValueError(f"the rotated part has an even width, not {self.rot}")
        self.row = self.kv_rank + self.rot                 # what a token's cache row holds
        self.direct = self.q_rank == 0                     # queries straight from the input
        if (self.rot or self.share_kv or sink) and not self.direct:
            raise ValueError("a rotated part, a term in the denominator and a shared cache go with direct queries")
        self.gate_group = 0 if not gate else (1 if gate == "element" else self.vd)
        self.has_gate = bool(gate)
        self.sink_name = f"{name}.{sink}" if sink else None
        self.sinks = self.inv_freq = None
        downs = [] if self.direct else [(f"{name}.dq", self.q_rank)]
        if not self.share_kv:
            downs.append((f"{name}.dkv", self.row))
        if gate:
            downs.append((f"{name}.g", self.nh * self.vd // self.gate_group))
        self.down = Linear(width, downs, False, weight_suffix=weight_suffix) if downs else None     # one product reads x
        if self.direct:
            self.uq = Linear(width, [(f"{name}.q", self.nh * (self.hd + self.rot))], False, weight_suffix=weight_suffix)
        else:
            self.uq = Linear(self.q_rank, [(f"{name}.uq", self.nh * self.hd)], False, weight_suffix=weight_suffix)
        self.o = Linear(self.nh * self.vd, [(f"{name}.o", width)], False, weight_suffix=weight_suffix)
        self.norm_names = (f"{name}.dq{norm_suffix}", f"{name}.dkv{norm_suffix}")
        self.uk_name, self.uv_name = f"{name}.uk{weight_suffix}", f"{name}.uv{weight_suffix}"

    def children(self):
        return tuple(p for p in (self.down, self.uq, self.o) if p is not None)

    def own_weight_specs(self):
        specs = [] if self.direct else [WeightSpec(self.norm_names[0], (self.q_rank,), "norm")]
        if not self.share_kv:
            specs.append(WeightSpec(self.norm_names[1], (self.kv_rank,), "norm"))
        if self.sink_name:
            specs.append(WeightSpec(self.sink_name, (self.nh,), "bias"))
        return specs + [WeightSpec(self.uk_name, (self.nh * self.hd, self.kv_rank), "matrix"),
                        WeightSpec(self.uv_name, (self.nh * self.vd, self.kv_rank), "matrix")]

    def bind_own(self, tensors, rt: Runtime):
        self.q_norm = None if self.direct else to_f32_vector(tensors[self.norm_names[0]], rt)
        self.c_norm = None if self.share_kv else to_f32_vector(tensors[self.norm_names[1]], rt)
        if self.sink_name:
            self.sinks = to_f32_vector(tensors[self.sink_name], rt)
        if self.rot:
            from .rope import inverse_frequencies
            self.inv_freq = inverse_frequencies(self.rot, self.rot_base).to(torch.float32).to(rt.device).contiguous()
        uk = to_compute(tensors[self.uk_name], rt).view(self.nh, self.hd, self.kv_rank)
        # carrying a query into the latent's space multiplies by W_uk,h^T: [H, kv_rank, dim]
        self.uk_t = uk.transpose(1, 2).contiguous()
        self.uv = to_compute(tensors[self.uv_name], rt).view(self.nh, self.vd, self.kv_rank).contiguous()
        # long portions: every head's keys, then every head's values, in one product over the latents in sight
        self.ukv = None
        if not self.direct and rt.dtype == torch.bfloat16 and self.hd == self.vd and self.hd % 16 == 0 and self.hd <= 256 and rt.device.type == "cuda":
            self.ukv = torch.cat([uk.reshape(self.nh * self.hd, self.kv_rank), self.uv.view(self.nh * self.vd, self.kv_rank)], 0).contiguous()
        # the direct form: a head's key is [W_uk,h c | rotated part], as wide as its query; values are padded to that width
        wide = self.hd + self.rot
        if self.direct and rt.dtype == torch.bfloat16 and wide % 16 == 0 and wide <= 256 and self.vd <= wide and rt.device.type == "cuda":
            self.ukv = torch.cat([uk.reshape(self.nh * self.hd, self.kv_rank), self.uv.view(self.nh * self.vd, self.kv_rank)], 0).contiguous()

    def weight_bytes(self):
        return super().weight_bytes() + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()

    def cache_spec(self):
        return PagedKVSpec(1, self.row, self.window, 0, 0, True)

    def forward_direct(self, x, ctx, cache):
        """The form with direct queries (and, where rot_dim > 0, a rotated part beside the latent)."""
        k, rt = self.rt.k, self.rt
        g = ctx.groups[cache.group]
        T, r, R = x.shape[0], self.kv_rank, self.rot
        q = self.uq.forward(x)                                                   # [T, H * (dim + R)]
        down = self.down.forward(x, out_dtype=torch.float32) if self.down is not None else None
        store = cache.writable and not self.share_kv
        long = (self.ukv is not None and not ctx.all_decode and ctx.max_q_len >= self.LONG_PORTION
                and cache.kv.dtype == torch.bfloat16 and hasattr(k, "paged_attention_wide"))
        # a long portion carries its rotated query parts to [T, H, dim + R] instead: the heads' own keys are read out
        lat_r = self.hd if long else r
        q_lat = torch.empty((T, self.nh * (lat_r + R)), dtype=torch.float32, device=x.device)
        # the latent's norm and the rotation of the shared key part into the token's cache row; the queries'
        # rotated parts into the places behind their latent parts
        k.latent_rope_prepare(q, down[:, :self.row] if store else None, ctx.positions, self.inv_freq, self.c_norm, self.eps,
                              g.slot_mapping if store else None, cache.kv if store else None, q_lat, self.nh, self.hd, R, r,
                              ctx.status, q_offset=lat_r)
        if long:
            heads = self.attend_long_direct(q, q_lat, ctx, cache, g)
            if self.has_gate:
                k.sigmoid_gate(heads, down[:, 0 if self.share_kv else self.row:], self.gate_group)
            return self.o.forward(heads)
        k.head_linear(q, self.uk_t, torch.float32, x_head_stride=self.hd + R, out=q_lat, out_head_stride=self.row)
        opts = dict(sinks=self.sinks) if self.sinks is not None else {}
        wide = getattr(k, "wide_attention_takes", None) if (not opts or getattr(k, "WIDE_HAS_SINKS", False)) else None
        if wide is not None and wide(q_lat, cache.kv, self.row, self.row, None):
            o_lat = k.paged_attention_wide(q_lat, cache.kv, ctx, g, self.nh, 1, self.row, self.scale, 0.0, self.window, **opts)
        else:
            o_lat = k.paged_attention_general(q_lat, cache.kv, ctx, g, self.nh, 1, self.row, self.row, self.scale,
                                              0.0, self.window, g.page_size, values_are_keys=True, **opts)
        heads = k.head_linear(o_lat, self.uv, rt.dtype, x_head_stride=self.row)  # [T, H * vdim]
        if self.has_gate:
            at = 0 if self.share_kv else self.row
            k.sigmoid_gate(heads, down[:, at:], self.gate_group)
        return self.o.forward(heads)

    def forward(self, x, ctx, cache):
        if self.direct:
            return self.forward_direct(x, ctx, cache)
        k, rt = self.rt.k, self.rt
        g = ctx.groups[cache.group]
        down = self.down.forward(x, out_dtype=torch.float32)
        cq = k.rmsnorm_rows(down[:, :self.q_rank], self.q_norm, self.eps, out_dtype=rt.dtype)
        if cache.writable:
            k.rmsnorm_rows(down[:, self.q_rank: self.q_rank + self.kv_rank], self.c_norm, self.eps, out=cache.kv,
                           row_map=g.slot_mapping, status=ctx.status)
        if self.ukv is not None and not ctx.all_decode and ctx.max_q_len >= self.LONG_PORTION and cache.kv.dtype == torch.bfloat16 \
                and hasattr(k, "paged_attention_wide"):
            heads = self.attend_long(cq, ctx, cache, g)
            if self.has_gate:
                k.sigmoid_gate(heads, down[:, self.q_rank + self.kv_rank:], self.vd)
            return self.o.forward(heads)
        q = self.uq.forward(cq)
        q_lat = k.head_linear(q, self.uk_t, torch.float32)                       # [T, H * kv_rank], 32-bit
        wide = getattr(k, "wide_attention_takes", None)
        if wide is not None and wide(q_lat, cache.kv, self.kv_rank, self.kv_rank, None):
            o_lat = k.paged_attention_wide(q_lat, cache.kv, ctx, g, self.nh, 1, self.kv_rank, self.scale, 0.0, self.window)
        else:
            o_lat = k.paged_attention_general(q_lat, cache.kv, ctx, g, self.nh, 1, self.kv_rank, self.kv_rank, self.scale,
                                              0.0, self.window, g.page_size, values_are_keys=True)
        heads = k.head_linear(o_lat, self.uv, rt.dtype)                          # [T, H * vdim]
        if self.has_gate:
            k.sigmoid_gate(heads, down[:, self.q_rank + self.kv_rank:], self.vd)
        return self.o.forward(heads)

    def pages_in_sight(self, ctx, g):
        """(row, block) of every page of positions that a row of this step may see, as device index vectors."""
        ps = g.page_size
        rows, blks = [], []
        for r in range(ctx.R):
            c = ctx.h_row_ctx[r]
            n = ctx.h_row_start[r + 1] - ctx.h_row_start[r]
            if ctx.h_row_slot[r] < 0 or n <= 0:
                continue
            lo = max(0, c - self.window + 1) if self.window > 0 else 0
            for b in range(lo // ps, (c + n - 1) // ps + 1):
                rows.append(r)
                blks.append(b)
        # one copy from pinned memory, so that the host does not fall into step with the device
        both = torch.tensor([rows, blks], dtype=torch.long, pin_memory=True).to(g.block_tables.device, non_blocking=True)
        return both[0], both[1], len(rows)

    def attend_long_direct(self, q, q_wide, ctx, cache, g):
        """The direct form over a long portion: per head, keys [W_uk,h c | the row's rotated part] and values W_uv,h c
        (padded with zeros to the keys' width, which the tiled kernel wants equal) of every page in sight, read out of
        the cached rows into pages that live for the step.  q [T, H * (dim + R)] as projected; q_wide (32-bit, same
        shape) holds the rotated query parts already and takes the unrotated ones here.  -> [T, H * vdim]."""
        from types import SimpleNamespace
        k, ps = self.rt.k, g.page_size
        T, H, D, R, Dv, r = q.shape[0], self.nh, self.hd, self.rot, self.vd, self.kv_rank
        E = D + R
        # which pages are in sight, and the step's block table over them, serve every layer of the step with this sight
        # over this cache group (a layer that reads another's cache among them)
        key = ("pages in sight", id(g), self.window)
        seen = ctx.scratch.get(key)
        if seen is None:
            rows_t, blks_t, n = self.pages_in_sight(ctx, g)
            pages = g.block_tables[rows_t, blks_t].long().clamp_(min=0)
            table = torch.full_like(g.block_tables, -1)
            table[rows_t, blks_t] = torch.arange(n, dtype=torch.int32, device=q.device)
            seen = ctx.scratch[key] = (pages, n, SimpleNamespace(block_tables=table, page_size=ps, window=self.window))
        pages, n, group = seen
        cached = cache.kv.view(cache.kv.shape[0], ps, self.row)[pages]           # [pages in sight, page, kv_rank + R]
        kv = k.linear(cached[..., :r].reshape(-1, r), self.ukv, None, torch.bfloat16)       # [n * page, H * (dim + vdim)]
        own = torch.zeros((n, 2, H, ps, E), dtype=torch.bfloat16, device=q.device)
        own[:, 0, :, :, :D] = kv[:, :H * D].view(n, ps, H, D).permute(0, 2, 1, 3)
        if R:
            own[:, 0, :, :, D:] = cached[..., r:].unsqueeze(1)
        own[:, 1, :, :, :Dv] = kv[:, H * D:].view(n, ps, H, Dv).permute(0, 2, 1, 3)
        q_wide.view(T, H, E)[..., :D] = q.view(T, H, E)[..., :D]
        opts = dict(sinks=self.sinks) if self.sinks is not None else {}
        out = k.paged_attention_wide(q_wide, own, ctx, group, H, H, E, self.scale, 0.0, self.window, **opts)
        return out.view(T, H, E)[..., :Dv].reshape(T, H * Dv)

    def attend_long(self, cq, ctx, cache, g):
        """Keys and values of every position a row of this step may see, read out of the cached latents into pages
        that live for the step (one per page of positions in sight, whole pages: what lies outside a row's sight on
        them is never loaded), and attention with the heads' own sizes.  -> [T, H * vdim]."""
        from types import SimpleNamespace
        k, ps = self.rt.k, g.page_size
        dev = cq.device
        rows, blks = [], []
        for r in range(ctx.R):
            c = ctx.h_row_ctx[r]
            n = ctx.h_row_start[r + 1] - ctx.h_row_start[r]
            if ctx.h_row_slot[r] < 0 or n <= 0:
                continue
            lo = max(0, c - self.window + 1) if self.window > 0 else 0
            for b in range(lo // ps, (c + n - 1) // ps + 1):
                rows.append(r)
                blks.append(b)
        # one copy from pinned memory, so that the host does not fall into step with the device
        both = torch.tensor([rows, blks], dtype=torch.long, pin_memory=True).to(dev, non_blocking=True)
        rows_t, blks_t = both[0], both[1]
        pages = g.block_tables[rows_t, blks_t].long().clamp_(min=0)
        latents = cache.kv.view(cache.kv.shape[0], ps, self.kv_rank)[pages]      # [pages in sight, page, kv_rank]
        kv = k.linear(latents.view(-1, self.kv_rank), self.ukv, None, torch.bfloat16)
        kv = kv.view(len(rows), ps, 2, self.nh, self.hd).permute(0, 2, 3, 1, 4).contiguous()      # pages of [2, H, page, dim]
        table = torch.full_like(g.block_tables, -1)
        table[rows_t, blks_t] = torch.arange(len(rows), dtype=torch.int32, device=dev)
        own = SimpleNamespace(block_tables=table, page_size=ps, window=self.window)
        ctx.scratch.setdefault("pages of a step", []).append(own)        # kept for the step: its identity keys cached views
        q = self.uq.forward(cq, out_dtype=torch.float32)
        return k.paged_attention_wide(q, kv, ctx, own, self.nh, self.nh, self.hd, self.scale, 0.0, self.window)
