"""Plain PyTorch statements of every kernel, with the kernels' own signatures.

Two uses.  The GPU tests run each CUDA kernel alone against the function of the same name
here.  The CPU tests put this module in the place of `fastmlx_b200.kernels`, so that the
cache manager, the step function, the scheduler and the replay program can be checked
against the plain model without a GPU.  It is test code: nothing in the package imports it.
"""
from __future__ import annotations

import torch

F64 = torch.float64


def gather_rows(table, ids, status, code=4):
    return table[ids.long()].clone()


def embedding(ids, table, status, out_dtype=None):
    if ((ids < 0) | (ids >= table.shape[0])).any():
        status[0] = 1
        ids = ids.clamp(0, table.shape[0] - 1)
    out = table[ids.long()].clone()
    return out.to(out_dtype) if out_dtype is not None else out


def add_rmsnorm(x, residual, weight, eps, stream_dtype=None, out_dtype=None):
    act = x.dtype if x is not None else (out_dtype or residual.dtype)
    if residual is not None:
        h = residual.to(F64) if x is None else (x.to(F64) + residual.to(F64))
        residual.copy_(h.to(residual.dtype))
    elif stream_dtype is not None and stream_dtype != act:
        residual = x.to(stream_dtype)
    else:
        residual = x
    h = residual.to(F64)
    out = h * torch.rsqrt((h * h).mean(-1, keepdim=True) + eps) * weight.to(F64)
    return out.to(act), residual


def silu_mul(gate_up, block=None):
    inter = gate_up.shape[1] // 2
    b = block or inter
    v = gate_up.reshape(gate_up.shape[0], inter // b, 2, b).to(F64)
    g, u = v[:, :, 0, :].reshape(-1, inter), v[:, :, 1, :].reshape(-1, inter)
    return (g * torch.sigmoid(g) * u).to(gate_up.dtype)


def linear(x, w, bias, out_dtype):
    y = x.to(F64) @ w.to(F64).t()
    if bias is not None:
        y = y + bias.to(F64)
    return y.to(out_dtype)


gemm_simple = linear


def rope_kv_write(qkv, positions, inv_freq, rotary_dim, traditional, slot_mapping, kv, nh, nkv, hd, status):
    T = qkv.shape[0]
    if rotary_dim > 0:
        ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(F64)
        cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        heads = qkv[:, :(nh + nkv) * hd].reshape(T, nh + nkv, hd).to(F64)
        out = heads.clone()
        r = rotary_dim
        if traditional:
            a, b = heads[..., 0:r:2], heads[..., 1:r:2]
            out[..., 0:r:2] = a * cos - b * sin
            out[..., 1:r:2] = b * cos + a * sin
        else:
            a, b = heads[..., :r // 2], heads[..., r // 2:r]
            out[..., :r // 2] = a * cos - b * sin
            out[..., r // 2:r] = b * cos + a * sin
        qkv[:, :(nh + nkv) * hd] = out.reshape(T, -1).to(qkv.dtype)
    if kv is None or slot_mapping is None or nkv == 0:
        return
    page_size = kv.shape[3]
    k = qkv[:, nh * hd:(nh + nkv) * hd].reshape(T, nkv, hd)
    v = qkv[:, (nh + nkv) * hd:(nh + 2 * nkv) * hd].reshape(T, nkv, hd)
    for t in range(T):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        if s >= kv.shape[0] * page_size:
            status[0] = 2
            continue
        kv[s // page_size, 0, :, s % page_size, :] = k[t]
        kv[s // page_size, 1, :, s % page_size, :] = v[t]


def paged_attention(qkv, kv, ctx, group, nh, nkv, hd, scale, window):
    """Each token attends over the pages of its own row, keys lo..position."""
    T = qkv.shape[0]
    page_size = kv.shape[3]
    out = torch.zeros(T, nh * hd, dtype=F64)
    q = qkv[:, :nh * hd].reshape(T, nh, hd).to(F64)
    rep = nh // nkv
    for t in range(T):
        pos = int(ctx.positions[t])
        if pos < 0:
            continue
        bt = group.block_tables[int(ctx.token_row[t])]
        lo = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(lo, pos + 1)
        pages = bt[(js // page_size).long()].long()
        if (pages < 0).any():
            ctx.status[0] = 3
            continue
        K = kv[pages, 0, :, (js % page_size).long(), :].to(F64)       # [n, nkv, hd]
        V = kv[pages, 1, :, (js % page_size).long(), :].to(F64)
        for h in range(nh):
            s = (K[:, h // rep, :] @ q[t, h]) * scale
            p = torch.softmax(s, dim=0)
            out[t, h * hd:(h + 1) * hd] = p @ V[:, h // rep, :]
    return out.to(qkv.dtype)


paged_attention_simple = paged_attention


def sample(logits, temperature=None, uniform=None, keep=None):
    rows, V = logits.shape
    out = torch.empty(rows, dtype=torch.int32)
    for r in range(rows):
        row = logits[r].to(F64).clone()
        if keep is not None:
            row[keep[r] == 0] = float("-inf")
        T = float(temperature[r]) if temperature is not None else 0.0
        top = int(torch.argmax(row))          # torch returns the first maximal index
        if not T > 0:
            out[r] = top
            continue
        w = torch.exp((row - row[top]) / T)
        c = torch.cumsum(w, 0)
        target = float(uniform[r]) * float(c[-1])
        idx = int(torch.searchsorted(c, torch.tensor(target, dtype=F64), right=True))
        out[r] = min(idx, V - 1)
    return out


def argmax(logits):
    return sample(logits)


def paged_attention_by_rows(q, kv, rows, block_tables, nh, nkv, hd, scale, window=0):
    """The same statement as `paged_attention`, one request at a time instead of one token at a
    time, for contexts of thousands of keys.  rows: (keys before this step, tokens of this
    step) per request; q [T, nh*hd] holds the steps' tokens in row order.  float64 on the CPU."""
    page_size = kv.shape[3]
    out = torch.zeros(q.shape[0], nh * hd, dtype=F64)
    rep = nh // nkv
    at = 0
    for r, (c, ql) in enumerate(rows):
        n = c + ql
        js = torch.arange(n)
        pages = block_tables[r][(js // page_size).long()].long()
        assert (pages >= 0).all()
        K = kv[pages, 0, :, (js % page_size).long(), :].to(F64)       # [n, nkv, hd]
        V = kv[pages, 1, :, (js % page_size).long(), :].to(F64)
        qi = torch.arange(c, n)
        visible = js[None, :] <= qi[:, None]
        if window > 0:
            visible &= js[None, :] > (qi[:, None] - window)
        qr = q[at:at + ql].reshape(ql, nh, hd).to(F64)
        for h in range(nh):
            s = (qr[:, h, :] @ K[:, h // rep, :].t()) * scale
            s = s.masked_fill(~visible, float("-inf"))
            out[at:at + ql, h * hd:(h + 1) * hd] = torch.softmax(s, dim=-1) @ V[:, h // rep, :]
        at += ql
    return out.to(q.dtype)


# ----------------------------------------------------------------------------- general attention route, latents, experts
def _rotate(heads, positions, inv_freq, rotary_dim, traditional):
    if not rotary_dim:
        return heads
    ang = (positions.to(torch.float32)[:, None] * inv_freq.to(torch.float32)[None, :]).to(F64)
    cos, sin = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out, r = heads.clone(), rotary_dim
    if traditional:
        a, b = heads[..., 0:r:2], heads[..., 1:r:2]
        out[..., 0:r:2] = a * cos - b * sin
        out[..., 1:r:2] = b * cos + a * sin
    else:
        a, b = heads[..., :r // 2], heads[..., r // 2:r]
        out[..., :r // 2] = a * cos - b * sin
        out[..., r // 2:r] = b * cos + a * sin
    return out


def qk_prepare(qkv, positions, inv_freq, rotary_dim, traditional, norm_eps, slot_mapping, kv, nh, nkv, hd, vd, status,
               bias=None, q_weight=None, k_weight=None, norm_first=False, whole=False, values_from_keys=False):
    T = qkv.shape[0]
    n_qk = (nh + nkv) * hd
    row = qkv[:, :n_qk + (0 if values_from_keys else nkv * vd)].to(F64)
    if bias is not None:
        row = row + bias.to(F64)
    if values_from_keys:                       # a token's values are its keys as they were projected
        row = torch.cat([row, row[:, nh * hd:n_qk]], 1)
    heads = row[:, :n_qk].reshape(T, nh + nkv, hd)
    w = torch.ones(nh + nkv, hd, dtype=F64)
    if q_weight is not None:
        w[:nh], w[nh:] = q_weight.to(F64).reshape(-1, hd), k_weight.to(F64).reshape(-1, hd)

    def norm(h):
        if norm_eps is None:
            return h
        if whole:                              # q and k each over the whole projection, all heads at once
            ms = torch.cat([(h[:, :nh] ** 2).mean((1, 2), keepdim=True).expand(T, nh, 1),
                            (h[:, nh:] ** 2).mean((1, 2), keepdim=True).expand(T, nkv, 1)], 1) if nkv else \
                (h ** 2).mean((1, 2), keepdim=True)
            return h / torch.sqrt(ms + norm_eps) * w
        return h / torch.sqrt((h * h).mean(-1, keepdim=True) + norm_eps) * w

    heads = _rotate(norm(heads), positions, inv_freq, rotary_dim, traditional) if norm_first \
        else norm(_rotate(heads, positions, inv_freq, rotary_dim, traditional))
    q = heads[:, :nh].reshape(T, nh * hd).to(torch.float32)
    if kv is not None and slot_mapping is not None and nkv:
        pages = kv.shape[0]
        ps = kv[0].numel() // (nkv * (hd + vd))
        flat = kv.view(pages, -1)
        for t in range(T):
            s = int(slot_mapping[t])
            if s < 0:
                continue
            if s >= pages * ps:
                status[0] = 2
                continue
            pg, off = s // ps, s % ps
            for g in range(nkv):
                flat[pg, (g * ps + off) * hd:(g * ps + off + 1) * hd] = heads[t, nh + g].to(kv.dtype)
                at = nkv * ps * hd + (g * ps + off) * vd
                flat[pg, at:at + vd] = row[t, n_qk + g * vd:n_qk + (g + 1) * vd].to(kv.dtype)
    return q


def paged_attention_general(q, kv, ctx, group, nh, nkv, hd, vd, scale, softcap, window, page_size, out=None,
                            keep_first=0, values_are_keys=False, gate=None, chunk=0, sinks=None, gate_group=1):
    T = q.shape[0]
    flat = kv.reshape(-1)
    res = torch.zeros(T, nh * vd, dtype=F64)
    rep = nh // nkv
    page_elems = nkv * page_size * (hd if values_are_keys else hd + vd)
    for t in range(T):
        pos = int(ctx.positions[t])
        if pos < 0:
            continue
        bt = group.block_tables[int(ctx.token_row[t])]
        lo = max(0, pos - window + 1) if window > 0 else 0
        if chunk > 0:
            lo = pos - pos % chunk
        js = torch.tensor([j for j in range(pos + 1) if j >= lo or j < keep_first])
        pages = bt[(js // page_size).long()].long()
        if (pages < 0).any():
            ctx.status[0] = 3
            continue
        for g in range(nkv):
            at = pages * page_elems + (g * page_size + js % page_size) * hd
            K = flat[at[:, None] + torch.arange(hd)[None, :]].to(F64)
            if values_are_keys:
                V = K
            else:
                at = pages * page_elems + nkv * page_size * hd + (g * page_size + js % page_size) * vd
                V = flat[at[:, None] + torch.arange(vd)[None, :]].to(F64)
            for h in range(g * rep, (g + 1) * rep):
                s = (K @ q[t, h * hd:(h + 1) * hd].to(F64)) * scale
                if softcap and softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                if sinks is not None:          # one more term in the denominator, with no value
                    sk = sinks[h].to(F64)
                    m = torch.maximum(s.max(), sk)
                    e = torch.exp(s - m)
                    res[t, h * vd:(h + 1) * vd] = (e / (e.sum() + torch.exp(sk - m))) @ V
                else:
                    res[t, h * vd:(h + 1) * vd] = torch.softmax(s, 0) @ V
    if gate is not None:
        res = res * torch.sigmoid(gate.to(F64)).repeat_interleave(gate_group, dim=1)
    res = res.to(kv.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def dyt_step(y, post, mult, add, residual, pre, out_dtype, out=None, keep_stream=True):
    ref = y if y is not None else residual
    s = residual.to(F64) if residual is not None else torch.zeros(ref.shape, dtype=F64)
    if y is not None:
        v = y.to(F64)
        if post:
            v = torch.tanh(post[0] * v) * post[1].to(F64) + post[2].to(F64)
        s = s + mult * v
    if add is not None:
        s = s + add.to(F64)
    if residual is None:
        residual = s.to(torch.float32)
    else:
        residual.copy_(s.to(torch.float32))
    if pre is False:
        return None, residual
    s = residual.to(F64)
    o = (torch.tanh(pre[0] * s) * pre[1].to(F64) + pre[2].to(F64)) if pre else s
    if out is not None:
        out.copy_(o.to(out.dtype))
        return out, residual
    return o.to(out_dtype), residual


def rmsnorm_rows(x, weight, eps, out=None, out_dtype=None, row_map=None, status=None):
    h = x.to(F64)
    y = h / torch.sqrt((h * h).mean(-1, keepdim=True) + eps) * weight.to(F64)
    if row_map is None:
        if out is None:
            return y.to(out_dtype or x.dtype)
        out.copy_(y.to(out.dtype))
        return out
    rows = out.view(-1, x.shape[1])
    for t in range(x.shape[0]):
        r = int(row_map[t])
        if r < 0:
            continue
        if r >= rows.shape[0]:
            status[0] = 2
            continue
        rows[r] = y[t].to(out.dtype)
    return out


def sigmoid_gate(o, gate, group=1):
    g = torch.sigmoid(gate.to(F64)).repeat_interleave(group, dim=1)
    o.copy_((o.to(F64) * g).to(o.dtype))
    return o


def moe_route(logits, top, groups=1, keep=1, want_chosen=False, experts=None, correction=None, scale=1.0):
    T, E = logits.shape[0], int(experts if experts is not None else logits.shape[1])
    s = torch.softmax(logits[:, :E].to(torch.float32), -1)
    pick = s if correction is None else s + correction.to(torch.float32)
    w = torch.zeros(T, E, dtype=torch.float32)
    chosen = torch.full((T, top), -1, dtype=torch.int32)
    for t in range(T):
        ok = [True] * E
        if groups > 1 and keep < groups:
            per = E // groups
            best = [max(float(s[t, e]) for e in range(g * per, (g + 1) * per)) for g in range(groups)]
            kept = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
            ok = [e // per in kept for e in range(E)]
        order = sorted((e for e in range(E) if ok[e]), key=lambda e: (-float(pick[t, e]), e))[:top]
        for i, e in enumerate(order):
            w[t, e] = s[t, e] * scale
            chosen[t, i] = e
    return (w, chosen) if want_chosen else w


def moe_plain_act(u, weights, E, ff, act, shared_gate=None, out=None):
    T, F = u.shape
    x = u.to(F64)
    if act == "relu2":
        a = torch.relu(x) ** 2
    elif act == "gelu_tanh":
        a = 0.5 * x * (1.0 + torch.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))
    else:
        a = _silu(x)
    w = weights.to(F64).repeat_interleave(ff, dim=1)
    if F > E * ff:
        sg = torch.sigmoid(shared_gate[:, :1].to(F64)) if shared_gate is not None else torch.ones(T, 1, dtype=F64)
        w = torch.cat([w, sg.expand(T, F - E * ff)], 1)
    res = (a * w).to(u.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def embed_scaled(ids, table, scale, status):
    if ((ids < 0) | (ids >= table.shape[0])).any():
        status[0] = 1
        ids = ids.clamp(0, table.shape[0] - 1)
    return (table[ids.long()].to(F64) * scale).to(torch.float32)


def rmsnorm_pair_mean(a, b, wa, wb, eps, out_dtype):
    def n(x, w):
        x = x.to(F64)
        return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.to(F64)
    return (0.5 * (n(a, wa) + n(b, wb))).to(out_dtype)


def retention_prepare(proj, positions, inv_freq, decay, H, D, P, rot, k_scale):
    T = proj.shape[0]
    row = proj.to(F64)
    q = _rotate(row[:, :H * D].reshape(T, H, D), positions, inv_freq, rot, False)
    k = _rotate(row[:, H * D:2 * H * D].reshape(T, H, D), positions, inv_freq, rot, False) * k_scale
    v = row[:, 2 * H * D:2 * H * D + H * P]
    xbc = torch.cat([v, k.reshape(T, -1), q.reshape(T, -1)], 1).to(torch.float32)
    dd = torch.cat([torch.ones(T, H), decay.to(torch.float32)[None, :].expand(T, H)], 1).contiguous()
    return xbc, dd


def retention_gate_norm(o, gate, eps, H, P, out_dtype, out=None):
    T = o.shape[0]
    v = o.to(F64).reshape(T, H, P)
    v = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(T, H * P) * _silu(gate.to(F64))
    res = v.to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def sigmoid_attention(q, kv, ctx, group, nh, nkv, hd, vd, scale, softcap, window, page_size, head_bias, mix, out=None,
                      out_dtype=None):
    T = q.shape[0]
    flat = kv.reshape(-1)
    part = torch.zeros(T, nh, nkv, vd, dtype=F64)              # head g's weights over the values of key/value head c
    rep = nh // nkv
    page_elems = nkv * page_size * (hd + vd)
    for t in range(T):
        pos = int(ctx.positions[t])
        if pos < 0:
            continue
        bt = group.block_tables[int(ctx.token_row[t])]
        lo = max(0, pos - window + 1) if window > 0 else 0
        js = torch.arange(lo, pos + 1)
        pages = bt[(js // page_size).long()].long()
        if (pages < 0).any():
            ctx.status[0] = 3
            continue
        Ks, Vs = [], []
        for c in range(nkv):
            at = pages * page_elems + (c * page_size + js % page_size) * hd
            Ks.append(flat[at[:, None] + torch.arange(hd)[None, :]].to(F64))
            at = pages * page_elems + nkv * page_size * hd + (c * page_size + js % page_size) * vd
            Vs.append(flat[at[:, None] + torch.arange(vd)[None, :]].to(F64))
        for h in range(nh):
            s = (Ks[h // rep] @ q[t, h * hd:(h + 1) * hd].to(F64)) * scale
            if softcap and softcap > 0:
                s = softcap * torch.tanh(s / softcap)
            w = torch.sigmoid(s + (head_bias[h].to(F64) if head_bias is not None else 0.0))
            for c in range(nkv):
                part[t, h, c] = w @ Vs[c]
    res = torch.zeros(T, nh, vd, dtype=F64)
    for h in range(nh):
        res[:, h] = torch.einsum("g,tgv->tv", mix[h].to(F64), part[:, :, h // rep])
    res = res.reshape(T, nh * vd).to(out_dtype or kv.dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def moe_expert_act(gu, weights, E, ff, limit, limit_shared=0.0, out=None, block=0):
    T, F = gu.shape[0], gu.shape[1] // 2
    if block:
        v = gu.reshape(T, F // block, 2, block).to(F64)
        g, u = v[:, :, 0].reshape(T, F), v[:, :, 1].reshape(T, F)
    else:
        g, u = gu[:, :F].to(F64), gu[:, F:].to(F64)
    lim = torch.full((F,), float(limit), dtype=F64)
    lim[E * ff:] = float(limit_shared)
    w = torch.ones(T, F, dtype=F64)
    w[:, :E * ff] = weights.to(F64).repeat_interleave(ff, dim=1)
    g = torch.minimum(g, lim)
    u = torch.maximum(torch.minimum(u, lim), -lim)
    y = (w * g * torch.sigmoid(1.702 * g) * (u + 1)).to(gu.dtype)
    if out is not None:
        out.copy_(y)
        return out
    return y


def head_linear(x, w, out_dtype, x_head_stride=None, out=None, out_head_stride=None):
    H, N, K = w.shape
    T = x.shape[0]
    xs = x_head_stride or K
    xh = x.reshape(T, H, xs)[:, :, :K]
    res = torch.einsum("thk,hnk->thn", xh.to(F64), w.to(F64))
    if out is None:
        return res.reshape(T, H * N).to(out_dtype)
    out.view(T, H, out_head_stride or N)[:, :, :N] = res.to(out.dtype)
    return out


# ----------------------------------------------------------------------------- bigram embedding, rotated latents, state space
def embed_bigram(ids, table, bigram, ctx, state, buckets, mul_prev, mul_cur):
    T = ids.shape[0]
    out = torch.zeros(T, table.shape[1], dtype=torch.float32)
    last = {}
    for t in range(T):
        r = int(ctx.token_row[t])
        slot, pos = int(ctx.row_slot[r]), int(ctx.positions[t])
        if slot < 0 or pos < 0:
            continue
        tok = int(ids[t])
        if not 0 <= tok < table.shape[0]:
            ctx.status[0] = 1
            continue
        first = t == int(ctx.row_start[r])
        prev = int(state[slot, 0]) if first else int(ids[t - 1])
        row = buckets if pos == 0 else (prev * mul_prev + tok * mul_cur) % buckets
        out[t] = (table[tok].to(F64) + bigram[row].to(F64)).to(torch.float32)
        last[slot] = tok
    for slot, tok in last.items():
        state[slot, 0] = tok
    return out


def latent_rope_prepare(q, dkv, positions, inv_freq, norm_w, eps, slot_mapping, kv, q_lat, H, D, R, r, status, q_offset=None):
    T = q.shape[0]
    row = r + R
    if R:
        off = r if q_offset is None else q_offset
        qr = q.reshape(T, H, D + R)[:, :, D:].to(F64)
        q_lat.view(T, H, off + R)[:, :, off:] = _rotate(qr, positions, inv_freq, R, False).to(q_lat.dtype)
    if kv is None or dkv is None:
        return
    c = dkv[:, :r].to(F64)
    c = c / torch.sqrt((c * c).mean(-1, keepdim=True) + eps) * norm_w.to(F64)
    both = c
    if R:
        kr = _rotate(dkv[:, r:row].to(F64).reshape(T, 1, R), positions, inv_freq, R, False).reshape(T, R)
        both = torch.cat([c, kr], 1)
    flat = kv.view(-1, row)
    for t in range(T):
        s = int(slot_mapping[t])
        if s < 0:
            continue
        if s >= flat.shape[0]:
            status[0] = 2
            continue
        flat[s] = both[t].to(kv.dtype)


def _silu(z):
    return z * torch.sigmoid(z)


def ssm_prepare(proj, conv_w, conv_b, a_log, dt_bias, ctx, state, conv_off, H, G, N, P, taps):
    T = proj.shape[0]
    inner = H * P
    C = inner + 2 * G * N
    xbc = torch.zeros(T, C, dtype=torch.float32)
    dd = torch.zeros(T, 2 * H, dtype=torch.float32)
    w, b = conv_w.to(F64), conv_b.to(F64)
    for r in range(ctx.R):
        slot = int(ctx.row_slot[r])
        a, e = int(ctx.row_start[r]), int(ctx.row_start[r + 1])
        if slot < 0 or e <= a:
            continue
        hist = state[slot, conv_off:conv_off + (taps - 1) * C].to(F64).reshape(taps - 1, C)
        u = torch.cat([hist, proj[a:e, inner:inner + C].to(F64)], 0)            # [taps-1 + n, C]
        for t in range(e - a):
            xbc[a + t] = _silu((u[t:t + taps] * w.t()).sum(0) + b).to(torch.float32)
        state[slot, conv_off:conv_off + (taps - 1) * C] = u[u.shape[0] - (taps - 1):].reshape(-1).to(torch.float32)
        dt = torch.nn.functional.softplus(proj[a:e, inner + C:inner + C + H].to(F64) + dt_bias.to(F64), threshold=40.0)
        dd[a:e, :H] = dt.to(torch.float32)
        dd[a:e, H:] = torch.exp(-torch.exp(a_log.to(F64)) * dt).to(torch.float32)
    return xbc, dd


def ssm_scan(xbc, dd, d_skip, ctx, state, H, G, N, P):
    T = xbc.shape[0]
    inner = H * P
    y = torch.zeros(T, inner, dtype=torch.float32)
    per = H // G
    for r in range(ctx.R):
        slot = int(ctx.row_slot[r])
        a, e = int(ctx.row_start[r]), int(ctx.row_start[r + 1])
        if slot < 0 or e <= a:
            continue
        S = state[slot, :H * P * N].to(F64).reshape(H, P, N)                   # S^T of every head
        for t in range(a, e):
            x = xbc[t, :inner].to(F64).reshape(H, P)
            B = xbc[t, inner:inner + G * N].to(F64).reshape(G, N).repeat_interleave(per, 0)
            Cm = xbc[t, inner + G * N:].to(F64).reshape(G, N).repeat_interleave(per, 0)
            dt, decay = dd[t, :H].to(F64), dd[t, H:].to(F64)
            S = decay[:, None, None] * S + dt[:, None, None] * x[:, :, None] * B[:, None, :]
            y[t] = ((S * Cm[:, None, :]).sum(-1) + d_skip.to(F64)[:, None] * x).reshape(-1).to(torch.float32)
        state[slot, :H * P * N] = S.reshape(-1).to(torch.float32)
    return y


def gated_group_rmsnorm(y, z, weight, eps, groups, out_dtype, out=None):
    T, n = y.shape
    v = y.to(F64) * _silu(z.to(F64))
    v = v.reshape(T, groups, n // groups)
    v = (v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(T, n) * weight.to(F64)
    res = v.to(out_dtype)
    if out is not None:
        out.copy_(res)
        return out
    return res


def act_mul(gate_up, kind, block=None):
    inter = gate_up.shape[1] // 2
    b = block or inter
    v = gate_up.reshape(gate_up.shape[0], inter // b, 2, b).to(F64)
    g, u = v[:, :, 0, :].reshape(-1, inter), v[:, :, 1, :].reshape(-1, inter)
    if kind == "silu":
        a = _silu(g)
    elif kind == "gelu_tanh":
        a = 0.5 * g * (1.0 + torch.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3)))
    else:
        raise ValueError(kind)
    return (a * u).to(gate_up.dtype)
