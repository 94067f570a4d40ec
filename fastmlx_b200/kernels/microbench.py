"""Times one kernel alone on synthetic inputs (CUDA events around a captured graph of
launches), for tuning and for profiler captures on a small case.

    python -m fastmlx_b200.kernels.microbench --kernel attn_decode --batch 8 --ctx 8192
    python -m fastmlx_b200.kernels.microbench --kernel attn_prefill --batch 1 --qlen 2048
    python -m fastmlx_b200.kernels.microbench --kernel gemv --M 8 --N 2048 --K 8192
    python -m fastmlx_b200.kernels.microbench --kernel gemm --M 2048 --N 16384 --K 2048
    python -m fastmlx_b200.kernels.microbench --kernel sample --batch 8 --N 128256
    python -m fastmlx_b200.kernels.microbench --kernel recurrence --batch 1 --qlen 2048 --nh 64 --hd 64 --state 128
    python -m fastmlx_b200.kernels.microbench --kernel attn_masked --batch 64 --qlen 1 --ctx 4096 --hd 64
    python -m fastmlx_b200.kernels.microbench --kernel attn_mixed --batch 64 --qlen 1 --ctx 4096 --hd 64
"""
from __future__ import annotations

import argparse
from types import SimpleNamespace

import torch

from .. import kernels as k

DEV = "cuda"


def _time_graph(fn, launches: int, replays: int) -> float:
    """Microseconds per call of fn, from a CUDA graph holding `launches` calls."""
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for _ in range(launches):
            fn()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (replays * launches) * 1e3


def _attention_inputs(a, qlen):
    B, ctx_len, nh, nkv, hd, ps = a.batch, a.ctx, a.nh, a.nkv, a.hd, a.page
    per = -(-(ctx_len + qlen) // ps)
    num_pages = B * per + 8
    kv = torch.randn(num_pages, 2, nkv, ps, hd, device=DEV, dtype=torch.bfloat16)
    bt = torch.randperm(num_pages, device=DEV)[:B * per].int().view(B, per).contiguous()
    T = B * qlen
    qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=DEV, dtype=torch.bfloat16)
    pos = torch.cat([torch.arange(ctx_len, ctx_len + qlen) for _ in range(B)]).int().to(DEV)
    ctx = SimpleNamespace(positions=pos, token_row=torch.arange(B).repeat_interleave(qlen).int().to(DEV),
                          status=torch.zeros(4, dtype=torch.int32, device=DEV),
                          row_start=(torch.arange(B + 1) * qlen).int().to(DEV),
                          row_ctx=torch.full((B,), ctx_len, dtype=torch.int32, device=DEV), R=B, max_q_len=qlen,
                          max_ctx_after=ctx_len + qlen, all_decode=qlen == 1, n_splits=0, scratch={})
    return qkv, kv, ctx, SimpleNamespace(block_tables=bt)


def _flush():
    """A buffer larger than L2, written between timed launches."""
    buf = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=DEV)
    return lambda: buf.fill_(1)


def _time_events(fn, reps: int, flush=None) -> float:
    """Median microseconds of fn alone: events around each launch, L2 flushed before it."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(reps):
        if flush is not None:
            flush()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) * 1e3)
    return sorted(out)[len(out) // 2]


def _rows_ctx(B, qlen, ctx_len=0):
    T = B * qlen
    return SimpleNamespace(T=T, R=B, positions=torch.cat([torch.arange(ctx_len, ctx_len + qlen) for _ in range(B)]).int().to(DEV),
                           token_row=torch.arange(B).repeat_interleave(qlen).int().to(DEV),
                           row_start=(torch.arange(B + 1) * qlen).int().to(DEV), row_slot=torch.arange(B).int().to(DEV),
                           row_ctx=torch.full((B,), ctx_len, dtype=torch.int32, device=DEV),
                           status=torch.zeros(4, dtype=torch.int32, device=DEV), max_q_len=qlen, max_ctx_after=ctx_len + qlen,
                           all_decode=qlen == 1, decode_rows=B if qlen == 1 else 0, scratch={})


def _recurrence(a) -> int:
    """The state-space recurrence and the gated delta rule side by side at like sizes: --nh heads of --hd values over
    --state rows of state, --groups groups; --batch requests of --qlen tokens each.  Per kernel: microseconds (events,
    L2 flushed) and the bytes it must move over that time."""
    H, P, N, G, taps, B, q = a.nh, a.hd, a.state, a.groups, a.taps, a.batch, a.qlen
    T = B * q
    ctx = _rows_ctx(B, q)
    flush = _flush()
    gen = lambda *s: torch.randn(*s, device=DEV)
    # ---- state space
    inner, C = H * P, H * P + 2 * G * N
    proj = gen(T, 2 * inner + 2 * G * N + H).bfloat16()
    conv_w, conv_b = gen(C, taps) * 0.5, gen(C) * 0.1
    a_log, dt_bias, d_skip = torch.log(torch.rand(H, device=DEV) * 0.9 + 0.05), gen(H) * 0.5 - 1, gen(H)
    slot = -(-(inner * N + (taps - 1) * C) // 4) * 4
    state = gen(B, slot) * 0.1
    norm_w = torch.rand(inner, device=DEV) + 0.5
    xbc, dd = k.ssm_prepare(proj, conv_w, conv_b, a_log, dt_bias, ctx, state, inner * N, H, G, N, P, taps)
    y = k.ssm_scan(xbc, dd, d_skip, ctx, state, H, G, N, P)
    rows = [("ssm_prepare", lambda: k.ssm_prepare(proj, conv_w, conv_b, a_log, dt_bias, ctx, state, inner * N, H, G, N, P, taps),
             T * (C + H) * 2 + T * (C + 2 * H) * 4 + B * (taps - 1) * C * 8),
            ("ssm_scan", lambda: k.ssm_scan(xbc, dd, d_skip, ctx, state, H, G, N, P), 2 * B * inner * N * 4 + T * (C + 2 * H + inner) * 4),
            ("gated_group_rmsnorm", lambda: k.gated_group_rmsnorm(y, proj[:, :inner], norm_w, 1e-6, G, torch.bfloat16),
             T * inner * (4 + 2 + 2))]
    # ---- delta rule: H heads of vdim P over keys of N values, G key heads
    Cd = 2 * G * N + H * P
    projd, ab = gen(T, Cd).bfloat16(), gen(T, 2 * H)
    conv_d = gen(Cd, taps) * 0.5
    slot_d = -(-(H * P * N + (taps - 1) * Cd) // 4) * 4
    state_d = gen(B, slot_d) * 0.1
    qkv, gb = k.delta_prepare(projd, ab, conv_d, a_log, dt_bias, ctx, state_d, H * P * N, H, G, N, P, taps)
    o = k.delta_rule(qkv, gb, ctx, state_d, H, G, N, P)
    gate, w_d = gen(T, inner).bfloat16(), torch.rand(P, device=DEV) + 0.5
    rows += [("delta_prepare", lambda: k.delta_prepare(projd, ab, conv_d, a_log, dt_bias, ctx, state_d, H * P * N, H, G, N, P, taps),
              T * Cd * 2 + T * 2 * H * 4 + T * (Cd + 2 * H) * 4 + B * (taps - 1) * Cd * 8),
             ("delta_rule", lambda: k.delta_rule(qkv, gb, ctx, state_d, H, G, N, P), 2 * B * inner * N * 4 + T * (Cd + 2 * H + inner) * 4),
             ("gated_rmsnorm", lambda: k.gated_rmsnorm(o, gate, w_d, 1e-6, H, P, torch.bfloat16), T * inner * (4 + 2 + 2))]
    for name, fn, nbytes in rows:
        if not name.startswith(a.only):
            continue
        us = _time_events(fn, a.replays, flush)
        print(f"{name} B={B} qlen={q} heads={H} vdim={P} state={N} groups={G} taps={taps}: {us:.1f} us, {nbytes / 1e6:.1f} MB, "
              f"{nbytes / us / 1e3:.0f} GB/s")
    print("status", ctx.status.tolist())
    return 0


def _attn_masked(a) -> int:
    """The tiled two-term attention kernel over bfloat16 pages with a sliding window (keys and values apart) and with
    runs of positions, one more term in the denominator and values that are read from a second plane, at equal sizes;
    then over pages of keys that are the values too (a latent of --hd values per token), with a learned term or none."""
    B, q, c, nh, nkv, hd, ps, span = a.batch, a.qlen, a.ctx if a.ctx != 8192 or a.qlen == 1 else 0, a.nh, a.nkv, a.hd, a.page, a.span
    ctx = _rows_ctx(B, q, c)
    per = -(-(c + q) // ps)
    flush = _flush()
    grp = SimpleNamespace(block_tables=torch.randperm(B * per + 8, device=DEV)[:B * per].int().view(B, per).contiguous(), page_size=ps)
    kv = torch.randn(B * per + 8, 2, nkv, ps, hd, device=DEV).bfloat16()
    qq = torch.randn(B * q, nh * hd, device=DEV)
    sinks0, sinks = torch.zeros(nh, device=DEV), torch.randn(nh, device=DEV)
    seen = sum(min(p + 1, span) for p in range(c, c + q)) * B                 # keys in sight, windowed
    seen_c = sum(p % span + 1 for p in range(c, c + q)) * B                  # in runs of positions
    flops = lambda n: 4.0 * nh * hd * n
    kvb = lambda n_rows: B * min(c + q, n_rows) * nkv * hd * 2 * 2
    cases = [("window", lambda: k.paged_attention_wide(qq, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 30.0, span), seen, kvb(span + q)),
             ("runs of positions, one more term", lambda: k.paged_attention_wide(qq, kv, ctx, grp, nh, nkv, hd, hd ** -0.5, 30.0, 0, chunk=span, sinks=sinks0),
              seen_c, kvb((c + q - 1) % span + 1 if q == 1 else span))]
    lat = torch.randn(B * per + 8, 1, 1, ps, hd, device=DEV).bfloat16()
    every = sum(p + 1 for p in range(c, c + q)) * B
    cases += [("latent, causal", lambda: k.paged_attention_wide(qq, lat, ctx, grp, nh, 1, hd, hd ** -0.5, 0.0, 0), every, B * (c + q) * hd * 2),
              ("latent, causal, a learned term", lambda: k.paged_attention_wide(qq, lat, ctx, grp, nh, 1, hd, hd ** -0.5, 0.0, 0, sinks=sinks),
               every, B * (c + q) * hd * 2)]
    for name, fn, n, nbytes in cases:
        if not name.startswith(a.only):
            continue
        us = _time_events(fn, a.replays, flush)
        print(f"attn_masked {name} B={B} qlen={q} ctx={c} nh={nh} nkv={nkv} hd={hd} span={span}: {us:.1f} us, "
              f"{flops(n) / us / 1e6:.1f} TFLOP/s of the attention's own flops, {nbytes / us / 1e3:.0f} GB/s of keys and values")
    print("status", ctx.status.tolist())
    return 0


def _attn_mixed(a) -> int:
    """Sigmoid attention whose heads' weights are mixed (the tiled kernel that owns all heads of a tile of tokens, and
    with --simple also the kernel of one warp per token, head and value head), and a retention's three kernels
    (prepare, the state-space scan with a group per head, gated norm per head) at the same head sizes: --batch requests
    of --qlen tokens behind --ctx tokens."""
    B, q, c, nh, nkv, hd, ps = a.batch, a.qlen, a.ctx if a.ctx != 8192 or a.qlen == 1 else 0, a.nh, a.nkv, a.hd, a.page
    ctx = _rows_ctx(B, q, c)
    per = -(-(c + q) // ps)
    flush = _flush()
    grp = SimpleNamespace(block_tables=torch.randperm(B * per + 8, device=DEV)[:B * per].int().view(B, per).contiguous(), page_size=ps)
    kv = torch.randn(B * per + 8, 2, nkv, ps, hd, device=DEV).bfloat16()
    qq = torch.randn(B * q, nh * hd, device=DEV)
    mix = (torch.eye(nh, device=DEV) + 0.1 * torch.randn(nh, nh, device=DEV)).contiguous()
    bias = torch.randn(nh, device=DEV) - 3.0
    every = sum(p + 1 for p in range(c, c + q)) * B                          # (query, key) pairs in sight
    fma = every * (nh * hd + nh * nh + nh * hd)                              # scores, the mix, the values: 32-bit multiply-adds
    kvb = B * (c + q) * nkv * hd * 2 * 2
    cases = [("tiled", lambda: k.sigmoid_attention(qq, kv, ctx, grp, nh, nkv, hd, hd, hd ** -0.5, 30.0, 0, ps, bias, mix, tiled=True))]
    if a.simple:
        cases.append(("one warp per token, head and value head",
                      lambda: k.sigmoid_attention(qq, kv, ctx, grp, nh, nkv, hd, hd, hd ** -0.5, 30.0, 0, ps, bias, mix, tiled=False)))
    for name, fn in cases:
        us = _time_events(fn, a.replays, flush)
        print(f"attn_mixed {name} B={B} qlen={q} ctx={c} nh={nh} nkv={nkv} hd={hd}: {us:.1f} us, {fma / us / 1e6:.2f} TFMA/s of "
              f"32-bit multiply-adds, {kvb / us / 1e3:.0f} GB/s of keys and values")
    # ---- the retention beside it: nh heads of hd values over hd rows of state
    H, D, P, T = nh, hd, hd, B * q
    proj = torch.randn(T, 2 * H * D + 2 * H * P, device=DEV)
    inv = torch.rand(D // 2, device=DEV)
    decay = torch.rand(H, device=DEV) * 0.1 + 0.9
    state = torch.randn(B, H * P * D, device=DEV) * 0.1
    zero = torch.zeros(H, device=DEV)
    xbc, dd = k.retention_prepare(proj, ctx.positions, inv, decay, H, D, P, D, D ** -0.5)
    o = k.ssm_scan(xbc, dd, zero, ctx, state, H, H, D, P)
    rows = [("retention_prepare", lambda: k.retention_prepare(proj, ctx.positions, inv, decay, H, D, P, D, D ** -0.5),
             T * (2 * H * D + H * P) * 8 + T * 2 * H * 4),
            ("ssm_scan, a group per head", lambda: k.ssm_scan(xbc, dd, zero, ctx, state, H, H, D, P),
             2 * B * H * P * D * 4 + T * (2 * H * D + 2 * H * P + 2 * H) * 4),
            ("retention_gate_norm", lambda: k.retention_gate_norm(o, proj[:, 2 * H * D + H * P:], 1e-6, H, P, torch.bfloat16),
             T * H * P * (4 + 4 + 2))]
    for name, fn, nbytes in rows:
        us = _time_events(fn, a.replays, flush)
        print(f"{name} B={B} qlen={q} heads={H} dim={D} vdim={P}: {us:.1f} us, {nbytes / 1e6:.1f} MB, {nbytes / us / 1e3:.0f} GB/s")
    print("status", ctx.status.tolist())
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--kernel", required=True, choices=["attn_decode", "attn_prefill", "gemv", "gemm", "sample", "recurrence", "attn_masked", "attn_mixed"])
    ap.add_argument("--simple", action="store_true", help="attn_mixed: time the kernel of one warp per token, head and value head too")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--ctx", type=int, default=8192, help="tokens already in the cache")
    ap.add_argument("--qlen", type=int, default=2048, help="tokens per row (attn_prefill)")
    ap.add_argument("--nh", type=int, default=32)
    ap.add_argument("--nkv", type=int, default=8)
    ap.add_argument("--hd", type=int, default=64)
    ap.add_argument("--page", type=int, default=16)
    ap.add_argument("--state", type=int, default=128, help="recurrence: rows of state per column (the delta rule's key size)")
    ap.add_argument("--groups", type=int, default=8, help="recurrence: groups that share B and C (the delta rule's key heads)")
    ap.add_argument("--taps", type=int, default=4)
    ap.add_argument("--span", type=int, default=1024, help="attn_masked: the window, and the length of a run of positions")
    ap.add_argument("--splits", type=int, default=0, help="0: the engine's own choice")
    ap.add_argument("--M", type=int, default=8)
    ap.add_argument("--N", type=int, default=2048)
    ap.add_argument("--K", type=int, default=8192)
    ap.add_argument("--dual", action="store_true", help="gemv: the gate/up product with SiLU-mul")
    ap.add_argument("--resident", action="store_true", help="one weight matrix, reused (it may stay in L2)")
    ap.add_argument("--only", default="", help="time only the implementations whose name starts so")
    ap.add_argument("--launches", type=int, default=10, help="kernel launches per graph")
    ap.add_argument("--replays", type=int, default=5)
    a = ap.parse_args(argv)
    if a.kernel == "recurrence":
        return _recurrence(a)
    if a.kernel == "attn_masked":
        return _attn_masked(a)
    if a.kernel == "attn_mixed":
        return _attn_mixed(a)
    if a.kernel == "attn_decode":
        qkv, kv, ctx, grp = _attention_inputs(a, 1)
        splits = a.splits or k.decode_splits(a.batch, a.nkv, a.ctx + 1, a.hd)
        # as in a model, where every layer has a cache of its own: more K and V than L2 holds
        copies = 1 if a.resident else max(1, int(400e6 // kv.numel() // 2) + 1)
        kvs = [kv] + [torch.randn_like(kv) for _ in range(copies - 1)]
        at = [0]

        def f():
            at[0] = (at[0] + 1) % copies
            return k.paged_attention_decode(qkv, kvs[at[0]], ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, 0, splits=splits)
        us = _time_graph(f, a.launches, a.replays)
        nbytes = a.batch * (a.ctx + 1) * a.nkv * a.hd * 2 * 2
        print(f"attn_decode B={a.batch} ctx={a.ctx} nh={a.nh} nkv={a.nkv} hd={a.hd} page={a.page} splits={splits}: "
              f"{us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of K and V")
    elif a.kernel == "attn_prefill":
        a.ctx = a.ctx if a.ctx != 8192 else 0
        qkv, kv, ctx, grp = _attention_inputs(a, a.qlen)
        flops = 4 * a.nh * a.hd * a.batch * (a.qlen * a.ctx + a.qlen * (a.qlen + 1) / 2)
        impls = [("mma.sync", lambda: k.paged_attention_prefill(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, 0))]
        if k.tc_attention_ok(a.nh, a.nkv, a.hd, a.page, 0):
            impls.append(("tcgen05, one query tile per CTA",
                          lambda: k.paged_attention_prefill_tc(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=1)))
            if (128 if a.hd == 64 else 64) % a.page == 0:
                impls.append(("tcgen05, two query tiles per CTA",
                              lambda: k.paged_attention_prefill_tc(qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=2, ksplits=1)))
                for ks in (2, 4):
                    if ks * qkv.shape[0] * a.nh * (a.hd + 2) > k.ATTN_SCRATCH_FLOATS:
                        continue
                    impls.append((f"tcgen05, two query tiles per CTA, keys in {ks} shares", (lambda ks: lambda: k.paged_attention_prefill_tc(
                        qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5, variant=2, ksplits=ks))(ks)))
                impls.append(("tcgen05, the library's choice", lambda: k.paged_attention_prefill_tc(
                    qkv, kv, ctx, grp, a.nh, a.nkv, a.hd, a.hd ** -0.5)))
        for name, f in impls:
            us = _time_graph(f, a.launches, a.replays)
            print(f"attn_prefill {name} B={a.batch} ctx={a.ctx} qlen={a.qlen} nh={a.nh} nkv={a.nkv} hd={a.hd}: {us:.1f} us, "
                  f"{flops / us / 1e6:.0f} TFLOP/s")
        print("status", ctx.status.tolist())
    elif a.kernel == "sample":
        # filters and draw over --batch rows of --N logits: the reference's default (top_p 0.95), top_p with top_k, none
        rows, V = a.batch, a.N
        logits = torch.randn(rows, V, device=DEV) * 2
        f = lambda v, dt=torch.float32: torch.full((rows,), v, dtype=dt, device=DEV)
        T, u = f(1.0), torch.rand(rows, device=DEV)
        cases = [("no filter", ()), ("top_p 0.95", (f(0.95), f(0.0), f(0, torch.int32), f(1, torch.int32))),
                 ("top_p 0.9, top_k 50", (f(0.9), f(0.0), f(50, torch.int32), f(1, torch.int32)))]
        for name, args in cases:
            if not name.startswith(a.only):
                continue
            if k.filter_sample_takes(V):
                us = _time_graph(lambda: k.filter_sample(logits, T, u, *args), a.launches, a.replays)
                print(f"sample rows={rows} V={V} {name}, one kernel on a cluster per row: {us:.1f} us")
            us = _time_graph(lambda: k.sample(logits, T, u, k.filter_mask(logits, *args) if args else None), a.launches, a.replays)
            print(f"sample rows={rows} V={V} {name}, filter kernel then sampling kernel: {us:.1f} us")
    elif a.kernel == "gemm":
        copies = 1 if a.resident else max(1, int(300e6 // (a.N * a.K * 2)) + 1)        # more weight than L2 holds
        ws = [torch.randn(a.N, a.K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(a.M, a.K, device=DEV, dtype=torch.bfloat16)
        st = torch.zeros(4, dtype=torch.int32, device=DEV)
        flops = 2.0 * a.M * a.N * a.K
        at = [0]

        def rotating(fn):
            def f():
                at[0] = (at[0] + 1) % copies
                return fn(ws[at[0]])
            return f
        impls = [("cublas", lambda w: torch.mm(x, w.t())),
                 ("tcgen05 bn128", lambda w: k.gemm_tcgen05(x, w, st, bn=128)),
                 ("tcgen05 bn256", lambda w: k.gemm_tcgen05(x, w, st, bn=256))]
        for name, fn in impls:
            if not name.startswith(a.only):
                continue
            us = _time_graph(rotating(fn), a.launches, a.replays)
            print(f"gemm M={a.M} N={a.N} K={a.K} {name}: {us:.1f} us, {flops / us / 1e6:.0f} TFLOP/s")
        print("status", st.tolist())
    else:
        copies = 1 if a.resident else max(1, int(300e6 // (a.N * a.K * 2)) + 1)        # more weight than L2 holds
        ws = [torch.randn(a.N, a.K, device=DEV, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(a.M, a.K, device=DEV, dtype=torch.bfloat16)
        st = torch.zeros(4, dtype=torch.int32, device=DEV)
        k.set_status_word(x.device, st)
        at = [0]

        def rotating(fn):
            def f():
                at[0] = (at[0] + 1) % copies
                return fn(ws[at[0]])
            return f
        impls = [("cublas", lambda w: torch.mm(x, w.t()))]
        if a.M <= 16:
            impls.append(("gemv 8 features", lambda w: k.gemv(x, w, wide=8, warps=8)))
            impls.append(("gemv 16 features", lambda w: k.gemv(x, w, wide=16, warps=8)))
            impls.append(("gemv 32 features", lambda w: k.gemv(x, w, wide=32, warps=8)))
            impls.append(("gemv 8 features, 16 warps", lambda w: k.gemv(x, w, wide=8, warps=16)))
            impls.append(("gemv 16 features, 16 warps", lambda w: k.gemv(x, w, wide=16, warps=16)))
        if a.dual:                      # N rows of gate and up in blocks of 128, SiLU-mul in the epilogue
            impls = [(f"gemv gate/up {wd} features", (lambda wd: lambda w: k.gemv(x, w, block=128, wide=wd))(wd))
                     for wd in (8, 16, 32) if a.M <= 16]
            impls.append(("library product, then SiLU-mul", lambda w: k.silu_mul(torch.mm(x, w.t()), 128)))
        for name, fn in impls:
            if not name.startswith(a.only):
                continue
            us = _time_graph(rotating(fn), a.launches, a.replays)
            print(f"gemv M={a.M} N={a.N} K={a.K} {name}: {us:.1f} us, {a.N * a.K * 2 / us / 1e3:.0f} GB/s of weights")
        print("status", st.tolist())
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
