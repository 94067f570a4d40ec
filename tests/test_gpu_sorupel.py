"""Sorupel on the GPU against the plain model of tests/plain_sorupel.py: whole prompts against decoding token by
token, portions down to two tokens, mixed batches over pools and slots that are used again, each mixer alone through
the cache manager (edges of a run of positions, a far key among hundreds, the first tokens, terms without a value,
state carried over long decoding), the bigram embedding's state, and greedy generation through the engine."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_sorupel as ps
import tiny
import tiny_sorupel as ts
import traces

pytestmark = pytest.mark.gpu

# Largest |difference| as a fraction of the largest |logit| of the plain model (float64).  32-bit: float32
# sums against float64.  bfloat16: weights are bfloat16 in both; the engine rounds activations.
TOL = {"float32": 2e-5, "bfloat16": 4e-2}
CASES = {
    "S1": dict(lens=[1, 2, 7, 45, 38, 100, 39, 76, 131], page=16, max_tokens=448),
    "S2": dict(lens=[3, 17, 72, 140, 71, 33, 90], page=16, max_tokens=384),
    "S3": dict(lens=[5, 64, 33, 230, 20, 101, 70], page=32, max_tokens=512),
    "S4": dict(lens=[4, 40, 23, 66, 35, 80], page=16, max_tokens=256),
}


def _prompts(name):
    return {f"r{i}": tiny.rand_tokens(n, ts.CONFIGS[name]["vocab"], 300 + i) for i, n in enumerate(CASES[name]["lens"])}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("sorupel")
    out = {}
    for name, cfg in ts.CONFIGS.items():
        d = ts.make_model_dir(root, cfg, seed=29)
        W = tiny.load_plain_weights(d)
        prompts = _prompts(name)
        out[name] = (d, W, prompts, {r: ps.forward(cfg, W, t) for r, t in prompts.items()})
    return out


def _run(model_dir, dtype, steps, max_tokens, page, max_live=4):
    from fastmlx_b200.engine.replay import Replayer
    rp = Replayer(model_dir, dtype, max_tokens, page_size=page, max_live=max_live)
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    assert not rp.manager.requests and all(g.pool.used_pages == 0 for g in rp.manager.groups)
    return outs, rp


def _compare(steps, outs, prompts, ref, tol):
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max(dim=1).values / ref[rid].abs().max().item()
        bad = torch.nonzero(err > tol)
        assert bad.numel() == 0, (f"request {rid}: first wrong position {int(bad[0])} of {len(toks)}, "
                                  f"error {err[int(bad[0])].item():.3e} (allowed {tol:.1e})")


CUTS = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions, "mixed": traces.mixed,
        "ones": lambda p: traces.tail_decoded(p, tail=10 ** 6)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["S1", "S2", "S3", "S4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "ones"])
def test_replay(models, name, dtype, cut):
    d, W, prompts, ref = models[name]
    case = CASES[name]
    steps = CUTS[cut](prompts)
    outs, rp = _run(d, dtype, steps, case["max_tokens"], case["page"])
    _compare(steps, outs, prompts, ref, TOL[dtype])
    if cut == "mixed":
        need = sum(-(-len(t) // case["page"]) for t in prompts.values())
        assert any(need > g.pool.num_pages for g in rp.manager.groups), "the pools are too large for pages to be used again"
        assert len(prompts) > rp.manager.max_requests, "too many slots for one to be used again"


@pytest.mark.parametrize("name", ["S1", "S4"])
def test_cuts_agree_in_32_bit(models, name):
    """The logits at a place do not depend on the cut, the batch, the pages or the slot beyond the order of 32-bit
    sums: far inside the allowance against the plain model."""
    d, W, prompts, ref = models[name]
    case = CASES[name]
    base_steps = traces.whole(prompts)
    base = traces.collect(base_steps, _run(d, "float32", base_steps, case["max_tokens"], case["page"])[0])
    for cut in ("tail", "portions", "mixed"):
        steps = CUTS[cut](prompts)
        rows = traces.collect(steps, _run(d, "float32", steps, case["max_tokens"], case["page"])[0])
        for rid in prompts:
            scale = float(ref[rid].abs().max())
            for i, row in rows[rid].items():
                assert np.abs(row - base[rid][i]).max() <= 4e-6 * scale, (cut, rid, i, np.abs(row - base[rid][i]).max())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_carries_state_and_passes_runs_of_positions(models, dtype):
    """190 tokens decoded one by one behind a short prompt: several runs of positions (37 and 5 long) begin among the
    decoded tokens, the recurrence's state and the previous token are carried through every step."""
    d, W, prompts, ref = models["S1"]
    toks = tiny.rand_tokens(200, ts.S1["vocab"], 77)
    sub = {"long": toks}
    want = {"long": ps.forward(ts.S1, W, toks)}
    steps = traces.tail_decoded(sub, tail=190)
    outs, _ = _run(d, dtype, steps, 256, 16)
    _compare(steps, outs, sub, want, TOL[dtype])


# ----------------------------------------------------------------------------- each mixer alone
class Rig:
    """A one-layer model's mixer part over the engine's cache manager: requests are fed the mixer's inputs in given
    portions, from and into the pages and state slots that the manager hands out."""

    def __init__(self, root, kind, mixer, overrides, width, dtype, page=16, max_tokens=640, max_live=5, eps=1e-6, seed=3):
        from fastmlx_b200.engine.replay import Replayer
        from fastmlx_b200.weights import safetensors_io as st
        self.cfg = ts.one_layer(kind, mixer, width=width, eps=eps)
        self.mixer_cfg, self.eps, self.page = mixer, eps, page
        tensors = ts.lively_tensors(self.cfg, seed)
        for name, t in overrides.items():
            assert tensors["l0.mix." + name].shape == t.shape, name
            tensors["l0.mix." + name] = t.to(torch.bfloat16)
        d = os.path.join(str(root), f"rig_{kind}_{dtype}_{seed}")
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(self.cfg, f)
        st.write_file(os.path.join(d, "model.safetensors"), tensors, {"format": "pt"})
        self.W = {n[len("l0.mix."):]: t.double() for n, t in tensors.items() if n.startswith("l0.mix.")}
        self.rp = Replayer(d, dtype, max_tokens, page_size=page, max_live=max_live)
        self.part = self.rp.model.layers[0].mixer
        m = self.rp.manager
        m.reserve(m.add_request("spare"), 3 * page)          # the first pages and slot 0 are not the requests' own

    def feed(self, hs, lens_by_step, ids=None):
        """hs[r]: request r's inputs [n_r, width] (float64, representable in the run's type).  -> outputs per request."""
        from fastmlx_b200.engine.batch import StepEntry, build_context
        m, rt = self.rp.manager, self.rp.rt
        ids = ids or [f"q{r}" for r in range(len(hs))]
        reqs = [m.add_request(i) for i in ids]
        got, at = [[] for _ in hs], [0] * len(hs)
        for step_lens in lens_by_step:
            live = [(r, n) for r, n in enumerate(step_lens) if n > 0]
            entries = [StepEntry(reqs[r], [0] * n, []) for r, n in live]
            for e in entries:
                m.reserve(e.request, len(e.tokens))
            ctx = build_context(entries, m, rt.device, self.rp.step_fn.status)
            x = torch.cat([hs[r][at[r]:at[r] + n] for r, n in live]).to(rt.dtype).to(rt.device).contiguous()
            y = self.part.forward(x, ctx, ctx.caches[0]).double().cpu()
            off = 0
            for r, n in live:
                got[r].append(y[off:off + n])
                off += n
                at[r] += n
                m.commit(reqs[r])
            m.check()
        self.rp.step_fn.check_status()
        for i in ids:
            m.free(i)
        return [torch.cat(x) for x in got]


def _close(got, want, tol):
    err = (got - want).abs().max(dim=1).values / want.abs().max().item()
    bad = torch.nonzero(err > tol)
    assert bad.numel() == 0, f"first wrong position {int(bad[0])} of {got.shape[0]}: {err[int(bad[0])].item():.3e} (allowed {tol:.1e})"


def _rounded(x):
    return x.bfloat16().double()


@pytest.mark.parametrize("dtype,D,scale", [("float32", 64, 0.4), ("bfloat16", 64, 0.4), ("bfloat16", 40, 0.6)],
                         ids=["float32", "bfloat16-tiled", "bfloat16"])
@pytest.mark.parametrize("edge", ["inside", "outside"])
@pytest.mark.parametrize("how", ["prompt", "portions", "decoded"])
def test_chunked_attention_edge_of_a_run(tmp_path, dtype, D, scale, edge, how):
    """Every query of a run of 37 positions points at one key: the run's first position, or the position before it.
    Its value (the key as projected) must be the output, or must not be in it.  Queries read the first D inputs and
    keys the next D, so that the two can be set apart; pages of earlier runs go back to the pool on the way."""
    size, H, n = 37, 2, 150
    width = 2 * D
    mixer = ts.attention(H, 1, D, scale, softcap=40.0, chunk=size, rot=(16, 10000.0))
    eye, zero = torch.eye(D), torch.zeros(D, D)
    over = {"q": torch.cat([torch.cat([eye, zero], 1)] * H, 0), "k": torch.cat([zero, eye], 1), "o": torch.eye(width),
            "q.norm": torch.ones(H * D), "k.norm": torch.ones(D)}
    rig = Rig(tmp_path, "attention", mixer, over, width, dtype)
    g = torch.Generator().manual_seed(D)
    h0 = torch.randn(n, width, generator=g, dtype=torch.float64)
    runs = -(-n // size)
    u = torch.zeros(runs, D, dtype=torch.float64)
    u[:, 16:] = torch.randn(runs, D - 16, generator=g, dtype=torch.float64)     # on the dimensions that do not turn
    u = u / u.norm(dim=1, keepdim=True)
    for p in range(n):
        h0[p, :D] = 8.0 * u[p // size] + 0.3 * h0[p, :D]
    for c in range(runs):
        j = c * size if edge == "inside" else c * size - 1
        if j >= 0:
            h0[j, D:] = 8.0 * u[c]
    hs = [_rounded(h0), _rounded(torch.randn(40, width, generator=g, dtype=torch.float64))]
    want = [ps.chunked_attention(h, rig.W, mixer, rig.eps) for h in hs]
    steps = {"prompt": [[n, 40]], "portions": [[31, 3], [2, 1], [37, 30], [38, 2], [42, 4]],
             "decoded": [[60, 1]] + [[1, 0]] * 90}[how]
    got = rig.feed(hs, steps)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for r in range(2):
        _close(got[r], want[r][:got[r].shape[0]], tol)
    # the oracle itself shows the edge: where the key is seen, a head's output is the key's value times its gate
    p = 100
    gate = torch.sigmoid(hs[0][p] @ rig.W["g"].T)
    near = (want[0][p, :D] / gate[0] - 8.0 * u[p // size]).abs().max().item()
    assert (near < 0.1) == (edge == "inside"), near


@pytest.mark.parametrize("dtype,R", [("float32", 8), ("bfloat16", 8), ("bfloat16", 16)], ids=["float32", "bfloat16", "bfloat16-tiled"])
def test_latent_attention_far_key_first_tokens_and_learned_sink(tmp_path, dtype, R):
    """Every query points at the latent of position 1: far back among hundreds for late queries, the first tokens for
    early ones.  One head's learned term in the denominator is as large as that score, so that it takes a known
    share; the other's is small.  Three requests of unequal length, page borders, single tokens and portions."""
    H, D, r = 2, 32, 32
    width = 128
    mixer = ts.latent(H, D, R, D, r, 0.2, 10000.0)
    pick = lambda rows, lo, s=1.0: torch.cat([torch.zeros(rows, lo), s * torch.eye(rows), torch.zeros(rows, width - lo - rows)], 1)
    wq = torch.cat([torch.cat([pick(D, 0), pick(R, 80, 0.3)], 0)] * H, 0)                # per head [D from 0.. | R from 80..]
    over = {"q": wq, "dkv": torch.cat([pick(r, 32), pick(R, 64, 0.3)], 0), "dkv.norm": torch.ones(r),
            "uk": torch.cat([torch.eye(r)] * H, 0), "uv": torch.cat([torch.eye(r)] * H, 0),
            "sink": torch.tensor([0.0, 30.0]), "o": torch.cat([torch.eye(H * D), torch.zeros(width - H * D, H * D)], 0)}
    rig = Rig(tmp_path, "latent_attention", mixer, over, width, dtype)
    g = torch.Generator().manual_seed(R)
    lens = [397, 22, 129]
    hs = [torch.randn(n, width, generator=g, dtype=torch.float64) for n in lens]
    c1 = ps.rms_norm(_rounded(hs[0])[1, 32:64], rig.eps)
    hs[0][:, :D] = 5.0 * c1
    hs = [_rounded(h) for h in hs]
    want = [ps.latent_attention(h, rig.W, mixer, rig.eps)[0] for h in hs]
    got = rig.feed(hs, [[330, 5, 64], [1, 1, 64], [2, 0, 1], [64, 16, 0]])
    tol = 2e-5 if dtype == "float32" else 3e-2
    for a, b in zip(got, want):
        _close(a, b, tol)
    # the oracle: head 0 gives the latent of position 1, head 1 its share beside the learned term
    p = 390
    gate = torch.sigmoid(hs[0][p] @ rig.W["g"].T)
    c1 = ps.rms_norm(hs[0][1, 32:64], rig.eps)
    s = (5.0 * c1 @ c1) * 0.2
    share = 1.0 / (1.0 + math.exp(30.0 - float(s)))
    assert (want[0][p, :D] / gate[:D] - c1).abs().max().item() < 0.05
    assert (want[0][p, D:2 * D] / gate[D:] - share * c1).abs().max().item() < 0.05 and 0.5 < share < 0.95


@pytest.mark.parametrize("kind,mixer", [
    ("latent_attention", ts.latent(20, 16, 16, 16, 176, 0.2, 5000.0)),       # cache rows of 192 values, 20 heads on them
    ("latent_attention", ts.latent(32, 16, 32, 16, 224, 0.15, 5000.0)),      # rows of 256, 32 heads
    ("latent_attention", ts.latent(12, 16, 16, 16, 128, 0.2, 5000.0)),       # rows of 144, heads that fit one warp's rows
    ("attention", ts.attention(24, 1, 64, 0.3, softcap=20.0, chunk=150, rot=(32, 3000.0))),
    ("attention", ts.attention(40, 2, 64, 0.3, chunk=90, rot=(16, 3000.0))),
    ("attention", ts.attention(64, 2, 32, 0.3, softcap=20.0, chunk=400)),
], ids=["latent-20x192", "latent-32x256", "latent-12x144", "attention-24:1", "attention-40:2", "attention-64:2"])
def test_single_tokens_with_many_heads_on_one_key_head(tmp_path, kind, mixer):
    """Single tokens of 17 to 32 query heads per key head share a tile's keys out over pairs of warps, and cache rows
    wider than 128 values keep the queries' terms in shared memory: three requests of unequal length, decoded one by
    one side by side behind prompts, short enough for one block per row and long enough for shares of the keys."""
    width = 96
    rig = Rig(tmp_path, kind, mixer, {}, width, "bfloat16", max_tokens=1024)
    g = torch.Generator().manual_seed(11)
    lens = [420, 37, 150]
    hs = [_rounded(torch.randn(n, width, generator=g, dtype=torch.float64)) for n in lens]
    plain = ps.latent_attention if kind == "latent_attention" else ps.chunked_attention
    want = [plain(h, rig.W, mixer, rig.eps) for h in hs]
    want = [w[0] if isinstance(w, tuple) else w for w in want]
    steps = [[380, 3, 120]] + [[1, 1, 1]] * 30 + [[1, 0, 0]] * 10
    got = rig.feed(hs, steps)
    for a, b in zip(got, want):
        _close(a, b[:a.shape[0]], 3e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(4, 10, 12, 2, 2, 3), (1, 64, 8, 1, 1, 4), (6, 32, 64, 3, 4, 2), (3, 7, 100, 1, 3, 5),
                                   (4, 5, 9, 4, 1, 1), (2, 8, 300, 1, 1, 2)], ids=lambda s: "x".join(map(str, s)))
def test_state_space_mixer_alone(tmp_path, dtype, shape):
    """(heads, vdim, state, groups, norm parts, taps).  Three requests in portions of one, two and many tokens; one
    head decays so slowly that the first token still counts after 300; then the slots are given back and taken again by
    new requests, which must start from zero state and an empty convolution."""
    H, P, N, G, parts, taps = shape
    width = 48
    mixer = ts.mamba(H, P, N, G, parts, taps)
    slow = torch.full((H,), -1.0)
    slow[0] = -9.0                                   # exp(-exp(-9) dt) is 1 - 1e-4 dt: nothing is forgotten
    rig = Rig(tmp_path, "mamba2", mixer, {"A_log": slow}, width, dtype, seed=H * 10 + taps)
    g = torch.Generator().manual_seed(N)
    lens = [300, 41, 9]
    hs = [_rounded(torch.randn(n, width, generator=g, dtype=torch.float64)) for n in lens]
    want = [ps.state_space(h, rig.W, mixer, rig.eps) for h in hs]
    steps = [[200, 1, 2], [1, 2, 1], [2, 30, 1], [1, 1, 2], [64, 7, 3], [32, 0, 0]]
    tol = 2e-5 if dtype == "float32" else 3e-2
    for a, b in zip(rig.feed(hs, steps), want):
        _close(a, b, tol)
    # the first token's mark on the last output of the long request: the plain model with token 0 changed differs
    other = hs[0].clone()
    other[0] = -other[0]
    assert (ps.state_space(other, rig.W, mixer, rig.eps)[-1] - want[0][-1]).abs().max() > 1e-3 * want[0].abs().max()
    # slots that held state are used again
    again = [hs[2], hs[1]]
    for a, b in zip(rig.feed(again, [[4, 40], [5, 1]], ids=["n0", "n1"]), [want[2], want[1]]):
        _close(a, b, tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("buckets,mul_prev,mul_cur", [(53, 31, 7), (7, 1, 0), (1, 5, 3), (1000, 65537, 40503)])
def test_bigram_embedding_keeps_the_previous_token_per_request(tmp_path, dtype, buckets, mul_prev, mul_cur):
    """Rows of the bigram table through portions and single tokens; the first token of a sequence takes the last row,
    also in a slot that another request has just left."""
    from fastmlx_b200.engine.batch import StepEntry, build_context
    from fastmlx_b200.engine.replay import Replayer
    vocab = 61
    cfg = ts.one_layer("mamba2", ts.mamba(2, 4, 4, 1, 1, 2), width=40, vocab=vocab, embedding=ts.bigram(buckets, mul_prev, mul_cur))
    d = ts.make_model_dir(tmp_path, cfg, seed=buckets)
    W = {n: t.double() for n, t in tiny.load_plain_weights(d).items()}
    rp = Replayer(d, dtype, 256, page_size=16, max_live=3)
    m, model = rp.manager, rp.model
    seqs = {i: torch.tensor(tiny.rand_tokens(n, vocab, 40 + i)) for i, n in enumerate([30, 12, 5, 17])}
    want = {i: ps.embed(s, W, cfg) for i, s in seqs.items()}

    def feed(order, lens_by_step):
        reqs = {i: m.add_request(f"e{i}") for i in order}
        at = {i: 0 for i in order}
        for step_lens in lens_by_step:
            live = [(i, n) for i, n in zip(order, step_lens) if n > 0]
            entries = [StepEntry(reqs[i], seqs[i][at[i]:at[i] + n].tolist(), []) for i, n in live]
            for e in entries:
                m.reserve(e.request, len(e.tokens))
            ctx = build_context(entries, m, rp.rt.device, rp.step_fn.status)
            x = model.embed.forward(ctx.tokens, ctx, ctx.caches[model.embed_entry]).double().cpu()
            off = 0
            for i, n in live:
                assert torch.allclose(x[off:off + n], want[i][at[i]:at[i] + n], atol=1e-6 if dtype == "float32" else 2e-2), (i, at[i])
                off += n
                at[i] += n
                m.commit(reqs[i])
        rp.step_fn.check_status()
        return at

    at = feed([0, 1, 2], [[1, 5, 2], [1, 1, 3], [2, 0, 0], [20, 6, 0], [6, 0, 0]])
    assert at == {0: 30, 1: 12, 2: 5}
    m.free("e1")
    slot = m.requests["e0"].slot
    m.free("e0")
    feed([3], [[1], [2], [14]])                       # takes a slot that was just given back
    assert m.requests["e3"].slot in (slot, 0, 1, 2)
    first = ps.embed(seqs[3][:1], W, cfg)[0]
    assert torch.allclose(first, W["embed"][seqs[3][0]] + W["bigram"][buckets])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_product_with_gelu(dtype):
    """act(gate) * up over joined products, plain and in blocks of 128, against the tanh form written out."""
    from fastmlx_b200 import kernels as k
    g = torch.Generator().manual_seed(8)
    for ff, block in ((40, None), (256, 128), (328, None)):
        gu = (torch.randn(9, 2 * ff, generator=g) * 3).to(dtype)
        if block:
            a = gu.view(9, -1, 2, block)
            gate, up = a[:, :, 0].reshape(9, ff).double(), a[:, :, 1].reshape(9, ff).double()
        else:
            gate, up = gu[:, :ff].double(), gu[:, ff:].double()
        want = ps.gelu_tanh(gate) * up
        got = k.act_mul(gu.cuda(), "gelu_tanh", block).cpu().double()
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(got, want, rtol=tol, atol=tol), (ff, block)


def test_gelu_gated_product_in_the_products_epilogue():
    """The decode product (at most 16 rows) and the tensor-memory product of prompt portions apply gelu(gate) * up
    themselves over weights whose gate and up rows alternate in blocks of 128, as the separate kernel does."""
    from fastmlx_b200 import kernels as k
    dev = torch.device("cuda")
    g = torch.Generator().manual_seed(12)
    ff, width, block = 512, 256, 128
    w = (torch.randn(2 * ff, width, generator=g) * 0.15).bfloat16()
    rows = w.view(ff // block, 2, block, width).double()
    wg, wu = rows[:, 0].reshape(ff, width), rows[:, 1].reshape(ff, width)
    for M in (1, 5, 16, 384):
        x = torch.randn(M, width, generator=g).bfloat16()
        gate, up = (x.double() @ wg.T).bfloat16().double(), (x.double() @ wu.T).bfloat16().double()
        want = ps.gelu_tanh(gate) * up
        if M <= 16:
            got = k.gemv(x.to(dev), w.to(dev), block=block, act="gelu_tanh")
            silu = k.gemv(x.to(dev), w.to(dev), block=block)
            assert torch.allclose(silu.cpu().double(), ps.silu(gate) * up, rtol=2e-2, atol=2e-2)     # the other gate is as it was
        else:
            got = k.gemm_tcgen05(x.to(dev), w.to(dev), epilogue=k.EPI_GELU_MUL)
        assert got.shape == (M, ff)
        assert torch.allclose(got.cpu().double(), want, rtol=2e-2, atol=2e-2), M
        unfused = k.act_mul(k.linear(x.to(dev), w.to(dev), None, torch.bfloat16), "gelu_tanh", block)
        assert (got.float() - unfused.float()).abs().max().item() <= 2.0 ** -7 * want.abs().max().item()


# ----------------------------------------------------------------------------- the engine
def _plain_greedy(cfg, W, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        row = ps.forward(cfg, W, toks)[-1]
        top = torch.topk(row, 2).values
        margins.append(float(top[0] - top[1]) / float(row.abs().max()))
        out.append(int(torch.argmax(row)))
        toks.append(out[-1])
    return out, margins


@pytest.mark.parametrize("dtype,slack", [("float32", 1e-5), ("bfloat16", 4e-2)])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(models, dtype, slack, graphs):
    """Six prompts over three slots, portions of 16 tokens: the scheduler admits, cuts and batches; slots and
    pages are used again; decode steps replay CUDA graphs where asked."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["S1"]
    cfg = ts.S1
    prompts = [tiny.rand_tokens(n, cfg["vocab"], 500 + n) for n in (1, 9, 40, 23, 3, 57)]
    eng = Engine(d, dtype=dtype, block_size=16, max_cache_tokens=512, max_concurrent_requests=3, prefill_chunk=16,
                 cuda_graphs=graphs)
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0))
    for p, out in zip(prompts, outs):
        assert out.finished and out.completion_tokens == 12
        want, margins = _plain_greedy(cfg, W, p, 12)
        for i, (a, b) in enumerate(zip(out.output_token_ids, want)):
            if a != b:
                assert margins[i] < slack, (i, a, b, margins[i])
                break                                   # after a tie that went the other way the texts differ
    st = eng.stats()
    assert st["pages_used"] == 0
    if graphs:
        assert st["graph_replays"] > 0


def test_command_line_and_trace_program(models, tmp_path):
    """`python -m fastmlx_b200 generate` and bin/trace_run on a Sorupel folder, as a user runs them."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, W, prompts, ref = models["S4"]
    out = subprocess.run([sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids",
                          "5,6,7;9", "--max-tokens", "5", "--temperature", "0", "--max-cache-tokens", "256"], cwd=root,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(x) for x in out.stdout.splitlines() if x.startswith("{")]
    assert [len(x["output_token_ids"]) for x in lines] == [5, 5]
    want, margins = _plain_greedy(ts.S4, W, [5, 6, 7], 5)
    for i, (a, b) in enumerate(zip(lines[0]["output_token_ids"], want)):
        if a != b:
            assert margins[i] < 1e-5
            break
    sub = {r: prompts[r] for r in ("r1", "r2", "r3")}
    steps = traces.mixed(sub)
    outdir = tmp_path / "out"
    proc = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", d, "--dtype", "float32", "--out", str(outdir),
                           "--max-tokens", "256"], input="".join(json.dumps(s) + "\n" for s in steps), cwd=root,
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [x for x in proc.stdout.splitlines() if x.startswith("done ")] == [f"done {s['step']}" for s in steps]
    outs = [np.fromfile(outdir / f"{s['step']}.f32", dtype="<f4").reshape(-1, ts.S4["vocab"]) for s in steps]
    _compare(steps, outs, sub, ref, TOL["float32"])


def test_preemption_recomputes_state_and_changes_no_token(models):
    """A pool too small for three requests to grow together: the scheduler preempts the newest, frees its pages and its
    state slots, and recomputes it later from zero state and no previous token; in 32-bit every request still produces
    what it produces with room to spare."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["S2"]                        # its attention layer has no mask: every key is kept
    prompts = [tiny.rand_tokens(n, ts.S2["vocab"], 900 + n) for n in (30, 28, 25)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    tight = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=18, max_concurrent_requests=4)
    outs = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    roomy = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=64, max_concurrent_requests=4)
    assert [o.output_token_ids for o in outs] == [o.output_token_ids for o in roomy.generate(prompts, sp)]
    assert all(o.finish_reason == "length" and len(o.output_token_ids) == 40 for o in outs)
    assert tight.stats()["pages_used"] == 0
    tight.manager.check()
