"""Kafepel on the GPU against the plain model of tests/plain_kafepel.py: whole prompts against decoding token by
token, portions down to two tokens, mixed batches over pools and slots that are used again, each branch of the mixer
alone through the cache manager (a far key among hundreds, page borders, the first tokens, a head mix that moves one
head's weights to another's values, state carried over long decoding, decays of 0 and 1), the kernels alone against
their plain statements, and greedy generation through the engine."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_kafepel as pk
import plain_ops
import tiny
import tiny_kafepel as tk
import traces

pytestmark = pytest.mark.gpu

# Largest |difference| as a fraction of the largest |logit| of the plain model (float64).  32-bit: float32
# sums against float64 (a retention's read-out over one or two keys whose dot products nearly cancel, then divided by
# its own root mean square, is the worst place: a sequence's first tokens).  bfloat16: weights are bfloat16 in both;
# the engine rounds activations; at such a place the rounding of the layer's input shows several times larger, so a
# few positions (FEW of all that are compared) may pass the allowance, none by more than WORST times.
TOL = {"float32": 5e-5, "bfloat16": 4e-2}
FEW, WORST = 0.03, 5.0
CASES = {
    "K1": dict(lens=[1, 2, 7, 45, 38, 100, 39, 76, 131], page=16, max_tokens=448),
    "K2": dict(lens=[3, 17, 72, 140, 71, 33, 90], page=16, max_tokens=384),
    "K3": dict(lens=[5, 64, 33, 230, 20, 101, 70], page=32, max_tokens=512),
    "K4": dict(lens=[4, 40, 23, 66, 35, 80], page=16, max_tokens=256),
}


# A router that takes bfloat16 inputs sees its scores moved a little; where the plain model's own choice of experts is
# decided by less (in some layer), either choice is right, and what the other choice does to the stream is carried on
# by the recurrence for some tokens: such a position and the SPAN - 1 after it are not compared in bfloat16.
CLOSE_CALL, SPAN = 0.005, 12


def _unsure(cfg, W, toks):
    """-> (logits of the plain model, the positions that are not compared in bfloat16)."""
    margins = []
    ref = pk.forward(cfg, W, toks, margins=margins)
    skip = torch.zeros(len(toks), dtype=torch.bool)
    if margins:
        for u in torch.nonzero(torch.stack(margins).min(0).values < CLOSE_CALL).flatten().tolist():
            skip[u:u + SPAN] = True
    return ref, skip


def _prompts(name):
    return {f"r{i}": tiny.rand_tokens(n, tk.CONFIGS[name]["vocab"], 300 + i) for i, n in enumerate(CASES[name]["lens"])}


SKIP = {}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("kafepel")
    out = {}
    for name, cfg in tk.CONFIGS.items():
        d = tk.make_model_dir(root, cfg, seed=29)
        W = tiny.load_plain_weights(d)
        prompts = _prompts(name)
        both = {r: _unsure(cfg, W, t) for r, t in prompts.items()}
        SKIP[name] = {r: b[1] for r, b in both.items()}
        out[name] = (d, W, prompts, {r: b[0] for r, b in both.items()})
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


def _compare(steps, outs, prompts, ref, tol, skip=None):
    rows = traces.collect(steps, outs)
    total = sum(len(t) for t in prompts.values())
    compared = total - (sum(int(skip[r].sum()) for r in prompts) if skip is not None else 0)
    assert compared > 0.4 * total or total < 16, "too few positions are compared"
    over = 0
    for rid, toks in prompts.items():
        assert sorted(rows[rid]) == list(range(len(toks)))
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max(dim=1).values / ref[rid].abs().max().item()
        if skip is not None:
            err = err.masked_fill(skip[rid], 0.0)
        bad = torch.nonzero(err > (tol if skip is None else WORST * tol))
        assert bad.numel() == 0, (f"request {rid}: first wrong position {int(bad[0])} of {len(toks)}, "
                                  f"error {err[int(bad[0])].item():.3e} (allowed {tol:.1e})")
        over += int((err > tol).sum())
    assert over <= max(1, int(FEW * compared)), f"{over} of {compared} positions are over the allowance"


CUTS = {"whole": traces.whole, "tail": traces.tail_decoded, "portions": traces.portions, "mixed": traces.mixed,
        "ones": lambda p: traces.tail_decoded(p, tail=10 ** 6)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed", "ones"])
def test_replay(models, name, dtype, cut):
    d, W, prompts, ref = models[name]
    case = CASES[name]
    steps = CUTS[cut](prompts)
    outs, rp = _run(d, dtype, steps, case["max_tokens"], case["page"])
    _compare(steps, outs, prompts, ref, TOL[dtype], SKIP[name] if dtype == "bfloat16" else None)
    if cut == "mixed":
        need = sum(-(-len(t) // case["page"]) for t in prompts.values())
        assert any(need > g.pool.num_pages for g in rp.manager.groups), "the pools are too large for pages to be used again"
        assert len(prompts) > rp.manager.max_requests, "too many slots for one to be used again"


@pytest.mark.parametrize("name", ["K1", "K4"])
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
@pytest.mark.parametrize("name", ["K1", "K2"])
def test_long_decoding_carries_state(models, dtype, name):
    """190 tokens decoded one by one behind a short prompt: the retention's state is carried through every step and the
    attention's context grows over many pages."""
    d, W, prompts, ref = models[name]
    cfg = tk.CONFIGS[name]
    toks = tiny.rand_tokens(200, cfg["vocab"], 77)
    sub = {"long": toks}
    ref, skip = _unsure(cfg, W, toks)
    steps = traces.tail_decoded(sub, tail=190)
    outs, _ = _run(d, dtype, steps, 256, CASES[name]["page"])
    _compare(steps, outs, sub, {"long": ref}, TOL[dtype], {"long": skip} if dtype == "bfloat16" else None)


# ----------------------------------------------------------------------------- each branch alone
class Rig:
    """A one-layer model's mixer part over the engine's cache manager: requests are fed the mixer's inputs in given
    portions, from and into the pages and state slots that the manager hands out."""

    def __init__(self, root, lft, rgt, overrides, width, dtype, page=16, max_tokens=640, max_live=5, eps=1e-6, seed=3):
        from fastmlx_b200.engine.replay import Replayer
        from fastmlx_b200.weights import safetensors_io as st
        self.cfg = tk.one_layer(lft, rgt, width=width, eps=eps)
        self.eps, self.page = eps, page
        tensors = tk.lively_tensors(self.cfg, seed)
        for name, t in overrides.items():
            assert tensors["l0.mix." + name].shape == t.shape, name
            tensors["l0.mix." + name] = t.to(torch.bfloat16)
        d = os.path.join(str(root), f"rig_{dtype}_{seed}")
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


def _pair(h, W, cfg_mixer, eps):
    return pk.parallel_mixer(h, W, cfg_mixer, eps)


@pytest.mark.parametrize("dtype,H,G,D", [("float32", 4, 2, 32), ("bfloat16", 4, 2, 32), ("bfloat16", 32, 2, 16), ("bfloat16", 3, 3, 40)],
                         ids=["float32", "bfloat16-tiled", "bfloat16-sixteen-heads-a-key-head", "bfloat16-odd"])
@pytest.mark.parametrize("how", ["prompt", "portions", "decoded"])
def test_sigmoid_attention_far_key_first_tokens_and_head_mix(tmp_path, dtype, H, G, D, how):
    """Every query of head 0 points at the key of position 1 and at nothing else (the number in front of the sigmoid is
    -12, so every other weight vanishes): far back among hundreds for late queries, the first tokens for early ones.
    The head mix hands head 0's weights to the last head alone, which belongs to another key/value head where there
    are several: the output must be position 1's value of THAT head.  The retention branch's output projection is zero."""
    width = max(128, H * D)
    lft = tk.left(H, G, D, D, 1.0, softcap=60.0, rot=tk.rot(8, 10000.0))
    rgt = tk.right(8, 8, (0.9, 0.5))
    pick = lambda rows, lo, s=1.0: torch.cat([torch.zeros(rows, lo), s * torch.eye(rows), torch.zeros(rows, width - lo - rows)], 1)
    wq = torch.cat([pick(D, 0)] + [torch.zeros(D, width)] * (H - 1), 0)            # head 0 reads the first D inputs
    wk = torch.cat([pick(D, D)] + [torch.zeros(D, width)] * (G - 1), 0)            # key head 0 reads the next D
    talk = torch.zeros(H, H)
    talk[H - 1, 0] = 1.0
    over = {"left.q": wq, "left.k": wk, "left.q.norm": torch.ones(H * D), "left.k.norm": torch.ones(G * D),
            "left.pb": torch.full((H,), -12.0), "left.talk": talk, "left.out": torch.ones(width),
            "right.o": torch.zeros(width, 16)}
    rig = Rig(tmp_path, lft, rgt, over, width, dtype)
    g = torch.Generator().manual_seed(D)
    lens = [397, 22, 129]
    hs = [torch.randn(n, width, generator=g, dtype=torch.float64) for n in lens]
    u = torch.zeros(D, dtype=torch.float64)
    u[8:] = torch.randn(D - 8, generator=g, dtype=torch.float64)                   # on the dimensions that do not turn
    u = u / u.norm()
    for h in hs:
        h[:, :D] = 6.0 * u + 0.05 * h[:, :D]
        h[:, D:2 * D] = -3.0 * u + 0.05 * h[:, D:2 * D]                             # every key points away ...
        h[1, D:2 * D] = 6.0 * u                                                   # ... but position 1's
    hs = [_rounded(h) for h in hs]
    want = [_pair(h, rig.W, rig.cfg["layers"][0]["mixer"], rig.eps) for h in hs]
    steps = {"prompt": [lens], "portions": [[330, 5, 64], [1, 1, 64], [2, 0, 1], [64, 16, 0]],
             "decoded": [[300, 2, 100]] + [[1, 1 if s < 20 else 0, 1 if s < 29 else 0] for s in range(97)]}[how]
    got = rig.feed(hs, steps)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for a, b in zip(got, want):
        _close(a, b[:a.shape[0]], tol)
    # the oracle itself: the left branch's last head carries position 1's value of its own key/value head
    inner = pk.sigmoid_attention(hs[0], {k[5:]: v for k, v in rig.W.items() if k.startswith("left.")} | {"o": torch.eye(H * D, dtype=torch.float64)},
                                 lft, rig.eps)
    v1 = (hs[0][1] @ rig.W["left.v"].T).reshape(G, D)[G - 1]
    assert (inner[390, (H - 1) * D:] - v1).abs().max().item() < 0.05 * v1.abs().max().item()
    assert inner[390, :(H - 1) * D].abs().max().item() < 1e-9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(3, 12, 20, (0.9, 0.97, 0.75), 12), (4, 8, 8, (0.5, 1.0, 0.0, 0.99), 0), (1, 64, 8, (0.9375,), 8),
                                   (2, 128, 32, (0.999, 0.5), 64), (5, 7, 5, (0.9, 0.8, 0.7, 0.6, 0.5), 6)])
def test_retention_alone(tmp_path, dtype, shape):
    """The retention branch alone (the attention branch's output projection is zero): three requests of unequal length
    in portions and single tokens, state slots used again by a second round of requests."""
    H, D, P, decay, rot = shape
    width = 64
    lft = tk.left(2, 1, 16, 16, 0.25)
    rgt = tk.right(D, P, decay, rot=tk.rot(rot, 1000.0) if rot else None)
    over = {"left.o": torch.zeros(width, 32)}
    rig = Rig(tmp_path, lft, rgt, over, width, dtype, seed=H + D)
    g = torch.Generator().manual_seed(P)
    for round_ in range(2):
        lens = [150, 3, 41]
        hs = [_rounded(torch.randn(n, width, generator=g, dtype=torch.float64)) for n in lens]
        want = [_pair(h, rig.W, rig.cfg["layers"][0]["mixer"], rig.eps) for h in hs]
        got = rig.feed(hs, [[64, 2, 0], [1, 1, 17], [2, 0, 2], [50, 0, 1], [1, 0, 21]] + [[1, 0, 0]] * 32,
                       ids=[f"round{round_}_{r}" for r in range(3)])
        tol = 2e-5 if dtype == "float32" else 3e-2
        for a, b in zip(got, want):
            _close(a, b[:a.shape[0]], tol)


# ----------------------------------------------------------------------------- kernels alone
def _dev(t):
    return t.cuda() if t is not None else None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_norm_and_gated_head_norm(dtype):
    from fastmlx_b200 import kernels as k
    g = torch.Generator().manual_seed(4)
    a, b = (torch.randn(37, 100, generator=g) * s for s in (3.0, 0.01))
    wa, wb = torch.randn(100, generator=g), torch.randn(100, generator=g)
    got = k.rmsnorm_pair_mean(a.cuda(), b.cuda(), wa.cuda(), wb.cuda(), 1e-5, dtype).cpu().double()
    want = plain_ops.rmsnorm_pair_mean(a, b, wa, wb, 1e-5, torch.float64)
    assert (got - want).abs().max() <= (2e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()
    o = torch.randn(29, 3 * 20, generator=g)
    gate = torch.randn(29, 80, generator=g).to(dtype)[:, 10:70]                      # a slice of a wider buffer
    got = k.retention_gate_norm(o.cuda(), gate.cuda(), 1e-6, 3, 20, dtype).cpu().double()
    want = plain_ops.retention_gate_norm(o, gate, 1e-6, 3, 20, torch.float64)
    assert (got - want).abs().max() <= (2e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()


@pytest.mark.parametrize("rot", [0, 6, 16])
def test_retention_prepare(rot):
    from fastmlx_b200 import kernels as k
    from fastmlx_b200.parts import inverse_frequencies
    g = torch.Generator().manual_seed(rot)
    H, D, P, T = 3, 16, 10, 21
    proj = torch.randn(T, 2 * H * D + 2 * H * P + 5, generator=g)
    pos = torch.randint(0, 3000, (T,), generator=g, dtype=torch.int32)
    inv = inverse_frequencies(rot, 500.0).float() if rot else None
    decay = torch.tensor([0.5, 1.0, 0.0])
    xbc, dd = k.retention_prepare(proj.cuda(), pos.cuda(), _dev(inv), decay.cuda(), H, D, P, rot, 0.25)
    wx, wd = plain_ops.retention_prepare(proj, pos, inv, decay, H, D, P, rot, 0.25)
    assert torch.equal(dd.cpu(), wd)
    assert (xbc.cpu() - wx).abs().max() < 2e-5 * wx.abs().max()       # the angle is a 32-bit product of thousands of radians


def test_router_choice_by_corrected_scores_and_plain_experts():
    from fastmlx_b200 import kernels as k
    g = torch.Generator().manual_seed(8)
    T, E = 50, 7
    z = torch.randn(T, E + 1, generator=g)
    z[3, :E] = 0.0                                                                  # a tie of all: the lower indices win
    corr = torch.randn(E, generator=g) * 0.2
    for top in (1, 3, E):
        w, chosen = k.moe_route(z.cuda(), top, want_chosen=True, experts=E, correction=corr.cuda(), scale=1.5)
        ww, wc = plain_ops.moe_route(z, top, want_chosen=True, experts=E, correction=corr, scale=1.5)
        assert torch.equal(chosen.cpu(), wc) and (w.cpu() - ww).abs().max() < 1e-6
        assert (w.cpu() > 0).sum(1).eq(top).all()
    s = torch.softmax(z[:, :E], -1)
    plain_top = torch.topk(s, 3).indices.sort(1).values
    corrected = plain_ops.moe_route(z, 3, want_chosen=True, experts=E, correction=corr)[1].long().sort(1).values
    assert not torch.equal(plain_top, corrected), "the correction changes no choice: the test shows nothing"
    for dtype in (torch.float32, torch.bfloat16):
        for ff, shared in ((6, 9), (16, 24)):                                       # the second in 16-byte pieces
            u = torch.randn(T, E * ff + shared, generator=g).to(dtype)
            for act in ("relu2", "gelu_tanh", "silu"):
                for gate in (z[:, E:], None):
                    got = k.moe_plain_act(u.cuda(), ww.cuda(), E, ff, act, shared_gate=_dev(gate)).cpu().double()
                    want = plain_ops.moe_plain_act(u.double(), ww, E, ff, act, shared_gate=gate)
                    assert (got - want).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2) * want.abs().max()


def test_scaled_embedding_starts_the_stream_in_32_bit():
    from fastmlx_b200 import kernels as k
    table = torch.randn(40, 24).bfloat16()
    ids = torch.tensor([3, 39, 0, 3], dtype=torch.int32)
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    got = k.embed_scaled(ids.cuda(), table.cuda(), 1.7, status).cpu()
    assert got.dtype == torch.float32 and torch.equal(got, (table.float()[ids.long()] * 1.7))
    assert int(status[0]) == 0
    k.embed_scaled(torch.tensor([40], dtype=torch.int32).cuda(), table.cuda(), 1.7, status)
    assert int(status[0]) == 1


# ----------------------------------------------------------------------------- through the engine
def _plain_greedy(cfg, W, prompt, n):
    toks, out, margins = list(prompt), [], []
    for _ in range(n):
        row = pk.forward(cfg, W, toks)[-1]
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
    # in bfloat16 the configuration whose routed layer uses all of its experts: no choice can go the other way
    name = "K1" if dtype == "float32" else "K2"
    d, W, _, _ = models[name]
    cfg = tk.CONFIGS[name]
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
    """`python -m fastmlx_b200 generate` and bin/trace_run on a Kafepel folder, as a user runs them."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    d, W, prompts, ref = models["K4"]
    out = subprocess.run([sys.executable, "-m", "fastmlx_b200", "generate", "--model-dir", d, "--dtype", "float32", "--prompt-ids",
                          "5,6,7;9", "--max-tokens", "5", "--temperature", "0", "--max-cache-tokens", "256"], cwd=root,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [json.loads(x) for x in out.stdout.splitlines() if x.startswith("{")]
    assert [len(x["output_token_ids"]) for x in lines] == [5, 5]
    want, margins = _plain_greedy(tk.K4, W, [5, 6, 7], 5)
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
    outs = [np.fromfile(outdir / f"{s['step']}.f32", dtype="<f4").reshape(-1, tk.K4["vocab"]) for s in steps]
    _compare(steps, outs, sub, ref, TOL["float32"])


def test_preemption_recomputes_state_and_changes_no_token(models):
    """A pool too small for three requests to grow together: the scheduler preempts the newest, frees its pages and its
    state slot, and recomputes it later from zero state; in 32-bit every request still produces what it produces with
    room to spare."""
    from fastmlx_b200 import Engine, SamplingParams
    d, W, _, _ = models["K2"]
    prompts = [tiny.rand_tokens(n, tk.K2["vocab"], 900 + n) for n in (30, 28, 25)]
    sp = SamplingParams(max_tokens=40, temperature=0.0)
    tight = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=18, max_concurrent_requests=4)
    outs = tight.generate(prompts, sp)
    assert tight.stats()["preemptions"] > 0
    roomy = Engine(d, dtype="float32", block_size=8, initial_cache_blocks=64, max_concurrent_requests=4)
    assert [o.output_token_ids for o in outs] == [o.output_token_ids for o in roomy.generate(prompts, sp)]
    assert all(o.finish_reason == "length" and len(o.output_token_ids) == 40 for o in outs)
    assert tight.stats()["pages_used"] == 0
    tight.manager.check()
