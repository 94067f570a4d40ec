"""Sorupel without a GPU: configuration, registry, tensor names, the order of layers and whose cache each reads,
the cache manager's handling of runs of positions, the plain model's mechanisms against properties that follow
from their definitions, and the engine's own step function, cache and state manager and replay program over plain
statements of the kernels against the plain model."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_ops
import plain_sorupel as ps
import tiny
import tiny_sorupel as ts
import traces
from fastmlx_b200 import registry
from fastmlx_b200.cache.manager import CacheManager
from fastmlx_b200.config import ConfigError
from fastmlx_b200.config.sorupel import SorupelConfig
from fastmlx_b200.parts import (BigramEmbedding, Embedding, GQAAttention, LatentAttention, PagedKVSpec, PreNormBlock,
                                StateSpaceMixer)


def test_registry_finds_the_design_and_builds_its_layers():
    cfg, model = registry.build_model(ts.S1)
    assert isinstance(cfg, SorupelConfig) and cfg.vocab_size == 211 and cfg.width == 96 and cfg.norm_eps == 1e-6
    assert all(isinstance(b, PreNormBlock) for b in model.layers)
    assert [type(b.mixer) for b in model.layers] == [GQAAttention, LatentAttention, StateSpaceMixer, LatentAttention, GQAAttention]
    assert [b.ffn is not None for b in model.layers] == [True, True, True, False, True]
    assert isinstance(model.embed, BigramEmbedding) and (model.embed.buckets, model.embed.mul_prev, model.embed.mul_cur) == (53, 31, 7)
    a = model.layers[0].mixer
    assert (a.nh, a.nkv, a.hd, a.scale, a.softcap, a.chunk, a.sink) == (4, 2, 24, 0.3, 7.5, 37, 0.0)
    assert a.values_from_keys and a.qk_norm_whole and a.gate_per_head
    m = model.layers[2].mixer
    assert (m.H, m.P, m.N, m.G, m.norm_groups, m.taps) == (4, 10, 12, 2, 2, 3)
    # without a bigram table the embedding is the plain one and keeps no state
    _, plain = registry.build_model(ts.S2)
    assert type(plain.embed) is Embedding and plain.embed_entry is None


def test_layers_run_in_order_and_a_layer_may_read_another_layers_cache():
    _, model = registry.build_model(ts.S3)
    assert [(r.layer, r.cache_from) for r in model.schedule] == [(0, None), (1, None), (2, None), (3, None), (4, 0), (5, 3), (6, None)]
    needs = model.cache_needs()
    assert len(needs) == 8                                     # seven layers and the embedding's previous token
    assert needs[0][0] == PagedKVSpec(1, 96 + 16, 0, 0, 0, True) and needs[3][0] == PagedKVSpec(1, 48 + 16, 0, 0, 0, True)
    assert needs[4] == (None, None, 0) and needs[5] == (None, None, 3)
    assert needs[1][0] == PagedKVSpec(2, 64, 0, 0, 0, False, 100) and needs[6][0] == PagedKVSpec(4, 64, 0, 0, 0, False, 64)
    kv, state, src = needs[2]
    assert kv is None and src is None and state.dtype == torch.float32
    assert state.shape[0] >= 6 * 32 * 64 + (2 - 1) * (6 * 32 + 2 * 3 * 64) and state.shape[0] % 4 == 0
    assert needs[7][0] is None and needs[7][1].dtype == torch.int32


def test_tensor_names_and_shapes():
    _, model = registry.build_model(ts.S1)
    specs = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert specs["embed"] == (211, 96) and specs["bigram"] == (54, 96) and specs["head"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["l0.mix.q"] == (96, 96) and specs["l0.mix.k"] == (48, 96) and "l0.mix.v" not in specs
    assert specs["l0.mix.q.norm"] == (96,) and specs["l0.mix.k.norm"] == (48,) and specs["l0.mix.g"] == (4, 96)
    assert specs["l0.mix.o"] == (96, 96) and specs["l0.mlp.gate"] == (160, 96) and specs["l0.mlp.down"] == (96, 160)
    assert specs["l1.mix.q"] == (3 * 24, 96) and specs["l1.mix.dkv"] == (48, 96) and specs["l1.mix.dkv.norm"] == (40,)
    assert specs["l1.mix.uk"] == (48, 40) and specs["l1.mix.uv"] == (72, 40) and specs["l1.mix.sink"] == (3,)
    assert specs["l1.mix.g"] == (72, 96) and specs["l1.mix.o"] == (96, 72)
    assert specs["l2.mix.in"] == (2 * 40 + 2 * 24 + 4, 96) and specs["l2.mix.conv"] == (88, 3) and specs["l2.mix.conv.b"] == (88,)
    assert specs["l2.mix.dt_bias"] == specs["l2.mix.A_log"] == specs["l2.mix.D"] == (4,) and specs["l2.mix.norm"] == (40,)
    assert specs["l2.mix.o"] == (96, 40)
    assert "l3.mix.dkv" not in specs and "l3.mix.dkv.norm" not in specs and specs["l3.mix.uk"] == (40, 40)
    assert "l3.norm2" not in specs and "l3.mlp.gate" not in specs
    tensors = ts.lively_tensors(ts.S1, 3)
    model.check_weights(tensors)
    # a checkpoint that stores a second norm for a layer without a feed-forward is read all the same
    model.check_weights(dict(tensors, **{"l3.norm2": torch.ones(96)}))
    with pytest.raises(Exception):
        model.check_weights({k: v for k, v in tensors.items() if k != "l1.mix.sink"})


@pytest.mark.parametrize("breakage", [
    lambda c: c["layers"][0].update(type="window"),
    lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"].update(vdim=16),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26),
    lambda c: c["layers"][0]["mixer"]["mask"].update(size=0),
    lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
    lambda c: c["layers"][1]["mixer"]["rot"].update(dims=4),
    lambda c: c["layers"][2]["mixer"].update(groups=3),
    lambda c: c["layers"][2]["mixer"].update(norm_groups=3),
    lambda c: c["layers"][2]["mixer"].update(conv=0),
    lambda c: c["layers"][3]["mixer"].update(kv_from=3),
    lambda c: c["layers"][3]["mixer"].update(kv_from=2),
    lambda c: c["layers"][3]["mixer"].update(kv_rank=24),
    lambda c: c["layers"][3]["mixer"]["rot"].update(base=3.0),
    lambda c: c["layers"][4]["mlp"].update(kind="routed"),
    lambda c: c["embedding"]["bigram"].update(buckets=0),
    lambda c: c.pop("norm"),
    lambda c: c.update(vocab=0),
    lambda c: c.update(layers=[]),
])
def test_bad_configurations_are_refused(breakage):
    c = copy.deepcopy(ts.S1)
    breakage(c)
    with pytest.raises(ConfigError):
        SorupelConfig.from_dict(c)


# ---- the cache manager
def test_pages_of_earlier_runs_of_positions_go_back_to_the_pool():
    spec = PagedKVSpec(1, 8, chunk=20)
    m = CacheManager([(spec, None, None)], page_size=8, num_pages=6, max_requests=2, dtype=torch.float32)
    r = m.add_request("a")
    for n in (10, 9, 1, 1, 30, 1, 17, 1):
        m.reserve(r, n)
        m.commit(r)
        m.check()
        bt = r.tables[0]
        run_start = r.length - r.length % 20                       # the next query's run begins here
        for p, page in enumerate(bt.pages):
            assert (page >= 0) == ((p + 1) * 8 > run_start), (r.length, p, bt.pages)
    assert r.length == 70
    m.free("a")
    m.check()
    assert m.groups[0].pool.used_pages == 0
    # a pool that holds a run, a portion and a page serves a request of any length
    assert m.holds_alone(100000, 8) == 0


def test_runs_shorter_than_a_page_and_state_slots_used_again():
    _, model = registry.build_model(ts.S1)
    m = CacheManager(model.cache_needs(), page_size=16, num_pages=8, max_requests=2, dtype=torch.float32)
    # entries: attention (runs of 37), latent, state space (no pages), a reader of entry 1, attention (runs of 5), the embedding
    assert [e.kv is not None for e in m.entries] == [True, True, False, True, True, False]
    assert m.entries[3].kv.data_ptr() == m.entries[1].kv.data_ptr() and not m.entries[3].writable and m.entries[1].writable
    assert [e.state is not None for e in m.entries] == [False, False, True, False, False, True]
    assert m.entries[1].kv.shape[-1] == 48 and m.entries[1].kv.shape[1] == 1
    a = m.add_request("a")
    for _ in range(40):
        m.reserve(a, 1)
        m.commit(a)
        m.check()
    g5 = [g for g in m.groups if g.spec.chunk == 5][0]
    assert g5.pool.used_pages <= 2
    slot = a.slot
    m.entries[2].state[slot].fill_(3.0)
    m.entries[5].state[slot].fill_(7)
    m.free("a")
    b = m.add_request("b")
    assert b.slot == slot and float(m.entries[2].state[slot].abs().max()) == 0.0 and int(m.entries[5].state[slot].abs().max()) == 0


# ---- the plain model's mechanisms
def test_plain_runs_of_positions_start_at_position_zero():
    seen = ps.same_chunk(11, 4)
    assert seen[6].tolist() == [False] * 4 + [True] * 3 + [False] * 4
    assert seen[7].tolist() == [False] * 4 + [True] * 4 + [False] * 3
    assert seen[8].tolist() == [False] * 8 + [True] + [False] * 2
    assert seen[3].tolist() == [True] * 4 + [False] * 7
    assert torch.equal(ps.same_chunk(7, None), torch.tril(torch.ones(7, 7, dtype=torch.bool)))
    assert torch.equal(ps.same_chunk(5, 1), torch.eye(5, dtype=torch.bool))


def test_plain_softmax_with_a_term_that_has_no_value():
    s = torch.tensor([[1.0, 2.0, -1.0, 0.5]], dtype=torch.float64)
    seen = torch.tensor([[True, True, False, True]])
    p = ps.sink_softmax(s, seen, 0.7)
    e = [math.exp(1.0), math.exp(2.0), 0.0, math.exp(0.5)]
    total = sum(e) + math.exp(0.7)
    assert torch.allclose(p[0], torch.tensor([x / total for x in e], dtype=torch.float64))
    assert float(p.sum()) < 1.0 and float(p[0, 2]) == 0.0
    # a term of score 0 adds one; a very negative one adds nothing; large scores do not overflow
    assert torch.allclose(ps.sink_softmax(s, seen, 0.0)[0, 1], torch.tensor(math.exp(2.0) / (sum(e) + 1.0), dtype=torch.float64))
    assert torch.allclose(ps.sink_softmax(s, seen, -1e4).sum(), torch.tensor(1.0, dtype=torch.float64))
    big = ps.sink_softmax(torch.tensor([[900.0, 899.0]], dtype=torch.float64), torch.tensor([[True, True]]), 5.0)
    assert torch.isfinite(big).all() and abs(float(big.sum()) - 1.0) < 1e-12


def test_plain_rotation_pairs_a_dimension_with_the_one_half_the_rotated_width_on():
    x = torch.randn(5, 3, 12, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    y = ps.rotate_half(x, pos, 10000.0, 8)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    a = 7.0 * 10000.0 ** (-2.0 * 1 / 8)                 # pair 1 = dimensions (1, 5)
    assert torch.allclose(y[2, 0, 1], x[2, 0, 1] * math.cos(a) - x[2, 0, 5] * math.sin(a))
    assert torch.allclose(y[2, 0, 5], x[2, 0, 5] * math.cos(a) + x[2, 0, 1] * math.sin(a))
    q, k = torch.randn(1, 1, 8, dtype=torch.float64), torch.randn(1, 1, 8, dtype=torch.float64)
    s = [float((ps.rotate_half(q, torch.tensor([p + 9]), 50.0, 8) * ps.rotate_half(k, torch.tensor([p]), 50.0, 8)).sum())
         for p in (0, 31)]
    assert abs(s[0] - s[1]) < 1e-9                      # a score depends on the distance alone
    assert torch.equal(ps.rotate_half(x, pos, 10.0, 0), x)


def test_plain_bigram_rows():
    cfg = {"embedding": ts.bigram(7, 3, 2)}
    W = {"embed": torch.zeros(10, 2, dtype=torch.float64), "bigram": torch.arange(8, dtype=torch.float64)[:, None].repeat(1, 2)}
    x = ps.embed(torch.tensor([4, 9, 0, 5]), W, cfg)
    assert x[:, 0].tolist() == [7.0, (4 * 3 + 9 * 2) % 7, (9 * 3 + 0) % 7, (0 + 5 * 2) % 7]


def test_plain_convolution_sees_zeros_before_the_start_and_its_last_tap_is_the_current_token():
    u = torch.randn(6, 3, dtype=torch.float64)
    w = torch.randn(3, 4, dtype=torch.float64)
    b = torch.randn(3, dtype=torch.float64)
    y = ps.short_convolution(u, w, b)
    assert torch.allclose(y[0], u[0] * w[:, 3] + b)
    assert torch.allclose(y[2], u[2] * w[:, 3] + u[1] * w[:, 2] + u[0] * w[:, 1] + b)
    assert torch.allclose(y[5], u[5] * w[:, 3] + u[4] * w[:, 2] + u[3] * w[:, 1] + u[2] * w[:, 0] + b)


def test_plain_recurrence_equals_its_sum_over_earlier_tokens():
    """y_t = sum_{s <= t} (prod_{s < r <= t} a_r) dt_s (B_s . C_t) x_s + D x_t: the recurrence, unrolled."""
    m = ts.mamba(4, 5, 6, 2, 2, 3)
    T, width = 9, 16
    g = torch.Generator().manual_seed(4)
    inner, GN = 20, 12
    W = {"in": torch.randn(2 * inner + 2 * GN + 4, width, generator=g, dtype=torch.float64) / 4, "conv": torch.randn(inner + 2 * GN, 3, generator=g, dtype=torch.float64),
         "conv.b": torch.randn(inner + 2 * GN, generator=g, dtype=torch.float64) * 0.1, "dt_bias": torch.randn(4, generator=g, dtype=torch.float64),
         "A_log": torch.randn(4, generator=g, dtype=torch.float64), "D": torch.randn(4, generator=g, dtype=torch.float64),
         "norm": torch.ones(inner, dtype=torch.float64), "o": torch.eye(inner, dtype=torch.float64)}
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    got = ps.state_space(h, W, m, 1e-6)
    p = h @ W["in"].T
    z, dt = p[:, :inner], ps.softplus(p[:, 2 * inner + 2 * GN:] + W["dt_bias"])
    xbc = ps.silu(ps.short_convolution(p[:, inner:2 * inner + 2 * GN], W["conv"], W["conv.b"]))
    x, B, C = xbc[:, :inner].reshape(T, 4, 5), xbc[:, inner:inner + GN].reshape(T, 2, 6), xbc[:, inner + GN:].reshape(T, 2, 6)
    la = -torch.exp(W["A_log"]) * dt                                    # log decay [T, H]
    y = torch.zeros(T, 4, 5, dtype=torch.float64)
    for hd in range(4):
        grp = hd // 2
        for t in range(T):
            for s in range(t + 1):
                y[t, hd] += math.exp(float(la[s + 1:t + 1, hd].sum())) * dt[s, hd] * (B[s, grp] @ C[t, grp]) * x[s, hd]
            y[t, hd] += W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * ps.silu(z)
    want = torch.cat([ps.rms_norm(y[:, :10], 1e-6), ps.rms_norm(y[:, 10:], 1e-6)], 1)
    assert torch.allclose(got, want, atol=1e-10)


def test_plain_latent_attention_needs_the_latent_and_the_rotated_part_only():
    """Scores through the query carried into the latent's space, and values read out behind the weighted sum."""
    m = ts.latent(2, 6, 4, 5, 7, 0.3, 100.0)
    T, width = 8, 12
    g = torch.Generator().manual_seed(1)
    W = {n: torch.randn(*s, generator=g, dtype=torch.float64) / 2 for n, s in
         {"q": (20, width), "dkv": (11, width), "dkv.norm": (7,), "uk": (12, 7), "uv": (10, 7), "sink": (2,), "g": (10, width), "o": (width, 10)}.items()}
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    want, (c, kr) = ps.latent_attention(h, W, m, 1e-6)
    q = (h @ W["q"].T).reshape(T, 2, 10)
    qr = ps.rotate_half(q[..., 6:], torch.arange(T), 100.0, 4)
    row = torch.cat([c, kr], 1)                                         # what a token's cache row holds
    outs = []
    for hd in range(2):
        q_lat = torch.cat([q[:, hd, :6] @ W["uk"].view(2, 6, 7)[hd], qr[:, hd]], 1)
        pr = ps.sink_softmax(q_lat @ row.T * 0.3, ps.causal(T), W["sink"][hd])
        outs.append((pr @ row[:, :7]) @ W["uv"].view(2, 5, 7)[hd].T)
    via = (torch.cat(outs, 1) * torch.sigmoid(h @ W["g"].T)) @ W["o"].T
    assert torch.allclose(want, via, atol=1e-12)
    # a layer that reads another layer's cache takes its rows as they are
    again, _ = ps.latent_attention(h, W, m, 1e-6, cached=(c, kr))
    assert torch.equal(again, want)


def test_plain_attention_values_are_the_keys_before_norm_and_rotation():
    m = ts.attention(2, 1, 4, 0.5, softcap=3.0, chunk=3, rot=(4, 10.0))
    T, width = 5, 6
    g = torch.Generator().manual_seed(2)
    W = {"q": torch.randn(8, width, generator=g, dtype=torch.float64), "k": torch.randn(4, width, generator=g, dtype=torch.float64),
         "q.norm": torch.ones(8, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64),
         "g": torch.zeros(2, width, dtype=torch.float64), "o": torch.eye(8, dtype=torch.float64)}
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    y = ps.chunked_attention(h, W, m, 1e-6)
    k = h @ W["k"].T
    # position 3 opens a run: it sees itself alone, with weight e^s / (1 + e^s) < 1, and half of it passes the gate
    q3 = ps.rotate_half(ps.rms_norm(h[3:4] @ W["q"].T, 1e-6).reshape(1, 2, 4), torch.tensor([3]), 10.0, 4)
    k3 = ps.rotate_half(ps.rms_norm(k[3:4], 1e-6).reshape(1, 1, 4), torch.tensor([3]), 10.0, 4)
    for hd in range(2):
        s = 3.0 * math.tanh(float(q3[0, hd] @ k3[0, 0]) * 0.5 / 3.0)
        w = math.exp(s) / (1.0 + math.exp(s))
        assert torch.allclose(y[3, 4 * hd:4 * hd + 4], 0.5 * w * k[3])


def test_plain_forward_is_causal_and_gives_the_stream_after_every_layer():
    W = {n: t.double() for n, t in ts.lively_tensors(ts.S1, 5).items()}
    toks = tiny.rand_tokens(50, 211, 1)
    full, streams = ps.forward(ts.S1, W, toks, return_layers=True)
    assert streams.shape == (5, 50, 96)
    assert torch.allclose(ps.forward(ts.S1, W, toks[:17]), full[:17], atol=1e-10)


# ---- the engine over plain statements of the kernels
LENS = {"S1": [1, 2, 9, 45, 58, 80], "S2": [3, 50, 75], "S3": [5, 40, 110], "S4": [4, 41, 70]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("sorupel_cpu")
    out = {}
    for name, cfg in ts.CONFIGS.items():
        d = ts.make_model_dir(root, cfg, seed=11)
        W = tiny.load_plain_weights(d)
        prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab"], 500 + i) for i, n in enumerate(LENS[name])}
        out[name] = (d, prompts, {r: ps.forward(cfg, W, t) for r, t in prompts.items()})
    return out


@pytest.mark.parametrize("name", ["S1", "S2", "S3", "S4"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_engine_over_plain_kernels_matches_the_plain_model(models, name, cut):
    from fastmlx_b200.engine.replay import Replayer
    d, prompts, ref = models[name]
    steps = {"whole": traces.whole, "tail": lambda p: traces.tail_decoded(p, tail=12), "portions": traces.portions,
             "mixed": lambda p: traces.mixed(p, max_live=2)}[cut](prompts)
    rp = Replayer(d, "float32", 256, page_size=8, device="cpu", kernels=plain_ops, max_live=2)
    outs = []
    for st in steps:
        outs.append(rp.step(st))
        rp.manager.check()
    assert not rp.manager.requests and all(g.pool.used_pages == 0 for g in rp.manager.groups)
    rows = traces.collect(steps, outs)
    for rid, toks in prompts.items():
        got = torch.from_numpy(np.stack([rows[rid][i] for i in range(len(toks))])).double()
        err = (got - ref[rid]).abs().max() / ref[rid].abs().max()
        assert err < 2e-5, (rid, float(err))
