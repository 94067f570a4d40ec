"""Kafepel without a GPU: configuration, registry, tensor names, what the cache manager is asked for, the plain
model's mechanisms against properties that follow from their definitions, and the engine's own step function, cache
and state manager and replay program over plain statements of the kernels against the plain model."""
import copy
import math

import numpy as np
import pytest
import torch

import plain_kafepel as pk
import plain_ops
import tiny
import tiny_kafepel as tk
import traces
from fastmlx_b200 import registry
from fastmlx_b200.config import ConfigError
from fastmlx_b200.config.kafepel import KafepelConfig
from fastmlx_b200.parts import (Embedding, GQAAttention, MixerOnly, PagedKVSpec, PairMixer, PlainRoutedExperts, PreNormBlock,
                                RetentionMixer, SwiGLU)


def test_registry_finds_the_design_and_builds_its_layers():
    cfg, model = registry.build_model(tk.K1)
    assert isinstance(cfg, KafepelConfig) and cfg.vocab_size == 211 and cfg.width == 96 and cfg.norm_eps == 1e-6
    assert cfg.embedding_scale == 1.7 and isinstance(model.embed, Embedding) and model.embed.scale == 1.7 and model.embed.starts_stream
    assert [type(b) for b in model.layers] == [PreNormBlock, PreNormBlock, PreNormBlock, MixerOnly]
    assert all(isinstance(b.mixer, PairMixer) for b in model.layers)
    assert [type(b.ffn) for b in model.layers[:3]] == [SwiGLU, PlainRoutedExperts, PlainRoutedExperts]
    a, r = model.layers[0].mixer.left, model.layers[0].mixer.right
    assert isinstance(a, GQAAttention) and isinstance(r, RetentionMixer)
    assert (a.nh, a.nkv, a.hd, a.vd, a.scale, a.softcap) == (4, 2, 24, 16, 0.3, 7.5) and a.sigmoid and a.qk_norm_whole
    assert a.pos.rotary_dim == 8 and a.pos.scaling.factor == 8.0 and a.pos.scaling.original_max_position_embeddings == 64
    assert (r.H, r.D, r.P, r.decay_values, r.rot_dims, r.rot_base) == (3, 12, 20, (0.9, 0.97, 0.75), 12, 500.0)
    e = model.layers[1].ffn
    assert (e.E, e.top, e.ff, e.scale, e.shared_ff, e.activation) == (6, 2, 24, 1.75, 40, "relu2")
    assert model.layers[2].ffn.shared_ff == 0 and model.layers[2].ffn.gate_name is None
    assert model.layers[2].mixer.left.softcap == 30.0 and model.layers[1].mixer.left.softcap == 0.0
    # no embedding block: no multiplier, and the embedding is the plain gather
    _, plain = registry.build_model(tk.K2)
    assert plain.embed.scale == 1.0 and not plain.embed.starts_stream


def test_a_layer_asks_for_pages_and_for_a_state_slot():
    _, model = registry.build_model(tk.K1)
    needs = model.cache_needs()
    assert len(needs) == 4 and all(src is None for _, _, src in needs)
    assert needs[0][0] == PagedKVSpec(2, 24, 0, 16) and needs[1][0] == PagedKVSpec(3, 16, 0, 0) and needs[2][0] == PagedKVSpec(1, 8, 0, 24)
    for (kv, state, _), floats in zip(needs, (3 * 12 * 20, 4 * 8 * 8, 20 * 12, 2 * 16 * 16)):
        assert state.dtype == torch.float32 and state.shape[0] >= floats and state.shape[0] % 4 == 0
    assert model.graph_safe


def test_tensor_names_and_shapes():
    _, model = registry.build_model(tk.K1)
    specs = {s.name: tuple(s.shape) for s in model.weight_specs()}
    assert specs["embed"] == (211, 96) and specs["head"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["l0.mix.left.q"] == (96, 96) and specs["l0.mix.left.k"] == (48, 96) and specs["l0.mix.left.v"] == (32, 96)
    assert specs["l0.mix.left.q.norm"] == (96,) and specs["l0.mix.left.k.norm"] == (48,)
    assert specs["l0.mix.left.talk"] == (4, 4) and specs["l0.mix.left.pb"] == (4,) and specs["l0.mix.left.o"] == (96, 64)
    assert specs["l0.mix.right.q"] == specs["l0.mix.right.k"] == (36, 96)
    assert specs["l0.mix.right.v"] == specs["l0.mix.right.g"] == (60, 96) and specs["l0.mix.right.o"] == (96, 60)
    assert specs["l0.mix.left.out"] == specs["l0.mix.right.out"] == (96,)
    assert specs["l0.mlp.gate"] == specs["l0.mlp.up"] == (160, 96) and specs["l0.mlp.down"] == (96, 160)
    assert specs["l1.mlp.router"] == (6, 96) and specs["l1.mlp.correction"] == (6,)
    assert specs["l1.mlp.e5.up"] == (24, 96) and specs["l1.mlp.e5.down"] == (96, 24) and "l1.mlp.e6.up" not in specs
    assert specs["l1.mlp.shared.up"] == (40, 96) and specs["l1.mlp.shared.down"] == (96, 40) and specs["l1.mlp.shared.sg"] == (1, 96)
    assert "l2.mlp.shared.up" not in specs and "l2.mlp.shared.sg" not in specs
    assert "l3.norm2" not in specs and not any(n.startswith("l3.mlp") for n in specs)
    tensors = tk.lively_tensors(tk.K1, 3)
    model.check_weights(tensors)
    model.check_weights(dict(tensors, **{"l3.norm2": torch.ones(96)}))
    with pytest.raises(Exception):
        model.check_weights({k: v for k, v in tensors.items() if k != "l1.mlp.correction"})


@pytest.mark.parametrize("breakage", [
    lambda c: c["layers"][0].update(type="serial"),
    lambda c: c["layers"][0]["mixer"]["left"].update(kv_heads=3),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=7),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"].update(dims=26),
    lambda c: c["layers"][0]["mixer"]["left"]["rot"]["scaling"].update(factor=0),
    lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5]),
    lambda c: c["layers"][0]["mixer"]["right"].update(decay=[0.5, 0.5, 1.5]),
    lambda c: c["layers"][0]["mixer"].pop("right"),
    lambda c: c["layers"][1]["mlp"]["router"].update(top=7),
    lambda c: c["layers"][1]["mlp"].update(kind="sparse"),
    lambda c: c["layers"][1]["mlp"].pop("expert"),
    lambda c: c.pop("norm"),
    lambda c: c["embedding"].update(scale="big"),
    lambda c: c.update(layers=[]),
])
def test_bad_configurations_are_refused(breakage):
    cfg = copy.deepcopy(tk.K1)
    breakage(cfg)
    with pytest.raises(ConfigError):
        KafepelConfig.from_dict(cfg)


# ---- the plain model's mechanisms
def _weights(shapes, seed, scale=0.5):
    g = torch.Generator().manual_seed(seed)
    return {n: torch.randn(*s, generator=g, dtype=torch.float64) * scale for n, s in shapes.items()}, g


def test_plain_frequency_bands_are_rescaled_by_wavelength():
    rot = tk.rot(16, 10000.0, (8.0, 1.0, 4.0, 64))
    f0 = pk.rotary_frequencies(tk.rot(16, 10000.0), torch.float64)
    f = pk.rotary_frequencies(rot, torch.float64)
    wl = 2 * math.pi / f0
    assert torch.equal(f[wl < 16], f0[wl < 16]) and (wl < 16).any()                  # short waves stay
    assert torch.allclose(f[wl > 64], f0[wl > 64] / 8.0) and (wl > 64).any()         # long waves slow down by the factor
    mid = (wl >= 16) & (wl <= 64)
    assert mid.any() and ((f[mid] < f0[mid]) & (f[mid] > f0[mid] / 8.0)).all()


def test_plain_rotation_pairs_a_dimension_with_the_one_half_the_rotated_width_on():
    u = torch.zeros(3, 1, 10, dtype=torch.float64)
    u[:, 0, 1] = 1.0
    u[:, 0, 9] = 5.0
    r = pk.rotate(u, tk.rot(6, 100.0))
    f1 = 100.0 ** (-2.0 / 6)
    for p in range(3):
        assert math.isclose(float(r[p, 0, 1]), math.cos(p * f1), abs_tol=1e-12)
        assert math.isclose(float(r[p, 0, 4]), math.sin(p * f1), abs_tol=1e-12)
        assert float(r[p, 0, 9]) == 5.0 and float(r[p, 0, 0]) == 0.0


def test_plain_sigmoid_attention_is_a_sum_of_unnormalised_weights_and_mixes_heads():
    m = tk.left(2, 1, 4, 3, 0.5, softcap=3.0, rot=tk.rot(4, 10.0))
    T, width = 6, 5
    W, g = _weights({"q": (8, width), "k": (4, width), "v": (3, width), "pb": (2,), "talk": (2, 2)}, 1)
    W.update({"q.norm": torch.ones(8, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64),
              "o": torch.eye(6, dtype=torch.float64)})
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    y = pk.sigmoid_attention(h, W, m, 1e-6)
    q = pk.rotate(pk.rms_norm(h @ W["q"].T, 1e-6).reshape(T, 2, 4), m["rot"])
    k = pk.rotate(pk.rms_norm(h @ W["k"].T, 1e-6).reshape(T, 1, 4), m["rot"])
    v = h @ W["v"].T
    t = 4
    a = torch.zeros(2, 3, dtype=torch.float64)                    # each head's own unmixed sum over the keys it sees
    for hd in range(2):
        for j in range(t + 1):
            s = 3.0 * math.tanh(float(q[t, hd] @ k[j, 0]) * 0.5 / 3.0)
            a[hd] += 1.0 / (1.0 + math.exp(-(s + float(W["pb"][hd])))) * v[j]
    assert torch.allclose(y[t].reshape(2, 3), W["talk"] @ a, atol=1e-12)
    # doubling the number of identical keys doubles the output: nothing is normalised over the keys
    W1 = dict(W, talk=torch.eye(2, dtype=torch.float64))
    m0 = tk.left(2, 1, 4, 3, 0.5)
    same = torch.ones(4, width, dtype=torch.float64)
    y1 = pk.sigmoid_attention(same, W1, m0, 1e-6)
    assert torch.allclose(y1[3], 4.0 * y1[0], atol=1e-12) and torch.allclose(y1[1], 2.0 * y1[0], atol=1e-12)


def test_plain_retention_equals_its_sum_over_earlier_tokens():
    m = tk.right(4, 3, (0.9, 0.0, 1.0), rot=tk.rot(2, 10.0))
    T, width = 7, 5
    W, g = _weights({"q": (12, width), "k": (12, width), "v": (9, width), "g": (9, width)}, 2)
    W["o"] = torch.eye(9, dtype=torch.float64)
    h = torch.randn(T, width, generator=g, dtype=torch.float64)
    y = pk.retention(h, W, m, 1e-6)
    q = pk.rotate((h @ W["q"].T).reshape(T, 3, 4), m["rot"])
    k = pk.rotate((h @ W["k"].T).reshape(T, 3, 4), m["rot"]) * 0.5
    v = (h @ W["v"].T).reshape(T, 3, 3)
    o = torch.zeros(T, 3, 3, dtype=torch.float64)
    for t in range(T):
        for hd, d in enumerate((0.9, 0.0, 1.0)):
            for s in range(t + 1):
                o[t, hd] += (d ** (t - s) if t > s else 1.0) * float(q[t, hd] @ k[s, hd]) * v[s, hd]
    want = pk.rms_norm(o, 1e-6).reshape(T, 9) * pk.silu(h @ W["g"].T)
    assert torch.allclose(y, want, atol=1e-10)
    # a decay of 0 forgets everything but the token itself
    assert torch.allclose(o[5, 1], float(q[5, 1] @ k[5, 1]) * v[5, 1])


def test_plain_router_chooses_by_corrected_scores_and_weighs_by_scores():
    mlp = tk.moe(4, 2, 1.5, 3, shared=2)
    width = 5
    W, g = _weights({f"e{e}.{n}": s for e in range(4) for n, s in (("up", (3, width)), ("down", (width, 3)))}, 3)
    W.update(_weights({"router": (4, width), "shared.up": (2, width), "shared.down": (width, 2), "shared.sg": (1, width)}, 4)[0])
    h = torch.randn(1, width, generator=g, dtype=torch.float64)
    s = torch.softmax(h @ W["router"].T, -1)[0]
    order = torch.argsort(s, descending=True).tolist()
    # a correction that lifts the weakest expert above all others changes the choice, not the weights
    W["correction"] = torch.zeros(4, dtype=torch.float64)
    W["correction"][order[3]] = 10.0
    y = pk.routed_feed_forward(h, W, mlp)
    want = sum(1.5 * s[e] * pk.expert(h, pk.sub(W, f"e{e}.")) for e in (order[3], order[0]))
    want = want + torch.sigmoid(h @ W["shared.sg"].T) * pk.expert(h, pk.sub(W, "shared."))
    assert torch.allclose(y, want, atol=1e-12)
    assert torch.equal(pk.expert(-torch.ones(1, 1, dtype=torch.float64), {"up": torch.ones(3, 1, dtype=torch.float64),
                                                                        "down": torch.ones(1, 3, dtype=torch.float64)}),
                       torch.zeros(1, 1, dtype=torch.float64))          # the square of relu: nothing passes below zero


def test_plain_forward_is_causal_and_gives_the_stream_after_every_layer():
    W = {n: t.double() for n, t in tk.lively_tensors(tk.K1, 5).items()}
    toks = tiny.rand_tokens(50, 211, 1)
    full, streams = pk.forward(tk.K1, W, toks, return_layers=True)
    assert streams.shape == (4, 50, 96)
    assert torch.allclose(pk.forward(tk.K1, W, toks[:17]), full[:17], atol=1e-10)


# ---- the engine over plain statements of the kernels
LENS = {"K1": [1, 2, 9, 45, 58, 80], "K2": [3, 50, 75], "K3": [5, 40, 110], "K4": [4, 41, 70]}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("kafepel_cpu")
    out = {}
    for name, cfg in tk.CONFIGS.items():
        d = tk.make_model_dir(root, cfg, seed=11)
        W = tiny.load_plain_weights(d)
        prompts = {f"r{i}": tiny.rand_tokens(n, cfg["vocab"], 500 + i) for i, n in enumerate(LENS[name])}
        out[name] = (d, prompts, {r: pk.forward(cfg, W, t) for r, t in prompts.items()})
    return out


@pytest.mark.parametrize("name", ["K1", "K2", "K3", "K4"])
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
