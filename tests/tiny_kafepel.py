"""Small Kafepel configurations for the tests: they differ from one another in every size and option, and use values
that a usual model makes equal or 1 (as many kv heads as heads, one head, values of another width than keys, a
retention whose keys are wider or narrower than its values, a rotation over the whole head, over a part or none,
rescaled frequency bands or none, no cap, one chosen expert or all, no shared expert, no feed-forward, an embedding
multiplier that is no power of two, decays of 0 and 1), and weights of a size at which every mechanism matters."""
import json
import os

import torch


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def left(heads, kv_heads, dim, vdim, scale, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    return m


def right(dim, vdim, decay, rot=None):
    m = {"heads": len(decay), "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = rot
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, scale, ff, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff},
            "shared": {"ff": shared} if shared else None}


def layer(lft, rgt, mlp=None):
    return {"type": "parallel", "mixer": {"left": lft, "right": rgt}, "mlp": mlp}


K1 = {
    "architecture": "Kafepel", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.7},
    "layers": [
        layer(left(4, 2, 24, 16, 0.3, softcap=7.5, rot=rot(8, 10000.0, (8.0, 1.0, 4.0, 64))),
              right(12, 20, (0.9, 0.97, 0.75), rot=rot(12, 500.0)), dense(160)),
        layer(left(3, 3, 16, 16, 0.25, rot=rot(16, 50.0)), right(8, 8, (0.5, 1.0, 0.0, 0.99)), moe(6, 2, 1.75, 24, shared=40)),
        layer(left(6, 1, 8, 24, 0.35, softcap=30.0), right(20, 12, (0.95,), rot=rot(4, 100.0)), moe(5, 1, 0.7, 16)),
        layer(left(2, 1, 32, 32, 0.17, softcap=3.0, rot=rot(32, 500.0, (2.0, 1.0, 2.0, 32))), right(16, 16, (0.8, 0.9), rot=rot(16, 500.0))),
    ],
}
K2 = {
    "architecture": "Kafepel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer(left(1, 1, 16, 8, 0.25), right(64, 8, (0.9375,)), moe(3, 3, 1.0, 32, shared=8)),
        layer(left(2, 2, 16, 32, 0.25, rot=rot(8, 100.0)), right(8, 32, (0.99, 0.6), rot=rot(8, 100.0)), dense(128)),
    ],
}
# sizes that the tiled kernels and the blocked products take: 64-wide heads, feed-forwards in blocks of 128
K3 = {
    "architecture": "Kafepel", "vocab": 130, "width": 128, "norm": {"eps": 1e-4}, "embedding": {"scale": 0.25},
    "layers": [
        layer(left(8, 2, 64, 64, 0.125, softcap=12.0, rot=rot(64, 250000.0, (3.0, 1.0, 2.0, 128))),
              right(64, 64, (0.97, 0.98, 0.99, 0.995), rot=rot(64, 250000.0)), dense(256)),
        layer(left(4, 4, 64, 64, 0.11, softcap=20.0, rot=rot(16, 30000.0)), right(32, 64, (0.9, 0.99), rot=rot(32, 30000.0)),
              moe(8, 2, 1.5, 64, shared=128)),
        layer(left(2, 1, 128, 64, 0.09, rot=rot(128, 777.0)), right(128, 32, (0.999, 0.5, 0.9), rot=rot(64, 777.0)), moe(4, 3, 2.0, 128)),
    ],
}
# sizes that are multiples of nothing
K4 = {
    "architecture": "Kafepel", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "layers": [
        layer(left(3, 3, 20, 14, 0.22, softcap=9.0, rot=rot(6, 777.0)), right(7, 5, (0.9, 0.8, 0.7, 0.6, 0.5), rot=rot(6, 777.0)),
              moe(7, 3, 1.3, 9, shared=11)),
        layer(left(6, 2, 10, 18, 0.3), right(9, 100, (0.93,)), dense(45)),
    ],
}
CONFIGS = {"K1": K1, "K2": K2, "K3": K3, "K4": K4}


def one_layer(lft, rgt, width=48, vocab=61, mlp=None, eps=1e-6, scale=None):
    cfg = {"architecture": "Kafepel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [layer(lft, rgt, mlp)]}
    if scale is not None:
        cfg["embedding"] = {"scale": scale}
    return cfg


def lively_tensors(config, seed, dtype=torch.bfloat16):
    """Weights at which every mechanism counts: matrices that keep activations of order one, a head mix away from the
    identity, numbers per head that keep the sigmoids away from 0 and 1, corrections that change some choices, norm
    weights away from one."""
    from fastmlx_b200 import registry
    _, model = registry.build_model(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in model.weight_specs():
        t = torch.randn(tuple(spec.shape), generator=g, dtype=torch.float32)
        name = spec.name
        if spec.kind == "head_mix":
            t = torch.eye(spec.shape[0]) * 0.8 + 0.4 * t
        elif spec.kind == "head_bias":
            t = t * 0.7 - 2.0
        elif name.endswith(".correction"):
            t = t * 0.15
        elif name.endswith(".router"):
            t = t * 1.5 / spec.shape[-1] ** 0.5
        elif spec.kind == "matrix":
            t = t / spec.shape[-1] ** 0.5
            if ".mix.left.q" in name or ".mix.left.k" in name:
                t = t * 2.0
        elif spec.kind == "embedding":
            t = t * 0.7
        elif spec.kind == "bias":
            t = t * 0.1
        elif spec.kind == "norm":
            t = 1.0 + 0.2 * t
        out[name] = t.to(dtype)
    return out


def make_model_dir(root, config, seed, tensors=None):
    """A folder with config.json and model.safetensors of lively weights (or of the tensors given)."""
    from fastmlx_b200.weights import safetensors_io as st
    d = os.path.join(str(root), f"kafepel_{config['vocab']}_{config['width']}_{len(config['layers'])}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    st.write_file(os.path.join(d, "model.safetensors"), tensors if tensors is not None else lively_tensors(config, seed),
                  {"format": "pt"})
    return d
