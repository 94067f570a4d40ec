"""Small Sorupel configurations for the tests: they differ from one another in every size and option, and use
values that a usual model makes equal or 1 (as many kv heads as heads, one head, values of another width than
keys, a state of another size than the values, one group or as many groups as heads, a rotation over the whole
head or none, runs of positions shorter than a page, no mask, no cap, no feed-forward, no bigram table, two
layers that read two different layers' caches), and weights of a size at which every mechanism matters."""
import json
import os

import torch


def attention(heads, kv_heads, dim, scale, softcap=None, chunk=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot_dim, "base": base}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def mamba(heads, vdim, state, groups, norm_groups, conv):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def bigram(buckets, mul_prev, mul_cur):
    return {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


S1 = {
    "architecture": "Sorupel", "vocab": 211, "width": 96, "norm": {"eps": 1e-6}, "embedding": bigram(53, 31, 7),
    "layers": [
        layer("attention", attention(4, 2, 24, 0.3, softcap=7.5, chunk=37, rot=(8, 10000.0)), ff=160),
        layer("latent_attention", latent(3, 16, 8, 24, 40, 0.2, 500.0), ff=160),
        layer("mamba2", mamba(4, 10, 12, 2, 2, 3), ff=72),
        layer("latent_attention", latent(5, 8, 8, 16, 40, 0.25, 500.0, kv_from=1)),
        layer("attention", attention(3, 1, 32, 0.17, softcap=30.0, chunk=5, rot=(32, 500.0)), ff=64),
    ],
}
S2 = {
    "architecture": "Sorupel", "vocab": 97, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        layer("mamba2", mamba(1, 64, 8, 1, 1, 4)),
        layer("attention", attention(2, 2, 16, 0.25), ff=128),
        layer("latent_attention", latent(1, 32, 4, 8, 24, 0.15, 100.0), ff=40),
    ],
}
# sizes that the tiled kernels take: 64-wide heads, cache rows of 112 and 64 values, a feed-forward in blocks of 128
S3 = {
    "architecture": "Sorupel", "vocab": 130, "width": 128, "norm": {"eps": 1e-4}, "embedding": bigram(1000, 3, 1),
    "layers": [
        layer("latent_attention", latent(4, 32, 16, 32, 96, 0.14, 1000000.0), ff=256),
        layer("attention", attention(8, 2, 64, 0.125, softcap=12.0, chunk=100, rot=(16, 30000.0)), ff=128),
        layer("mamba2", mamba(6, 32, 64, 3, 4, 2), ff=128),
        layer("latent_attention", latent(2, 48, 16, 64, 48, 0.1, 777.0)),
        layer("latent_attention", latent(8, 16, 16, 16, 96, 0.2, 1000000.0, kv_from=0), ff=96),
        layer("latent_attention", latent(3, 32, 16, 40, 48, 0.12, 777.0, kv_from=3)),
        layer("attention", attention(4, 4, 64, 0.11, chunk=64, rot=(64, 100.0))),
    ],
}
# sizes that are multiples of nothing
S4 = {
    "architecture": "Sorupel", "vocab": 101, "width": 50, "norm": {"eps": 1e-5}, "embedding": bigram(7, 1, 0),
    "layers": [
        layer("mamba2", mamba(3, 7, 100, 1, 3, 5), ff=45),
        layer("attention", attention(3, 3, 20, 0.22, softcap=9.0, chunk=33, rot=(6, 777.0)), ff=45),
        layer("latent_attention", latent(2, 10, 6, 14, 21, 0.3, 50.0)),
        layer("mamba2", mamba(4, 5, 9, 4, 1, 2)),
    ],
}
CONFIGS = {"S1": S1, "S2": S2, "S3": S3, "S4": S4}


def one_layer(kind, mixer, width=48, vocab=61, ff=None, embedding=None, eps=1e-6):
    cfg = {"architecture": "Sorupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": [layer(kind, mixer, ff)]}
    if embedding:
        cfg["embedding"] = embedding
    return cfg


def lively_tensors(config, seed, dtype=torch.bfloat16):
    """Weights at which every mechanism counts: matrices that keep activations of order one, sinks and skips of
    order one, decay rates spread over (0, 1), norm weights away from one."""
    from fastmlx_b200 import registry
    _, model = registry.build_model(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in model.weight_specs():
        t = torch.randn(tuple(spec.shape), generator=g, dtype=torch.float32)
        name = spec.name
        if name.endswith(".sink"):
            t = t * 1.5
        elif spec.kind == "matrix":
            t = t / spec.shape[-1] ** 0.5
            if name.endswith((".mix.q", ".mix.k")):
                t = t * 2.0
        elif spec.kind == "embedding":
            t = t * 0.7
        elif spec.kind == "bias":
            t = t * 0.1
        elif spec.kind == "norm":
            t = 1.0 + 0.2 * t
        elif spec.kind == "conv":
            t = t * 0.5
        elif spec.kind == "log_rate":
            t = torch.log(torch.sigmoid(t) * 0.98 + 0.02)
        elif spec.kind == "rate_bias":
            t = t * 0.5 - 1.0
        out[name] = t.to(dtype)
    return out


def make_model_dir(root, config, seed):
    """A folder with config.json and model.safetensors of lively weights."""
    from fastmlx_b200.weights import safetensors_io as st
    d = os.path.join(str(root), f"sorupel_{config['vocab']}_{config['width']}_{len(config['layers'])}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    st.write_file(os.path.join(d, "model.safetensors"), lively_tensors(config, seed), {"format": "pt"})
    return d
