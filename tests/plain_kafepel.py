"""A plain, slow Kafepel: one function per mechanism, written from the design's equations.

Nothing here is shared with the package's compute path: it reads a configuration dict and a dict of
tensors, works on one whole sequence at a time in float64 (or the dtype asked for), builds every mask
as a dense [T, T] table and walks the recurrence token by token.  The engine's results are compared
with it.

Notation.  x[t] is the residual stream at token t.  A layer is x <- x + mixer(N1(x)), then (where it has a
feed-forward) x <- x + ff(N2(x)), every N an RMS norm with a plain weight.  The mixer runs two branches on the
same input: attention whose weights are sigmoids, mixed across heads, and a retention (a linear recurrence with
one fixed decay per head); each branch's output is RMS-normed over the width and the mixer returns half their sum.
The feed-forward is a gated dense one or a routed mixture of small squared-relu experts with a gated shared expert.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def silu(z):
    return z * torch.sigmoid(z)


def rotary_frequencies(rot, dtype):
    """f_i = base^(-2i/dims); with a `scaling` block the frequencies are rescaled by wavelength l = 2 pi / f:
    kept where l < original/high, divided by factor where l > original/low, blended linearly in between."""
    dims = int(rot["dims"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = float(rot["base"]) ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        out = f.clone()
        for j in range(f.numel()):
            wl = 2 * math.pi / float(f[j])
            if wl < orig / high:
                continue
            if wl > orig / low:
                out[j] = f[j] / factor
            else:
                s = (orig / wl - low) / (high - low)
                out[j] = (1 - s) * f[j] / factor + s * f[j]
        f = out
    return f


def rotate(u, rot):
    """u[T, heads, dim]: the first rot.dims dimensions of each head turn by position * f_i, dimension i paired with
    i + dims/2; the rest pass."""
    if not rot or not int(rot.get("dims", 0)):
        return u
    T, dims = u.shape[0], int(rot["dims"])
    half = dims // 2
    f = rotary_frequencies(rot, u.dtype)
    a = torch.arange(T, dtype=u.dtype)[:, None] * f[None, :]          # [T, half]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    lo, hi = u[..., :half], u[..., half:dims]
    return torch.cat([lo * c - hi * s, hi * c + lo * s, u[..., dims:]], dim=-1)


def sigmoid_attention(h, W, m, eps):
    """Left branch.  q and k are RMS-normed over the whole projection (weights of that width), rotated; scores are
    scaled and capped; a visible key's weight is sigmoid(score + pb[head]); the heads' weight tables are mixed by
    `talk`; head hd applies its mixed weights to the values of key/value head hd // (heads / kv_heads)."""
    T = h.shape[0]
    H, G, D, Dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = rms_norm(h @ W["q"].T, eps, W["q.norm"]).reshape(T, H, D)
    k = rms_norm(h @ W["k"].T, eps, W["k.norm"]).reshape(T, G, D)
    v = (h @ W["v"].T).reshape(T, G, Dv)
    q, k = rotate(q, m.get("rot")), rotate(k, m.get("rot"))
    per = H // G
    cap = m.get("softcap")
    visible = torch.tril(torch.ones(T, T, dtype=torch.bool))
    weights = torch.zeros(H, T, T, dtype=h.dtype)
    for hd in range(H):
        s = (q[:, hd] @ k[:, hd // per].T) * float(m["scale"])
        if cap:
            s = float(cap) * torch.tanh(s / float(cap))
        weights[hd] = torch.where(visible, torch.sigmoid(s + W["pb"][hd]), torch.zeros_like(s))
    mixed = torch.einsum("hg,gij->hij", W["talk"], weights)
    out = torch.stack([mixed[hd] @ v[:, hd // per] for hd in range(H)], dim=1)      # [T, H, Dv]
    return out.reshape(T, H * Dv) @ W["o"].T


def retention(h, W, m, eps):
    """Right branch.  Per head, with S [dim, vdim] starting at zero: S <- decay S + k v^T, o = S^T q, k scaled by
    dim^-1/2 after its rotation; o divided by its root mean square per head, times silu(W_g h), then W_o."""
    T = h.shape[0]
    H, D, Dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = rotate((h @ W["q"].T).reshape(T, H, D), m.get("rot"))
    k = rotate((h @ W["k"].T).reshape(T, H, D), m.get("rot")) * D ** -0.5
    v = (h @ W["v"].T).reshape(T, H, Dv)
    o = torch.zeros(T, H, Dv, dtype=h.dtype)
    S = torch.zeros(H, D, Dv, dtype=h.dtype)
    decay = [float(d) for d in m["decay"]]
    for t in range(T):
        for hd in range(H):
            S[hd] = decay[hd] * S[hd] + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S[hd].T @ q[t, hd]
    o = rms_norm(o, eps).reshape(T, H * Dv) * silu(h @ W["g"].T)
    return o @ W["o"].T


def sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix)}


def parallel_mixer(h, W, m, eps):
    left = rms_norm(sigmoid_attention(h, sub(W, "left."), m["left"], eps), eps, W["left.out"])
    right = rms_norm(retention(h, sub(W, "right."), m["right"], eps), eps, W["right.out"])
    return 0.5 * (left + right)


def dense_feed_forward(h, W):
    return (silu(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def expert(h, W):
    return (torch.relu(h @ W["up"].T) ** 2) @ W["down"].T


def routed_feed_forward(h, W, mlp, margins=None):
    """softmax scores over all experts; the `top` largest of score + correction are chosen; a chosen expert weighs
    score * router.scale (no renormalisation); the shared expert is added times sigmoid(sg . h).  `margins`, a list,
    receives [T]: by how much (in choice scores) each token's choice is decided, the gap between the last expert
    chosen and the first one left out (infinite where all are chosen)."""
    r = mlp["router"]
    E, top = int(r["experts"]), int(r["top"])
    s = torch.softmax(h @ W["router"].T, dim=-1)
    choice = s + W["correction"] if "correction" in W else s
    idx = torch.topk(choice, top, dim=-1).indices                    # [T, top]
    if margins is not None:
        ranked = torch.sort(choice, dim=-1, descending=True).values
        margins.append(ranked[:, top - 1] - ranked[:, top] if top < E else torch.full_like(ranked[:, 0], float("inf")))
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in idx[t].tolist():
            out[t] += s[t, e] * float(r.get("scale", 1.0)) * expert(h[t:t + 1], sub(W, f"e{e}."))[0]
    if mlp.get("shared"):
        sw = sub(W, "shared.")
        out = out + torch.sigmoid(h @ sw["sg"].T) * expert(h, sw)
    return out


def forward(cfg, tensors, ids, dtype=torch.float64, return_layers=False, margins=None):
    """Logits [T, vocab] of one whole sequence; with `return_layers` also the stream after every layer; `margins`, a
    list, receives every router's margins (see `routed_feed_forward`)."""
    W = {k: v.to(dtype) if v.is_floating_point() else v for k, v in tensors.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    eps = float(cfg["norm"]["eps"])
    x = W["embed"][ids] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        x = x + parallel_mixer(rms_norm(x, eps, W[f"l{i}.norm1"]), sub(W, f"l{i}.mix."), layer["mixer"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            h = rms_norm(x, eps, W[f"l{i}.norm2"])
            w = sub(W, f"l{i}.mlp.")
            x = x + (dense_feed_forward(h, w) if mlp["kind"] == "dense" else routed_feed_forward(h, w, mlp, margins))
        streams.append(x)
    logits = rms_norm(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
