"""A plain, slow Sorupel: one function per mechanism, written from the design's equations.

Nothing here is shared with the package's compute path: it reads a configuration dict and a
dict of tensors, works on one whole sequence at a time in float64 (or the dtype asked for),
builds every mask as a dense [T, T] table and walks every recurrence token by token.  The
engine's results are compared with it.

Notation.  x[t] is the residual stream at token t, ids[t] its token.  A layer is
x <- x + mixer(N1(x)), then (where it has a feed-forward) x <- x + ff(N2(x)), every N an RMS
norm with a plain weight.  Three mixers: chunked attention whose values are its keys, attention
over a cached latent with a rotated key part shared by the heads, and a state-space recurrence
with a matrix of state per head.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, eps, weight=None):
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def embed(ids, W, cfg):
    """x[t] = E[ids[t]] + B[(ids[t-1] * mul_prev + ids[t] * mul_cur) mod buckets]; the first token of a sequence
    takes row `buckets` of B, its last one."""
    x = W["embed"][ids]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        n = int(bg["buckets"])
        rows = torch.full_like(ids, n)
        rows[1:] = (ids[:-1] * int(bg["mul_prev"]) + ids[1:] * int(bg["mul_cur"])) % n
        x = x + W["bigram"][rows]
    return x


def rotate_half(x, positions, base, dims):
    """x [T, H, D]: dimension i pairs with i + dims/2, i < dims/2, and the pair turns by positions * base^(-2i/dims);
    dimensions from `dims` on pass."""
    if not dims:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def causal(T):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return j <= i


def same_chunk(T, size):
    """[T, T]: query i sees key j <= i of its own chunk, chunks counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size:
        seen = seen & ((i // size) == (j // size))
    return seen


def sink_softmax(s, seen, sink):
    """Rows of s over the keys in sight, with one more term exp(sink) in the denominator that has no value."""
    s = s.masked_fill(~seen, -math.inf)
    sink = torch.as_tensor(sink, dtype=s.dtype)
    m = torch.maximum(s.max(-1, keepdim=True).values, sink)
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink - m))


def chunked_attention(h, W, m, eps, positions=None):
    """Grouped queries; the values are the keys as projected (no norm, no rotation); q and k are RMS-normed over
    the whole projection; capped scores; softmax with one added to the denominator; one gate value per head."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T) if positions is None else positions
    q = h @ W["q"].T
    k = h @ W["k"].T
    v = k.reshape(T, G, D)
    q = rms_norm(q, eps, W["q.norm"]).reshape(T, H, D)
    k = rms_norm(k, eps, W["k.norm"]).reshape(T, G, D)
    rot = m.get("rot") or {}
    q = rotate_half(q, pos, rot.get("base", 1.0), rot.get("dims", 0))
    k = rotate_half(k, pos, rot.get("base", 1.0), rot.get("dims", 0))
    seen = same_chunk(T, (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ W["g"].T)                       # [T, H]
    cap = m.get("softcap")
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        p = sink_softmax(s, seen, 0.0)
        outs.append((p @ v[:, g]) * gate[:, hd:hd + 1])
    return torch.cat(outs, -1) @ W["o"].T


def latent_of(h, W, m, eps, positions=None):
    """What a latent-attention layer caches per token: the normed latent c and the rotated key part."""
    T = h.shape[0]
    r, R = m["kv_rank"], m["rot_dim"]
    pos = torch.arange(T) if positions is None else positions
    d = h @ W["dkv"].T
    c = rms_norm(d[:, :r], eps, W["dkv.norm"])
    kr = rotate_half(d[:, r:r + R].reshape(T, 1, R), pos, m["rot"]["base"], R).reshape(T, R)
    return c, kr


def latent_attention(h, W, m, eps, cached=None, positions=None):
    """Per head keys [W_uk c | rotated part shared by the heads], values W_uv c; causal; a learned sink per head;
    an element-wise gate.  `cached` = (c, rotated key part) of the layer whose cache this layer reads."""
    T = h.shape[0]
    H, D, R, Dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T) if positions is None else positions
    c, kr = cached if cached is not None else latent_of(h, W, m, eps, positions)
    q = (h @ W["q"].T).reshape(T, H, D + R)
    qn = q[..., :D]
    qr = rotate_half(q[..., D:], pos, m["rot"]["base"], R)
    kn = (c @ W["uk"].T).reshape(T, H, D)
    v = (c @ W["uv"].T).reshape(T, H, Dv)
    seen = causal(T)
    outs = []
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        p = sink_softmax(s, seen, W["sink"][hd].to(s.dtype))
        outs.append(p @ v[:, hd])
    o = torch.cat(outs, -1) * torch.sigmoid(h @ W["g"].T)
    return o @ W["o"].T, (c, kr)


def short_convolution(u, taps_w, bias):
    """u [T, C], taps_w [C, taps]: y[t] = sum_i w[:, taps-1-i] u[t-i] + b, zeros before the start."""
    T, C = u.shape
    taps = taps_w.shape[1]
    y = torch.zeros_like(u) + bias
    for i in range(taps):
        shifted = torch.zeros_like(u)
        if i < T:
            shifted[i:] = u[:T - i]
        y = y + shifted * taps_w[:, taps - 1 - i]
    return y


def state_space(h, W, m, eps):
    """The state-space mixer: per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T, y_t = S_t^T C_t + D x_t,
    then y silu(z), an RMS norm over `norm_groups` equal parts of the row, a weight, the output projection."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    p = h @ W["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, W["conv"], W["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    dt = softplus(dt + W["dt_bias"])                          # [T, H]
    decay = torch.exp(-torch.exp(W["A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=h.dtype)
    S = torch.zeros(H, N, P, dtype=h.dtype)
    per = H // G
    for t in range(T):
        for hd in range(H):
            g = hd // per
            S[hd] = decay[t, hd] * S[hd] + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S[hd].T @ C[t, g] + W["D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    ng = m["norm_groups"]
    y = rms_norm(y.reshape(T, ng, inner // ng), eps).reshape(T, inner) * W["norm"]
    return y @ W["o"].T


def gated_feed_forward(h, W):
    return (gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, ids, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one whole sequence; with `return_layers` also the stream after every layer."""
    W = {k: v.to(dtype) if v.is_floating_point() else v for k, v in tensors.items()}
    ids = torch.as_tensor(ids, dtype=torch.long)
    eps = float(cfg["norm"]["eps"])
    x = embed(ids, W, cfg)
    caches = {}
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        h = rms_norm(x, eps, W[f"l{i}.norm1"])
        w = sub(W, f"l{i}.mix.")
        if layer["type"] == "attention":
            y = chunked_attention(h, w, m, eps)
        elif layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, caches[i] = latent_attention(h, w, m, eps, caches[src] if src is not None else None)
        elif layer["type"] == "mamba2":
            y = state_space(h, w, m, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + gated_feed_forward(rms_norm(x, eps, W[f"l{i}.norm2"]), sub(W, f"l{i}.mlp."))
        streams.append(x)
    logits = rms_norm(x, eps, W["final.norm"]) @ W["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
