"""A plain, slow Medirax: one function per mechanism, written from the design's equations.

Nothing here is shared with the package's compute path: it reads a configuration dict and
a dict of tensors, works on one sequence at a time in float64 (or the dtype asked for) and
keeps its own caches as Python lists.  The engine's results are compared with it.

Notation.  x[t] is the residual stream at token t.  A layer is parallel: with
h = norm(x), x <- x + mixer(h) + ff(h).  Layers run in the order of the `layers` list,
and the layers loop.start .. loop.stop-1 run loop.times times in a row (same weights, a
cache of its own for every pass).
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, eps, weight=None, offset=0.0):
    """x / sqrt(mean(x^2) + eps) (* (offset + weight))."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    if weight is not None:
        y = y * (offset + weight)
    return y


def unit_vector(x, eps=1e-6):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def relu_squared(x):
    return torch.relu(x) ** 2


def causal_conv_silu(x, w):
    """x [T, C], w [C, taps] (the last column multiplies the current token), zeros before
    the start; then silu."""
    T, C = x.shape
    taps = w.shape[1]
    padded = torch.cat([x.new_zeros(taps - 1, C), x], 0)
    y = x.new_zeros(T, C)
    for j in range(taps):
        y = y + padded[j: j + T] * w[:, j]
    return silu(y)


def rotate_half_partial(x, positions, base, dims):
    """x [T, H, D]: the first `dims` dimensions of every head are rotated, dimension i with
    i + dims/2 by the angle p * base^(-2i/dims); the rest pass."""
    if dims == 0:
        return x
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    f = torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def delta_mixer(h, W, m, eps):
    """Gated delta rule over one whole sequence h [T, width]; W maps '.q' ... to tensors."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv_silu(h @ W["q"].T, W["q.conv"]).view(T, G, D)
    k = causal_conv_silu(h @ W["k"].T, W["k.conv"]).view(T, G, D)
    v = causal_conv_silu(h @ W["v"].T, W["v.conv"]).view(T, H, Dv)
    q = unit_vector(q) * D ** -0.5
    k = unit_vector(k)
    beta = torch.sigmoid(h @ W["b"].T)                                       # [T, H]
    decay = torch.exp(-torch.exp(W["A_log"]) * torch.nn.functional.softplus(h @ W["a"].T + W["dt_bias"]))
    gate = silu(h @ W["g"].T).view(T, H, Dv)
    out = h.new_zeros(T, H, Dv)
    for head in range(H):
        kv = head // (H // G)
        S = h.new_zeros(D, Dv)
        for t in range(T):
            S = decay[t, head] * S
            u = beta[t, head] * (v[t, head] - S.T @ k[t, kv])
            S = S + torch.outer(k[t, kv], u)
            out[t, head] = S.T @ q[t, kv]
    out = rms_norm(out, eps, W["norm"]) * gate
    return out.reshape(T, H * Dv) @ W["o"].T


def attention_mixer(h, W, m, eps):
    """Sliding-window attention with capped scores over one whole sequence."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ W["q"].T + W["q.b"]).view(T, H, D)
    k = (h @ W["k"].T + W["k.b"]).view(T, G, D)
    v = (h @ W["v"].T + W["v.b"]).view(T, G, Dv)
    rot = m.get("rot") or {"base": 1.0, "dims": 0}
    q = rms_norm(rotate_half_partial(q, pos, rot["base"], rot["dims"]), eps)
    k = rms_norm(rotate_half_partial(k, pos, rot["base"], rot["dims"]), eps)
    cap = m.get("softcap")
    window = (m.get("mask") or {}).get("size")
    out = h.new_zeros(T, H, Dv)
    for head in range(H):
        kv = head // (H // G)
        s = (q[:, head] @ k[:, kv].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        d = pos[:, None] - pos[None, :]
        seen = d >= 0
        if window:
            seen = seen & (d < window)
        s = s.masked_fill(~seen, -math.inf)
        out[:, head] = torch.softmax(s, -1) @ v[:, kv]
    return out.reshape(T, H * Dv) @ W["o"].T + W["o.b"]


def dense_ff(h, W):
    return relu_squared(h @ W["up"].T) @ W["down"].T


def layer_order(config):
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sub(tensors, prefix, dtype):
    return {n[len(prefix):]: t.to(dtype) for n, t in tensors.items() if n.startswith(prefix)}


def forward(config, tensors, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence; `streams`, a list, receives the residual
    stream after every layer run."""
    eps = config["norm"]["eps"]
    x = tensors["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    for i in layer_order(config):
        spec = config["layers"][i]
        h = rms_norm(x, eps, tensors[f"l{i}.norm1"].to(dtype), 1.0)
        W = sub(tensors, f"l{i}.mix.", dtype)
        mixer = {"delta": delta_mixer, "attention": attention_mixer}[spec["type"]]
        y = mixer(h, W, spec["mixer"], eps)
        if spec.get("mlp"):
            y = y + dense_ff(h, sub(tensors, f"l{i}.mlp.", dtype))
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = rms_norm(x, eps, tensors["final.norm"].to(dtype), 1.0)
    return (x @ tensors["head"].to(dtype).T) * config["logit_scale"]
