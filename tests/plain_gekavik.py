"""A plain, slow Gekavik: one function per mechanism, written from the design's equations.

Nothing here is shared with the package's compute path: it reads a configuration dict and a
dict of tensors, works on one whole sequence at a time in float64 (or the dtype asked for), and
builds every mask as a dense [T, T] table.  The engine's results are compared with it.

Notation.  x[t] is the residual stream at token t, e[t] the embedding of token t, r the
residual multiplier.  A layer is x <- x + r * N1b(mixer(N1(x))), then (where it has a
feed-forward) x <- x + r * N2b(ff(N2(x))), every N a dynamic tanh.  Layers run in the order of
the `layers` list; the layers loop.start .. loop.stop-1 run loop.times times in a row, and in
front of pass p the stream is replaced by W_in [x ; e] + step[p].
"""
from __future__ import annotations

import math

import torch


def dynamic_tanh(x, alpha, w, b):
    """tanh(alpha x) w + b: no mean, no variance."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x, eps, weight):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_pairs(x, positions, base, dims):
    """x [T, H, D]: dimensions (2i, 2i+1), i < dims/2, turn by positions * base^(-2i/dims); the rest pass."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=x.dtype)
    a = positions.to(x.dtype)[:, None] * (torch.tensor(float(base), dtype=x.dtype) ** (-2.0 * i / dims))[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def visible(T, size=None, keep_first=0):
    """[T, T] table: query i sees key j when j <= i and (i - j < size or j < keep_first)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if size:
        seen = seen & ((i - j < size) | (j < keep_first))
    return seen


def softmax_attention(q, k, v, scale, seen):
    """q [T, D], k [T, D], v [T, Dv] of one head."""
    s = (q @ k.T) * scale
    s = s.masked_fill(~seen, -math.inf)
    return torch.softmax(s, -1) @ v


def attention_mixer(h, W, m, eps):
    """Grouped queries with biased projections, q and k normalised per head (a weight shared by the
    heads) before the rotation, a window that keeps the first tokens, and an element-wise output gate."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rms_norm((h @ W["q"].T + W["q.b"]).view(T, H, D), eps, W["q.norm"])
    k = rms_norm((h @ W["k"].T + W["k.b"]).view(T, G, D), eps, W["k.norm"])
    v = (h @ W["v"].T + W["v.b"]).view(T, G, Dv)
    rot = m.get("rot") or {}
    q = rotate_pairs(q, pos, rot.get("base", 1.0), rot.get("dims", 0))
    k = rotate_pairs(k, pos, rot.get("base", 1.0), rot.get("dims", 0))
    mask = m.get("mask") or {}
    seen = visible(T, mask.get("size"), mask.get("keep_first", 0))
    out = h.new_zeros(T, H, Dv)
    for head in range(H):
        g = head // (H // G)
        out[:, head] = softmax_attention(q[:, head], k[:, g], v[:, g], m["scale"], seen)
    out = out.reshape(T, H * Dv) * torch.sigmoid(h @ W["g"].T)
    return out @ W["o"].T


def latent_attention_mixer(h, W, m, eps):
    """Keys and values of every head are read out of one normalised latent per token; the queries pass a
    latent of their own; no positions; a plain window; one gate value per head."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ W["dq"].T, eps, W["dq.norm"])
    q = (cq @ W["uq"].T).view(T, H, D)
    c = rms_norm(h @ W["dkv"].T, eps, W["dkv.norm"])
    k = (c @ W["uk"].T).view(T, H, D)
    v = (c @ W["uv"].T).view(T, H, Dv)
    seen = visible(T, (m.get("mask") or {}).get("size"), 0)
    gate = torch.sigmoid(h @ W["g"].T)                                       # [T, H]
    out = h.new_zeros(T, H, Dv)
    for head in range(H):
        out[:, head] = softmax_attention(q[:, head], k[:, head], v[:, head], m["scale"], seen) * gate[:, head, None]
    return out.reshape(T, H * Dv) @ W["o"].T


def expert(h, gate, up, down, limit):
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ down.T


def route(z, top, groups, keep, margins=None):
    """z [T, E] router logits -> weights [T, E], zero where an expert is not chosen: softmax scores; a group
    of neighbouring experts scores as its best member; only the `keep` best groups may be chosen from.
    `margins`, a list, receives [T]: by how much (in logits) each token's choice is decided, the smaller of the
    gap between the last kept group and the first that is not, and between the last chosen expert and the next."""
    T, E = z.shape
    s = torch.softmax(z, -1)
    allowed = torch.ones_like(s, dtype=torch.bool)
    gap = torch.full((T,), math.inf, dtype=z.dtype)
    if groups and groups > 1 and keep < groups:
        per = E // groups
        best = s.view(T, groups, per).max(-1).values
        kept = torch.zeros(T, groups, dtype=torch.bool)
        kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
        allowed = kept[:, :, None].expand(T, groups, per).reshape(T, E)
        zb = z.view(T, groups, per).max(-1).values.sort(-1, descending=True).values
        gap = zb[:, keep - 1] - zb[:, keep]
    if margins is not None:
        zs = z.masked_fill(~allowed, -math.inf).sort(-1, descending=True).values
        if top < E:
            gap = torch.minimum(gap, zs[:, top - 1] - zs[:, top])
        margins.append(gap)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    w = torch.zeros_like(s)
    w.scatter_(1, chosen, s.gather(1, chosen))
    return w


def moe_ff(h, W, mlp, margins=None):
    r = mlp["router"]
    z = h @ W["router"].T
    g = r.get("groups") or {}
    w = route(z, r["top"], g.get("count", 1), g.get("keep", 1), margins)
    out = torch.zeros_like(h)
    for e in range(r["experts"]):
        rows = torch.nonzero(w[:, e] > 0).flatten()
        if rows.numel():
            y = expert(h[rows], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"], mlp["expert"]["limit"])
            out[rows] += w[rows, e, None] * y
    if mlp.get("shared"):
        out = out + expert(h, W["shared.gate"], W["shared.up"], W["shared.down"], mlp["shared"]["limit"])
    return out


def sub(tensors, prefix, dtype):
    return {n[len(prefix):]: t.to(dtype) for n, t in tensors.items() if n.startswith(prefix)}


def norm_of(tensors, name, dtype):
    return float(tensors[name + ".alpha"]), tensors[name].to(dtype), tensors[name + ".b"].to(dtype)


def layer_passes(config):
    """[(layer index, pass number or None)]: a pass number stands at the first layer of each pass of the loop."""
    n = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for p in range(times):
        order += [(i, p if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(config, tensors, tokens, dtype=torch.float64, streams=None, margins=None):
    """Logits [T, vocab] of one whole sequence; `streams`, a list, receives the residual stream after
    every layer run; `margins`, a list, every router's margins (see `route`)."""
    eps, r = config["norm"]["eps"], config["residual_mult"]
    emb = tensors["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    x = emb
    for i, p in layer_passes(config):
        spec = config["layers"][i]
        if p is not None:
            x = torch.cat([x, emb], -1) @ tensors["loop.in"].to(dtype).T + tensors["loop.step"].to(dtype)[p]
        mixer = {"attention": attention_mixer, "latent_attention": latent_attention_mixer}[spec["type"]]
        y = mixer(dynamic_tanh(x, *norm_of(tensors, f"l{i}.norm1", dtype)), sub(tensors, f"l{i}.mix.", dtype),
                  spec["mixer"], eps)
        x = x + r * dynamic_tanh(y, *norm_of(tensors, f"l{i}.norm1b", dtype))
        if spec.get("mlp"):
            y = moe_ff(dynamic_tanh(x, *norm_of(tensors, f"l{i}.norm2", dtype)), sub(tensors, f"l{i}.mlp.", dtype),
                       spec["mlp"], margins)
            x = x + r * dynamic_tanh(y, *norm_of(tensors, f"l{i}.norm2b", dtype))
        if streams is not None:
            streams.append(x.clone())
    x = dynamic_tanh(x, *norm_of(tensors, "final.norm", dtype))
    return x @ tensors["head"].to(dtype).T
