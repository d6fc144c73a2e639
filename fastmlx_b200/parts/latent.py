"""Attention whose keys and values are read out of one cached latent per token."""
from __future__ import annotations

import torch

from .base import Mixer, PagedKVSpec, Runtime, WeightSpec, to_compute, to_f32_vector
from .linear import Linear


class LatentAttention(Mixer):
    """Per token one latent c = rmsnorm(W_dkv x) w of `kv_rank` values is cached; head h has keys k = W_uk,h c and
    values v = W_uv,h c.  The queries pass a latent of their own, q = W_uq (rmsnorm(W_dq x) w).  No positions
    enter.  A query sees itself and the window - 1 tokens before it (window 0: every earlier token).  Head h's
    output is multiplied by sigmoid(W_g x)_h where a gate is named, and the heads go through W_o.

    Only c lies in the pages (one "kv head" of size kv_rank, whose keys are its values too), and neither k nor
    v is ever formed: since q_h . (W_uk,h c) = (W_uk,h^T q_h) . c, each query is carried into the latent's space
    (one small product per head), attention runs over the latents with all heads sharing them, and the heads'
    outputs, weighted sums of latents, are read out through W_uv,h afterwards.  Scores and weights are 32-bit
    (the queries stay in 32-bit from their product to the scores).

    Tensors, under `name`: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g (optional), o."""

    supports_cuda_graph = True

    def __init__(self, width: int, num_heads: int, head_dim: int, v_head_dim: int, q_rank: int, kv_rank: int,
                 eps: float, name: str, scale: float | None = None, window: int = 0, gate: bool = True,
                 weight_suffix: str = "", norm_suffix: str = ".norm"):
        self.width, self.nh, self.hd, self.vd = int(width), int(num_heads), int(head_dim), int(v_head_dim)
        self.q_rank, self.kv_rank, self.eps = int(q_rank), int(kv_rank), float(eps)
        self.scale = float(scale) if scale is not None else float(head_dim) ** -0.5
        self.window = int(window)
        self.name, self.wsfx = name, weight_suffix
        downs = [(f"{name}.dq", self.q_rank), (f"{name}.dkv", self.kv_rank)]
        if gate:
            downs.append((f"{name}.g", self.nh))
        self.has_gate = bool(gate)
        self.down = Linear(width, downs, False, weight_suffix=weight_suffix)         # one product reads x
        self.uq = Linear(self.q_rank, [(f"{name}.uq", self.nh * self.hd)], False, weight_suffix=weight_suffix)
        self.o = Linear(self.nh * self.vd, [(f"{name}.o", width)], False, weight_suffix=weight_suffix)
        self.norm_names = (f"{name}.dq{norm_suffix}", f"{name}.dkv{norm_suffix}")
        self.uk_name, self.uv_name = f"{name}.uk{weight_suffix}", f"{name}.uv{weight_suffix}"

    def children(self):
        return (self.down, self.uq, self.o)

    def own_weight_specs(self):
        return [WeightSpec(self.norm_names[0], (self.q_rank,), "norm"), WeightSpec(self.norm_names[1], (self.kv_rank,), "norm"),
                WeightSpec(self.uk_name, (self.nh * self.hd, self.kv_rank), "matrix"),
                WeightSpec(self.uv_name, (self.nh * self.vd, self.kv_rank), "matrix")]

    def bind_own(self, tensors, rt: Runtime):
        self.q_norm, self.c_norm = (to_f32_vector(tensors[n], rt) for n in self.norm_names)
        uk = to_compute(tensors[self.uk_name], rt).view(self.nh, self.hd, self.kv_rank)
        # carrying a query into the latent's space multiplies by W_uk,h^T: [H, kv_rank, dim]
        self.uk_t = uk.transpose(1, 2).contiguous()
        self.uv = to_compute(tensors[self.uv_name], rt).view(self.nh, self.vd, self.kv_rank).contiguous()

    def weight_bytes(self):
        return super().weight_bytes() + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()

    def cache_spec(self):
        return PagedKVSpec(1, self.kv_rank, self.window, 0, 0, True)

    def forward(self, x, ctx, cache):
        k, rt = self.rt.k, self.rt
        g = ctx.groups[cache.group]
        down = self.down.forward(x, out_dtype=torch.float32)
        cq = k.rmsnorm_rows(down[:, :self.q_rank], self.q_norm, self.eps, out_dtype=rt.dtype)
        if cache.writable:
            k.rmsnorm_rows(down[:, self.q_rank: self.q_rank + self.kv_rank], self.c_norm, self.eps, out=cache.kv,
                           row_map=g.slot_mapping, status=ctx.status)
        q = self.uq.forward(cq)
        q_lat = k.head_linear(q, self.uk_t, torch.float32)                       # [T, H * kv_rank], 32-bit
        wide = getattr(k, "wide_attention_takes", None)
        if wide is not None and wide(q_lat, cache.kv, self.kv_rank, self.kv_rank, None):
            o_lat = k.paged_attention_wide(q_lat, cache.kv, ctx, g, self.nh, 1, self.kv_rank, self.scale, 0.0, self.window)
        else:
            o_lat = k.paged_attention_general(q_lat, cache.kv, ctx, g, self.nh, 1, self.kv_rank, self.kv_rank, self.scale,
                                              0.0, self.window, g.page_size, values_are_keys=True)
        heads = k.head_linear(o_lat, self.uv, rt.dtype)                          # [T, H * vdim]
        if self.has_gate:
            k.sigmoid_gate(heads, down[:, self.q_rank + self.kv_rank:], self.vd)
        return self.o.forward(heads)
