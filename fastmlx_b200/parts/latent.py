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

    That form reads kv_rank values per key and head, which suits single tokens (the cache is what a decode step
    reads).  A long portion of a prompt multiplies kv_rank / dim times more than it must, so steps with a portion of
    LONG_PORTION tokens or more (bfloat16, head sizes the tiled kernel takes) read the keys and values of the tokens in
    sight out of the latents once per step, into pages of their own that live for the step, and attend over those
    with the heads' own sizes.  The cache holds latents either way.

    Tensors, under `name`: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g (optional), o."""

    supports_cuda_graph = True
    LONG_PORTION = 128

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
        # long portions: every head's keys, then every head's values, in one product over the latents in sight
        self.ukv = None
        if rt.dtype == torch.bfloat16 and self.hd == self.vd and self.hd % 16 == 0 and self.hd <= 256 and rt.device.type == "cuda":
            self.ukv = torch.cat([uk.reshape(self.nh * self.hd, self.kv_rank), self.uv.view(self.nh * self.vd, self.kv_rank)], 0).contiguous()

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
        if self.ukv is not None and not ctx.all_decode and ctx.max_q_len >= self.LONG_PORTION and cache.kv.dtype == torch.bfloat16 \
                and hasattr(k, "paged_attention_wide"):
            heads = self.attend_long(cq, ctx, cache, g)
            if self.has_gate:
                k.sigmoid_gate(heads, down[:, self.q_rank + self.kv_rank:], self.vd)
            return self.o.forward(heads)
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

    def attend_long(self, cq, ctx, cache, g):
        """Keys and values of every position a row of this step may see, read out of the cached latents into pages
        that live for the step (one per page of positions in sight, whole pages: what lies outside a row's sight on
        them is never loaded), and attention with the heads' own sizes.  -> [T, H * vdim]."""
        from types import SimpleNamespace
        k, ps = self.rt.k, g.page_size
        dev = cq.device
        rows, blks = [], []
        for r in range(ctx.R):
            c = ctx.h_row_ctx[r]
            n = ctx.h_row_start[r + 1] - ctx.h_row_start[r]
            if ctx.h_row_slot[r] < 0 or n <= 0:
                continue
            lo = max(0, c - self.window + 1) if self.window > 0 else 0
            for b in range(lo // ps, (c + n - 1) // ps + 1):
                rows.append(r)
                blks.append(b)
        # one copy from pinned memory, so that the host does not fall into step with the device
        both = torch.tensor([rows, blks], dtype=torch.long, pin_memory=True).to(dev, non_blocking=True)
        rows_t, blks_t = both[0], both[1]
        pages = g.block_tables[rows_t, blks_t].long().clamp_(min=0)
        latents = cache.kv.view(cache.kv.shape[0], ps, self.kv_rank)[pages]      # [pages in sight, page, kv_rank]
        kv = k.linear(latents.view(-1, self.kv_rank), self.ukv, None, torch.bfloat16)
        kv = kv.view(len(rows), ps, 2, self.nh, self.hd).permute(0, 2, 3, 1, 4).contiguous()      # pages of [2, H, page, dim]
        table = torch.full_like(g.block_tables, -1)
        table[rows_t, blks_t] = torch.arange(len(rows), dtype=torch.int32, device=dev)
        own = SimpleNamespace(block_tables=table, page_size=ps, window=self.window)
        ctx.scratch.setdefault("pages of a step", []).append(own)        # kept for the step: its identity keys cached views
        q = self.uq.forward(cq, out_dtype=torch.float32)
        return k.paged_attention_wide(q, kv, ctx, own, self.nh, self.nh, self.hd, self.scale, 0.0, self.window)
