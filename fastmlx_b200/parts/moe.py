"""A routed feed-forward: a router that chooses a few small experts per token, and an optional expert for all."""
from __future__ import annotations

import torch

from .base import FeedForward, Part, Runtime, WeightSpec, to_compute


class RoutedExperts(FeedForward):
    """y = sum over the token's chosen experts of s_e expert_e(x) (+ shared(x)).

    Router: logits z = W_r x and scores s = softmax(z) over all experts, in 32-bit; the experts form `groups`
    equal groups of neighbours, a group scores as its best member, and only experts of the `keep` best groups may
    be chosen; the `top` best of those are, with their scores as weights (not renormalised).

    Expert (no biases): g = min(W_gate x, limit), u = clamp(W_up x, -limit, limit), W_down (g sigmoid(1.702 g) (u + 1)).
    The shared expert has the same form with a width and a limit of its own and weight 1.

    All experts' gate and up matrices are stacked into one matrix and their down matrices laid side by side.  A step
    runs the stacked product for every token, the activation kernel zeroes the columns of experts a token did not
    choose and scales the others by the token's weight, and one product with the down matrices gives the weighted
    sum, added up inside the product's 32-bit accumulators.  No token's result depends on what else is in the
    batch, nothing loops on the host, and a decode step can be captured.  It reads every expert's weights and
    multiplies experts / top times more than needed, which is the right trade for experts as small as a tile of
    the product and the wrong one for large ones.

    Tensors, under `name`: router; e<i>.gate, e<i>.up, e<i>.down; shared.gate, shared.up, shared.down."""

    supports_cuda_graph = True

    def __init__(self, width: int, experts: int, top: int, ff: int, limit: float, name: str, groups: int = 1,
                 keep: int = 1, shared_ff: int = 0, shared_limit: float = 0.0, weight_suffix: str = "",
                 expert_prefix: str = "e", shared_name: str = "shared", router_name: str = "router",
                 proj_names=("gate", "up", "down")):
        self.width, self.E, self.top, self.ff, self.limit = int(width), int(experts), int(top), int(ff), float(limit)
        self.groups, self.keep = max(1, int(groups)), max(1, int(keep))
        if self.E % self.groups or not 0 < self.top <= self.E:
            raise ValueError(f"{experts} experts do not form {groups} equal groups, or top={top} is out of range")
        if self.top > (self.E // self.groups) * min(self.keep, self.groups):
            raise ValueError(f"top={top} experts cannot come from {keep} groups of {self.E // self.groups}")
        self.shared_ff, self.shared_limit = int(shared_ff), float(shared_limit)
        self.F = self.E * self.ff + self.shared_ff
        g, u, d = proj_names
        pre = [f"{name}.{expert_prefix}{i}" for i in range(self.E)] + ([f"{name}.{shared_name}"] if self.shared_ff else [])
        widths = [self.ff] * self.E + ([self.shared_ff] if self.shared_ff else [])
        self.gate_names = [(f"{p}.{g}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.up_names = [(f"{p}.{u}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.down_names = [(f"{p}.{d}{weight_suffix}", w) for p, w in zip(pre, widths)]
        self.router_name = f"{name}.{router_name}{weight_suffix}"

    def own_weight_specs(self):
        specs = [WeightSpec(self.router_name, (self.E, self.width), "matrix")]
        specs += [WeightSpec(n, (w, self.width), "matrix") for n, w in self.gate_names + self.up_names]
        specs += [WeightSpec(n, (self.width, w), "matrix") for n, w in self.down_names]
        return specs

    def bind_own(self, tensors, rt: Runtime):
        self.router = to_compute(tensors[self.router_name], rt)
        self.gate_up = torch.cat([to_compute(tensors[n], rt) for n, _ in self.gate_names + self.up_names], 0).contiguous()
        self.down = torch.cat([to_compute(tensors[n], rt) for n, _ in self.down_names], 1).contiguous()

    def weight_bytes(self):
        return sum(t.numel() * t.element_size() for t in (self.router, self.gate_up, self.down))

    def route(self, x):
        """-> the tokens' weights over the experts, 32-bit [T, E], zero where an expert is not chosen."""
        k = self.rt.k
        return k.moe_route(k.linear(x, self.router, None, torch.float32), self.top, self.groups, self.keep)

    def forward(self, x, ctx):
        k = self.rt.k
        w = self.route(x)
        gu = k.linear(x, self.gate_up, None, self.rt.dtype)
        act = k.moe_expert_act(gu, w, self.E, self.ff, self.limit, self.shared_limit)
        return k.linear(act, self.down, None, self.rt.dtype)
