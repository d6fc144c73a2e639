"""What stands in front of each pass of a looped run of layers."""
from __future__ import annotations

import torch

from .base import Part, Runtime, WeightSpec, to_compute, to_f32_vector
from .norm import Pending, settle


class LoopInput(Part):
    """Owns the tensors of a loop's entry: W_in [width, 2 width] and a vector per pass, step [times, width].
    In front of pass p the stream x is replaced by W_in [x ; e] + step[p], e being the token embeddings as the
    embedding left them (`ctx.scratch["embedding"]`, which the model keeps for the step)."""

    def __init__(self, width: int, times: int, in_name: str, step_name: str):
        self.width, self.times, self.in_name, self.step_name = int(width), int(times), in_name, step_name

    def own_weight_specs(self):
        return [WeightSpec(self.in_name, (self.width, 2 * self.width), "matrix"),
                WeightSpec(self.step_name, (self.times, self.width), "bias")]

    def bind_own(self, tensors, rt: Runtime):
        self.weight = to_compute(tensors[self.in_name], rt)
        self.steps = to_f32_vector(tensors[self.step_name], rt)

    def weight_bytes(self):
        return self.weight.numel() * self.weight.element_size()


class LoopPass(Part):
    """The entry of pass `index`, as a layer of the model's schedule that has no cache: it settles what the layer
    before left pending, writes the stream beside the embeddings, and hands the product on as the start of a
    new stream, with the pass's vector still to be added (the next norm's kernel adds it)."""

    supports_cuda_graph = True

    def __init__(self, entry: LoopInput, index: int):
        self.entry, self.index = entry, int(index)

    def children(self):
        return (self.entry,) if self.index == 0 else ()       # the tensors are declared and bound once

    def cache_spec(self):
        return None

    def state_spec(self):
        return None

    def forward(self, delta, residual, ctx, cache):
        e, rt, d = self.entry, self.entry.rt, self.entry.width
        x0 = ctx.scratch["embedding"]
        # one buffer per forward pass, shared by the loop's passes: the embeddings are copied beside the stream's place
        # once.  A context may be run twice (the warm-up before a capture, then the capture): the copy belongs to each run.
        made_for, joined = ctx.scratch.get("stream beside embeddings", (None, None))
        if made_for is not x0:
            joined = torch.empty((x0.shape[0], 2 * d), dtype=rt.dtype, device=x0.device)
            joined[:, d:].copy_(x0)
            ctx.scratch["stream beside embeddings"] = (x0, joined)
        settle(delta, residual, rt, out=joined[:, :d])
        y = rt.k.linear(joined, e.weight, None, torch.float32)
        return Pending(y, None, 1.0, e.steps[self.index]), None
