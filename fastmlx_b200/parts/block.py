"""The arrangement of norm, mixer and feed-forward in one layer."""
from __future__ import annotations

import torch

from .base import FeedForward, Mixer, Norm, Part
from .linear import JoinedLinear
from .norm import Pending


class PreNormBlock(Part):
    """h += mixer(norm1(h)); h += ffn(norm2(h)) (tamnd/fastmlx compute/models/llama.go:402-429).
    The stream is carried as (delta, residual): each norm first adds the delta to the
    residual in 32-bit, then normalises the sum, so the add costs no pass of its own."""

    def __init__(self, mixer: Mixer, ffn: FeedForward, norm1: Norm, norm2: Norm):
        self.mixer, self.ffn, self.norm1, self.norm2 = mixer, ffn, norm1, norm2

    def children(self):
        return (self.norm1, self.mixer, self.norm2, self.ffn)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        delta, residual = self.mixer.forward_in_block(delta, residual, self.norm1, ctx, cache)
        return self.ffn.forward_in_block(delta, residual, self.norm2, ctx)

    def emit(self, b, delta, stream, pos):
        """Native program: (delta register, stream register or None) -> (delta', stream)."""
        x, stream = self.norm1.emit(b, delta, stream)
        y = self.mixer.emit(b, x, pos)
        b.release(x)
        x, stream = self.norm2.emit(b, y, stream)
        z = self.ffn.emit(b, x)
        b.release(x)
        return z, stream


class ParallelBlock(Part):
    """h = norm(x); x <- x + (mixer(h) + ffn(h)): one norm, and both sublayers read its output.

    Mixer and feed-forward are built with `output=False`: their output projections are joined
    into one product over [mixer's heads | feed-forward's hidden layer], so that the two
    sublayers' outputs are added inside the product's 32-bit accumulators, and the block's
    output is rounded once before the 32-bit residual sum takes it.  `ffn` may be None."""

    def __init__(self, mixer: Mixer, ffn: FeedForward | None, norm: Norm, width: int):
        self.mixer, self.ffn, self.norm = mixer, ffn, norm
        pieces = [mixer.out_piece] + ([ffn.out_piece] if ffn is not None else [])
        self.out = JoinedLinear(width, pieces)

    def children(self):
        return tuple(p for p in (self.norm, self.mixer, self.ffn, self.out) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        h, residual = self.norm.forward(delta, residual)
        joined = torch.empty((h.shape[0], self.out.in_features), dtype=self.rt.dtype, device=h.device)
        m = self.mixer.inner_features
        self.mixer.forward_inner(h, ctx, cache, out=joined[:, :m] if self.ffn is not None else joined)
        if self.ffn is not None:
            self.ffn.forward_inner(h, ctx, out=joined[:, m:])
        return self.out.forward(joined), residual


class SandwichBlock(Part):
    """x <- x + r * norm1b(mixer(norm1(x))); x <- x + r * norm2b(ffn(norm2(x))): a norm in front of and behind each
    sublayer, and a multiplier r on what enters the stream.  `ffn` (with its two norms) may be None.

    The block hands its last sublayer's output on as a `Pending` sum, so that the norm behind a sublayer, the
    scaled sum into the 32-bit stream and the norm in front of the next sublayer are one kernel; its norms must
    take a `Pending` (`DynamicTanh` does)."""

    def __init__(self, mixer: Mixer, ffn: FeedForward | None, norm1: Norm, norm1b: Norm, norm2: Norm | None,
                 norm2b: Norm | None, mult: float = 1.0):
        self.mixer, self.ffn, self.mult = mixer, ffn, float(mult)
        self.norm1, self.norm1b, self.norm2, self.norm2b = norm1, norm1b, norm2, norm2b
        if ffn is not None and (norm2 is None or norm2b is None):
            raise ValueError("a feed-forward needs the norms around it")

    def children(self):
        parts = [self.norm1, self.mixer, self.norm1b]
        if self.ffn is not None:
            parts += [self.norm2, self.ffn, self.norm2b]
        return tuple(parts)

    def cache_spec(self):
        return self.mixer.cache_spec()

    def state_spec(self):
        return self.mixer.state_spec()

    @property
    def supports_cuda_graph(self):
        return bool(getattr(self.mixer, "supports_cuda_graph", False)) and \
            bool(getattr(self.ffn, "supports_cuda_graph", True))

    def forward(self, delta, residual, ctx, cache):
        h, residual = self.norm1.forward(delta, residual)
        pending = Pending(self.mixer.forward(h, ctx, cache), self.norm1b, self.mult)
        if self.ffn is None:
            return pending, residual
        h, residual = self.norm2.forward(pending, residual)
        return Pending(self.ffn.forward(h, ctx), self.norm2b, self.mult), residual
