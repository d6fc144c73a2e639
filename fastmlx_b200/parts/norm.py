"""Norms with the residual sum fused in front of them: RMSNorm, and the dynamic tanh."""
from __future__ import annotations

import torch

from dataclasses import dataclass

from .base import Norm, Runtime, WeightSpec, to_f32_vector


class RMSNorm(Norm):
    """x * rsqrt(mean(x^2) + eps) * w; the weight is a plain multiplier
    (tamnd/fastmlx compute/models/llama.go:402,425,432 -> mlxgo/binding_cgo.go:382-396).
    Sum of squares, rsqrt and the residual sum are 32-bit."""

    def __init__(self, width: int, eps: float, name: str, offset: float = 0.0, suffix: str = ".weight"):
        """`offset`: the multiplier is offset + w (1 for a weight that is stored around zero), added once,
        in 32-bit, when the weight is bound.  `suffix` completes the tensor's name."""
        self.width, self.eps, self.name = int(width), float(eps), name
        self.offset, self.tensor = float(offset), name + suffix

    def own_weight_specs(self):
        return [WeightSpec(self.tensor, (self.width,), "norm0" if self.offset else "norm")]

    def bind_own(self, tensors, rt: Runtime):
        self.weight = to_f32_vector(tensors[self.tensor], rt)
        if self.offset:
            self.weight = (self.weight + self.offset).contiguous()

    def weight_bytes(self):
        return self.weight.numel() * 4

    def forward(self, x, residual):
        # Beside bfloat16 activations the stream (the running sum of every layer's output) is kept
        # in 32-bit: each layer's contribution is small against it, and rounding the sum to
        # bfloat16 twice a layer is what a deep model's logits would feel most.
        return self.rt.k.add_rmsnorm(x, residual, self.weight, self.eps, stream_dtype=torch.float32,
                                     out_dtype=self.rt.dtype)

    def emit(self, b, x, stream):
        from ..engine.native import BF16, F32, OP_ADD_RMSNORM
        out = b.reg(self.width)
        args = dict(out0=out, vec=b.ptr(self.weight), n=self.width, eps=self.eps)
        if stream is None and b.act == BF16:
            # the stream's first value, widened into a 32-bit register of its own
            stream = b.reg(self.width, F32)
            b.op(OP_ADD_RMSNORM, in0=x, in1=stream, init=1, **args)
            b.release(x)
        elif stream is None:
            b.op(OP_ADD_RMSNORM, in0=x, **args)          # x itself is the stream from here on
            stream = x
        else:
            b.op(OP_ADD_RMSNORM, in0=-1 if x is None else x, in1=stream, **args)
            b.release(x)
        return out, stream

    def fold(self):
        """(weight, eps) for a kernel that normalises its input rows itself."""
        return (self.weight, self.eps)


@dataclass
class Pending:
    """A sublayer's output that is not in the stream yet: the stream is residual + mult * norm(x) + add, where
    `norm` (a DynamicTanh or None) stands behind the sublayer and `add` is a vector or None.  A block hands this
    on instead of a finished sum, so that the next norm's kernel does the sum in the same pass."""
    x: torch.Tensor
    norm: "DynamicTanh | None" = None
    mult: float = 1.0
    add: torch.Tensor | None = None


class DynamicTanh(Norm):
    """tanh(alpha x) w + b with a scalar alpha, a weight and a bias: no mean and no variance are computed.
    Tensors: `<name>` (the weight), `<name>.b`, `<name>.alpha` (a scalar).  All in 32-bit.

    `forward(x, residual)` takes for x a tensor (added to the stream as it is) or a `Pending` (the norm behind
    the sublayer before, the stream's multiplier and a vector to add): one kernel adds it to the 32-bit stream
    and applies this norm to the sum."""

    def __init__(self, width: int, name: str, weight_suffix: str = "", bias_suffix: str = ".b", alpha_suffix: str = ".alpha"):
        self.width, self.name = int(width), name
        self.names = (name + weight_suffix, name + bias_suffix, name + alpha_suffix)

    def own_weight_specs(self):
        w, b, a = self.names
        return [WeightSpec(w, (self.width,), "norm"), WeightSpec(b, (self.width,), "bias"), WeightSpec(a, (), "alpha")]

    def bind_own(self, tensors, rt: Runtime):
        w, b, a = self.names
        self.weight, self.bias = to_f32_vector(tensors[w], rt), to_f32_vector(tensors[b], rt)
        self.alpha = float(tensors[a].float().item())

    def weight_bytes(self):
        return 8 * self.width

    def args(self):
        return (self.alpha, self.weight, self.bias)

    def forward(self, x, residual, out=None):
        p = x if isinstance(x, Pending) else Pending(x)
        return self.rt.k.dyt_step(p.x, p.norm.args() if p.norm is not None else None, p.mult, p.add, residual, self.args(),
                                  self.rt.dtype, out=out)


def settle(x, residual, rt: Runtime, out=None, out_dtype=None):
    """The stream with a pending output added, and (where `out_dtype` or `out` asks for it) a copy of the sum in
    the activations' type, e.g. into a slice of a wider buffer.  -> (copy or None, residual)."""
    p = x if isinstance(x, Pending) else Pending(x)
    want = out is not None or out_dtype is not None
    return rt.k.dyt_step(p.x, p.norm.args() if p.norm is not None else None, p.mult, p.add, residual,
                         None if want else False, out_dtype or rt.dtype, out=out)
