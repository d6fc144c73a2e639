"""The gated delta rule: a mixer with a matrix of state per head instead of a cache of keys."""
from __future__ import annotations

import torch

from .base import Mixer, Runtime, StateSpec, WeightSpec, to_f32_vector
from .linear import Linear


class GatedDeltaMixer(Mixer):
    """Per head, with S [dim, vdim] carried from token to token in 32-bit,

        S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

    where q and k (kv_heads x dim; head h reads group h // (heads / kv_heads)) and v (heads x
    vdim) are projections of the input that pass a short causal convolution per channel (`taps`
    taps, the last one the current token's, zeros before the start) and SiLU; q and k are then
    unit vectors (x / sqrt(sum x^2 + 1e-6)), q also times dim^-1/2; beta = sigmoid(W_b x) and
    g = exp(-exp(A_log) softplus(W_a x + dt_bias)) are one number per head.  Each head's o is
    divided by its root mean square (eps `norm_eps`), multiplied by a weight shared by the heads
    and by SiLU(W_g x), and goes through the output projection.

    Per request the part keeps, in one state slot of 32-bit floats, S^T of every head and the
    last taps-1 inputs of the convolutions; a step runs each request's tokens in order from what
    the steps before left there.  Everything from the convolution's output to o's norm is 32-bit.
    `names`: the tensors of (q, k, v, b, a, gate, o, A_log, dt_bias, norm); a convolution's taps
    are `<projection><conv_suffix>`.  `output=False` leaves the output projection to the block."""

    supports_cuda_graph = True

    def __init__(self, width: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, norm_eps: float, name: str,
                 names=("q", "k", "v", "b", "a", "g", "o", "A_log", "dt_bias", "norm"), conv_suffix: str = ".conv",
                 output: bool = True, weight_suffix: str = ".weight"):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are no multiple of {kv_heads} key heads")
        if not 1 <= taps <= 16:
            raise ValueError(f"a short convolution has 1 to 16 taps, not {taps}")
        if dim > 256:
            raise ValueError(f"the recurrence keeps up to 256 rows of state per column, not {dim}")
        self.H, self.G, self.D, self.Dv, self.taps = int(heads), int(kv_heads), int(dim), int(vdim), int(taps)
        self.eps = float(norm_eps)
        q, k, v, b, a, g, o, alog, dtb, norm = (f"{name}.{n}" for n in names)
        self.channels = 2 * self.G * self.D + self.H * self.Dv
        self.qkvg = Linear(width, [(q, self.G * self.D), (k, self.G * self.D), (v, self.H * self.Dv),
                                   (g, self.H * self.Dv)], weight_suffix=weight_suffix)
        self.ba = Linear(width, [(b, self.H), (a, self.H)], weight_suffix=weight_suffix)
        self.conv_names = [(q + conv_suffix, self.G * self.D), (k + conv_suffix, self.G * self.D),
                           (v + conv_suffix, self.H * self.Dv)]
        self.vec_names = (alog, dtb, norm)
        self.inner_features = self.H * self.Dv
        self.out_piece = (o + weight_suffix, self.inner_features, None)
        self.o = Linear(self.inner_features, [(o, width)], weight_suffix=weight_suffix) if output else None
        self.s_floats = self.H * self.Dv * self.D

    def children(self):
        return tuple(p for p in (self.qkvg, self.ba, self.o) if p is not None)

    def own_weight_specs(self):
        alog, dtb, norm = self.vec_names
        return [WeightSpec(n, (c, self.taps), "conv") for n, c in self.conv_names] + \
            [WeightSpec(alog, (self.H,), "log_rate"), WeightSpec(dtb, (self.H,), "rate_bias"),
             WeightSpec(norm, (self.Dv,), "norm")]

    def bind_own(self, tensors, rt: Runtime):
        self.conv_w = torch.cat([to_f32_vector(tensors[n], rt) for n, _ in self.conv_names], dim=0).contiguous()
        self.a_log, self.dt_bias, self.norm_w = (to_f32_vector(tensors[n], rt) for n in self.vec_names)

    def state_spec(self):
        # a multiple of four floats, so that every slot starts on 16 bytes
        n = self.s_floats + (self.taps - 1) * self.channels
        return StateSpec((-(-n // 4) * 4,), torch.float32)

    def forward_inner(self, x, ctx, cache, out=None):
        """The normalised, gated read-outs of all heads side by side, [T, heads * vdim]."""
        k = self.rt.k
        proj = self.qkvg.forward(x)
        ab = self.ba.forward(x, out_dtype=torch.float32)
        qkv, gb = k.delta_prepare(proj, ab, self.conv_w, self.a_log, self.dt_bias, ctx, cache.state, self.s_floats,
                                  self.H, self.G, self.D, self.Dv, self.taps)
        o = k.delta_rule(qkv, gb, ctx, cache.state, self.H, self.G, self.D, self.Dv)
        return k.gated_rmsnorm(o, proj[:, self.channels:], self.norm_w, self.eps, self.H, self.Dv, self.rt.dtype, out=out)

    def forward(self, x, ctx, cache):
        return self.o.forward(self.forward_inner(x, ctx, cache))
