"""Medirax, assembled from parts.

Every layer is a `ParallelBlock` (one norm whose weight is stored around zero; mixer and
feed-forward read its output, and their output projections are one joined product) around a
`GatedDeltaMixer` or a `GQAAttention` on its route with 32-bit scores (partial rotary
positions, q and k normalised after the rotation, capped scores, a sliding window), with a
`DenseMLP` of squared relu or none.  The schedule names a looped run of layers once per pass,
so that every pass has a cache or a state slot of its own.  Tensor names: `embed`,
`l<i>.norm1`, `l<i>.mix.<name>` (biases `<name>.b`, convolution taps `<name>.conv`),
`l<i>.mlp.up|down`, `final.norm`, `head`; matrices are stored [out, in] under their bare names.
"""
from __future__ import annotations

from .. import registry
from ..config.medirax import MediraxConfig
from ..parts import (DenseMLP, Embedding, GatedDeltaMixer, GQAAttention, LMHead, Model, NoPositionEncoding,
                     ParallelBlock, RMSNorm, RotaryEmbedding, Run)


def build_medirax(cfg: MediraxConfig) -> Model:
    d = cfg.width
    embed = Embedding(cfg.vocab, d, "embed", suffix="")
    layers = []
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}", spec.mixer
        if spec.type == "delta":
            mixer = GatedDeltaMixer(d, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, cfg.norm_eps, f"{p}.mix",
                                    output=False, weight_suffix="")
        else:
            pos = RotaryEmbedding(m.dim, m.rot_base, rotary_dim=m.rot_dims) if m.rot_dims else NoPositionEncoding()
            mixer = GQAAttention(d, m.heads, m.kv_heads, m.dim, pos, f"{p}.mix", bias=True, scale=m.scale,
                                 window=m.window, proj_names=("q", "k", "v", "o"), v_head_dim=m.vdim,
                                 softcap=m.softcap, qk_norm_eps=cfg.norm_eps, output=False, weight_suffix="",
                                 bias_suffix=".b")
        ffn = None
        if spec.mlp is not None:
            ffn = DenseMLP(d, spec.mlp.ff, f"{p}.mlp", activation="relu2", output=False, weight_suffix="")
        layers.append(ParallelBlock(mixer, ffn, RMSNorm(d, cfg.norm_eps, f"{p}.norm1", offset=1.0, suffix=""), d))
    head = LMHead(cfg.vocab, d, "head", suffix="", scale=cfg.logit_scale)
    return Model(embed, layers, RMSNorm(d, cfg.norm_eps, "final.norm", offset=1.0, suffix=""), head,
                 schedule=[Run(i) for i in cfg.layer_order()], vocab_size=cfg.vocab)


registry.register(["medirax", "Medirax"], MediraxConfig.from_dict, build_medirax, replace=True)
