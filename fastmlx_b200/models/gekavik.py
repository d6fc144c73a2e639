"""Gekavik, assembled from parts.

Every layer is a `SandwichBlock` (dynamic-tanh norms in front of and behind each sublayer, a multiplier on
what enters the stream) around a `GQAAttention` on its route with 32-bit scores (biases added in 32-bit, q and
k normalised with a weight before an interleaved rotation, a window that keeps the first tokens, an
element-wise output gate) or a `LatentAttention`, with `RoutedExperts` or no feed-forward.  The schedule names
a looped run of layers once per pass, so that every pass has a cache of its own, and puts a `LoopPass` in
front of each pass.  Tensor names: `embed`, `loop.in`, `loop.step`, `l<i>.norm1|norm1b|norm2|norm2b` (with
`.b` and `.alpha`), `l<i>.mix.<name>` (biases `<name>.b`, norm weights `<name>.norm`), `l<i>.mlp.router`,
`l<i>.mlp.e<j>.gate|up|down`, `l<i>.mlp.shared.gate|up|down`, `final.norm`, `head`; matrices are stored
[out, in] under their bare names.
"""
from __future__ import annotations

from .. import registry
from ..config.gekavik import GekavikConfig
from ..parts import (DynamicTanh, Embedding, GQAAttention, LatentAttention, LMHead, LoopInput, LoopPass, Model,
                     NoPositionEncoding, RotaryEmbedding, RoutedExperts, Run, SandwichBlock)


def build_gekavik(cfg: GekavikConfig) -> Model:
    d = cfg.width
    embed = Embedding(cfg.vocab, d, "embed", suffix="")
    layers = []
    drop = []
    for i, spec in enumerate(cfg.layers):
        p, m = f"l{i}", spec.mixer
        if spec.type == "attention":
            pos = RotaryEmbedding(m.dim, m.rot_base, traditional=True, rotary_dim=m.rot_dims) if m.rot_dims \
                else NoPositionEncoding()
            mixer = GQAAttention(d, m.heads, m.kv_heads, m.dim, pos, f"{p}.mix", bias=True, scale=m.scale,
                                 window=m.window, proj_names=("q", "k", "v", "o"), v_head_dim=m.vdim,
                                 qk_norm_eps=cfg.norm_eps, qk_norm_weights=("q.norm", "k.norm"), qk_norm_first=True,
                                 keep_first=m.keep_first, gate="g", late_bias=True, out_bias=False, weight_suffix="",
                                 bias_suffix=".b")
        else:
            mixer = LatentAttention(d, m.heads, m.dim, m.vdim, m.q_rank, m.kv_rank, cfg.norm_eps, f"{p}.mix",
                                    scale=m.scale, window=m.window)
        ffn = norm2 = norm2b = None
        if spec.mlp is not None:
            e = spec.mlp
            ffn = RoutedExperts(d, e.experts, e.top, e.ff, e.limit, f"{p}.mlp", groups=e.groups, keep=e.keep,
                                shared_ff=e.shared_ff, shared_limit=e.shared_limit)
            norm2, norm2b = DynamicTanh(d, f"{p}.norm2"), DynamicTanh(d, f"{p}.norm2b")
        else:
            drop.append(f"{p}.norm2")                 # a layer without a feed-forward uses no second pair of norms
        layers.append(SandwichBlock(mixer, ffn, DynamicTanh(d, f"{p}.norm1"), DynamicTanh(d, f"{p}.norm1b"), norm2, norm2b,
                                    cfg.residual_mult))
    schedule = []
    if cfg.loop is not None:
        entry = LoopInput(d, cfg.loop.times, "loop.in", "loop.step")
        first_pass = len(layers)
        layers += [LoopPass(entry, t) for t in range(cfg.loop.times)]
    for i, t in cfg.layer_passes():
        if t is not None:
            schedule.append(Run(first_pass + t))
        schedule.append(Run(i))
    head = LMHead(cfg.vocab, d, "head", suffix="")
    return Model(embed, layers, DynamicTanh(d, "final.norm"), head, schedule=schedule, vocab_size=cfg.vocab, drop=drop)


registry.register(["gekavik", "Gekavik"], GekavikConfig.from_dict, build_gekavik, replace=True)
