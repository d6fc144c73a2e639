"""Small Gekavik configurations for the tests, and weights that make faults show.

The configurations differ from one another in every size and option and use values that a usual model makes
equal or 1: as many kv heads as heads and one kv head, values wider and narrower than keys, a rotation over a
part of the head, the whole head or none, kept first tokens from none to more than a page, windows shorter than
a page and none at all, latents of different ranks for queries and keys, one expert per token and every group
kept, experts' limits that differ from the shared expert's, no shared expert, no feed-forward, no loop, a loop
from the first layer, a loop of one pass.
"""
import os

import torch


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def latent(heads, dim, vdim, q_rank, kv_rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def moe(experts, top, ff, limit, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    m = {"kind": "moe", "router": r, "expert": {"ff": ff, "limit": limit}}
    if shared is not None:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def layer(kind, mixer, mlp=None):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


G1 = {
    "architecture": "Gekavik", "vocab": 211, "width": 96, "residual_mult": 0.45, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attention(4, 2, 24, 40, 0.3, window=37, keep_first=3, rot=(8, 10000.0)),
              moe(8, 2, 48, 0.8, groups=(4, 2), shared=(32, 2.0))),
        layer("latent_attention", latent(3, 16, 24, 40, 48, 0.2, window=21), moe(6, 3, 16, 1.5, groups=(2, 1))),
        layer("attention", attention(2, 2, 32, 32, 0.17, window=5, keep_first=1, rot=(32, 500.0))),
        layer("latent_attention", latent(2, 32, 16, 24, 64, 0.15), moe(4, 1, 64, 3.0, shared=(48, 0.5))),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
G2 = {
    "architecture": "Gekavik", "vocab": 97, "width": 64, "residual_mult": 1.0, "norm": {"eps": 1e-6},
    "layers": [
        layer("latent_attention", latent(4, 16, 16, 32, 32, 0.25, window=70), moe(4, 2, 32, 1.0, groups=(2, 2))),
        layer("attention", attention(2, 1, 16, 48, 0.25), moe(3, 3, 24, 0.6)),
        layer("attention", attention(4, 1, 16, 16, 0.2, window=40, keep_first=19, rot=(4, 100.0)), moe(9, 2, 8, 2.0, groups=(3, 1))),
    ],
}
G3 = {
    "architecture": "Gekavik", "vocab": 130, "width": 128, "residual_mult": 0.2, "norm": {"eps": 1e-4},
    "layers": [
        layer("attention", attention(8, 2, 64, 16, 0.125, window=1000, keep_first=2, rot=(16, 1000000.0)),
              moe(16, 4, 32, 1.2, groups=(8, 3), shared=(64, 1.2))),
        layer("latent_attention", latent(8, 32, 32, 96, 128, 0.18, window=33)),
        layer("attention", attention(1, 1, 128, 64, 0.09, window=64, keep_first=0, rot=(128, 50000.0)), moe(2, 1, 128, 0.9)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}
# sizes that are multiples of nothing: rows of 25 and 50 bytes, 20-wide heads with 12-wide values, a latent of 36
G4 = {
    "architecture": "Gekavik", "vocab": 101, "width": 50, "residual_mult": 0.7, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attention(3, 3, 20, 12, 0.22, window=33, keep_first=5, rot=(6, 777.0)), moe(5, 2, 10, 1.0)),
        layer("latent_attention", latent(5, 12, 20, 30, 36, 0.3, window=18), moe(6, 2, 14, 0.75, groups=(3, 2), shared=(22, 1.0))),
    ],
    "loop": {"start": 1, "stop": 2, "times": 1},
}
CONFIGS = {"G1": G1, "G2": G2, "G3": G3, "G4": G4}
# experts as wide as a block of the grouped products (128 hidden columns), for the tests that force those products on
G5 = {
    "architecture": "Gekavik", "vocab": 150, "width": 128, "residual_mult": 0.5, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attention(4, 2, 32, 32, 0.2, window=50, keep_first=2, rot=(16, 5000.0)), moe(6, 2, 128, 1.1, shared=(128, 0.9))),
        layer("latent_attention", latent(4, 32, 32, 64, 64, 0.2, window=45), moe(8, 3, 256, 2.0, groups=(4, 2))),
    ],
}


def lively_tensors(config, seed, dtype=torch.bfloat16):
    """Random weights of a size at which every mechanism matters: embeddings and activations of the order of one,
    scores of a few units (so that a key that should not be seen, or is not seen though it should be, moves the
    output), router logits spread far enough apart that rounding does not change a token's experts."""
    from fastmlx_b200 import registry
    _, model = registry.build_model(config)
    g = torch.Generator().manual_seed(seed)
    out = {}
    for spec in model.weight_specs():
        t = torch.randn(tuple(spec.shape), generator=g, dtype=torch.float32)
        if spec.kind == "matrix":
            t = t / spec.shape[-1] ** 0.5
            if spec.name.endswith(".router"):
                t = t * 12.0
            elif spec.name == "loop.in":
                t = t * 1.4
        elif spec.kind == "bias":
            t = t * 0.1
        elif spec.kind == "norm":
            t = 1.0 + 0.2 * t
        elif spec.kind == "alpha":
            t = torch.sigmoid(t) + 0.5
        out[spec.name] = t.to(dtype)
    return out


def make_model_dir(root, config, seed):
    """A folder with config.json and model.safetensors of lively weights."""
    import json
    from fastmlx_b200.weights import safetensors_io as st
    d = os.path.join(str(root), f"gekavik_{config['vocab']}_{seed}")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(config, f)
    st.write_file(os.path.join(d, "model.safetensors"), lively_tensors(config, seed), {"format": "pt"})
    return d


def random_config(seed):
    """A configuration drawn from a seed: every size, count, constant and the order of layers vary."""
    import random
    rnd = random.Random(seed)
    width = rnd.choice([40, 48, 72, 96, 136, 200])
    n_layers = rnd.randint(2, 4)
    layers = []
    for _ in range(n_layers):
        if rnd.random() < 0.5:
            kv = rnd.choice([1, 2, 3])
            heads = kv * rnd.choice([1, 2, 4])
            dim = rnd.choice([8, 16, 24, 40, 64])
            vdim = rnd.choice([dim, dim, 16, 48])
            window = rnd.choice([None, 7, 30, 61, 100])
            keep = rnd.choice([None, 0, 1, 4, 17, 33]) if window else None
            rot = rnd.choice([None, (dim, 10000.0), (max(2, dim // 2 // 2 * 2), 300.0)])
            mixer = ("attention", attention(heads, kv, dim, vdim, rnd.choice([0.1, 0.2, dim ** -0.5]), window, keep, rot))
        else:
            dim = rnd.choice([8, 16, 32])
            mixer = ("latent_attention", latent(rnd.choice([1, 2, 3, 5]), dim, rnd.choice([dim, dim, 24]), rnd.choice([16, 40, 64]),
                                                rnd.choice([16, 36, 64, 128]), rnd.choice([0.15, 0.25]), rnd.choice([None, 9, 40, 90])))
        mlp = None
        if rnd.random() < 0.8:
            groups = rnd.choice([1, 2, 3, 4])
            per = rnd.choice([1, 2, 3])
            keep_g = rnd.randint(1, groups)
            top = rnd.randint(1, per * keep_g)
            mlp = moe(groups * per, top, rnd.choice([8, 20, 32, 64]), rnd.choice([0.5, 1.0, 4.0]),
                      (groups, keep_g) if rnd.random() < 0.7 else None, (rnd.choice([8, 24, 64]), rnd.choice([0.7, 2.0])) if rnd.random() < 0.6 else None)
            if mlp["router"].get("groups") is None:
                mlp["router"]["top"] = rnd.randint(1, groups * per)
        layers.append(layer(mixer[0], mixer[1], mlp))
    cfg = {"architecture": "Gekavik", "vocab": rnd.choice([61, 100, 257]), "width": width, "residual_mult": rnd.choice([0.25, 0.6, 1.0]),
           "norm": {"eps": rnd.choice([1e-6, 1e-5])}, "layers": layers}
    if rnd.random() < 0.7:
        a = rnd.randint(0, n_layers - 1)
        cfg["loop"] = {"start": a, "stop": rnd.randint(a + 1, n_layers), "times": rnd.randint(1, 3)}
    return cfg
