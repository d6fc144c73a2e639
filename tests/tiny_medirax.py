"""Small Medirax configurations for the tests: they differ from one another in every size and
option, and use values that a usual model makes equal or 1 (as many kv heads as heads, one kv
head, one head, values wider or narrower than keys, a rotation over the whole head or none, a
window shorter than a page, no window, no cap, no feed-forward, no loop, a loop of one pass)."""


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, window=None, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if window is not None:
        m["mask"] = {"size": window}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return m


def delta(heads, kv_heads, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv}


def layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


M1 = {
    "architecture": "Medirax", "vocab": 211, "width": 96, "logit_scale": 0.37, "norm": {"eps": 1e-6},
    "layers": [
        layer("attention", attention(4, 2, 24, 40, 0.3, softcap=7.5, window=37, rot=(8, 10000.0)), ff=160),
        layer("delta", delta(4, 2, 24, 40, 3), ff=160),
        layer("delta", delta(2, 2, 16, 16, 2)),
        layer("attention", attention(3, 1, 32, 32, 0.17, softcap=30.0, window=5, rot=(32, 500.0)), ff=64),
    ],
    "loop": {"start": 1, "stop": 3, "times": 2},
}
M2 = {
    "architecture": "Medirax", "vocab": 97, "width": 64, "logit_scale": 1.0, "norm": {"eps": 1e-5},
    "layers": [
        layer("delta", delta(1, 1, 64, 8, 4)),
        layer("attention", attention(2, 2, 16, 48, 0.25), ff=128),
        layer("attention", attention(4, 4, 16, 16, 0.2, softcap=50.0, window=70, rot=(4, 100.0))),
    ],
}
M3 = {
    "architecture": "Medirax", "vocab": 130, "width": 128, "logit_scale": 2.5, "norm": {"eps": 1e-4},
    "layers": [
        layer("delta", delta(6, 3, 128, 16, 1), ff=96),
        layer("attention", attention(8, 2, 64, 16, 0.125, softcap=12.0, window=1000, rot=(16, 1000000.0)), ff=96),
        layer("delta", delta(2, 1, 40, 72, 5), ff=200),
    ],
    "loop": {"start": 0, "stop": 3, "times": 1},
}
# sizes that are multiples of nothing: rows of 25 and 50 bytes, 20-wide heads with 12-wide values
M4 = {
    "architecture": "Medirax", "vocab": 101, "width": 50, "logit_scale": 0.8, "norm": {"eps": 1e-5},
    "layers": [
        layer("attention", attention(3, 3, 20, 12, 0.22, softcap=9.0, window=33, rot=(6, 777.0)), ff=45),
        layer("delta", delta(3, 1, 20, 12, 3), ff=45),
        layer("attention", attention(2, 1, 48, 48, 0.15, softcap=18.0, window=21, rot=(16, 10000.0))),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
CONFIGS = {"M1": M1, "M2": M2, "M3": M3, "M4": M4}
