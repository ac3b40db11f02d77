"""Small Lobuzen configurations for the tests.  They differ from one another in every size, in the order
of the layers and in every constant, and hold the cases a single model may hide: layers without a
feed-forward, a model without a token side, values wider and narrower than keys, one and several key/value
heads, layers without a window and with windows of one and two positions, a layer that reads another
layer's latent rows over a longer and over a shorter window than the owner's, routers with and without
groups, with groups of one expert, and with every expert chosen, sizes that are no multiple of four."""


def _attention(heads, kv_heads, dim, vdim, scale, window, mlp):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer, "mlp": mlp}


def _latent(heads, dim, vdim, rank, scale, window, mlp, kv_from=None):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if kv_from is not None:
        mixer["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": mixer, "mlp": mlp}


def _dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def _moe(ff, experts, top, count=None, keep=None):
    router = {"experts": experts, "top": top}
    if count is not None:
        router["groups"] = {"count": count, "keep": keep}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


LZ_A = {
    "architecture": "Lobuzen", "vocab": 97, "width": 64, "norm": {"eps": 1e-5}, "token_side": {"dim": 8},
    "layers": [
        _latent(4, 16, 24, 32, 0.3, 20, _moe(40, 8, 2, 4, 2)),
        _attention(4, 2, 16, 24, 0.25, 12, _dense(80, 1.5)),
        _latent(2, 8, 16, 32, 0.4, 33, _moe(24, 6, 3, 3, 2), kv_from=0),      # a longer window than the owner's
        _attention(2, 2, 24, 8, 0.2, None, None),
        _latent(4, 12, 12, 32, 0.3, 7, _dense(48, 0.75), kv_from=0),           # and a shorter one
    ],
}

# Keys and values of one size of 64, latent rows of 64 and 128: in bfloat16 the attention runs on the
# tensor-core kernels.  No token side; a router without groups.
LZ_B = {
    "architecture": "Lobuzen", "vocab": 211, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        _attention(4, 2, 64, 64, 0.125, 50, _moe(32, 4, 2)),
        _latent(8, 16, 32, 128, 0.25, 70, _dense(96, 3.0)),
        _latent(4, 32, 16, 64, 0.2, None, None),
        _attention(2, 1, 64, 64, 0.1, 17, _dense(64, 1.0)),
        _latent(16, 8, 8, 128, 0.35, 16, _moe(16, 8, 4, 2, 1), kv_from=1),
    ],
}

# Odd sizes: a width, head sizes, a latent size and feed-forward widths that are no multiple of four,
# windows of one and of two positions, every expert chosen, groups of one expert.
LZ_C = {
    "architecture": "Lobuzen", "vocab": 61, "width": 50, "norm": {"eps": 1e-4}, "token_side": {"dim": 3},
    "layers": [
        _attention(3, 3, 10, 6, 0.5, 2, _moe(33, 5, 5)),
        _latent(3, 6, 10, 22, 0.45, 1, _moe(9, 4, 2, 4, 3)),
        _attention(6, 2, 6, 14, 0.3, 9, _dense(77, 0.4)),
        _latent(1, 20, 18, 22, 0.3, 25, None, kv_from=1),
    ],
}

# A model of one layer, of a wide latent row and many heads on one key/value head.
LZ_D = {
    "architecture": "Lobuzen", "vocab": 40, "width": 96, "norm": {"eps": 1e-5}, "token_side": {"dim": 16},
    "layers": [
        _latent(24, 8, 8, 256, 0.3, 90, _moe(24, 12, 3, 3, 1)),
    ],
}

# Wider: products over a width that the kernels for few rows take whole, sixteen experts in four groups,
# 32 heads on one cached head (two groups of 16 on the tensor-core kernels), latent rows of a size that only
# the float32-arithmetic kernel takes, a reader of them.
LZ_E = {
    "architecture": "Lobuzen", "vocab": 500, "width": 384, "norm": {"eps": 1e-5}, "token_side": {"dim": 16},
    "layers": [
        _attention(6, 3, 64, 64, 0.125, 50, _dense(448, 2.5)),
        _latent(6, 32, 64, 96, 0.2, 100, _moe(160, 16, 4, 4, 2)),
        _attention(12, 1, 32, 48, 0.18, 30, _moe(96, 16, 6, 2, 1)),
        _latent(3, 64, 32, 96, 0.12, 60, _moe(160, 16, 4, 4, 2), kv_from=1),
        _latent(32, 16, 16, 64, 0.25, 80, _dense(320, 1.0)),
    ],
}

# Keys and values of 256 on the tensor-core kernels, latent rows of 48 (the float32-arithmetic kernel) under
# 16 and 20 heads, 32 experts of which 8 are chosen from 4 of 8 groups, one expert chosen from one group of
# two, a width that is no multiple of 128, readers with longer windows than their owners.
LZ_F = {
    "architecture": "Lobuzen", "vocab": 1000, "width": 320, "norm": {"eps": 1e-6}, "token_side": {"dim": 40},
    "layers": [
        _latent(16, 64, 64, 48, 0.125, 90, _moe(200, 32, 8, 8, 4)),
        _attention(16, 4, 256, 256, 0.0625, 64, _moe(72, 32, 8, 8, 4)),
        _attention(8, 8, 128, 128, 0.09, 33, _dense(200, 4.0)),
        _latent(20, 32, 48, 48, 0.18, 128, _dense(520, 0.5), kv_from=0),
        _latent(8, 32, 48, 256, 0.18, 40, _moe(64, 6, 1, 3, 1)),
        _latent(8, 24, 40, 256, 0.2, 100, None, kv_from=4),
    ],
}

CONFIGS = {"A": (LZ_A, 16), "B": (LZ_B, 16), "C": (LZ_C, 4), "D": (LZ_D, 32), "E": (LZ_E, 16), "F": (LZ_F, 16)}
LENGTHS = {
    "A": {"a": 70, "b": 45, "c": 100, "d": 37, "e": 64, "f": 1, "g": 150},
    "B": {"a": 70, "b": 33, "c": 130, "d": 2, "e": 64, "g": 200},
    "C": {"a": 41, "b": 2, "c": 23, "g": 70},
    "D": {"a": 70, "b": 1, "c": 140, "g": 230},
    "E": {"a": 300, "b": 64, "c": 129, "g": 260},
    "F": {"a": 150, "b": 65, "c": 17, "g": 120},
}
