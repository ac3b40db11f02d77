"""Small Bemuzen configurations for the tests.  They differ from one another in every size, in the
order of the layers and in every constant, and hold the cases a single model may hide: a layer
without a feed-forward, values wider or narrower than keys, one and several key/value heads, one and
several groups, one and several parts of the gated norm, two to four taps, head sizes that are no
multiple of 32, more value columns than one block of the recurrence holds."""


def _parallel(left: dict, right: dict, ff: int | None) -> dict:
    return {"type": "parallel", "mixer": {"left": left, "right": right},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _mamba(mixer: dict, ff: int | None) -> dict:
    return {"type": "mamba2", "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


BZ_A = {
    "architecture": "Bemuzen", "vocab": 97, "width": 64, "logit_scale": 0.5, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 53, "mul_prev": 5, "mul_cur": 3}},
    "layers": [
        _parallel({"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "q_temp": {"coef": 0.7, "every": 8}},
                  {"heads": 2, "dim": 8, "vdim": 16, "decay": [0.9, 0.5]}, 80),
        _mamba({"heads": 2, "vdim": 16, "state": 8, "groups": 1, "conv": 4, "norm_groups": 1}, 48),
        _parallel({"heads": 2, "kv_heads": 2, "dim": 24, "vdim": 8, "scale": 0.2, "q_temp": {"coef": 0.25, "every": 5}},
                  {"heads": 4, "dim": 12, "vdim": 8, "decay": [0.99, 0.7, 0.95, 0.3]}, None),
    ],
}

BZ_B = {
    "architecture": "Bemuzen", "vocab": 211, "width": 96, "logit_scale": 1.5, "norm": {"eps": 1e-6},
    "embedding": {"bigram": {"buckets": 127, "mul_prev": 1, "mul_cur": 11}},
    "layers": [
        _mamba({"heads": 6, "vdim": 8, "state": 12, "groups": 3, "conv": 2, "norm_groups": 3}, None),
        _parallel({"heads": 6, "kv_heads": 6, "dim": 20, "vdim": 12, "scale": 0.25, "q_temp": {"coef": 1.0, "every": 16}},
                  {"heads": 3, "dim": 36, "vdim": 40, "decay": [0.8, 0.999, 0.6]}, 112),
        _mamba({"heads": 4, "vdim": 12, "state": 20, "groups": 4, "conv": 3, "norm_groups": 2}, 64),
        _mamba({"heads": 3, "vdim": 16, "state": 16, "groups": 1, "conv": 4, "norm_groups": 4}, 64),
    ],
}

BZ_C = {
    "architecture": "Bemuzen", "vocab": 300, "width": 128, "logit_scale": 0.125, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 401, "mul_prev": 13, "mul_cur": 1}},
    "layers": [
        _parallel({"heads": 3, "kv_heads": 1, "dim": 64, "vdim": 128, "scale": 0.125, "q_temp": {"coef": 0.4, "every": 32}},
                  {"heads": 2, "dim": 40, "vdim": 72, "decay": [0.97, 0.9]}, 160),
        _mamba({"heads": 2, "vdim": 80, "state": 72, "groups": 2, "conv": 4, "norm_groups": 2}, 96),
    ],
}

# Keys and values of one size of 64: in bfloat16 the softmax branch runs on the tensor-core kernels.
BZ_D = {
    "architecture": "Bemuzen", "vocab": 157, "width": 128, "logit_scale": 0.3, "norm": {"eps": 1e-5},
    "embedding": {"bigram": {"buckets": 89, "mul_prev": 2, "mul_cur": 9}},
    "layers": [
        _parallel({"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.125, "q_temp": {"coef": 0.3, "every": 48}},
                  {"heads": 2, "dim": 32, "vdim": 64, "decay": [0.98, 0.8]}, 96),
        _parallel({"heads": 2, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.2, "q_temp": {"coef": 0.5, "every": 100}},
                  {"heads": 1, "dim": 16, "vdim": 48, "decay": [0.93]}, None),
    ],
}

# Odd sizes: a width, head sizes and feed-forward widths that are no multiple of four (the kernels' forms
# of one element a thread, the library's products over odd rows), a convolution of one tap (no inputs to
# keep), as many groups as heads, a temperature that steps at every position, large hash constants.
BZ_E = {
    "architecture": "Bemuzen", "vocab": 61, "width": 50, "logit_scale": 2.0, "norm": {"eps": 1e-4},
    "embedding": {"bigram": {"buckets": 17, "mul_prev": 1000003, "mul_cur": 998244353}},
    "layers": [
        _mamba({"heads": 3, "vdim": 7, "state": 5, "groups": 3, "conv": 1, "norm_groups": 1}, 77),
        _parallel({"heads": 3, "kv_heads": 3, "dim": 10, "vdim": 6, "scale": 0.5, "q_temp": {"coef": 0.2, "every": 1}},
                  {"heads": 1, "dim": 6, "vdim": 9, "decay": [1.0]}, 33),
        _mamba({"heads": 2, "vdim": 9, "state": 33, "groups": 1, "conv": 5, "norm_groups": 3}, None),
    ],
}

CONFIGS = {"A": (BZ_A, 16), "B": (BZ_B, 8), "C": (BZ_C, 32), "D": (BZ_D, 16), "E": (BZ_E, 4)}
LENGTHS = {
    "A": {"a": 70, "b": 45, "c": 100, "d": 37, "e": 64, "f": 1, "g": 150},
    "B": {"a": 70, "b": 33, "c": 90, "d": 2, "e": 64, "g": 130},
    "C": {"a": 70, "b": 45, "c": 3, "d": 37, "g": 110},
    "D": {"a": 70, "b": 45, "c": 130, "d": 1, "g": 200},
    "E": {"a": 41, "b": 2, "c": 23, "g": 70},
}
