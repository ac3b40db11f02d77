"""A plain, slow statement of the Bemuzen decoder, one function per mechanism, token by token.

Everything is written from the design's equations with torch tensors on the CPU, in whatever
floating type the weights are handed over in (tests use float64 or float32); nothing here is
shared with the engine's parts or kernels.  ``PlainBemuzen`` keeps a request's state (previous
token, keys and values, recurrent states, the convolution's last inputs) in a dictionary, so
a prompt may be fed in any portions and must give the same rows.

Notation: ``h`` is a mixer's input row, ``W x`` a matrix stored ``[out, in]`` applied to a row.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by the root of (mean of squares + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return rms(x, eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.log1p(torch.exp(-z.abs())) + torch.clamp(z, min=0)


def bigram_row(previous: int | None, token: int, mul_prev: int, mul_cur: int, buckets: int) -> int:
    if previous is None:
        return buckets
    return (previous * mul_prev + token * mul_cur) % buckets


def query_temperature(position: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((position + 1) // every + 1)


def bias_slope(head: int, heads: int) -> float:
    return 2.0 ** (-8.0 * (head + 1) / heads)


def softmax_attention_row(q, keys, values, position: int, scale: float, slopes, group: int):
    """q ``[H, d]`` at ``position``; keys ``[n, G, d]`` and values ``[n, G, dv]`` of positions 0..n-1
    (n = position + 1).  Score of key j for head h: q.k * scale - slope_h * (position - j)."""
    heads = q.shape[0]
    out = []
    distance = torch.arange(position, -1, -1, dtype=q.dtype)
    for h in range(heads):
        g = h // group
        scores = (keys[:, g] @ q[h]) * scale - slopes[h] * distance
        weights = torch.softmax(scores, dim=0)
        out.append(weights @ values[:, g])
    return torch.cat(out)


def softmax_branch_step(w, cfg, eps, h, position, cache):
    """The softmax side of the paired mixer for one row; ``cache`` holds 'k' and 'v' lists."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = (w["q"] @ h).view(H, d)
    k = (w["k"] @ h).view(G, d)
    v = (w["v"] @ h).view(G, dv)
    q = norm_plain(q, w["q.norm"], eps) * query_temperature(position, cfg["q_temp"]["coef"], cfg["q_temp"]["every"])
    k = norm_plain(k, w["k.norm"], eps)
    cache.setdefault("k", []).append(k)
    cache.setdefault("v", []).append(v)
    slopes = [bias_slope(i, H) for i in range(H)]
    attended = softmax_attention_row(q, torch.stack(cache["k"]), torch.stack(cache["v"]), position,
                                     cfg["scale"], slopes, H // G)
    return w["o"] @ attended


def decayed_linear_attention_step(q, k, v, decay, state):
    """Per head: S <- decay S + k v^T (S is ``[d, dv]``), o = S^T q.  Returns o ``[H, dv]``."""
    out = []
    for h in range(q.shape[0]):
        state[h] = decay[h] * state[h] + torch.outer(k[h], v[h])
        out.append(state[h].T @ q[h])
    return torch.stack(out)


def linear_branch_step(w, cfg, eps, h, cache):
    H, d, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = silu(w["q"] @ h).view(H, d)
    k = silu(w["k"] @ h).view(H, d)
    v = silu(w["v"] @ h).view(H, dv)
    if "S" not in cache:
        cache["S"] = [torch.zeros(d, dv, dtype=h.dtype) for _ in range(H)]
    o = decayed_linear_attention_step(q, k, v, cfg["decay"], cache["S"]).reshape(-1)
    o = norm_plain(o, w["norm"], eps) * torch.sigmoid(w["g"] @ h)
    return w["o"] @ o


def paired_mixer_step(w, cfg, eps, h, position, cache):
    left = {k[len("left."):]: v for k, v in w.items() if k.startswith("left.") and k != "left.out"}
    right = {k[len("right."):]: v for k, v in w.items() if k.startswith("right.") and k != "right.out"}
    a = softmax_branch_step(left, cfg["left"], eps, h, position, cache.setdefault("left", {}))
    b = linear_branch_step(right, cfg["right"], eps, h, cache.setdefault("right", {}))
    return 0.5 * (norm_plain(a, w["left.out"], eps) + norm_plain(b, w["right.out"], eps))


def causal_conv_step(x, weight, bias, history):
    """``weight`` ``[C, taps]``, last column for the current input; ``history`` the last taps - 1
    inputs (oldest first, zeros before the start), updated in place."""
    taps = weight.shape[1]
    window = torch.stack(history + [x], dim=1) if taps > 1 else x[:, None]      # [C, taps]
    out = (window * weight).sum(1) + bias
    if taps > 1:
        history.pop(0)
        history.append(x)
    return out


def selective_scan_step(x, B, C, dt, a_log, D, group, state):
    """x ``[H, dv]``, B and C ``[G, N]``, dt ``[H]`` (already through softplus).  Per head:
    S <- exp(-exp(a_log) dt) S + dt B x^T (S is ``[N, dv]``), y = S^T C + D x."""
    out = []
    for h in range(x.shape[0]):
        g = h // group
        state[h] = torch.exp(-torch.exp(a_log[h]) * dt[h]) * state[h] + dt[h] * torch.outer(B[g], x[h])
        out.append(state[h].T @ C[g] + D[h] * x[h])
    return torch.stack(out)


def mamba2_step(w, cfg, eps, h, cache):
    H, dv, N, G = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = H * dv
    taps = cfg["conv"]
    proj = w["in"] @ h
    z, xbc, dt = proj[:inner], proj[inner:2 * inner + 2 * G * N], proj[2 * inner + 2 * G * N:]
    if "conv" not in cache:
        cache["conv"] = [torch.zeros_like(xbc) for _ in range(taps - 1)]
        cache["S"] = [torch.zeros(N, dv, dtype=h.dtype) for _ in range(H)]
    xbc = silu(causal_conv_step(xbc, w["conv"], w["conv.b"], cache["conv"]))
    x = xbc[:inner].view(H, dv)
    B = xbc[inner:inner + G * N].view(G, N)
    C = xbc[inner + G * N:].view(G, N)
    dt = softplus(dt + w["dt_bias"])
    y = selective_scan_step(x, B, C, dt, w["A_log"], w["D"], H // G, cache["S"]).reshape(-1)
    y = y * silu(z)
    parts = cfg["norm_groups"]
    y = rms(y.view(parts, inner // parts), eps).reshape(-1) * w["norm"]
    return w["o"] @ y


def gated_feed_forward(w, h):
    return w["down"] @ (silu(w["gate"] @ h) * (w["up"] @ h))


class PlainBemuzen:
    """``config``: the parsed config.json; ``weights``: name -> tensor (any float type; integer
    tables untouched).  ``step(state, tokens)`` returns ``(logits [T, vocab], residual after every
    layer [L, T, width])`` for the next ``tokens`` of the request whose ``state`` dict is given."""

    def __init__(self, config: dict, weights: dict, dtype=torch.float64) -> None:
        self.config = config
        self.eps = float(config["norm"]["eps"])
        self.w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
        self.dtype = dtype

    def _sub(self, prefix: str) -> dict:
        return {k[len(prefix):]: v for k, v in self.w.items() if k.startswith(prefix)}

    def step(self, state: dict, tokens: list[int]):
        cfg, eps = self.config, self.eps
        bigram = cfg["embedding"]["bigram"]
        rows, trail = [], []
        for token in tokens:
            position = state.get("position", 0)
            x = self.w["embed"][token] + self.w["bigram"][bigram_row(
                state.get("previous"), token, bigram["mul_prev"], bigram["mul_cur"], bigram["buckets"])]
            after = []
            for index, layer in enumerate(cfg["layers"]):
                name = f"l{index}."
                cache = state.setdefault(index, {})
                h = norm_one_plus(x, self.w[name + "norm1"], eps)
                mix = self._sub(name + "mix.")
                if layer["type"] == "parallel":
                    mixed = paired_mixer_step(mix, layer["mixer"], eps, h, position, cache)
                elif layer["type"] == "mamba2":
                    mixed = mamba2_step(mix, layer["mixer"], eps, h, cache)
                else:
                    raise ValueError(layer["type"])
                x = x + norm_one_plus(mixed, self.w[name + "norm1b"], eps)
                if layer.get("mlp") is not None:
                    h = norm_one_plus(x, self.w[name + "norm2"], eps)
                    x = x + norm_one_plus(gated_feed_forward(self._sub(name + "mlp."), h), self.w[name + "norm2b"], eps)
                after.append(x)
            trail.append(torch.stack(after))
            rows.append(self.w["head"] @ norm_one_plus(x, self.w["final.norm"], eps) * cfg["logit_scale"])
            state["previous"] = token
            state["position"] = position + 1
        return torch.stack(rows), torch.stack(trail, dim=1)
