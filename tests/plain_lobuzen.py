"""A plain, slow statement of the Lobuzen decoder, one function per mechanism, token by token.

Written from the design's equations with torch tensors on the CPU, in whatever floating type the
weights are handed over in (tests use float64 or float32); nothing here is shared with the engine's
parts or kernels.  ``PlainLobuzen`` keeps a request's past (keys and values of the attention layers,
the latent rows of the latent layers) in a dictionary, so a prompt may be fed in any portions and
must give the same rows.

Notation: ``h`` is a sublayer's input row (the residual stream itself: this design has no norm in
front of a sublayer), ``W x`` a matrix stored ``[out, in]`` applied to a row.
"""

from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by the root of (mean of squares + eps)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def visible(position: int, window: int | None) -> range:
    """The positions a query at ``position`` sees: itself and the ``window - 1`` before it."""
    first = 0 if window is None else max(0, position - window + 1)
    return range(first, position + 1)


def softmax_with_sink(scores: torch.Tensor, sink=None) -> torch.Tensor:
    """Weights over the given scores; with a sink the denominator also holds ``exp(sink)``, which
    has no key and no value."""
    top = scores.max() if sink is None else torch.maximum(scores.max(), sink)
    e = torch.exp(scores - top)
    total = e.sum() if sink is None else e.sum() + torch.exp(sink - top)
    return e / total


def attention_step(w, cfg, eps, h, position, cache):
    """Grouped attention without positions: queries and keys divided by their root mean square per
    head (no weight), window, ordinary softmax.  ``cache`` holds lists 'k' and 'v', one entry a
    position."""
    H, G, d, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    q = rms((w["q"] @ h).view(H, d), eps)
    k = rms((w["k"] @ h).view(G, d), eps)
    v = (w["v"] @ h).view(G, dv)
    cache.setdefault("k", []).append(k)
    cache.setdefault("v", []).append(v)
    window = (cfg.get("mask") or {}).get("size")
    seen = list(visible(position, window))
    keys = torch.stack([cache["k"][j] for j in seen])       # [n, G, d]
    values = torch.stack([cache["v"][j] for j in seen])
    out = []
    for head in range(H):
        g = head // (H // G)
        weights = softmax_with_sink((keys[:, g] @ q[head]) * cfg["scale"])
        out.append(weights @ values[:, g])
    return w["o"] @ torch.cat(out)


def latent_row(w, eps, h):
    """The row a latent layer caches: the down projection, RMS-normed with a plain weight."""
    return rms(w["dkv"] @ h, eps) * w["dkv.norm"]


def latent_attention_step(w, cfg, eps, h, position, latents):
    """Attention whose keys and values are made from cached latent rows by the layer's own up
    projections; softmax with a sink per head.  ``latents``: the list of latent rows, one a position,
    this position's included (the layer's own or another layer's)."""
    H, d, dv = cfg["heads"], cfg["dim"], cfg["vdim"]
    q = (w["q"] @ h).view(H, d)
    window = (cfg.get("mask") or {}).get("size")
    c = torch.stack([latents[j] for j in visible(position, window)])    # [n, rank]
    keys = (c @ w["uk"].T).view(-1, H, d)
    values = (c @ w["uv"].T).view(-1, H, dv)
    out = []
    for head in range(H):
        weights = softmax_with_sink((keys[:, head] @ q[head]) * cfg["scale"], w["sink"][head])
        out.append(weights @ values[:, head])
    return w["o"] @ torch.cat(out)


def dense_feed_forward(w, cfg, h):
    """Capped gate and up: ``g = min(gate, limit)``, ``u = clamp(up, -limit, limit)``,
    ``down(g * sigmoid(1.702 g) * (u + 1))``."""
    limit = cfg["limit"]
    g = torch.clamp(w["gate"] @ h, max=limit)
    u = torch.clamp(w["up"] @ h, min=-limit, max=limit)
    return w["down"] @ (g * torch.sigmoid(1.702 * g) * (u + 1.0))


def route(w, router, h):
    """The chosen experts and their weights for one row.  Scores are sigmoids of the router's
    logits; the choice is made on score + correction, among the experts of the best groups only (a
    group's mark is the sum of its two largest choice scores); the weights are the plain scores of
    the chosen experts, not renormalised."""
    experts, top = router["experts"], router["top"]
    scores = torch.sigmoid(w["router"].to(torch.float64) @ h.to(torch.float64))
    choice = scores + w["correction"].to(torch.float64)
    groups = router.get("groups")
    if groups:
        count, keep = groups["count"], groups["keep"]
        per = experts // count
        marks = torch.stack([torch.topk(choice[g * per:(g + 1) * per], min(2, per)).values.sum() for g in range(count)])
        kept = torch.topk(marks, keep).indices.tolist()
        allowed = torch.full_like(choice, -math.inf)
        for g in kept:
            allowed[g * per:(g + 1) * per] = choice[g * per:(g + 1) * per]
        choice = allowed
    chosen = torch.topk(choice, top).indices.tolist()
    return chosen, [scores[e].to(h.dtype) for e in chosen]


def expert_feed_forward(w, index, h):
    p = f"e{index}."
    return w[p + "down"] @ (silu(w[p + "gate"] @ h) * (w[p + "up"] @ h))


def routed_feed_forward(w, cfg, h):
    chosen, weights = route(w, cfg["router"], h)
    return sum(weight * expert_feed_forward(w, e, h) for e, weight in zip(chosen, weights))


def token_side(w, side_row, eps, x):
    """What the layer adds for the token itself: ``rms(proj(gelu(gate x) * e)) * norm``."""
    y = w["proj"] @ (gelu_tanh(w["gate"] @ x) * side_row)
    return rms(y, eps) * w["norm"]


def _sub(weights: dict, prefix: str) -> dict:
    return {name[len(prefix):]: t for name, t in weights.items() if name.startswith(prefix)}


class PlainLobuzen:
    def __init__(self, config: dict, weights: dict, dtype=torch.float64):
        self.config = config
        self.eps = config["norm"]["eps"]
        self.weights = {name: (t.to(dtype) if t.is_floating_point() else t) for name, t in weights.items()}
        self.side_dim = (config.get("token_side") or {}).get("dim")
        self.requests: dict = {}

    def release(self, request) -> None:
        self.requests.pop(request, None)

    def step_row(self, request, token: int, trail: list | None = None) -> torch.Tensor:
        """Feed the request's next token; returns the logits row.  ``trail`` receives the residual
        stream after every layer."""
        w, eps = self.weights, self.eps
        state = self.requests.setdefault(request, {"position": 0, "layers": {}})
        position = state["position"]
        x = w["embed"][token].clone()
        for index, layer in enumerate(self.config["layers"]):
            p = f"l{index}."
            mix = _sub(w, p + "mix.")
            cache = state["layers"].setdefault(index, {})
            if layer["type"] == "attention":
                mixed = attention_step(mix, layer["mixer"], eps, x, position, cache)
            elif layer["type"] == "latent_attention":
                source = layer["mixer"].get("kv_from")
                if source is None:
                    cache.setdefault("c", []).append(latent_row(mix, eps, x))
                    latents = cache["c"]
                else:
                    latents = state["layers"][source]["c"]
                mixed = latent_attention_step(mix, layer["mixer"], eps, x, position, latents)
            else:
                raise ValueError(layer["type"])
            x = x + rms(mixed, eps) * w[p + "norm1"]
            mlp = layer.get("mlp")
            if mlp is not None:
                ff = _sub(w, p + "mlp.")
                y = dense_feed_forward(ff, mlp, x) if mlp["kind"] == "dense" else routed_feed_forward(ff, mlp, x)
                x = x + rms(y, eps) * w[p + "norm2"]
            if self.side_dim:
                row = w["side.embed"][token, index * self.side_dim:(index + 1) * self.side_dim]
                x = x + token_side(_sub(w, p + "side."), row, eps, x)
            if trail is not None:
                trail.append(x.clone())
        state["position"] = position + 1
        return w["embed"] @ (rms(x, eps) * w["final.norm"])

    def run(self, request, tokens, trail: list | None = None) -> torch.Tensor:
        rows = []
        for token in tokens:
            layers: list = []
            rows.append(self.step_row(request, int(token), layers))
            if trail is not None:
                trail.append(torch.stack(layers))
        return torch.stack(rows)
