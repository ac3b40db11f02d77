"""Lobuzen: a decoder whose sublayers read the residual stream itself and are normalised behind, with two
kinds of attention (grouped heads with unit-norm queries and keys; cached latent rows with a sink) and dense
or routed feed-forwards, as a description made of parts.

What the design fixes, and so what is written here rather than read from config.json:

* a layer is ``h += norm1(mixer(h))``, then, where it has one, ``h += norm2(ff(h))``, then, where the model
  has a token side, ``h += side_norm(proj(gelu_tanh(gate h) * e))`` with ``e`` the layer's columns of the token's
  row of one table; all norms (and the model's last one) are RMSNorm with a plain weight;
* the attention mixer rotates nothing, divides queries and keys by their root mean square per head (no
  weight), has grouped key/value heads, an optional window and an ordinary softmax;
* the latent mixer caches one RMS-normed row per position and makes keys and values from it by up
  projections per head; every head's softmax has a sink; a layer may read another layer's rows;
* the dense feed-forward is ``down(g sigmoid(1.702 g) (u + 1))`` with ``g = min(gate h, limit)`` and ``u =
  clamp(up h, -limit, limit)``; an expert is ``down(silu(gate h) * up h)``; the router scores are sigmoids, a
  group's mark is the sum of its two largest choice scores, the weights are not renormalised;
* the logits are the embedding table times the normalised stream.

Tensor names: ``embed``, ``side.embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down`` or
``l<i>.mlp.router|correction|e<j>.gate|up|down``, ``l<i>.side.gate|proj|norm``, ``final.norm``; matrices are stored
``[out, in]``.
"""

from __future__ import annotations

import math

import torch

from ..config.lobuzen_config import AttentionMixerConfig, DenseMlpConfig, LatentMixerConfig, LobuzenConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

SWISH_SLOPE = 1.702         # of the dense feed-forward's gate
UP_OFFSET = 1.0             # added to the dense feed-forward's capped up projection
GROUP_TOP = 2               # choice scores that make a group's mark


def _norm(config: LobuzenConfig, name: str) -> PartSpec:
    # The tensor is the norm's own name (no ".weight" behind it).
    return PartSpec("rms_norm", {"eps": config.norm_eps, "weight_name": ""}, name=name)


def _longest(windows) -> int | None:
    """The window a cache must keep for layers that read it over these windows."""
    windows = list(windows)
    return None if any(w is None for w in windows) else max(windows)


def _mixer(config: LobuzenConfig, index: int) -> PartSpec:
    mixer = config.layers[index].mixer
    if isinstance(mixer, AttentionMixerConfig):
        return PartSpec("biased_attention", {
            "num_heads": mixer.heads, "num_kv_heads": mixer.kv_heads, "head_dim": mixer.dim, "value_dim": mixer.vdim,
            "scale": mixer.scale, "slopes": None, "window": mixer.window, "qk_norm_eps": config.norm_eps,
            "qk_norm_weights": False, "q_temperature": None, "weight_names": ("q", "k", "v", "o", "", ""),
        }, name="mix")
    readers = [other.mixer.window for other in config.layers
               if isinstance(other.mixer, LatentMixerConfig) and other.mixer.kv_from == index]
    return PartSpec("latent_attention", {
        "num_heads": mixer.heads, "head_dim": mixer.dim, "value_dim": mixer.vdim, "latent_dim": mixer.kv_rank,
        "scale": mixer.scale, "window": mixer.window, "cache_window": _longest([mixer.window, *readers]),
        "norm_eps": config.norm_eps, "sinks": True, "own_latent": mixer.kv_from is None,
    }, name="mix")


def _feed_forward(mlp) -> PartSpec:
    if isinstance(mlp, DenseMlpConfig):
        return PartSpec("capped_gated", {"intermediate_size": mlp.ff, "limit": mlp.limit, "slope": SWISH_SLOPE,
                                         "up_offset": UP_OFFSET}, name="mlp")
    return PartSpec("routed_experts", {
        "num_experts": mlp.experts, "top": mlp.top, "intermediate_size": mlp.ff, "group_count": mlp.group_count,
        "group_keep": mlp.group_keep, "group_top": GROUP_TOP, "correction": True}, name="mlp")


def build_spec(config: LobuzenConfig) -> ModelSpec:
    layers, schedule = [], []
    for index, layer in enumerate(config.layers):
        norms = {"post_mixer": _norm(config, "norm1")}
        feed_forward = None
        if layer.mlp is not None:
            norms["post_feed_forward"] = _norm(config, "norm2")
            feed_forward = _feed_forward(layer.mlp)
        side = None
        if config.side_dim is not None:
            norms["post_side"] = _norm(config, "side.norm")
            side = PartSpec("gated_token_rows", {
                "dim": config.side_dim, "column": index * config.side_dim,
                "table_width": len(config.layers) * config.side_dim, "table_name": "/side.embed"}, name="side")
        layers.append(LayerSpec(name=f"l{index}", block=PartSpec("post_norm"), mixer=_mixer(config, index),
                                feed_forward=feed_forward, position=PartSpec("none"), norms=norms, side=side))
        # one execution per layer, so a layer's number is also its place in the schedule
        schedule.append(ScheduleEntry(layer=index, cache_from=getattr(layer.mixer, "kv_from", None)))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("token_embedding", {"weight_name": "embed"}, name=""),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=_norm(config, "final.norm"),
        output_head=PartSpec("linear_head", {"tied": True}, name="head"),
    )


def random_weights(config: LobuzenConfig, seed: int, *, std: float | None = None, norm_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Seeded random tensors under the checkpoint's names: matrices ``N(0, std)`` (``std`` defaults to
    ``fan_in ** -0.5``, which keeps activations of order one through any width), norm weights ``1 + N(0,
    norm_std)``, sinks and the router's correction ``N(0, 0.5)`` and ``N(0, 0.1)``."""
    generator = torch.Generator(device=device).manual_seed(seed)

    def normal(shape, mean: float, spread: float) -> torch.Tensor:
        return (mean + torch.empty(shape, dtype=torch.float32, device=device).normal_(
            0.0, 1.0, generator=generator) * spread).to(dtype)

    def matrix(rows: int, cols: int) -> torch.Tensor:
        return normal((rows, cols), 0.0, std if std is not None else 1.0 / math.sqrt(cols))

    hidden = config.hidden_size
    weights = {"embed": normal((config.vocab_size, hidden), 0.0, 1.0)}
    if config.side_dim is not None:
        weights["side.embed"] = normal((config.vocab_size, len(config.layers) * config.side_dim), 0.0, 1.0)
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        mixer = layer.mixer
        weights[p + "norm1"] = normal((hidden,), 1.0, norm_std)
        weights[p + "mix.q"] = matrix(mixer.heads * mixer.dim, hidden)
        weights[p + "mix.o"] = matrix(hidden, mixer.heads * mixer.vdim)
        if isinstance(mixer, AttentionMixerConfig):
            weights[p + "mix.k"] = matrix(mixer.kv_heads * mixer.dim, hidden)
            weights[p + "mix.v"] = matrix(mixer.kv_heads * mixer.vdim, hidden)
        else:
            if mixer.kv_from is None:
                weights[p + "mix.dkv"] = matrix(mixer.kv_rank, hidden)
                weights[p + "mix.dkv.norm"] = normal((mixer.kv_rank,), 1.0, norm_std)
            weights[p + "mix.uk"] = matrix(mixer.heads * mixer.dim, mixer.kv_rank)
            weights[p + "mix.uv"] = matrix(mixer.heads * mixer.vdim, mixer.kv_rank)
            weights[p + "mix.sink"] = normal((mixer.heads,), 0.0, 0.5)
        mlp = layer.mlp
        if mlp is not None:
            weights[p + "norm2"] = normal((hidden,), 1.0, norm_std)
            if isinstance(mlp, DenseMlpConfig):
                weights[p + "mlp.gate"] = matrix(mlp.ff, hidden)
                weights[p + "mlp.up"] = matrix(mlp.ff, hidden)
                weights[p + "mlp.down"] = matrix(hidden, mlp.ff)
            else:
                weights[p + "mlp.router"] = matrix(mlp.experts, hidden)
                weights[p + "mlp.correction"] = normal((mlp.experts,), 0.0, 0.1)
                for expert in range(mlp.experts):
                    weights[p + f"mlp.e{expert}.gate"] = matrix(mlp.ff, hidden)
                    weights[p + f"mlp.e{expert}.up"] = matrix(mlp.ff, hidden)
                    weights[p + f"mlp.e{expert}.down"] = matrix(hidden, mlp.ff)
        if config.side_dim is not None:
            weights[p + "side.gate"] = matrix(config.side_dim, hidden)
            weights[p + "side.proj"] = matrix(hidden, config.side_dim)
            weights[p + "side.norm"] = normal((hidden,), 1.0, norm_std)
    weights["final.norm"] = normal((hidden,), 1.0, norm_std)
    return weights


register_architecture("Lobuzen", LobuzenConfig, build_spec, random_weights)
