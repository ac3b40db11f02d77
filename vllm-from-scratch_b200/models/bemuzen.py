"""Bemuzen: a decoder whose layers mix tokens either by two mixers side by side (softmax attention
with a distance bias beside decayed linear attention) or by a selective scan, as a description made
of parts.

What the design fixes, and so what is written here rather than read from config.json:

* the embedding is a token row plus a row of a hashed table of (previous token, token) pairs;
* every layer is ``h += post(mixer(pre(h)))`` and, where it has one, ``h += post(ff(pre(h)))``, with all
  four norms (and the model's last one) RMSNorm whose stored vector lies around zero (weight ``1 + w``);
* the softmax branch normalises queries and keys per head with plain weights, rotates nothing, scales
  the queries by a temperature that grows with the logarithm of the position, and subtracts
  ``2 ** (-8 (h + 1) / H) * distance`` from the scores of head h;
* the linear branch and the selective scan activate with silu, gate with sigmoid / silu, and keep
  their state in float32;
* the feed-forward is ``down(silu(gate x) * up x)``; the logits are multiplied by ``logit_scale``.

Tensor names: ``embed``, ``bigram``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm``, ``head``; matrices are stored ``[out, in]``.
"""

from __future__ import annotations

import math

import torch

from ..config.bemuzen_config import BemuzenConfig, Mamba2MixerConfig, ParallelMixerConfig
from ..config.registry import register_architecture
from ..parts.attention import power_of_two_slopes
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry


def _norm(config: BemuzenConfig, name: str) -> PartSpec:
    # The tensor is the norm's own name (no ".weight" behind it) and is stored around zero.
    return PartSpec("rms_norm", {"eps": config.norm_eps, "offset": 1.0, "weight_name": ""}, name=name)


def _mixer(config: BemuzenConfig, mixer: ParallelMixerConfig | Mamba2MixerConfig) -> PartSpec:
    if isinstance(mixer, Mamba2MixerConfig):
        return PartSpec("selective_scan", {
            "num_heads": mixer.heads, "value_dim": mixer.vdim, "state_dim": mixer.state, "groups": mixer.groups,
            "conv_taps": mixer.conv, "norm_groups": mixer.norm_groups, "norm_eps": config.norm_eps,
        }, name="mix")
    left, right = mixer.left, mixer.right
    softmax = PartSpec("biased_attention", {
        "num_heads": left.heads, "num_kv_heads": left.kv_heads, "head_dim": left.dim, "value_dim": left.vdim,
        "scale": left.scale, "slopes": tuple(power_of_two_slopes(left.heads)), "qk_norm_eps": config.norm_eps,
        "q_temperature": (left.q_temp_coef, left.q_temp_every),
        "weight_names": ("q", "k", "v", "o", "q.norm", "k.norm"),
    }, name="left")
    linear = PartSpec("decayed_linear_attention", {
        "num_heads": right.heads, "head_dim": right.dim, "value_dim": right.vdim, "decay": right.decay,
        "norm_eps": config.norm_eps,
    }, name="right")
    return PartSpec("paired_mixers", {"branches": (softmax, linear), "eps": config.norm_eps}, name="mix")


def build_spec(config: BemuzenConfig) -> ModelSpec:
    layers = []
    for index, layer in enumerate(config.layers):
        norms = {"mixer": _norm(config, "norm1"), "post_mixer": _norm(config, "norm1b")}
        feed_forward = None
        if layer.ff is not None:
            norms.update({"feed_forward": _norm(config, "norm2"), "post_feed_forward": _norm(config, "norm2b")})
            feed_forward = PartSpec("gated_silu", {"intermediate_size": layer.ff,
                                                   "weight_names": ("gate", "up", "down")}, name="mlp")
        layers.append(LayerSpec(name=f"l{index}", block=PartSpec("sandwich_norm"), mixer=_mixer(config, layer.mixer),
                                feed_forward=feed_forward, position=PartSpec("none"), norms=norms))
    return ModelSpec(
        hidden_size=config.hidden_size,
        vocab_size=config.vocab_size,
        embedding=PartSpec("bigram_embedding", {
            "buckets": config.bigram_buckets, "mul_prev": config.bigram_mul_prev, "mul_cur": config.bigram_mul_cur,
            "weight_names": ("embed", "bigram")}, name=""),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=index) for index in range(len(layers))),
        final_norm=_norm(config, "final.norm"),
        output_head=PartSpec("linear_head", {"scale": config.logit_scale, "weight_name": ""}, name="head"),
    )


def random_weights(config: BemuzenConfig, seed: int, *, std: float | None = None, norm_std: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16, device: str | torch.device = "cpu"
                   ) -> dict[str, torch.Tensor]:
    """Seeded random tensors under the checkpoint's names: matrices ``N(0, std)`` (``std`` defaults to
    ``fan_in ** -0.5``, which keeps activations of order one through any width), vectors stored around
    zero ``N(0, norm_std)``, plain norm weights ``1 + N(0, norm_std)``, ``A_log`` and ``dt_bias`` spread so that
    the heads' decays differ."""
    generator = torch.Generator(device=device).manual_seed(seed)

    def normal(shape, mean: float, spread: float) -> torch.Tensor:
        return (mean + torch.empty(shape, dtype=torch.float32, device=device).normal_(
            0.0, 1.0, generator=generator) * spread).to(dtype)

    def matrix(rows: int, cols: int) -> torch.Tensor:
        return normal((rows, cols), 0.0, std if std is not None else 1.0 / math.sqrt(cols))

    hidden = config.hidden_size
    weights = {"embed": normal((config.vocab_size, hidden), 0.0, 1.0),
               "bigram": normal((config.bigram_buckets + 1, hidden), 0.0, 0.5)}
    for index, layer in enumerate(config.layers):
        p = f"l{index}."
        for name in ("norm1", "norm1b") + (("norm2", "norm2b") if layer.ff is not None else ()):
            weights[p + name] = normal((hidden,), 0.0, norm_std)
        mixer = layer.mixer
        if isinstance(mixer, Mamba2MixerConfig):
            inner = mixer.heads * mixer.vdim
            channels = inner + 2 * mixer.groups * mixer.state
            weights[p + "mix.in"] = matrix(inner + channels + mixer.heads, hidden)
            weights[p + "mix.conv"] = normal((channels, mixer.conv), 0.0, 0.5)
            weights[p + "mix.conv.b"] = normal((channels,), 0.0, 0.1)
            weights[p + "mix.dt_bias"] = normal((mixer.heads,), -1.0, 1.0)
            weights[p + "mix.A_log"] = normal((mixer.heads,), 0.0, 1.0)
            weights[p + "mix.D"] = normal((mixer.heads,), 1.0, 0.3)
            weights[p + "mix.norm"] = normal((inner,), 1.0, norm_std)
            weights[p + "mix.o"] = matrix(hidden, inner)
        else:
            left, right = mixer.left, mixer.right
            weights[p + "mix.left.q"] = matrix(left.heads * left.dim, hidden)
            weights[p + "mix.left.k"] = matrix(left.kv_heads * left.dim, hidden)
            weights[p + "mix.left.v"] = matrix(left.kv_heads * left.vdim, hidden)
            weights[p + "mix.left.q.norm"] = normal((left.dim,), 1.0, norm_std)
            weights[p + "mix.left.k.norm"] = normal((left.dim,), 1.0, norm_std)
            weights[p + "mix.left.o"] = matrix(hidden, left.heads * left.vdim)
            weights[p + "mix.left.out"] = normal((hidden,), 1.0, norm_std)
            weights[p + "mix.right.q"] = matrix(right.heads * right.dim, hidden)
            weights[p + "mix.right.k"] = matrix(right.heads * right.dim, hidden)
            weights[p + "mix.right.v"] = matrix(right.heads * right.vdim, hidden)
            weights[p + "mix.right.g"] = matrix(right.heads * right.vdim, hidden)
            weights[p + "mix.right.norm"] = normal((right.heads * right.vdim,), 1.0, norm_std)
            weights[p + "mix.right.o"] = matrix(hidden, right.heads * right.vdim)
            weights[p + "mix.right.out"] = normal((hidden,), 1.0, norm_std)
        if layer.ff is not None:
            weights[p + "mlp.gate"] = matrix(layer.ff, hidden)
            weights[p + "mlp.up"] = matrix(layer.ff, hidden)
            weights[p + "mlp.down"] = matrix(hidden, layer.ff)
    weights["final.norm"] = normal((hidden,), 0.0, norm_std)
    weights["head"] = matrix(config.vocab_size, hidden)
    return weights


register_architecture("Bemuzen", BemuzenConfig, build_spec, random_weights)
