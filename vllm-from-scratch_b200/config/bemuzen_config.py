"""Typed configuration of the Bemuzen decoder, read from its config.json.

The file names the design under ``architecture`` and gives every size and every constant that may
differ between two models of the design: ``vocab``, ``width``, ``logit_scale``, ``norm.eps``,
``embedding.bigram`` (``buckets``, ``mul_prev``, ``mul_cur``) and ``layers``, a list whose entries give
a layer's ``type`` (which mixer), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: ``kind``
and ``ff``, or null).  What the design fixes (the form of the norms, the slopes of the distance bias,
the activations) is code, in ``models/bemuzen.py`` and the parts it names.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .model_config import ConfigError


def _int(where: str, value: Any, least: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where} must be an integer of at least {least}, got {value!r}")
    return value


def _float(where: str, value: Any) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where} must be a number, got {value!r}")
    return float(value)


def _keys(where: str, raw: Any, wanted: tuple[str, ...]) -> Mapping[str, Any]:
    if not isinstance(raw, Mapping):
        raise ConfigError(f"config.json: {where} must be an object, got {raw!r}")
    missing = [key for key in wanted if key not in raw]
    if missing:
        raise ConfigError(f"config.json: {where} lacks {', '.join(missing)}")
    return raw


@dataclass(frozen=True)
class SoftmaxBranchConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: float
    q_temp_every: int

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "SoftmaxBranchConfig":
        raw = _keys(where, raw, ("heads", "kv_heads", "dim", "vdim", "scale", "q_temp"))
        temp = _keys(where + ".q_temp", raw["q_temp"], ("coef", "every"))
        heads, kv_heads = _int(where + ".heads", raw["heads"]), _int(where + ".kv_heads", raw["kv_heads"])
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        return cls(heads, kv_heads, _int(where + ".dim", raw["dim"]), _int(where + ".vdim", raw["vdim"]),
                   _float(where + ".scale", raw["scale"]), _float(where + ".q_temp.coef", temp["coef"]),
                   _int(where + ".q_temp.every", temp["every"]))

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, "q_temp": {"coef": self.q_temp_coef, "every": self.q_temp_every}}


@dataclass(frozen=True)
class LinearBranchConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple[float, ...]

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "LinearBranchConfig":
        raw = _keys(where, raw, ("heads", "dim", "vdim", "decay"))
        heads = _int(where + ".heads", raw["heads"])
        decay = raw["decay"]
        if not isinstance(decay, (list, tuple)) or len(decay) != heads:
            raise ConfigError(f"config.json: {where}.decay must list one constant per head ({heads})")
        return cls(heads, _int(where + ".dim", raw["dim"]), _int(where + ".vdim", raw["vdim"]),
                   tuple(_float(where + ".decay", value) for value in decay))

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: SoftmaxBranchConfig
    right: LinearBranchConfig

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "ParallelMixerConfig":
        raw = _keys(where, raw, ("left", "right"))
        return cls(SoftmaxBranchConfig.from_dict(where + ".left", raw["left"]),
                   LinearBranchConfig.from_dict(where + ".right", raw["right"]))

    def to_dict(self) -> dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict()}


@dataclass(frozen=True)
class Mamba2MixerConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "Mamba2MixerConfig":
        raw = _keys(where, raw, ("heads", "vdim", "state", "groups", "conv", "norm_groups"))
        made = cls(*(_int(f"{where}.{key}", raw[key]) for key in ("heads", "vdim", "state", "groups", "conv", "norm_groups")))
        if made.heads % made.groups:
            raise ConfigError(f"config.json: {where}.heads ({made.heads}) must be a multiple of groups ({made.groups})")
        if (made.heads * made.vdim) % made.norm_groups:
            raise ConfigError(f"config.json: {where}: heads * vdim must divide into norm_groups ({made.norm_groups})")
        return made

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                "conv": self.conv, "norm_groups": self.norm_groups}


_MIXERS = {"parallel": ParallelMixerConfig, "mamba2": Mamba2MixerConfig}


@dataclass(frozen=True)
class BemuzenLayerConfig:
    type: str
    mixer: ParallelMixerConfig | Mamba2MixerConfig
    ff: int | None                  # None: the layer has no feed-forward

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "BemuzenLayerConfig":
        raw = _keys(where, raw, ("type", "mixer"))
        kind = raw["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(_MIXERS))})")
        mlp = raw.get("mlp")
        ff = None
        if mlp is not None:
            mlp = _keys(where + ".mlp", mlp, ("kind", "ff"))
            if mlp["kind"] != "dense":
                raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r}: only 'dense' is part of the design")
            ff = _int(where + ".mlp.ff", mlp["ff"])
        return cls(kind, _MIXERS[kind].from_dict(where + ".mixer", raw["mixer"]), ff)

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.ff is None else {"kind": "dense", "ff": self.ff}}


@dataclass(frozen=True)
class BemuzenConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    logit_scale: float
    norm_eps: float
    bigram_buckets: int
    bigram_mul_prev: int
    bigram_mul_cur: int
    layers: tuple[BemuzenLayerConfig, ...]
    initializer_range: float = 0.05

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "BemuzenConfig":
        raw = _keys("the file", raw, ("architecture", "vocab", "width", "logit_scale", "norm", "embedding", "layers"))
        norm = _keys("norm", raw["norm"], ("eps",))
        bigram = _keys("embedding.bigram", _keys("embedding", raw["embedding"], ("bigram",))["bigram"],
                       ("buckets", "mul_prev", "mul_cur"))
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        eps = _float("norm.eps", norm["eps"])
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        return cls(
            architecture=str(raw["architecture"]), vocab_size=_int("vocab", raw["vocab"]),
            hidden_size=_int("width", raw["width"]), logit_scale=_float("logit_scale", raw["logit_scale"]),
            norm_eps=eps, bigram_buckets=_int("embedding.bigram.buckets", bigram["buckets"]),
            bigram_mul_prev=_int("embedding.bigram.mul_prev", bigram["mul_prev"], 0),
            bigram_mul_cur=_int("embedding.bigram.mul_cur", bigram["mul_cur"], 0),
            layers=tuple(BemuzenLayerConfig.from_dict(f"layers[{index}]", layer) for index, layer in enumerate(layers)),
            initializer_range=float(raw.get("initializer_range", 0.05)))

    @classmethod
    def from_json(cls, path: str | Path) -> "BemuzenConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> dict[str, Any]:
        """config.json content that reads back to an equal object."""
        return {
            "architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
            "logit_scale": self.logit_scale, "norm": {"eps": self.norm_eps},
            "embedding": {"bigram": {"buckets": self.bigram_buckets, "mul_prev": self.bigram_mul_prev,
                                     "mul_cur": self.bigram_mul_cur}},
            "layers": [layer.to_dict() for layer in self.layers],
            "initializer_range": self.initializer_range,
        }

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def summary(self) -> list[str]:
        """A few lines that describe the model to a reader of the command line's output."""
        kinds = [layer.type + ("" if layer.ff is not None else " (no feed-forward)") for layer in self.layers]
        runs: list[list] = []
        for kind in kinds:
            if runs and runs[-1][0] == kind:
                runs[-1][1] += 1
            else:
                runs.append([kind, 1])
        return [f"{len(self.layers)} layers, width={self.hidden_size}, vocabulary={self.vocab_size}, "
                f"bigram buckets={self.bigram_buckets}",
                "order of layers: " + ", ".join(f"{count} x {kind}" for kind, count in runs)]
