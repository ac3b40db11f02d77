"""Typed configuration of the Lobuzen decoder, read from its config.json.

The file names the design under ``architecture`` and gives every size and every constant that may
differ between two models of the design: ``vocab``, ``width``, ``norm.eps``, ``token_side.dim`` (absent
or null: the layers add nothing for the token itself) and ``layers``, a list whose entries give a
layer's ``type`` (which mixer), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: ``kind`` dense
with ``ff`` and ``limit``, or ``kind`` moe with ``expert.ff`` and ``router``; or null).  What the design fixes
(a norm behind every sublayer and none in front, the form of the activations, the unit norm of queries
and keys, two scores to a group's mark) is code, in ``models/lobuzen.py`` and the parts it names.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .bemuzen_config import _float, _int, _keys
from .model_config import ConfigError


def _window(where: str, raw: Mapping[str, Any]) -> int | None:
    mask = raw.get("mask")
    if mask is None:
        return None
    mask = _keys(where + ".mask", mask, ("size",))
    return None if mask["size"] is None else _int(where + ".mask.size", mask["size"])


def _mask(window: int | None) -> dict[str, Any]:
    return {} if window is None else {"mask": {"size": window}}


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "AttentionMixerConfig":
        raw = _keys(where, raw, ("heads", "kv_heads", "dim", "vdim", "scale"))
        heads, kv_heads = _int(where + ".heads", raw["heads"]), _int(where + ".kv_heads", raw["kv_heads"])
        if heads % kv_heads:
            raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        return cls(heads, kv_heads, _int(where + ".dim", raw["dim"]), _int(where + ".vdim", raw["vdim"]),
                   _float(where + ".scale", raw["scale"]), _window(where, raw))

    def to_dict(self) -> dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                "scale": self.scale, **_mask(self.window)}


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int | None
    kv_from: int | None             # the layer whose cached latent rows this one reads, if not its own

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "LatentMixerConfig":
        raw = _keys(where, raw, ("heads", "dim", "vdim", "kv_rank", "scale"))
        kv_from = raw.get("kv_from")
        return cls(_int(where + ".heads", raw["heads"]), _int(where + ".dim", raw["dim"]),
                   _int(where + ".vdim", raw["vdim"]), _int(where + ".kv_rank", raw["kv_rank"]),
                   _float(where + ".scale", raw["scale"]), _window(where, raw),
                   None if kv_from is None else _int(where + ".kv_from", kv_from, 0))

    def to_dict(self) -> dict[str, Any]:
        made = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank,
                "scale": self.scale, **_mask(self.window)}
        if self.kv_from is not None:
            made["kv_from"] = self.kv_from
        return made


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "dense", "ff": self.ff, "limit": self.limit}


@dataclass(frozen=True)
class MoeMlpConfig:
    ff: int                         # of one expert
    experts: int
    top: int
    group_count: int
    group_keep: int

    def to_dict(self) -> dict[str, Any]:
        return {"kind": "moe", "expert": {"ff": self.ff},
                "router": {"experts": self.experts, "top": self.top,
                           "groups": {"count": self.group_count, "keep": self.group_keep}}}


def _mlp(where: str, raw: Any) -> DenseMlpConfig | MoeMlpConfig | None:
    if raw is None:
        return None
    raw = _keys(where, raw, ("kind",))
    if raw["kind"] == "dense":
        raw = _keys(where, raw, ("ff", "limit"))
        limit = _float(where + ".limit", raw["limit"])
        if limit <= 0:
            raise ConfigError(f"config.json: {where}.limit must be positive, got {limit}")
        return DenseMlpConfig(_int(where + ".ff", raw["ff"]), limit)
    if raw["kind"] == "moe":
        raw = _keys(where, raw, ("expert", "router"))
        expert = _keys(where + ".expert", raw["expert"], ("ff",))
        router = _keys(where + ".router", raw["router"], ("experts", "top"))
        experts, top = _int(where + ".router.experts", router["experts"]), _int(where + ".router.top", router["top"])
        count = keep = 1
        if router.get("groups") is not None:
            groups = _keys(where + ".router.groups", router["groups"], ("count", "keep"))
            count, keep = _int(where + ".router.groups.count", groups["count"]), _int(where + ".router.groups.keep", groups["keep"])
        if experts % count or keep > count:
            raise ConfigError(f"config.json: {where}.router: {experts} experts in {count} groups of which {keep} are kept")
        if top > keep * (experts // count):
            raise ConfigError(f"config.json: {where}.router: top={top} experts cannot come from {keep} groups of {experts // count}")
        return MoeMlpConfig(_int(where + ".expert.ff", expert["ff"]), experts, top, count, keep)
    raise ConfigError(f"config.json: {where}.kind {raw['kind']!r}: 'dense' and 'moe' are part of the design")


_MIXERS = {"attention": AttentionMixerConfig, "latent_attention": LatentMixerConfig}


@dataclass(frozen=True)
class LobuzenLayerConfig:
    type: str
    mixer: AttentionMixerConfig | LatentMixerConfig
    mlp: DenseMlpConfig | MoeMlpConfig | None

    @classmethod
    def from_dict(cls, where: str, raw: Any) -> "LobuzenLayerConfig":
        raw = _keys(where, raw, ("type", "mixer"))
        kind = raw["type"]
        if kind not in _MIXERS:
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                              f"({', '.join(sorted(_MIXERS))})")
        return cls(kind, _MIXERS[kind].from_dict(where + ".mixer", raw["mixer"]), _mlp(where + ".mlp", raw.get("mlp")))

    def to_dict(self) -> dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class LobuzenConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    side_dim: int | None            # None: no per-layer token input
    layers: tuple[LobuzenLayerConfig, ...]

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LobuzenConfig":
        raw = _keys("the file", raw, ("architecture", "vocab", "width", "norm", "layers"))
        norm = _keys("norm", raw["norm"], ("eps",))
        eps = _float("norm.eps", norm["eps"])
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        layers = raw["layers"]
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        side = raw.get("token_side")
        side_dim = None
        if side is not None:
            side = _keys("token_side", side, ("dim",))
            side_dim = None if side["dim"] is None else _int("token_side.dim", side["dim"])
        made = cls(str(raw["architecture"]), _int("vocab", raw["vocab"]), _int("width", raw["width"]), eps, side_dim,
                   tuple(LobuzenLayerConfig.from_dict(f"layers[{index}]", layer) for index, layer in enumerate(layers)))
        for index, layer in enumerate(made.layers):
            mixer = layer.mixer
            if isinstance(mixer, LatentMixerConfig) and mixer.kv_from is not None:
                where = f"layers[{index}].mixer.kv_from"
                if mixer.kv_from >= index:
                    raise ConfigError(f"config.json: {where}={mixer.kv_from} must name an earlier layer")
                owner = made.layers[mixer.kv_from].mixer
                if not isinstance(owner, LatentMixerConfig) or owner.kv_from is not None:
                    raise ConfigError(f"config.json: {where}={mixer.kv_from} names a layer that caches no latent rows of its own")
                if owner.kv_rank != mixer.kv_rank:
                    raise ConfigError(f"config.json: {where}: kv_rank {mixer.kv_rank} differs from the owner's {owner.kv_rank}")
        return made

    @classmethod
    def from_json(cls, path: str | Path) -> "LobuzenConfig":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    def to_dict(self) -> dict[str, Any]:
        """config.json content that reads back to an equal object."""
        made = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "layers": [layer.to_dict() for layer in self.layers]}
        if self.side_dim is not None:
            made["token_side"] = {"dim": self.side_dim}
        return made

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def summary(self) -> list[str]:
        """A few lines that describe the model to a reader of the command line's output."""
        def kind(layer: LobuzenLayerConfig) -> str:
            mlp = "no feed-forward" if layer.mlp is None else "dense" if isinstance(layer.mlp, DenseMlpConfig) else "experts"
            return f"{layer.type} ({mlp})"
        runs: list[list] = []
        for name in map(kind, self.layers):
            if runs and runs[-1][0] == name:
                runs[-1][1] += 1
            else:
                runs.append([name, 1])
        return [f"{len(self.layers)} layers, width={self.hidden_size}, vocabulary={self.vocab_size}, "
                f"token side={'none' if self.side_dim is None else self.side_dim}",
                "order of layers: " + ", ".join(f"{count} x {name}" for name, count in runs)]
