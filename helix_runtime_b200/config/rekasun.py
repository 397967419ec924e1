"""Typed configuration of the Rekasun decoder, read from its ``config.json``.

The document is nested: sizes of the model at the top (``vocab``, ``width``), constants in
small objects (``embedding.scale``, ``norm.eps``), a list ``layers`` whose entries name the
kind of mixer (``type``), the mixer's sizes (``mixer``) and the feed-forward (``mlp``, null
for none), and an optional ``loop`` (``start``, ``stop``, ``times``): layers ``start`` to
``stop - 1`` run ``times`` times in a row with the same weights.  Every size and constant is
read from the document; layers may differ from one another in every one of them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
import math

from .keys import COUNT, REAL, TEXT, Key, Kind, read_keys

ARCHITECTURE = "Rekasun"
DEFAULT_MAX_POSITIONS = 1 << 17


# a constant that multiplies: any finite number
FACTOR = Kind(lambda value: isinstance(value, (int, float)) and not isinstance(value, bool)
              and math.isfinite(float(value)), float, "must be a finite number")


def _whole(value: Any) -> bool:
    return isinstance(value, int) and not isinstance(value, bool) and value >= 0


def _object(document: Mapping[str, Any], name: str, where: str = "") -> Mapping[str, Any]:
    value = document.get(name)
    if not isinstance(value, dict):
        raise ConfigError(f"config field {where + name!r} must be an object")
    return value


@dataclasses.dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float             # scores are (q . k) * scale
    conv: int                # taps of the causal filter on q, k and v (1: none)
    window: int              # a position sees the last `window` positions, itself included
    keep_first: int          # and the first `keep_first` positions, whatever their distance

    KEYS = (Key("heads", COUNT), Key("kv_heads", COUNT), Key("dim", COUNT), Key("vdim", COUNT),
            Key("scale", REAL), Key("conv", COUNT, default=1))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "AttentionMixerConfig":
        values = read_keys(document, cls.KEYS, where)
        mask = _object(document, "mask", where)
        size, keep = mask.get("size"), mask.get("keep_first", 0)
        if not (_whole(size) and size > 0):
            raise ConfigError(f"config field '{where}mask.size' must be a positive integer")
        if not _whole(keep):
            raise ConfigError(f"config field '{where}mask.keep_first' must be a whole number")
        if values["heads"] % values["kv_heads"]:
            raise ConfigError(f"config field '{where}heads' must be a multiple of "
                              f"'{where}kv_heads'")
        return cls(window=int(size), keep_first=int(keep), **values)

    def to_dict(self) -> Dict[str, Any]:
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
                "vdim": self.vdim, "scale": self.scale, "conv": self.conv,
                "mask": {"size": self.window, "keep_first": self.keep_first}}


MIXER_CONFIGS = {"attention": AttentionMixerConfig}


@dataclasses.dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    kind: str = "dense"

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "DenseMlpConfig":
        values = read_keys(document, (Key("ff", COUNT), Key("kind", TEXT, default="dense")), where)
        if values["kind"] != "dense":
            raise ConfigError(f"config field '{where}kind' is {values['kind']!r}; this engine "
                              f"runs 'dense' feed-forwards")
        return cls(**values)

    def to_dict(self) -> Dict[str, Any]:
        return {"ff": self.ff, "kind": self.kind}


@dataclasses.dataclass(frozen=True)
class RekasunLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[DenseMlpConfig]

    @classmethod
    def from_dict(cls, document: Any, index: int) -> "RekasunLayerConfig":
        where = f"layers[{index}]."
        if not isinstance(document, dict):
            raise ConfigError(f"config field 'layers[{index}]' must be an object")
        kind = document.get("type")
        if kind not in MIXER_CONFIGS:
            raise ConfigError(f"config field '{where}type' is {kind!r}; known: "
                              + ", ".join(sorted(MIXER_CONFIGS)))
        mixer = MIXER_CONFIGS[kind].from_dict(_object(document, "mixer", where), where + "mixer.")
        mlp = document.get("mlp")
        if mlp is not None and not isinstance(mlp, dict):
            raise ConfigError(f"config field '{where}mlp' must be an object or null")
        return cls(kind, mixer, None if mlp is None else DenseMlpConfig.from_dict(mlp, where + "mlp."))

    def to_dict(self) -> Dict[str, Any]:
        return {"type": self.type, "mixer": self.mixer.to_dict(),
                "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclasses.dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclasses.dataclass(frozen=True)
class RekasunConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[RekasunLayerConfig, ...]
    loop: Optional[LoopConfig] = None
    max_positions: int = DEFAULT_MAX_POSITIONS

    architecture = ARCHITECTURE

    def __post_init__(self) -> None:
        if not self.layers:
            raise ConfigError("config field 'layers' must name at least one layer")
        if self.loop is not None:
            loop = self.loop
            if not 0 <= loop.start < loop.stop <= len(self.layers) or loop.times < 1:
                raise ConfigError(f"config field 'loop' ({loop.start}, {loop.stop}, {loop.times}) "
                                  f"does not fit {len(self.layers)} layers")

    @classmethod
    def from_dict(cls, document: Mapping[str, Any]) -> "RekasunConfig":
        values = read_keys(document, (Key("vocab", COUNT), Key("width", COUNT),
                                      Key("max_positions", COUNT, default=DEFAULT_MAX_POSITIONS)))
        scale = read_keys(document.get("embedding") or {}, (Key("scale", FACTOR, default=1.0),),
                          "embedding.")["scale"]
        eps = read_keys(_object(document, "norm"), (Key("eps", REAL),), "norm.")["eps"]
        layers = document.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a list of layers")
        loop = document.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not all(_whole(loop.get(k)) for k in ("start", "stop", "times")):
                raise ConfigError("config field 'loop' must give whole numbers start, stop, times")
            loop = LoopConfig(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        return cls(vocab=values["vocab"], width=values["width"], embedding_scale=scale,
                   norm_eps=eps, loop=loop, max_positions=values["max_positions"],
                   layers=tuple(RekasunLayerConfig.from_dict(layer, index)
                                for index, layer in enumerate(layers)))

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.loop is not None:
            document["loop"] = dataclasses.asdict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            document["max_positions"] = self.max_positions
        return document

    def layer_runs(self) -> Tuple[Tuple[int, bool], ...]:
        """The layers in the order they run, as ``(layer, starts_a_repeat)``: the second is
        true for the first layer of every pass through the loop but the first pass."""
        count = len(self.layers)
        if self.loop is None:
            return tuple((layer, False) for layer in range(count))
        loop = self.loop
        runs = [(layer, False) for layer in range(loop.start)]
        for turn in range(loop.times):
            runs.extend((layer, turn > 0 and layer == loop.start)
                        for layer in range(loop.start, loop.stop))
        runs.extend((layer, False) for layer in range(loop.stop, count))
        return tuple(runs)
