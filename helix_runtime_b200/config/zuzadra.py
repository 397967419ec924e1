"""Typed configuration of the Zuzadra decoder, read from its ``config.json``.

The document is nested: ``vocab`` and ``width`` at the top, ``norm.eps``, an optional
``streams`` (the number of residual streams joined by hyper-connections; left out: one
residual and no connection weights), a list ``layers`` whose entries name the mixer
(``type``: ``mamba2`` or ``parallel``), its sizes (``mixer``) and the feed-forward (``mlp``,
null for none), and an optional ``loop`` (``start``, ``stop``, ``times``): layers ``start`` to
``stop - 1`` run ``times`` times in a row with the same weights, every run with its own cache
and state.  Every size and constant is read from the document; layers may differ from one
another in every one of them.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, Mapping, Optional, Tuple

from .errors import ConfigError
from .keys import COUNT, REAL, TEXT, Key, read_keys
from .rekasun import FACTOR, DenseMlpConfig, LoopConfig, _object, _whole

ARCHITECTURE = "Zuzadra"
DEFAULT_MAX_POSITIONS = 1 << 17
ROTARY_LAYOUTS = ("halves", "interleaved")


@dataclasses.dataclass(frozen=True)
class StateSpaceMixerConfig:
    heads: int
    vdim: int                # width of a head
    state: int               # rows of a head's state matrix
    groups: int              # groups of heads that share B and C
    conv: int                # taps of the causal filter on x, B and C
    norm_groups: int         # equal parts the gated output is normed in

    KEYS = (Key("heads", COUNT), Key("vdim", COUNT), Key("state", COUNT),
            Key("groups", COUNT, default=1), Key("conv", COUNT, default=1),
            Key("norm_groups", COUNT, default=1))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "StateSpaceMixerConfig":
        values = read_keys(document, cls.KEYS, where)
        if values["heads"] % values["groups"]:
            raise ConfigError(f"config field '{where}heads' must be a multiple of '{where}groups'")
        if (values["heads"] * values["vdim"]) % values["norm_groups"]:
            raise ConfigError(f"config field '{where}norm_groups' must divide heads * vdim")
        return cls(**values)

    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)


@dataclasses.dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float             # scores are (q . k) * scale
    window: int              # a position sees the last `window` positions, itself included
    rot_base: float
    rot_dims: int            # leading coordinates of a head that are rotated
    rot_layout: str          # which coordinates pair up: halves or interleaved

    KEYS = (Key("heads", COUNT), Key("kv_heads", COUNT), Key("dim", COUNT), Key("vdim", COUNT),
            Key("scale", REAL))

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "WindowAttentionConfig":
        values = read_keys(document, cls.KEYS, where)
        size = _object(document, "mask", where).get("size")
        if not (_whole(size) and size > 0):
            raise ConfigError(f"config field '{where}mask.size' must be a positive integer")
        rot = _object(document, "rot", where)
        rotation = read_keys(rot, (Key("base", REAL), Key("dims", COUNT),
                                   Key("layout", TEXT, default="halves")), where + "rot.")
        if rotation["layout"] not in ROTARY_LAYOUTS:
            raise ConfigError(f"config field '{where}rot.layout' is {rotation['layout']!r}; known: "
                              + ", ".join(ROTARY_LAYOUTS))
        if rotation["dims"] % 2 or rotation["dims"] > values["dim"]:
            raise ConfigError(f"config field '{where}rot.dims' must be even and at most "
                              f"'{where}dim'")
        if values["vdim"] % 2:
            raise ConfigError(f"config field '{where}vdim' must be even: values are rotated in pairs")
        if values["heads"] % values["kv_heads"]:
            raise ConfigError(f"config field '{where}heads' must be a multiple of "
                              f"'{where}kv_heads'")
        return cls(window=int(size), rot_base=rotation["base"], rot_dims=rotation["dims"],
                   rot_layout=rotation["layout"], **values)

    def to_dict(self) -> Dict[str, Any]:
        rot = {"base": self.rot_base, "dims": self.rot_dims}
        if self.rot_layout != "halves":
            rot["layout"] = self.rot_layout
        return {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim,
                "vdim": self.vdim, "scale": self.scale, "mask": {"size": self.window}, "rot": rot}


@dataclasses.dataclass(frozen=True)
class TimeMixConfig:
    heads: int
    dim: int
    rank: Optional[int] = None    # rows of the decay's first small matrix; None: the checkpoint's

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "TimeMixConfig":
        return cls(**read_keys(document, (Key("heads", COUNT), Key("dim", COUNT),
                                          Key("rank", COUNT, default=None)), where))

    def to_dict(self) -> Dict[str, Any]:
        document = {"heads": self.heads, "dim": self.dim}
        if self.rank is not None:
            document["rank"] = self.rank
        return document


@dataclasses.dataclass(frozen=True)
class ParallelMixerConfig:
    left: WindowAttentionConfig
    right: TimeMixConfig
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, document: Mapping[str, Any], where: str) -> "ParallelMixerConfig":
        scales = read_keys(document, (Key("left_scale", FACTOR, default=1.0),
                                      Key("right_scale", FACTOR, default=1.0)), where)
        return cls(left=WindowAttentionConfig.from_dict(_object(document, "left", where),
                                                        where + "left."),
                   right=TimeMixConfig.from_dict(_object(document, "right", where),
                                                 where + "right."), **scales)

    def to_dict(self) -> Dict[str, Any]:
        return {"left": self.left.to_dict(), "right": self.right.to_dict(),
                "left_scale": self.left_scale, "right_scale": self.right_scale}


MIXER_CONFIGS = {"mamba2": StateSpaceMixerConfig, "parallel": ParallelMixerConfig}


@dataclasses.dataclass(frozen=True)
class ZuzadraLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[DenseMlpConfig]

    @classmethod
    def from_dict(cls, document: Any, index: int) -> "ZuzadraLayerConfig":
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
class ZuzadraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZuzadraLayerConfig, ...]
    streams: Optional[int] = None           # None: one residual, no hyper-connection weights
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
    def from_dict(cls, document: Mapping[str, Any]) -> "ZuzadraConfig":
        values = read_keys(document, (Key("vocab", COUNT), Key("width", COUNT),
                                      Key("streams", COUNT, default=None),
                                      Key("max_positions", COUNT, default=DEFAULT_MAX_POSITIONS)))
        eps = read_keys(_object(document, "norm"), (Key("eps", REAL),), "norm.")["eps"]
        layers = document.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config field 'layers' must be a list of layers")
        loop = document.get("loop")
        if loop is not None:
            if not isinstance(loop, dict) or not all(_whole(loop.get(k)) for k in ("start", "stop", "times")):
                raise ConfigError("config field 'loop' must give whole numbers start, stop, times")
            loop = LoopConfig(int(loop["start"]), int(loop["stop"]), int(loop["times"]))
        return cls(vocab=values["vocab"], width=values["width"], norm_eps=eps,
                   streams=values["streams"], loop=loop, max_positions=values["max_positions"],
                   layers=tuple(ZuzadraLayerConfig.from_dict(layer, index)
                                for index, layer in enumerate(layers)))

    def to_dict(self) -> Dict[str, Any]:
        document: Dict[str, Any] = {
            "architecture": self.architecture, "vocab": self.vocab, "width": self.width,
            "norm": {"eps": self.norm_eps},
            "layers": [layer.to_dict() for layer in self.layers],
        }
        if self.streams is not None:
            document["streams"] = self.streams
        if self.loop is not None:
            document["loop"] = dataclasses.asdict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            document["max_positions"] = self.max_positions
        return document

    def with_checkpoint_sizes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "ZuzadraConfig":
        """The configuration with the sizes it leaves open read from tensor shapes: the rank of
        a time-mixing layer's decay is the row count of ``l<i>.mix.right.w1``."""
        layers = []
        for index, layer in enumerate(self.layers):
            if layer.type == "parallel" and layer.mixer.right.rank is None:
                shape = shapes.get(f"l{index}.mix.right.w1")
                if shape is not None and len(shape) == 2:
                    right = dataclasses.replace(layer.mixer.right, rank=int(shape[0]))
                    layer = dataclasses.replace(
                        layer, mixer=dataclasses.replace(layer.mixer, right=right))
            layers.append(layer)
        return dataclasses.replace(self, layers=tuple(layers))

    @staticmethod
    def random_scale(name: str, shape: Tuple[int, ...]):
        """What a model with random weights holds in its vectors and small tables (None: ones):
        norm weights are stored around zero, streams are read evenly and mixed by the identity,
        state-space heads decay at rates from 1/16 to 1 with steps around 0.1, time-mix channels
        keep 0.95 of their state per token, blends take half of the previous token."""
        import math

        import torch
        leaf = name.rsplit(".", 1)[-1]
        if leaf in ("norm1", "norm2") or name in ("final.norm",) or leaf in ("b", "w0"):
            return {"w0": -3.0}.get(leaf, 0.0)
        if leaf == "in" and ".hc" in name:
            return 1.0 / shape[0]
        if leaf == "mix" and ".hc" in name:
            return torch.eye(shape[0])
        if leaf == "A_log":
            return torch.linspace(math.log(1.0 / 16.0), 0.0, shape[0])
        if leaf == "dt_bias":
            return -2.25
        if leaf == "conv":
            taps = torch.full(shape, 0.1)
            taps[:, -1] = 1.0
            return taps
        if leaf in ("r", "k", "v", "g", "w") and ".mu." in name:
            return 0.5
        if leaf in ("act", "u"):
            return 0.5
        return None

    def layer_runs(self) -> Tuple[int, ...]:
        """The layers in the order they run."""
        count = len(self.layers)
        if self.loop is None:
            return tuple(range(count))
        loop = self.loop
        return tuple(range(loop.start)) + tuple(range(loop.start, loop.stop)) * loop.times \
            + tuple(range(loop.stop, count))
