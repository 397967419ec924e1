"""The Zuzadra decoder as a list of parts.

A layer is pre-norm over residual streams: each sublayer (mixer, then feed-forward) reads a
weighted sum of the streams through an RMS norm whose weight is stored around zero
(``1 + w``), its output is multiplied by a per-channel layer scale, and all streams are
rewritten from the old ones and that output (hyper-connections; without ``streams`` in the
configuration there is one residual and only the layer scale).  Mixers: ``mamba2``, a
selective state-space layer; ``parallel``, a sliding-window attention (per-head query/key
norm, partial rotary encoding, values rotated by their position and the output turned back)
beside a time-mixing layer with a decayed outer-product state, summed with two constants.
The feed-forward is two matrices with biases around the xIELU activation.  A stretch of
layers may run several times with the same weights (``loop``); every run owns its cache and
state.  The model ends with the same kind of norm over the sum of the streams and an untied
head.

Tensor names: ``embed``; per layer ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``,
``l<i>.hc{1,2}.{in,out,mix}``; ``l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}`` (mamba2);
``l<i>.mix.left.{q,k,v,o,q.norm,k.norm}`` and ``l<i>.mix.right.{mu.{r,k,v,g,w},r,k,v,g,w1,w2,
w0,u,norm,o}`` (parallel; the rank of the decay's two small matrices is read from the
checkpoint); ``l<i>.mlp.{up,up.b,down,down.b,act}``; ``final.norm``, ``head``.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

from ..config.errors import ConfigError
from ..config.registry import register_architecture
from ..config.spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry
from ..config.zuzadra import (ARCHITECTURE, ParallelMixerConfig, StateSpaceMixerConfig,
                              ZuzadraConfig)

PAIRING_OF_LAYOUT = {"halves": "half_split", "interleaved": "adjacent"}


def _state_space_mixer(prefix: str, mixer: StateSpaceMixerConfig, config: ZuzadraConfig) -> PartSpec:
    roles = {"in": "in", "filter": "conv", "filter_bias": "conv.b", "dt_bias": "dt_bias",
             "a_log": "A_log", "skip": "D", "norm": "norm", "o": "o"}
    return PartSpec("state_space", {
        "heads": mixer.heads, "head_width": mixer.vdim, "state_size": mixer.state,
        "groups": mixer.groups, "filter_taps": mixer.conv, "norm_groups": mixer.norm_groups,
        "eps": config.norm_eps,
    }, {role: f"{prefix}.mix.{name}" for role, name in roles.items()})


def _parallel_mixer(prefix: str, mixer: ParallelMixerConfig, config: ZuzadraConfig) -> PartSpec:
    left, right = mixer.left, mixer.right
    pairing = PAIRING_OF_LAYOUT[left.rot_layout]
    position = PartSpec("computed_rotary", {
        "theta": left.rot_base, "head_dim": left.dim, "rotary_dim": left.rot_dims,
        "pairing": pairing, "qk_norm": True, "eps": config.norm_eps,
        "rotate_values": True, "value_dim": left.vdim,
    }, {"q_norm": f"{prefix}.mix.left.q.norm", "k_norm": f"{prefix}.mix.left.k.norm"})
    attention = PartSpec("paged_attention", {
        "num_heads": left.heads, "num_kv_heads": left.kv_heads, "head_dim": left.dim,
        "value_dim": left.vdim, "scale": left.scale, "window": left.window,
        "position": position,
    }, {name: f"{prefix}.mix.left.{name}" for name in ("q", "k", "v", "o")})
    names = {f"mu_{s}": f"{prefix}.mix.right.mu.{s}" for s in ("r", "k", "v", "g", "w")}
    names.update({name: f"{prefix}.mix.right.{name}"
                  for name in ("r", "k", "v", "g", "w1", "w2", "w0", "norm", "o")})
    names["bonus"] = f"{prefix}.mix.right.u"
    if right.rank is None:
        raise ConfigError(f"layer {prefix}: the rank of the decay's small matrices is neither in "
                          "the configuration ('rank') nor read from a checkpoint")
    time_mix = PartSpec("time_mix", {
        "heads": right.heads, "head_dim": right.dim, "eps": config.norm_eps,
        "decay_rank": right.rank,
    }, names)
    return PartSpec("side_by_side", {"mixers": (attention, time_mix),
                                     "scales": (mixer.left_scale, mixer.right_scale)})


# one builder per value of a layer's ``type``
MIXER_SPECS: Dict[str, Callable[[str, object, ZuzadraConfig], PartSpec]] = {
    "mamba2": _state_space_mixer, "parallel": _parallel_mixer}


def _connection(config: ZuzadraConfig, prefix: str, which: int) -> PartSpec:
    names = {"scale": f"{prefix}.ls{which}"}
    weighted = config.streams is not None
    if weighted:
        names.update({"read": f"{prefix}.hc{which}.in", "write": f"{prefix}.hc{which}.out",
                      "mixing": f"{prefix}.hc{which}.mix"})
    return PartSpec("streams", {"streams": config.streams or 1, "weighted": weighted,
                                "layer_scale": True}, names)


def build_zuzadra_spec(config: ZuzadraConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("rms", {"eps": config.norm_eps, "one_plus": True}, {"weight": name})

    blocks = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        feed_forward = feed_forward_norm = feed_forward_connection = None
        if layer.mlp is not None:
            feed_forward = PartSpec("dense_mlp", {"intermediate_size": layer.mlp.ff,
                                                  "activation": "xielu", "bias": True},
                                    {"up": f"{prefix}.mlp.up", "up_bias": f"{prefix}.mlp.up.b",
                                     "down": f"{prefix}.mlp.down",
                                     "down_bias": f"{prefix}.mlp.down.b",
                                     "act": f"{prefix}.mlp.act"})
            feed_forward_norm = norm(f"{prefix}.norm2")
            feed_forward_connection = _connection(config, prefix, 2)
        blocks.append(BlockSpec(
            arrangement="streams",
            mixer_norm=norm(f"{prefix}.norm1"),
            mixer=MIXER_SPECS[layer.type](prefix, layer.mixer, config),
            feed_forward_norm=feed_forward_norm,
            feed_forward=feed_forward,
            mixer_connection=_connection(config, prefix, 1),
            feed_forward_connection=feed_forward_connection,
        ))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": config.vocab}, {"weight": "embed"}),
        blocks=tuple(blocks),
        schedule=tuple(ScheduleEntry(block=layer) for layer in config.layer_runs()),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear", {"vocab_size": config.vocab, "tied": False}, {"weight": "head"}),
        streams=config.streams or 1,
    )


register_architecture(ARCHITECTURE, ZuzadraConfig.from_dict, build_zuzadra_spec,
                      aliases=("zuzadra",),
                      sizes_from_checkpoint=ZuzadraConfig.with_checkpoint_sizes)
