"""The Rekasun decoder as a list of parts.

A layer is a parallel block: one LayerNorm (weight and bias), whose output both the mixer and
the gated feed-forward (gelu_tanh) read, and one residual sum.  The mixer of ``type``
``attention`` is grouped-query attention without position encoding: q, k and v pass a short
causal filter over time right after their projection, scores are scaled by the layer's own
constant, a position sees the last ``mask.size`` positions and the first ``mask.keep_first``
ones, and the concatenated heads are gated with ``sigmoid(g h)`` before the output
projection.  The embedding is scaled by a constant.  A stretch of layers may run several
times in a row with the same weights (``loop``); every run of a layer owns its cache and
state, and the embedding's output is added to the residual stream before every repeat.
The model ends with a LayerNorm and an untied head.

Tensor names: ``embed``, ``l<i>.norm1`` (bias ``.b``), ``l<i>.mix.{q,k,v,g,o}``,
``l<i>.mix.{q,k,v}.conv``, ``l<i>.mlp.{gate,up,down}``, ``final.norm`` (bias ``.b``), ``head``.
"""
from __future__ import annotations

from typing import Callable, Dict

from ..config.registry import register_architecture
from ..config.rekasun import ARCHITECTURE, AttentionMixerConfig, RekasunConfig
from ..config.spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry


def _attention_mixer(prefix: str, mixer: AttentionMixerConfig) -> PartSpec:
    names = {name: f"{prefix}.mix.{name}" for name in ("q", "k", "v", "o", "g")}
    if mixer.conv > 1:
        names.update({f"{name}_conv": f"{prefix}.mix.{name}.conv" for name in ("q", "k", "v")})
    return PartSpec("paged_attention", {
        "num_heads": mixer.heads,
        "num_kv_heads": mixer.kv_heads,
        "head_dim": mixer.dim,
        "value_dim": mixer.vdim,
        "scale": mixer.scale,
        "window": mixer.window,
        "keep_first": mixer.keep_first,
        "short_conv": mixer.conv,
        "output_gate": "sigmoid",
        "position": PartSpec("none", {"head_dim": mixer.dim}),
    }, names)


# one builder per value of a layer's ``type``
MIXER_SPECS: Dict[str, Callable[[str, object], PartSpec]] = {"attention": _attention_mixer}


def build_rekasun_spec(config: RekasunConfig) -> ModelSpec:
    blocks = []
    for index, layer in enumerate(config.layers):
        prefix = f"l{index}"
        feed_forward = None
        if layer.mlp is not None:
            feed_forward = PartSpec("gated_mlp", {"intermediate_size": layer.mlp.ff,
                                                  "activation": "gelu_tanh"},
                                    {name: f"{prefix}.mlp.{name}" for name in ("gate", "up", "down")})
        blocks.append(BlockSpec(
            arrangement="parallel",
            mixer_norm=PartSpec("layer_norm", {"eps": config.norm_eps},
                                {"weight": f"{prefix}.norm1", "bias": f"{prefix}.norm1.b"}),
            mixer=MIXER_SPECS[layer.type](prefix, layer.mixer),
            feed_forward=feed_forward,
        ))
    return ModelSpec(
        architecture=config.architecture,
        hidden_size=config.width,
        vocab_size=config.vocab,
        max_positions=config.max_positions,
        embedding=PartSpec("token_table", {"vocab_size": config.vocab,
                                           "scale": config.embedding_scale}, {"weight": "embed"}),
        blocks=tuple(blocks),
        schedule=tuple(ScheduleEntry(block=layer, add_embedding=repeat)
                       for layer, repeat in config.layer_runs()),
        final_norm=PartSpec("layer_norm", {"eps": config.norm_eps},
                            {"weight": "final.norm", "bias": "final.norm.b"}),
        lm_head=PartSpec("linear", {"vocab_size": config.vocab, "tied": False}, {"weight": "head"}),
    )


register_architecture(ARCHITECTURE, RekasunConfig.from_dict, build_rekasun_spec,
                      aliases=("rekasun",))
