"""Small Zuzadra configurations for the tests and how their model folders are made.

They differ in every size and constant, and inside a model the layers differ too:

* ``streams3``: three residual streams; a state-space layer with two groups, a 3-tap filter and
  its output normed in two parts; a parallel layer with grouped key/value heads, a window of
  24 that spans pages of 8, half of the head rotated, unequal scales; a state-space layer
  without a feed-forward; layers 1 and 2 run three times.
* ``single``: no streams key (one residual, layer scale only), width 120; a parallel layer with
  one key/value head, the whole head rotated with interleaved pairs, a window (7) smaller than
  a page, scales of one; a state-space layer with a filter of one tap (none) and a state of 24
  rows (no power of two); no loop.
* ``fast``: the shapes the tensor-core kernels take (width 256, heads of 64, feed-forward 512),
  two streams, sharp attention (scores spread by about six) over a window of 44, prompts of
  hundreds of tokens, the parallel layer run twice.
* ``recurrent``: state-space layers only (no keys or values anywhere, so the cache manager has
  no pages to hand out), one residual stream WITH connection weights, a state of one row in its
  second layer, the first layer run twice.
* ``odd``: sizes no fast kernel takes: width 90, five streams, heads of 20 with values of 12, a
  time-mix head of 12 (three heads), a decay rank of 5, a filter of five taps, an odd
  vocabulary, one stream count that is no power of two, a loop that runs once.

Weights are drawn so that nothing is trivial: attention is sharp, some state-space heads and
time-mix channels decay slowly (far tokens matter) and some fast, filters and biases are not
zero, norm weights are not one, streams mix.
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from helix_runtime_b200.weights.random_init import write_model_folder


def _ssm(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state,
                                        "groups": groups, "conv": conv, "norm_groups": norm_groups}}


def _parallel(heads, kv_heads, dim, vdim, window, rot_dims, base, right_heads, right_dim,
              left_scale, right_scale, layout=None, sharp=2.0):
    rot = {"base": base, "dims": rot_dims}
    if layout is not None:
        rot["layout"] = layout
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                 "scale": sharp / math.sqrt(dim), "mask": {"size": window}, "rot": rot},
        "right": {"heads": right_heads, "dim": right_dim},
        "left_scale": left_scale, "right_scale": right_scale}}


def _layer(mixer, ff):
    return dict(mixer, mlp=None if ff is None else {"ff": ff, "kind": "dense"})


CONFIGS = {
    "streams3": {
        "architecture": "Zuzadra", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "streams": 3,
        "layers": [_layer(_ssm(4, 16, 16, groups=2, conv=3, norm_groups=2), 96),
                   _layer(_parallel(4, 2, 16, 8, 24, 8, 10000.0, 2, 16, 0.7, 1.3), 80),
                   _layer(_ssm(2, 24, 8, conv=2), None)],
        "loop": {"start": 1, "stop": 3, "times": 3},
    },
    "single": {
        "architecture": "Zuzadra", "vocab": 333, "width": 120, "norm": {"eps": 1e-6},
        "layers": [_layer(_parallel(5, 1, 24, 24, 7, 24, 500.0, 5, 8, 1.0, 1.0,
                                    layout="interleaved"), 200),
                   _layer(_ssm(3, 20, 24, conv=1), 144)],
    },
    "fast": {
        "architecture": "Zuzadra", "vocab": 512, "width": 256, "norm": {"eps": 1e-5}, "streams": 2,
        "layers": [_layer(_ssm(8, 32, 64, groups=2, conv=4, norm_groups=4), 512),
                   _layer(_parallel(4, 2, 64, 64, 44, 32, 100000.0, 4, 64, 0.5, 0.9, sharp=6.0), 512),
                   _layer(_ssm(4, 64, 32, conv=4), 512)],
        "loop": {"start": 1, "stop": 2, "times": 2},
    },
    "recurrent": {
        "architecture": "Zuzadra", "vocab": 150, "width": 48, "norm": {"eps": 1e-5}, "streams": 1,
        "layers": [_layer(_ssm(3, 8, 12, conv=3), 64),
                   _layer(_ssm(2, 16, 1, groups=2, conv=2, norm_groups=2), None)],
        "loop": {"start": 0, "stop": 1, "times": 2},
    },
    "odd": {
        "architecture": "Zuzadra", "vocab": 131, "width": 90, "norm": {"eps": 1e-4}, "streams": 5,
        "layers": [_layer(_parallel(3, 3, 20, 12, 33, 10, 77.0, 3, 12, 1.5, 0.4), 70),
                   _layer(_ssm(5, 6, 40, groups=5, conv=5, norm_groups=3), 50)],
        "loop": {"start": 1, "stop": 2, "times": 1},
    },
}
PAGE_SIZE = {"streams3": 8, "single": 16, "fast": 16, "odd": 8, "recurrent": 16}
SEED = {"streams3": 21, "single": 22, "fast": 23, "odd": 24, "recurrent": 25}
DECAY_RANK = {"streams3": 8, "single": 16, "fast": 32, "odd": 5, "recurrent": 1}


def tensors_for(config: dict, seed: int, storage_dtype: torch.dtype, decay_rank: int):
    rng = np.random.default_rng(seed)
    width = config["width"]
    streams = config.get("streams")

    def matrix(rows, columns, gain=1.0):
        return torch.tensor(rng.normal(size=(rows, columns)) * gain / math.sqrt(columns),
                            dtype=torch.float32).to(storage_dtype)

    def vector(size, mean, spread):
        return torch.tensor(mean + spread * rng.normal(size=size), dtype=torch.float32) \
            .to(storage_dtype)

    def uniform(size, low, high):
        return torch.tensor(rng.uniform(low, high, size=size), dtype=torch.float32).to(storage_dtype)

    tensors = {"embed": matrix(config["vocab"], width, math.sqrt(width)),
               "final.norm": vector(width, 0.0, 0.2), "head": matrix(config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}", layer["mixer"]
        for which in (1, 2):
            if which == 2 and layer["mlp"] is None:
                continue
            tensors[f"{prefix}.norm{which}"] = vector(width, 0.0, 0.2)
            tensors[f"{prefix}.ls{which}"] = vector(width, 0.6, 0.15)
            if streams is not None:
                tensors[f"{prefix}.hc{which}.in"] = vector(streams, 1.0 / streams, 0.2)
                tensors[f"{prefix}.hc{which}.out"] = vector(streams, 0.8, 0.3)
                tensors[f"{prefix}.hc{which}.mix"] = torch.tensor(
                    0.9 * np.eye(streams) + 0.15 * rng.normal(size=(streams, streams)),
                    dtype=torch.float32).to(storage_dtype)
        if layer["type"] == "mamba2":
            heads, vdim, state, groups = (mixer[k] for k in ("heads", "vdim", "state", "groups"))
            inner, channels = heads * vdim, heads * vdim + 2 * groups * state
            tensors[f"{prefix}.mix.in"] = matrix(2 * inner + 2 * groups * state + heads, width)
            taps = rng.normal(size=(channels, mixer["conv"])) * 0.4
            taps[:, -1] += 1.0
            tensors[f"{prefix}.mix.conv"] = torch.tensor(taps, dtype=torch.float32).to(storage_dtype)
            tensors[f"{prefix}.mix.conv.b"] = vector(channels, 0.0, 0.2)
            tensors[f"{prefix}.mix.dt_bias"] = uniform(heads, -3.0, 0.5)
            # slow and fast heads: rates from 0.02 to 4
            tensors[f"{prefix}.mix.A_log"] = uniform(heads, math.log(0.02), math.log(4.0))
            tensors[f"{prefix}.mix.D"] = vector(heads, 1.0, 0.3)
            tensors[f"{prefix}.mix.norm"] = vector(inner, 1.0, 0.2)
            tensors[f"{prefix}.mix.o"] = matrix(width, inner, 0.7)
        else:
            left, right = mixer["left"], mixer["right"]
            tensors[f"{prefix}.mix.left.q"] = matrix(left["heads"] * left["dim"], width)
            tensors[f"{prefix}.mix.left.k"] = matrix(left["kv_heads"] * left["dim"], width)
            tensors[f"{prefix}.mix.left.v"] = matrix(left["kv_heads"] * left["vdim"], width)
            tensors[f"{prefix}.mix.left.q.norm"] = vector(left["dim"], 1.0, 0.2)
            tensors[f"{prefix}.mix.left.k.norm"] = vector(left["dim"], 1.0, 0.2)
            tensors[f"{prefix}.mix.left.o"] = matrix(width, left["heads"] * left["vdim"], 0.7)
            a = right["heads"] * right["dim"]
            for s in "rkvgw":
                tensors[f"{prefix}.mix.right.mu.{s}"] = uniform(width, 0.0, 1.0)
            for s in "rkvg":
                tensors[f"{prefix}.mix.right.{s}"] = matrix(a, width)
            tensors[f"{prefix}.mix.right.w1"] = matrix(decay_rank, width)
            tensors[f"{prefix}.mix.right.w2"] = matrix(a, decay_rank, 0.5)
            # decays from 0.999 (exp(-exp(-7))) to 0.2 (exp(-exp(0.5)))
            tensors[f"{prefix}.mix.right.w0"] = uniform(a, -7.0, 0.5)
            tensors[f"{prefix}.mix.right.u"] = torch.tensor(
                0.5 + 0.3 * rng.normal(size=(right["heads"], right["dim"])),
                dtype=torch.float32).to(storage_dtype)
            tensors[f"{prefix}.mix.right.norm"] = vector(a, 1.0, 0.2)
            tensors[f"{prefix}.mix.right.o"] = matrix(width, a, 0.7)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            tensors[f"{prefix}.mlp.up"] = matrix(ff, width, 1.5)
            tensors[f"{prefix}.mlp.up.b"] = vector(ff, 0.0, 0.3)
            tensors[f"{prefix}.mlp.down"] = matrix(width, ff, 0.5)
            tensors[f"{prefix}.mlp.down.b"] = vector(width, 0.0, 0.2)
            tensors[f"{prefix}.mlp.act"] = vector(2, 0.3, 0.5)
    return tensors


def make_folder(directory: str, name: str, storage_dtype: str = "float32") -> str:
    path = os.path.join(directory, f"zuzadra_{name}_{storage_dtype}")
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        dtype = torch.bfloat16 if storage_dtype == "bfloat16" else torch.float32
        write_model_folder(path, CONFIGS[name],
                           tensors_for(CONFIGS[name], SEED[name], dtype, DECAY_RANK[name]))
    return path
