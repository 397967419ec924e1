"""Small Rekasun configurations for the tests and how their model folders are made.

They differ in every size and constant, and inside a model the layers differ too:

* ``mixed``: three layers of different shapes (so three cache groups): grouped heads with a
  3-tap filter, a window of 24 and 4 kept keys; equal query and key/value heads whose values
  are twice as wide as their keys, a 2-tap filter, a window (7) smaller than a page, nothing
  kept and no feed-forward; one key/value head with values half as wide as the keys, a 4-tap
  filter and more kept keys (20) than a page holds.  Layers 0 and 1 run three times.
* ``plain``: width 120 (heads of 24, held in rows of 32), no filter in its first layer, a
  window longer than any test sequence, no loop, embedding scale 1; a second layer whose
  kept keys cover its whole window.
* ``fast``: the shapes the tensor-core kernels are built for (width 256, heads of 64, a
  feed-forward of 512, pages of 16), a window of 48 with 8 kept keys, the middle layer run
  twice, prompts of hundreds of tokens.

* ``odd``: sizes the fast kernels do not take: a width (90) that is no multiple of 8, heads
  of 20 with values of 12, five filter taps, an odd vocabulary, a loop that runs once.

Weights are drawn so that attention is sharp (scores spread by about two), filters and
biases are not trivial, and norm weights are not one.
"""
from __future__ import annotations

import math
import os

import numpy as np
import torch

from helix_runtime_b200.weights.random_init import write_model_folder


def _attention(heads, kv_heads, dim, vdim, conv, size, keep_first):
    return {"type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv,
                      "scale": 2.0 / math.sqrt(dim), "mask": {"size": size, "keep_first": keep_first}}}


def _layer(mixer, ff):
    return dict(mixer, mlp=None if ff is None else {"ff": ff, "kind": "dense"})


CONFIGS = {
    "mixed": {
        "architecture": "Rekasun", "vocab": 200, "width": 64,
        "embedding": {"scale": 2.5}, "norm": {"eps": 1e-5},
        "layers": [_layer(_attention(4, 2, 16, 16, 3, 24, 4), 96),
                   _layer(_attention(4, 4, 16, 32, 2, 7, 0), None),
                   _layer(_attention(2, 1, 32, 16, 4, 40, 20), 80)],
        "loop": {"start": 0, "stop": 2, "times": 3},
    },
    "plain": {
        "architecture": "Rekasun", "vocab": 333, "width": 120,
        "embedding": {"scale": 1.0}, "norm": {"eps": 1e-6},
        "layers": [_layer(_attention(5, 5, 24, 24, 1, 1000, 0), 200),
                   _layer(_attention(5, 1, 24, 24, 3, 16, 16), 144)],
    },
    "fast": {
        "architecture": "Rekasun", "vocab": 512, "width": 256,
        "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
        "layers": [_layer(_attention(4, 2, 64, 64, 3, 48, 8), 512),
                   _layer(_attention(4, 2, 64, 64, 3, 48, 8), 512),
                   _layer(_attention(4, 4, 64, 64, 2, 100, 0), 512)],
        "loop": {"start": 1, "stop": 2, "times": 2},
    },
    "odd": {
        "architecture": "Rekasun", "vocab": 131, "width": 90,
        "embedding": {"scale": 0.7}, "norm": {"eps": 1e-4},
        "layers": [_layer(_attention(3, 3, 20, 12, 5, 33, 1), 70),
                   _layer(_attention(6, 2, 20, 12, 5, 33, 1), 50)],
        "loop": {"start": 1, "stop": 2, "times": 1},
    },
}
PAGE_SIZE = {"mixed": 8, "plain": 16, "fast": 16, "odd": 8}
SEED = {"mixed": 11, "plain": 12, "fast": 13, "odd": 14}


def tensors_for(config: dict, seed: int, storage_dtype: torch.dtype):
    rng = np.random.default_rng(seed)
    width = config["width"]

    def matrix(rows, columns, gain=1.0):
        return torch.tensor(rng.normal(size=(rows, columns)) * gain / math.sqrt(columns),
                            dtype=torch.float32).to(storage_dtype)

    def vector(size, mean, spread):
        return torch.tensor(mean + spread * rng.normal(size=size), dtype=torch.float32)

    tensors = {"embed": matrix(config["vocab"], width, math.sqrt(width)),
               "final.norm": vector(width, 1.0, 0.2), "final.norm.b": vector(width, 0.0, 0.2),
               "head": matrix(config["vocab"], width)}
    for index, layer in enumerate(config["layers"]):
        prefix, mixer = f"l{index}", layer["mixer"]
        q_rows, k_rows = mixer["heads"] * mixer["dim"], mixer["kv_heads"] * mixer["dim"]
        v_rows, o_columns = mixer["kv_heads"] * mixer["vdim"], mixer["heads"] * mixer["vdim"]
        tensors[f"{prefix}.norm1"] = vector(width, 1.0, 0.2)
        tensors[f"{prefix}.norm1.b"] = vector(width, 0.0, 0.2)
        tensors[f"{prefix}.mix.q"] = matrix(q_rows, width)
        tensors[f"{prefix}.mix.k"] = matrix(k_rows, width)
        tensors[f"{prefix}.mix.v"] = matrix(v_rows, width)
        tensors[f"{prefix}.mix.g"] = matrix(o_columns, width, 2.0)
        tensors[f"{prefix}.mix.o"] = matrix(width, o_columns, 0.5)
        if mixer["conv"] > 1:
            for name, rows in (("q", q_rows), ("k", k_rows), ("v", v_rows)):
                taps = rng.normal(size=(rows, mixer["conv"])) * 0.5
                taps[:, -1] += 1.0
                tensors[f"{prefix}.mix.{name}.conv"] = torch.tensor(taps, dtype=torch.float32) \
                    .to(storage_dtype)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            tensors[f"{prefix}.mlp.gate"] = matrix(ff, width, 1.5)
            tensors[f"{prefix}.mlp.up"] = matrix(ff, width)
            tensors[f"{prefix}.mlp.down"] = matrix(width, ff, 0.5)
    return tensors


def make_folder(directory: str, name: str, storage_dtype: str = "float32") -> str:
    path = os.path.join(directory, f"rekasun_{name}_{storage_dtype}")
    if not os.path.exists(os.path.join(path, "model.safetensors")):
        dtype = torch.bfloat16 if storage_dtype == "bfloat16" else torch.float32
        write_model_folder(path, CONFIGS[name], tensors_for(CONFIGS[name], SEED[name], dtype))
    return path
