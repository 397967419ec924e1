"""Randomly drawn Rekasun configurations through the engine against the plain implementation:
heads, key/value heads, key and value sizes, taps, windows, kept keys, widths (also ones the
tensor-core products do not take), feed-forward sizes, layer counts and loops all vary, and
every model is replayed as mixed batches over a pool made for its live requests only."""
from __future__ import annotations

import math
import os

import numpy as np
import pytest
import torch

import plain_rekasun
import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200.weights.random_init import write_model_folder
from rekasun_configs import tensors_for

pytestmark = pytest.mark.gpu


def draw_config(seed: int) -> dict:
    rng = np.random.default_rng(1000 + seed)
    width = int(rng.choice([40, 64, 72, 100, 128, 136, 256]))
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        kv_heads = int(rng.choice([1, 2, 3, 4]))
        heads = kv_heads * int(rng.choice([1, 2, 4]))
        dim = int(rng.choice([8, 16, 24, 32, 48, 64, 96, 128]))
        vdim = int(rng.choice([dim, dim, 8, 16, 32, 64, 80]))
        window = int(rng.choice([1, 2, 5, 16, 17, 31, 40, 64, 90, 300]))
        keep = int(rng.choice([0, 0, 1, 3, 8, 16, 25, 70]))
        layers.append({
            "type": "attention",
            "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                      "conv": int(rng.choice([1, 2, 3, 4])), "scale": 2.0 / math.sqrt(dim),
                      "mask": {"size": window, "keep_first": keep}},
            "mlp": None if rng.random() < 0.2 else
            {"ff": int(rng.choice([48, 100, 128, 200, 384])), "kind": "dense"}})
    config = {"architecture": "Rekasun", "vocab": int(rng.choice([97, 256, 300])), "width": width,
              "embedding": {"scale": float(rng.choice([1.0, 0.5, 3.0]))},
              "norm": {"eps": float(rng.choice([1e-6, 1e-5, 1e-3]))}, "layers": layers}
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return config


def relative_error(got: np.ndarray, want: np.ndarray) -> float:
    difference = got.astype(np.float64) - want
    difference -= difference.mean(axis=-1, keepdims=True)
    spread = want - want.mean(axis=-1, keepdims=True)
    return float(np.sqrt((difference ** 2).mean(axis=-1)).max() / np.sqrt((spread ** 2).mean()))


@pytest.mark.parametrize("seed", range(int(os.environ.get("HELIX_SWEEP_SEEDS", "12"))))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration_in_mixed_batches(seed, dtype, model_root):
    config = draw_config(seed)
    folder = os.path.join(model_root, f"rekasun_sweep_{seed}_{dtype}")
    storage = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_model_folder(folder, config, tensors_for(config, 50 + seed, storage))
    plain = plain_rekasun.PlainRekasun(folder, precision=dtype)
    # every third model also gets a long request fed in long portions (the prompt kernels'
    # two-lane query tiles, windows that start beyond the first key tile)
    long_one = seed % 3 == 0
    lengths = (1, 7, 45, 130, 77) + ((700,) if long_one else ())
    requests = {f"r{index}": random_tokens(config["vocab"], length, seed=seed * 10 + index)
                for index, length in enumerate(lengths)}
    expected = {name: plain.logits(tokens) for name, tokens in requests.items()}
    steps = traces.mixed(requests, max_live=3, seed=seed,
                         chunk_choices=(2, 3, 7, 16, 33, 64) + ((300, 129) if long_one else ()))
    page = int(np.random.default_rng(seed).choice([8, 16]))
    pages = -(-traces.live_token_need(steps, round_to=page) // page)
    harness = Harness(folder, dtype, page, num_pages=pages, max_requests=3, max_tokens=1024)
    positions = {}
    worst = 0.0
    for step in steps:
        rows = traces.labels(step, positions)
        out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        for name in step["end"]:
            harness.end(name)
        want = np.stack([expected[name][position] for name, position in rows])
        if dtype == "float32":
            assert_close(out, want, f"seed {seed} step {step['step']} rows {rows[:3]}",
                         atol=5e-4, rtol=5e-4)
        else:
            assert np.isfinite(out).all()
            worst = max(worst, relative_error(out, want))
    harness.cache.check()
    assert not harness.cache.live_requests()
    # bfloat16: against the plain implementation that rounds where the engine stores, what is
    # left is a few per cent of the logits' spread at most (a wrong key or a lost state moves
    # them by their whole spread)
    assert worst < 0.06, f"seed {seed}: {worst:.3f} of the logits' spread"
