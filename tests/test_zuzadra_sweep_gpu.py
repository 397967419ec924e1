"""Randomly drawn Zuzadra configurations through the engine against the plain implementation:
stream counts (and none), the order and number of layers, loops, every size of both mixers
(heads, groups, state rows, head widths, taps, norm groups; query, key/value and value sizes,
windows, rotated coordinates, pair layouts; time-mix heads and ranks), widths the tensor-core
products do not take, feed-forward sizes and constants all vary, and every model is replayed as
mixed batches over a pool made for its live requests only."""
from __future__ import annotations

import math
import os

import numpy as np
import pytest
import torch

import plain_zuzadra
import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close
from helix_runtime_b200.weights.random_init import write_model_folder
from zuzadra_configs import tensors_for

pytestmark = pytest.mark.gpu


def draw_config(seed: int):
    rng = np.random.default_rng(2000 + seed)
    pick = lambda values: values[int(rng.integers(0, len(values)))]
    width = pick([40, 64, 72, 100, 128, 136, 256])
    layers = []
    for _ in range(int(rng.integers(1, 5))):
        if rng.random() < 0.5:
            groups = pick([1, 1, 2, 3])
            heads = groups * pick([1, 2, 4])
            vdim = pick([4, 8, 12, 16, 20, 32, 64])
            norm_groups = pick([g for g in (1, 2, 3, 4, heads) if (heads * vdim) % g == 0])
            mixer = {"type": "mamba2", "mixer": {
                "heads": heads, "vdim": vdim, "state": pick([1, 4, 8, 16, 17, 24, 32, 48, 64, 130]),
                "groups": groups, "conv": pick([1, 2, 3, 4, 6]), "norm_groups": norm_groups}}
        else:
            kv_heads = pick([1, 2, 3, 4])
            heads = kv_heads * pick([1, 2, 4])
            dim = pick([8, 16, 24, 32, 48, 64, 96, 128])
            vdim = pick([dim, dim, 8, 16, 32, 64, 80])
            rot = {"base": float(pick([100.0, 10000.0, 250000.0])),
                   "dims": pick([d for d in (2, 4, 8, dim // 2, dim) if d % 2 == 0 and d <= dim])}
            if rng.random() < 0.3:
                rot["layout"] = "interleaved"
            mixer = {"type": "parallel", "mixer": {
                "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                         "scale": pick([1.0, 2.0, 4.0]) / math.sqrt(dim),
                         "mask": {"size": pick([1, 2, 5, 16, 17, 31, 40, 64, 90, 300])}, "rot": rot},
                "right": {"heads": pick([1, 2, 3, 5]), "dim": pick([4, 8, 16, 20, 32, 64, 72])},
                "left_scale": float(pick([1.0, 0.5, 1.7])), "right_scale": float(pick([1.0, 0.3, 1.2]))}}
        mixer["mlp"] = None if rng.random() < 0.2 else \
            {"ff": pick([48, 100, 128, 200, 384]), "kind": "dense"}
        layers.append(mixer)
    config = {"architecture": "Zuzadra", "vocab": pick([97, 256, 300]), "width": width,
              "norm": {"eps": float(pick([1e-6, 1e-5, 1e-3]))}, "layers": layers}
    streams = pick([None, 1, 2, 3, 4, 7])
    if streams is not None:
        config["streams"] = streams
    if rng.random() < 0.7:
        start = int(rng.integers(0, len(layers)))
        stop = int(rng.integers(start + 1, len(layers) + 1))
        config["loop"] = {"start": start, "stop": stop, "times": int(rng.integers(1, 4))}
    return config, pick([3, 8, 16, 40])


def relative_error(got: np.ndarray, want: np.ndarray) -> np.ndarray:
    """Per row: the root mean square of the difference (its mean taken off) over the spread of
    the wanted logits."""
    difference = got.astype(np.float64) - want
    difference -= difference.mean(axis=-1, keepdims=True)
    spread = want - want.mean(axis=-1, keepdims=True)
    return np.sqrt((difference ** 2).mean(axis=-1)) / np.sqrt((spread ** 2).mean())


@pytest.mark.parametrize("seed", range(int(os.environ.get("HELIX_SWEEP_SEEDS", "12"))))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_configuration_in_mixed_batches(seed, dtype, model_root):
    config, rank = draw_config(seed)
    folder = os.path.join(model_root, f"zuzadra_sweep_{seed}_{dtype}")
    storage = torch.bfloat16 if dtype == "bfloat16" else torch.float32
    write_model_folder(folder, config, tensors_for(config, 70 + seed, storage, rank))
    plain = plain_zuzadra.PlainZuzadra(folder, precision=dtype)
    # every third model also gets a long request fed in long portions
    long_one = seed % 3 == 0
    lengths = (1, 7, 45, 130, 77) + ((500,) if long_one else ())
    requests = {f"r{index}": random_tokens(config["vocab"], length, seed=seed * 10 + index)
                for index, length in enumerate(lengths)}
    expected = {name: plain.logits(tokens) for name, tokens in requests.items()}
    # bfloat16: how far rounding the activations moves each row of the plain logits; a few
    # positions of some models are ill-conditioned (a group whose root mean square is small),
    # and there the engine may differ by a multiple of that, elsewhere by some per cent of the
    # logits' spread (a wrong key or a lost state moves them by their whole spread)
    moved = {}
    if dtype == "bfloat16":
        exact = plain_zuzadra.PlainZuzadra(folder, precision="float32")
        moved = {name: relative_error(expected[name], exact.logits(tokens).astype(np.float64))
                 for name, tokens in requests.items()}
    steps = traces.mixed(requests, max_live=3, seed=seed,
                         chunk_choices=(2, 3, 7, 16, 33, 64) + ((300, 129) if long_one else ()))
    page = int(np.random.default_rng(seed).choice([8, 16]))
    pages = -(-traces.live_token_need(steps, round_to=page) // page)
    harness = Harness(folder, dtype, page, num_pages=pages, max_requests=3, max_tokens=1024)
    positions = {}
    for step in steps:
        rows = traces.labels(step, positions)
        out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        for name in step["end"]:
            harness.end(name)
        want = np.stack([expected[name][position] for name, position in rows])
        if dtype == "float32":
            assert_close(out, want, f"seed {seed} step {step['step']} rows {rows[:3]}",
                         atol=6e-4, rtol=6e-4)
        else:
            assert np.isfinite(out).all()
            error = relative_error(out, want.astype(np.float64))
            allowed = np.array([max(0.08, 4.0 * moved[name][position]) for name, position in rows])
            bad = np.nonzero(error > allowed)[0]
            assert bad.size == 0, (f"seed {seed} step {step['step']}: row {rows[bad[0]]} differs by "
                                   f"{error[bad[0]]:.3f} of the logits' spread, allowed "
                                   f"{allowed[bad[0]]:.3f}")
    harness.cache.check()
    assert not harness.cache.live_requests()
