"""The Rekasun decoder through the engine's own model, cache manager and step function,
against the plain implementation: every way of cutting the same requests into steps gives
the plain logits at every position.  Pools are small, so pages and state slots are used again
(free pages are filled with NaN); windows give pages back while their kept first pages stay.
"""
from __future__ import annotations

import numpy as np
import pytest

import plain_rekasun
import traces
from conftest import random_tokens
from engine_harness import Harness, assert_close
from rekasun_configs import CONFIGS, PAGE_SIZE, make_folder

pytestmark = pytest.mark.gpu

LENGTHS = {"mixed": (1, 2, 9, 33, 90), "plain": (3, 17, 40, 75), "fast": (5, 70, 150, 310),
           "odd": (4, 11, 50, 120)}
CASES = [("mixed", "float32"), ("plain", "float32"), ("fast", "float32"), ("odd", "float32"),
         ("mixed", "bfloat16"), ("plain", "bfloat16"), ("fast", "bfloat16"), ("odd", "bfloat16")]
# float32: double against float32 sums.  bfloat16: the plain implementation rounds where the
# engine stores; what is left are activations that fall on the other side of a rounding
# boundary, which sharp attention carries into logits of spread one.
TOLERANCE = {"float32": dict(atol=3e-4, rtol=3e-4), "bfloat16": dict(atol=6e-2, rtol=3e-2)}


def make_requests(name: str, extra: int = 0):
    vocab = CONFIGS[name]["vocab"]
    return {f"r{index}": random_tokens(vocab, length + extra, seed=77 * len(name) + index)
            for index, length in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def models(model_root):
    cache = {}

    def get(name: str, dtype: str):
        if (name, dtype) not in cache:
            folder = make_folder(model_root, name, dtype)
            cache[(name, dtype)] = (folder, plain_rekasun.PlainRekasun(folder, precision=dtype))
        return cache[(name, dtype)]
    return get


@pytest.fixture(scope="module")
def expectations(models):
    cache = {}

    def get(name: str, dtype: str, extra: int = 0):
        if (name, dtype, extra) not in cache:
            plain = models(name, dtype)[1]
            cache[(name, dtype, extra)] = {request: plain.logits(tokens)
                                           for request, tokens in make_requests(name, extra).items()}
        return cache[(name, dtype, extra)]
    return get


def replay(harness: Harness, steps, expected, dtype: str, what: str):
    positions = {}
    for step in steps:
        rows = traces.labels(step, positions)
        out = harness.run([(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
        for name in step["end"]:
            harness.end(name)
        if rows:
            want = np.stack([expected[name][position] for name, position in rows])
            assert_close(out, want, f"{what} step {step['step']} rows {rows[:4]}...",
                         **TOLERANCE[dtype])
        harness.cache.check()
    assert not harness.cache.live_requests()


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_requests(name, dtype, models, expectations):
    harness = Harness(models(name, dtype)[0], dtype, PAGE_SIZE[name], num_pages=48)
    replay(harness, traces.whole(make_requests(name)), expectations(name, dtype), dtype,
           f"whole {name} {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_layers_of_different_sizes_keep_their_scratch(dtype, models):
    """Every layer's scratch buffers stay where they are from step to step (CUDA graphs point
    at them), also when the layers of a model differ in width."""
    harness = Harness(models("mixed", dtype)[0], dtype, PAGE_SIZE["mixed"], num_pages=48)
    tokens = make_requests("mixed")["r3"]
    harness.run([("a", tokens[:19], [18])])
    harness.run([("a", tokens[19:20], [0])])      # a portion and a single token: every path's buffers
    workspace = harness.step.workspace
    held, retired = workspace.bytes(), len(workspace._retired)
    for position in range(20, 30):
        harness.run([("a", tokens[position:position + 1], [0])])
    harness.run([("b", tokens[:17], [16])])
    harness.end("b")
    assert workspace.bytes() == held and len(workspace._retired) == retired
    harness.end("a")


@pytest.mark.parametrize("name,dtype", CASES)
def test_residual_stream_after_every_layer_run(name, dtype, models):
    folder, plain = models(name, dtype)
    harness = Harness(folder, dtype, PAGE_SIZE[name], num_pages=48)
    tokens = make_requests(name)["r3"]
    seen = []
    harness.model.after_entry = lambda index, rows: seen.append(rows.float().cpu().numpy().copy())
    harness.whole("a", tokens)
    states = plain.hidden_states(tokens)
    assert len(seen) == len(states)
    for index, (got, want) in enumerate(zip(seen, states)):
        spread = float(np.abs(want).max())
        tolerance = 2e-5 * spread if dtype == "float32" else 3e-2 * spread
        assert_close(got, want.astype(np.float32), f"{name} {dtype} layer run {index}",
                     atol=tolerance, rtol=0.0)


@pytest.mark.parametrize("name,dtype", CASES)
def test_tail_decoded_one_by_one(name, dtype, models, expectations):
    # 60 decoded tokens: every window of these models passes over decoded tokens
    harness = Harness(models(name, dtype)[0], dtype, PAGE_SIZE[name], num_pages=48)
    replay(harness, traces.tail_decoded(make_requests(name, extra=30), tail=60),
           expectations(name, dtype, 30), dtype, f"tail {name} {dtype}")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_changing_size(name, dtype, models, expectations):
    harness = Harness(models(name, dtype)[0], dtype, PAGE_SIZE[name], num_pages=48)
    replay(harness, traces.chunked(make_requests(name, extra=30)), expectations(name, dtype, 30),
           dtype, f"portions {name} {dtype}")


@pytest.mark.parametrize("name,dtype", CASES)
@pytest.mark.parametrize("seed", [0, 1])
def test_mixed_batches_over_a_small_pool(name, dtype, seed, models, expectations):
    requests = make_requests(name, extra=30)
    steps = traces.mixed(requests, max_live=3, seed=seed)
    page = PAGE_SIZE[name]
    pages = -(-traces.live_token_need(steps, round_to=page) // page)
    harness = Harness(models(name, dtype)[0], dtype, page, num_pages=pages, max_requests=3)
    replay(harness, steps, expectations(name, dtype, 30), dtype, f"mixed {name} {dtype}")
    stats = harness.cache.stats()
    assert all(group["reuses"] > 0 for group in stats["groups"]), "no page was used again"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_windowed_layer_needs_no_more_pages_than_its_window(dtype, models):
    """A long request over a pool that could never hold all of it: the windowed groups give
    pages back as the window passes them, the kept first pages stay, and the logits at the
    end are those of the whole sequence."""
    name = "mixed"
    folder, plain = models(name, dtype)
    tokens = random_tokens(CONFIGS[name]["vocab"], 200, seed=5)
    # the widest layer keeps 20 first keys (3 pages of 8) and sees 40 (6 pages) + the portion
    harness = Harness(folder, dtype, PAGE_SIZE[name], num_pages=14, max_requests=1)
    expected = plain.logits(tokens)
    cursor = 0
    for size in [13, 8, 8, 3, 11] * 10:
        size = min(size, len(tokens) - cursor)
        if size == 0:
            break
        out = harness.run([("long", tokens[cursor:cursor + size], range(size))])
        assert_close(out, expected[cursor:cursor + size], f"positions from {cursor}",
                     **TOLERANCE[dtype])
        cursor += size
        harness.cache.check()
    assert cursor == len(tokens)
    harness.end("long")


@pytest.mark.parametrize("name,dtype", [("mixed", "float32"), ("fast", "bfloat16")])
def test_greedy_generation_through_the_engine(name, dtype, models):
    """``Engine.generate``: scheduler, continuous batching, CUDA graphs and sampling, several
    requests at once.  Each generated token must be (within rounding) the best token of the
    plain logits for the sequence so far."""
    from helix_runtime_b200 import Engine
    folder, plain = models(name, dtype)
    vocab = CONFIGS[name]["vocab"]
    prompts = [random_tokens(vocab, length, seed=300 + length) for length in (3, 25, 61)]
    engine = Engine.from_pretrained(folder, dtype=dtype, page_size=PAGE_SIZE[name], num_pages=64,
                                    max_running_requests=3, max_tokens_per_iteration=64,
                                    max_prefill_chunk=24, poison_free_pages=True)
    results = engine.generate(prompts, max_new_tokens=24)
    slack = 1e-3 if dtype == "float32" else 0.12
    for prompt, result in zip(prompts, results):
        tokens = list(prompt)
        assert len(result.generated_tokens) == 24
        for token in result.generated_tokens:
            logits = plain.logits(tokens)[-1]
            assert logits[token] >= logits.max() - slack, \
                f"token {token} at position {len(tokens)} is not the plain model's choice"
            tokens.append(token)


@pytest.mark.parametrize("name,dtype", [("mixed", "float32"), ("fast", "bfloat16")])
def test_trace_replay_as_a_user_runs_it(name, dtype, models, expectations, tmp_path):
    """``bin/trace_run`` in a process of its own, fed a trace of mixed batches over a pool made
    for the live requests only; the logits it writes are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys

    from conftest import ROOT
    folder = models(name, dtype)[0]
    requests = make_requests(name, extra=30)
    expected = expectations(name, dtype, 30)
    steps = traces.mixed(requests, max_live=4, seed=7)
    out_dir = str(tmp_path / "out")
    process = subprocess.Popen(
        [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
         "--out", out_dir, "--max-tokens", str(traces.live_token_need(steps, 64))],
        stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, cwd=ROOT)
    try:
        positions = {}
        for step in steps:
            process.stdin.write(json.dumps(step) + "\n")
            process.stdin.flush()
            assert process.stdout.readline().strip() == f"done {step['step']}"
            rows = traces.labels(step, positions)
            data = np.fromfile(os.path.join(out_dir, f"{step['step']}.f32"), dtype="<f4")
            want = np.stack([expected[request][position] for request, position in rows])
            assert_close(data.reshape(want.shape), want, f"step {step['step']}", **TOLERANCE[dtype])
        process.stdin.close()
        assert process.wait(timeout=120) == 0
    finally:
        if process.poll() is None:
            process.kill()


def test_generation_from_the_command_line(models):
    """``bin/helix_generate`` chooses the model by ``config.json`` and prints the plain
    implementation's greedy tokens."""
    import os
    import subprocess
    import sys

    from conftest import ROOT
    folder, plain = models("mixed", "float32")
    prompt = random_tokens(CONFIGS["mixed"]["vocab"], 19, seed=3)
    done = subprocess.run(
        [sys.executable, os.path.join(ROOT, "bin", "helix_generate"), "--model", folder,
         "--dtype", "float32", "--max-new-tokens", "12", *[str(token) for token in prompt]],
        capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert done.returncode == 0, done.stderr
    lines = done.stdout.strip().splitlines()
    generated = [int(token) for token in lines[0].split(":")[1].split()]
    tokens = list(prompt)
    for token in generated:
        logits = plain.logits(tokens)[-1]
        assert logits[token] >= logits.max() - 1e-3
        tokens.append(token)
    assert len(generated) == 12 and lines[1] == "stop_reason: max_new_tokens"


@pytest.mark.parametrize("cuda_graphs", [False, True])
def test_the_next_turn_of_a_conversation_adopts_pages_kept_keys_and_filter_state(models, cuda_graphs):
    """Prefix sharing: a later prompt that goes on from an earlier one adopts the pages its
    windows still reach, the kept first pages, and the filters' state as it stood at the
    prefix's end, and computes only what is new; its tokens are the plain implementation's."""
    from helix_runtime_b200 import Engine
    folder, plain = models("mixed", "float32")
    vocab = CONFIGS["mixed"]["vocab"]
    engine = Engine.from_pretrained(folder, dtype="float32", page_size=8, num_pages=96,
                                    max_running_requests=3, max_tokens_per_iteration=32,
                                    max_prefill_chunk=11, cuda_graphs=cuda_graphs,
                                    prefix_cache_entries=4, poison_free_pages=True)

    def check(prompt, result):
        logits = plain.logits(prompt + result.generated_tokens[:-1])
        for index, token in enumerate(result.generated_tokens):
            row = logits[len(prompt) + index - 1]
            assert row[token] >= row.max() - 1e-3, f"token {index}"

    first = random_tokens(vocab, 45, seed=41)                 # its prefix: 40 tokens
    one = engine.generate([first], max_new_tokens=6)[0]
    check(first, one)
    second = first + one.generated_tokens + random_tokens(vocab, 30, seed=42)
    other = random_tokens(vocab, 13, seed=43)
    two, beside = engine.generate([second, other], max_new_tokens=8)
    check(second, two)
    check(other, beside)
    assert engine.request(two.request_id).reused_tokens == 40
    assert engine.request(beside.request_id).reused_tokens == 0
    engine.cache.check()
    engine.prefix.clear()
    engine.cache.check()
    assert all(group.pool.pages_in_use == 0 for group in engine.cache.groups)
