"""The kernels behind the Zuzadra mechanisms, one at a time, against the plain functions of
``plain_zuzadra`` (NumPy, double): residual streams, the biased activation, the causal filter,
both recurrences (whole sequences, and cut into portions that carry their state), the token
shift, the gated group norm, and the rotation from positions with normed heads and rotated
values.  Sizes are ones the models of the other tests do not have.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_zuzadra as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def device_tensor(array, dtype=torch.float32):
    return torch.tensor(np.asarray(array), dtype=torch.float32).to(dtype).cuda().contiguous()


def as_double(tensor):
    return tensor.float().cpu().numpy().astype(np.float64)


def batch(lengths, slots):
    """Device description of one step: request r brings lengths[r] tokens and owns slots[r]."""
    starts = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int32)
    token_request = np.concatenate([np.full(n, r) for r, n in enumerate(lengths)]).astype(np.int32)
    make = lambda a: torch.tensor(np.asarray(a, dtype=np.int32)).cuda()
    return make(token_request), make(slots), make(starts)


def close(got, want, atol, rtol=0.0):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape
    assert np.isfinite(got).all()
    error = np.abs(got - want)
    assert (error <= atol + rtol * np.abs(want)).all(), \
        f"worst error {error.max():.3e} at {np.unravel_index(error.argmax(), error.shape)}"


# ----------------------------------------------------------------- residual streams

@pytest.mark.parametrize("streams", [1, 3, 6])
@pytest.mark.parametrize("dtype", DTYPES)
def test_streams_read_norm_and_write(streams, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(streams)
    tokens, hidden, eps = 7, 52, 1e-5
    x = rng.normal(size=(tokens, streams, hidden))
    read, write = rng.normal(size=streams), rng.normal(size=streams)
    mixing = rng.normal(size=(streams, streams))
    weight, scale = rng.normal(size=hidden), rng.normal(size=hidden)
    y = rng.normal(size=(tokens, hidden))
    d_streams = device_tensor(x.reshape(tokens, streams * hidden))
    out = torch.empty((tokens, hidden), dtype=dtype, device="cuda")
    clear = torch.full((tokens, hidden), 3.0, dtype=torch.float32, device="cuda")
    ops.streams_read_norm(d_streams, device_tensor(read), streams, device_tensor(1.0 + weight), out,
                          eps, tokens, clear=clear)
    u = np.einsum("s,tsw->tw", read, x)
    want = plain.rms_norm_one_plus(u, weight, eps)
    close(as_double(out), want, 1e-5 if dtype == torch.float32 else 4e-2, 1e-5)
    assert float(clear.abs().max()) == 0.0
    # the cleared buffer may start from a vector (a bias) instead of zero
    start = rng.normal(size=hidden)
    ops.streams_read_norm(d_streams, device_tensor(read), streams, device_tensor(1.0 + weight), out,
                          eps, tokens, clear=clear, initial=device_tensor(start))
    close(as_double(clear), np.tile(start.astype(np.float32), (tokens, 1)), 0.0)
    close(as_double(out), want, 1e-5 if dtype == torch.float32 else 4e-2, 1e-5)
    # gathered rows, plain sum of the streams (the final norm)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device="cuda")
    gathered = torch.empty((3, hidden), dtype=dtype, device="cuda")
    ops.streams_read_norm(d_streams, None, streams, device_tensor(1.0 + weight), gathered, eps, 3,
                          rows=rows)
    want = plain.rms_norm_one_plus(x.sum(axis=1)[[5, 0, 5]], weight, eps)
    close(as_double(gathered), want, 1e-5 if dtype == torch.float32 else 4e-2, 1e-5)
    if dtype == torch.float32:
        ops.streams_write(d_streams, device_tensor(y), device_tensor(mixing), device_tensor(write),
                          device_tensor(scale), streams, tokens)
        want = np.einsum("sr,tsw->trw", mixing, x) + write[None, :, None] * (scale * y)[:, None, :]
        close(as_double(d_streams).reshape(tokens, streams, hidden), want, 1e-5, 1e-5)


def test_streams_spread_and_scaled_sum():
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 24))
    streams = torch.zeros((5, 3 * 24), dtype=torch.float32, device="cuda")
    ops.streams_spread(device_tensor(x), streams, 5, 3)
    close(as_double(streams).reshape(5, 3, 24), np.repeat(x[:, None], 3, axis=1), 1e-7)
    base, a, b = rng.normal(size=(5, 24)), rng.normal(size=(6, 24)), rng.normal(size=(6, 24))
    d_base, d_a, d_b = device_tensor(base), device_tensor(a), device_tensor(b)
    ops.scaled_sum(d_base, [d_a, d_b], [0.6, -1.1], 5)
    close(as_double(d_base), base + 0.6 * a[:5] - 1.1 * b[:5], 1e-6)
    assert float(d_a[:5].abs().max()) == 0.0 and float(d_b[:5].abs().max()) == 0.0
    close(as_double(d_a[5:]), a[5:], 1e-7)       # rows beyond the step are not touched


@pytest.mark.parametrize("dtype", DTYPES)
def test_biased_activation(dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(1)
    z = np.concatenate([rng.normal(size=(4, 40)) * 3.0, [[0.0] * 40], rng.normal(size=(1, 40)) * 1e-3])
    bias = rng.normal(size=40) * 0.3
    p, q = 0.4, -0.7
    out = torch.empty((6, 40), dtype=dtype, device="cuda")
    ops.biased_activation(device_tensor(z), device_tensor(bias), out, 6, ops.ACT_XIELU,
                          float(plain.softplus(p)), 0.5 + float(plain.softplus(q)))
    close(as_double(out), plain.xielu(z + bias, p, q), 2e-6 if dtype == torch.float32 else 2e-2,
          1e-6 if dtype == torch.float32 else 8e-3)
    ops.biased_activation(device_tensor(z), None, out, 6, ops.ACT_TANH)
    close(as_double(out), np.tanh(z), 2e-6 if dtype == torch.float32 else 8e-3)
    x = device_tensor(z)
    ops.add_bias(x, device_tensor(bias), 6)
    close(as_double(x), (z + bias).astype(np.float32), 1e-6)


# -------------------------------------------------------------------------- filter

@pytest.mark.parametrize("taps", [1, 2, 4, 5])
@pytest.mark.parametrize("dtype", DTYPES)
def test_causal_filter_in_portions_of_every_size(taps, dtype):
    """Two sequences side by side, cut into portions shorter and longer than the filter; the
    history travels in the state rows, and a slot that is used again starts from zeros."""
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(taps)
    channels, before, after = 37, 6, 3      # the filtered columns sit inside wider rows
    lengths = {"a": 23, "b": 9}
    raw = {k: as_double(device_tensor(rng.normal(size=(n, channels)), dtype)) for k, n in lengths.items()}
    weights, bias = rng.normal(size=(channels, taps)), rng.normal(size=channels)
    want = {k: plain.silu(plain.causal_filter_bias(v, weights, bias)) for k, v in raw.items()}
    state = torch.full((3, (taps - 1) * channels + 5), 7.0, dtype=torch.float32, device="cuda")
    slots = {"a": 2, "b": 0}
    state[[0, 2]] = 0.0
    cursor = {"a": 0, "b": 0}
    for sizes in ([1, 1], [2, 1], [1, 3], [7, 1], [5, 2], [3, 1], [4, 0]):
        live = [(k, s) for k, s in zip(("a", "b"), sizes) if s > 0]
        rows = np.concatenate([raw[k][cursor[k]:cursor[k] + s] for k, s in live])
        wide = np.concatenate([np.zeros((len(rows), before)), rows, np.zeros((len(rows), after))], axis=1)
        d_rows = device_tensor(wide, dtype)
        out = torch.empty((len(rows), channels), dtype=dtype, device="cuda")
        token_request, request_slot, request_start = batch([s for _, s in live], [slots[k] for k, _ in live])
        ops.causal_filter(d_rows[:, before:before + channels], out, device_tensor(weights),
                          device_tensor(bias), state if taps > 1 else None, len(rows), True,
                          token_request, request_slot, request_start)
        expected = np.concatenate([want[k][cursor[k]:cursor[k] + s] for k, s in live])
        close(as_double(out), expected, 2e-5 if dtype == torch.float32 else 3e-2, 1e-2 if dtype == torch.bfloat16 else 0)
        for k, s in live:
            cursor[k] += s
    assert cursor == {"a": 23, "b": 9}
    assert float(state[1].min()) == 7.0          # nobody's slot stays untouched


# --------------------------------------------------------------------- recurrences

def run_in_portions(lengths, portions, step_fn):
    """Feed requests of ``lengths`` tokens in rounds; ``portions[round][r]`` tokens of request
    r each round.  ``step_fn(spans)`` gets [(request, begin, end)] of one round."""
    cursor = [0] * len(lengths)
    for sizes in portions:
        spans = []
        for r, size in enumerate(sizes):
            size = min(size, lengths[r] - cursor[r])
            if size > 0:
                spans.append((r, cursor[r], cursor[r] + size))
                cursor[r] += size
        if spans:
            step_fn(spans)
    assert cursor == list(lengths)


PORTIONS = [[1, 2], [1, 1], [2, 40], [33, 1], [1, 0], [5, 7], [64, 64], [200, 200]]


@pytest.mark.parametrize("heads,width,rows,groups", [(4, 12, 16, 2), (2, 40, 24, 1), (3, 64, 128, 3),
                                                     (1, 8, 1, 1)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_state_space_scan(heads, width, rows, groups, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(heads * 100 + rows)
    lengths = [130, 57]
    inner, bc = heads * width, groups * rows
    data = []
    for n in lengths:
        rows_in = as_double(device_tensor(rng.normal(size=(n, inner + 2 * bc)), dtype))
        dt = as_double(device_tensor(rng.normal(size=(n, heads)), dtype))
        data.append((rows_in, dt))
    dt_bias, skip = rng.uniform(-3, 0.5, size=heads), rng.normal(size=heads)
    # one head that hardly forgets: a token hundreds of steps back still counts
    a_log = rng.uniform(np.log(0.3), np.log(3.0), size=heads)
    a_log[0] = np.log(0.004)
    want = []
    for rows_in, dt in data:
        n = len(dt)
        want.append(plain.state_space_scan(
            rows_in[:, :inner].reshape(n, heads, width), rows_in[:, inner:inner + bc].reshape(n, groups, rows),
            rows_in[:, inner + bc:].reshape(n, groups, rows), plain.softplus(dt + dt_bias), a_log, skip,
            groups).reshape(n, inner))
    state = torch.zeros((3, heads * ops.scan_state_floats(width, rows) + 3), dtype=torch.float32,
                        device="cuda")
    state[1] = float("nan")                       # a slot nobody owns is never read
    slots = [2, 0]
    got = [np.zeros_like(w) for w in want]

    def step(spans):
        x = np.concatenate([data[r][0][b:e] for r, b, e in spans])
        dt = np.concatenate([data[r][1][b:e] for r, b, e in spans])
        d_x, d_dt = device_tensor(x, dtype), device_tensor(dt, dtype)
        y = torch.empty((len(x), inner), dtype=torch.float32, device="cuda")
        _, request_slot, request_start = batch([e - b for _, b, e in spans], [slots[r] for r, _, _ in spans])
        ops.state_space_scan(d_x[:, :inner], d_x[:, inner:inner + bc], d_x[:, inner + bc:], d_dt,
                             device_tensor(dt_bias), device_tensor(a_log), device_tensor(skip), state,
                             y, request_start, request_slot, len(spans), heads, width, rows, groups)
        out, at = as_double(y), 0
        for r, b, e in spans:
            got[r][b:e] = out[at:at + e - b]
            at += e - b

    run_in_portions(lengths, PORTIONS, step)
    for r in range(2):
        spread = np.abs(want[r]).max()
        close(got[r], want[r], 3e-5 * spread)


@pytest.mark.parametrize("heads,dim", [(2, 16), (3, 12), (1, 64), (2, 40)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_outer_product_scan(heads, dim, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(heads * 10 + dim)
    lengths = [140, 31]
    a = heads * dim
    w0 = rng.uniform(-7.0, 0.5, size=a)
    bonus = rng.normal(size=(heads, dim))
    data, want = [], []
    for n in lengths:
        r, k, v = (as_double(device_tensor(rng.normal(size=(n, a)) * 0.5, dtype)) for _ in range(3))
        decay_log = rng.normal(size=(n, a)).astype(np.float32).astype(np.float64) * 0.3
        data.append((r, k, v, decay_log))
        w = np.exp(-np.exp(decay_log + w0))
        want.append(plain.decayed_outer_product_scan(
            r.reshape(n, heads, dim), k.reshape(n, heads, dim), v.reshape(n, heads, dim),
            w.reshape(n, heads, dim), bonus).reshape(n, a))
    state = torch.zeros((2, heads * ops.scan_state_floats(dim, dim)), dtype=torch.float32,
                        device="cuda")
    slots = [1, 0]
    got = [np.zeros_like(w) for w in want]

    def step(spans):
        parts = [np.concatenate([data[r][i][b:e] for r, b, e in spans]) for i in range(4)]
        d_r, d_k, d_v = (device_tensor(p, dtype) for p in parts[:3])
        o = torch.empty((len(parts[0]), a), dtype=torch.float32, device="cuda")
        _, request_slot, request_start = batch([e - b for _, b, e in spans], [slots[r] for r, _, _ in spans])
        ops.outer_product_scan(d_r, d_k, d_v, device_tensor(parts[3]), device_tensor(w0),
                               device_tensor(bonus), state, o, request_start, request_slot,
                               len(spans), heads, dim)
        out, at = as_double(o), 0
        for r, b, e in spans:
            got[r][b:e] = out[at:at + e - b]
            at += e - b

    run_in_portions(lengths, PORTIONS, step)
    for r in range(2):
        close(got[r], want[r], 3e-5 * np.abs(want[r]).max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_shift_carries_the_previous_row(dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(3)
    hidden, mixes = 44, 5
    lengths = [19, 6]
    h = [as_double(device_tensor(rng.normal(size=(n, hidden)), dtype)) for n in lengths]
    mu = rng.uniform(size=(mixes, hidden))
    want = [x[None] + (plain.shifted(x) - x)[None] * mu[:, None, :] for x in h]
    state = torch.zeros((2, hidden + 2), dtype=torch.float32, device="cuda")
    got = [np.zeros_like(w) for w in want]

    def step(spans):
        rows = device_tensor(np.concatenate([h[r][b:e] for r, b, e in spans]), dtype)
        out = torch.empty((mixes, len(rows) + 3, hidden), dtype=dtype, device="cuda")
        token_request, request_slot, request_start = batch([e - b for _, b, e in spans],
                                                            [1 - r for r, _, _ in spans])
        ops.token_shift(rows, device_tensor(mu), out, state, len(rows), token_request, request_slot,
                        request_start)
        values, at = as_double(out), 0
        for r, b, e in spans:
            got[r][:, b:e] = values[:, at:at + e - b]
            at += e - b

    run_in_portions(lengths, [[1, 1], [2, 1], [1, 0], [9, 2], [1, 1], [50, 50]], step)
    for r in range(2):
        close(got[r], want[r], 1e-6 if dtype == torch.float32 else 3e-2)


@pytest.mark.parametrize("groups", [1, 2, 5])
@pytest.mark.parametrize("gate_after", [False, True])
@pytest.mark.parametrize("dtype", DTYPES)
def test_gated_group_norm(groups, gate_after, dtype):
    from helix_runtime_b200.ops import library as ops
    rng = np.random.default_rng(groups)
    tokens, channels, eps = 6, 60, 1e-5
    y = rng.normal(size=(tokens, channels)).astype(np.float32).astype(np.float64)
    gate = as_double(device_tensor(rng.normal(size=(tokens, channels)), dtype))
    weight = rng.normal(size=channels)
    out = torch.empty((tokens, channels), dtype=dtype, device="cuda")
    ops.gated_group_norm(device_tensor(y), device_tensor(gate, dtype), device_tensor(weight), out,
                         tokens, groups, eps, gate_after)
    if gate_after:
        want = plain.grouped_unit_rms(y, groups, eps) * weight * plain.silu(gate)
    else:
        want = plain.grouped_unit_rms(y * plain.silu(gate), groups, eps) * weight
    close(as_double(out), want, 1e-5 if dtype == torch.float32 else 5e-2, 1e-5)


# ----------------------------------------------------------- rotation, normed heads

@pytest.mark.parametrize("layout", ["halves", "interleaved"])
@pytest.mark.parametrize("head_dim,value_dim,row_dim,rotary_dim", [(16, 16, 16, 16), (24, 12, 32, 8),
                                                                   (64, 48, 64, 32), (20, 12, 20, 0)])
def test_norm_rotation_and_rotated_values(layout, head_dim, value_dim, row_dim, rotary_dim):
    """Queries come back normed and rotated; keys and values are found in the pages, normed and
    rotated (values over all their coordinates); rotating a value back by its own position
    gives the projected value again."""
    from helix_runtime_b200.ops import library as ops
    from helix_runtime_b200.parts.position import ComputedRotary, PAIRINGS
    rng = np.random.default_rng(head_dim + rotary_dim)
    heads, kv_heads, page_size, num_pages, eps, base = 3, 2, 4, 9, 1e-5, 640.0
    positions = np.array([0, 1, 5, 130, 131, 4095], dtype=np.int32)
    tokens = len(positions)
    code = PAIRINGS["half_split" if layout == "halves" else "adjacent"]

    def padded(count, real):
        values = np.zeros((tokens, count, row_dim))
        values[:, :, :real] = rng.normal(size=(tokens, count, real))
        return values

    q, k, v = padded(heads, head_dim), padded(kv_heads, head_dim), padded(kv_heads, value_dim)
    q_norm, k_norm = rng.normal(size=head_dim), rng.normal(size=head_dim)
    qkv = device_tensor(np.concatenate([q.reshape(tokens, -1), k.reshape(tokens, -1),
                                        v.reshape(tokens, -1)], axis=1))
    # one request; position p lives in page table[p // page_size]
    table = torch.full((1, 1100), -1, dtype=torch.int32, device="cuda")
    for index, page in ((0, 3), (1, 7), (32, 1), (1023, 5)):
        table[0, index] = page
    shape = (num_pages, kv_heads, page_size, row_dim)
    k_cache = torch.zeros(shape, dtype=torch.float32, device="cuda")
    v_cache = torch.zeros(shape, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    zeros = torch.zeros(tokens, dtype=torch.int32, device="cuda")
    freq = ComputedRotary.frequencies(base, rotary_dim, "cuda")
    value_freq = ComputedRotary.frequencies(base, value_dim, "cuda")
    ops.norm_rotary_append(qkv, torch.tensor(positions).cuda(), zeros, zeros[:1], table, k_cache,
                           v_cache, freq, value_freq, device_tensor(q_norm), device_tensor(k_norm),
                           eps, tokens, heads, kv_heads, head_dim, value_dim, row_dim, rotary_dim,
                           code, code, page_size, num_pages, status)
    assert int(status.item()) == 0
    where = positions.astype(np.float64)
    want_q = plain.rotate_pairs(plain.unit_rms(q[..., :head_dim], eps) * q_norm, where, base,
                                rotary_dim, layout)
    want_k = plain.rotate_pairs(plain.unit_rms(k[..., :head_dim], eps) * k_norm, where, base,
                                rotary_dim, layout)
    want_v = plain.rotate_pairs(v[..., :value_dim], where, base, value_dim, layout)
    got_q = as_double(qkv)[:, :heads * row_dim].reshape(tokens, heads, row_dim)
    # angles are float32 products of position and frequency: at position 4095 they differ from
    # the double ones by up to 2e-4
    close(got_q[..., :head_dim], want_q, 2e-3)
    close(got_q[:-1, :, :head_dim], want_q[:-1], 1e-4)
    assert np.abs(got_q[..., head_dim:]).max(initial=0.0) == 0.0
    chunk = 4          # float32: 16-byte pieces of 4 coordinates, slot-major inside a piece
    pages = as_double(table)[0]
    for cache, want, real in ((k_cache, want_k, head_dim), (v_cache, want_v, value_dim)):
        stored = as_double(cache).reshape(num_pages, kv_heads, row_dim // chunk, page_size, chunk)
        for t, p in enumerate(positions):
            page, slot = int(pages[p // page_size]), p % page_size
            got = stored[page, :, :, slot, :].reshape(kv_heads, row_dim)
            close(got[:, :real], want[t], 2e-3 if p > 1000 else 1e-4)
            assert np.abs(got[:, real:]).max(initial=0.0) == 0.0
    # turning back: a "context" made of each token's own cached value returns the projection
    context = device_tensor(np.repeat(want_v_padded(want_v, row_dim)[:, :1], heads, axis=1)
                            .reshape(tokens, heads * row_dim))
    ops.rotate_back(context, torch.tensor(positions).cuda(), value_freq, tokens, heads, row_dim,
                    value_dim, code)
    back = as_double(context).reshape(tokens, heads, row_dim)
    close(back[:-1, :, :value_dim], np.repeat(v[:-1, :1, :value_dim], heads, axis=1), 2e-4)


def want_v_padded(values, row_dim):
    out = np.zeros(values.shape[:-1] + (row_dim,))
    out[..., :values.shape[-1]] = values
    return out
