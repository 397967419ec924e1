"""Plain, slow implementation of the Zuzadra decoder: whole sequences, no cache, NumPy in
double precision, one function per mechanism.  It shares no code with the engine (own
safetensors reader, own order of layers, own masks, own recurrences written token by token).

Notation.  The residual is kept as ``S`` streams ``X[s]`` (``[S, T, W]``), all equal to the
embedding at the start.  A sublayer ``f`` with read weights ``a[s]``, write weights ``b[t]``,
mixing matrix ``M[s, t]`` and layer scale ``l`` does ``u = sum_s a[s] X[s]``,
``y = l * f(norm(u))``, ``X[t] <- sum_s M[s, t] X[s] + b[t] y``.  Without streams it is
``x <- x + l * f(norm(x))``.  ``norm(x) = x / sqrt(mean(x^2) + eps) * (1 + w)``.

Mixers (``h`` is the normed input ``[T, W]``):

* state-space (``mamba2``): ``[z | x | B | C | dt] = h Win'``; ``x, B, C`` pass a causal
  per-channel filter with bias and silu; ``d_t = softplus(dt_t + bias)``;
  ``S_t = exp(-exp(A) d_t) S_(t-1) + d_t B_t x_t'``; ``y_t = S_t' C_t + D x_t``;
  ``out = groupnorm(y * silu(z)) * g`` through ``Wo``.
* ``parallel``: ``left_scale * attention(h) + right_scale * timemix(h)``.
  attention: per-head RMS norm of q and k, rotation of the first ``dims`` coordinates (pairs
  ``i, i + dims/2``), values rotated by their own position over all their coordinates and the
  head's sum turned back by the query's position, softmax over the last ``window`` keys.
  timemix: each of r, k, v, g, w reads ``h + (h_prev - h) mu``; ``w = exp(-exp(W2 tanh(W1 m) +
  w0))``; ``o_t = (S_(t-1) + diag(u) k_t v_t')' r_t``; ``S_t = diag(w_t) S_(t-1) + k_t v_t'``;
  each head's ``o`` over its root mean square, times a weight, times ``silu(Wg m_g)``, ``Wo``.

Feed-forward: ``Wdown act(Wup h + b) + b'`` with
``act(z) = softplus(p) z^2 + z/2`` for ``z > 0`` and
``(1/2 + softplus(q)) (exp(z) - 1 - z) + z/2`` otherwise.

``precision="bfloat16"`` rounds activations to bfloat16 where a bfloat16 engine stores them
(norm outputs, projections, filtered rows, mixes, attention output, normed heads, the
feed-forward's activation); sums, recurrences and the residual streams stay in double.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Callable, Dict, List, Optional

import numpy as np


def read_safetensors(path: str) -> Dict[str, np.ndarray]:
    with open(path, "rb") as source:
        (length,) = struct.unpack("<Q", source.read(8))
        header = json.loads(source.read(length).decode("utf-8"))
        payload = source.read()
    header.pop("__metadata__", None)
    tensors = {}
    for name, record in header.items():
        begin, end = record["data_offsets"]
        raw = payload[begin:end]
        if record["dtype"] == "F32":
            value = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif record["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << np.uint32(16)
            value = bits.view(np.float32).astype(np.float64)
        elif record["dtype"] == "I32":
            value = np.frombuffer(raw, dtype="<i4").astype(np.int64)
        else:
            raise ValueError(f"unsupported dtype {record['dtype']}")
        tensors[name] = value.reshape(tuple(record["shape"]))
    return tensors


def to_bfloat16(values: np.ndarray) -> np.ndarray:
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(values))


def identity(values: np.ndarray) -> np.ndarray:
    return values


# ------------------------------------------------------------------- small functions

def softplus(z):
    return np.logaddexp(0.0, z)


def silu(z):
    return z / (1.0 + np.exp(-z))


def unit_rms(x: np.ndarray, eps: float) -> np.ndarray:
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm_one_plus(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    return unit_rms(x, eps) * (1.0 + weight)


def xielu(z: np.ndarray, p: float, q: float) -> np.ndarray:
    positive = softplus(p) * z * z + 0.5 * z
    negative = (0.5 + softplus(q)) * np.expm1(np.minimum(z, 0.0)) - (0.5 + softplus(q)) * z + 0.5 * z
    return np.where(z > 0.0, positive, negative)


# ------------------------------------------------------------------- mechanisms

def causal_filter_bias(u: np.ndarray, taps: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """``u [T, C]``, ``taps [C, n]`` with the last column on the token itself, zeros before the
    sequence: ``y[t, c] = bias[c] + sum_j taps[c, j] u[t - (n - 1) + j, c]``."""
    length, n = u.shape[0], taps.shape[1]
    out = np.tile(bias[None, :], (length, 1)).astype(np.float64)
    for t in range(length):
        for j in range(n):
            source = t - (n - 1) + j
            if source >= 0:
                out[t] += taps[:, j] * u[source]
    return out


def state_space_scan(x: np.ndarray, b: np.ndarray, c: np.ndarray, step: np.ndarray,
                     a_log: np.ndarray, skip: np.ndarray, groups: int) -> np.ndarray:
    """``x [T, H, P]``, ``b, c [T, G, N]``, ``step [T, H]`` (already positive): the selective
    state-space recurrence, one ``N x P`` state per head, written token by token."""
    length, heads, width = x.shape
    per_group = heads // groups
    out = np.zeros((length, heads, width))
    for head in range(heads):
        group = head // per_group
        state = np.zeros((b.shape[2], width))
        rate = math.exp(a_log[head])
        for t in range(length):
            state = math.exp(-rate * step[t, head]) * state \
                + step[t, head] * np.outer(b[t, group], x[t, head])
            out[t, head] = state.T @ c[t, group] + skip[head] * x[t, head]
    return out


def grouped_unit_rms(y: np.ndarray, parts: int, eps: float) -> np.ndarray:
    """``y [T, C]`` cut into ``parts`` equal parts, each divided by its own root mean square."""
    length, channels = y.shape
    return unit_rms(y.reshape(length, parts, channels // parts), eps).reshape(length, channels)


def rotate_pairs(x: np.ndarray, positions: np.ndarray, base: float, dims: int, layout: str,
                 sign: float = 1.0) -> np.ndarray:
    """``x [T, ..., D]``: the first ``dims`` coordinates turn by ``sign * position * base^(-2m /
    dims)`` in pairs (``halves``: ``m`` with ``m + dims/2``; ``interleaved``: ``2m`` with
    ``2m + 1``); the rest pass."""
    out = x.copy()
    half = dims // 2
    for m in range(half):
        first, second = (m, m + half) if layout == "halves" else (2 * m, 2 * m + 1)
        angle = sign * positions * base ** (-2.0 * m / dims)
        shape = (-1,) + (1,) * (x.ndim - 2)
        cos, sin = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
        u, v = x[..., first], x[..., second]
        out[..., first] = u * cos - v * sin
        out[..., second] = v * cos + u * sin
    return out


def windowed_softmax_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float,
                               window: int) -> np.ndarray:
    """``q [T, H, D]``, ``k [T, G, D]``, ``v [T, G, E]``: position ``i`` sees ``j`` with
    ``0 <= i - j < window``; query head ``h`` reads key/value head ``h // (H / G)``."""
    length, heads, _ = q.shape
    per_group = heads // k.shape[1]
    out = np.zeros((length, heads, v.shape[2]))
    for head in range(heads):
        group = head // per_group
        for i in range(length):
            first = max(0, i - window + 1)
            scores = (k[first:i + 1, group] @ q[i, head]) * scale
            weights = np.exp(scores - scores.max())
            weights /= weights.sum()
            out[i, head] = weights @ v[first:i + 1, group]
    return out


def shifted(h: np.ndarray) -> np.ndarray:
    """The previous token's row; zeros for the first token."""
    return np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)


def decayed_outer_product_scan(r: np.ndarray, k: np.ndarray, v: np.ndarray, w: np.ndarray,
                               bonus: np.ndarray) -> np.ndarray:
    """``r, k, v, w [T, H, D]``, ``bonus [H, D]``: the read comes before the update, with the
    bonus on the current token only."""
    length, heads, dim = r.shape
    out = np.zeros((length, heads, dim))
    for head in range(heads):
        state = np.zeros((dim, dim))
        for t in range(length):
            pair = np.outer(k[t, head], v[t, head])
            out[t, head] = (state + bonus[head][:, None] * pair).T @ r[t, head]
            state = w[t, head][:, None] * state + pair
    return out


# ------------------------------------------------------------------------ the model

class PlainZuzadra:
    def __init__(self, folder: str, precision: str = "float32") -> None:
        with open(os.path.join(folder, "config.json")) as source:
            self.config = json.load(source)
        self.w = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.round: Callable[[np.ndarray], np.ndarray] = \
            to_bfloat16 if precision == "bfloat16" else identity
        self.eps = float(self.config["norm"]["eps"])
        self.streams = self.config.get("streams")
        self.after_layer: Optional[Callable[[int, np.ndarray], None]] = None

    # ---------------------------------------------------------------- sublayers

    def linear(self, name: str, x: np.ndarray, bias: bool = False) -> np.ndarray:
        out = x @ self.w[name].T
        return out + self.w[name + ".b"] if bias else out

    def state_space_mixer(self, prefix: str, sizes: dict, h: np.ndarray) -> np.ndarray:
        heads, width, state, groups = sizes["heads"], sizes["vdim"], sizes["state"], sizes["groups"]
        inner, length = heads * width, h.shape[0]
        rows = self.round(self.linear(f"{prefix}.in", h))
        z, xbc, dt = np.split(rows, [inner, 2 * inner + 2 * groups * state], axis=1)
        xbc = self.round(silu(causal_filter_bias(xbc, self.w[f"{prefix}.conv"],
                                                 self.w[f"{prefix}.conv.b"])))
        x, b, c = np.split(xbc, [inner, inner + groups * state], axis=1)
        step = softplus(dt + self.w[f"{prefix}.dt_bias"])
        y = state_space_scan(x.reshape(length, heads, width), b.reshape(length, groups, state),
                             c.reshape(length, groups, state), step, self.w[f"{prefix}.A_log"],
                             self.w[f"{prefix}.D"], groups).reshape(length, inner)
        gated = grouped_unit_rms(y * silu(z), sizes["norm_groups"], self.eps) * self.w[f"{prefix}.norm"]
        return self.linear(f"{prefix}.o", self.round(gated))

    def attention_mixer(self, prefix: str, sizes: dict, h: np.ndarray, positions: np.ndarray) -> np.ndarray:
        heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
        length = h.shape[0]
        rot = sizes["rot"]
        layout = rot.get("layout", "halves")
        q = self.round(self.linear(f"{prefix}.q", h)).reshape(length, heads, dim)
        k = self.round(self.linear(f"{prefix}.k", h)).reshape(length, groups, dim)
        v = self.round(self.linear(f"{prefix}.v", h)).reshape(length, groups, vdim)
        q = unit_rms(q, self.eps) * self.w[f"{prefix}.q.norm"]
        k = unit_rms(k, self.eps) * self.w[f"{prefix}.k.norm"]
        q = self.round(rotate_pairs(q, positions, rot["base"], rot["dims"], layout))
        k = self.round(rotate_pairs(k, positions, rot["base"], rot["dims"], layout))
        v = self.round(rotate_pairs(v, positions, rot["base"], vdim, layout))
        out = windowed_softmax_attention(q, k, v, sizes["scale"], sizes["mask"]["size"])
        out = rotate_pairs(out, positions, rot["base"], vdim, layout, sign=-1.0)
        return self.linear(f"{prefix}.o", self.round(out.reshape(length, heads * vdim)))

    def time_mixer(self, prefix: str, sizes: dict, h: np.ndarray) -> np.ndarray:
        heads, dim, length = sizes["heads"], sizes["dim"], h.shape[0]
        before = shifted(h)
        mix = {s: self.round(h + (before - h) * self.w[f"{prefix}.mu.{s}"]) for s in "rkvgw"}
        r = self.round(self.linear(f"{prefix}.r", mix["r"])).reshape(length, heads, dim)
        k = self.round(self.linear(f"{prefix}.k", mix["k"])).reshape(length, heads, dim)
        v = self.round(self.linear(f"{prefix}.v", mix["v"])).reshape(length, heads, dim)
        gate = silu(self.round(self.linear(f"{prefix}.g", mix["g"])))
        low = self.round(np.tanh(self.linear(f"{prefix}.w1", mix["w"])))
        w = np.exp(-np.exp(self.linear(f"{prefix}.w2", low) + self.w[f"{prefix}.w0"]))
        out = decayed_outer_product_scan(r, k, v, w.reshape(length, heads, dim), self.w[f"{prefix}.u"])
        out = unit_rms(out, self.eps).reshape(length, heads * dim) * self.w[f"{prefix}.norm"] * gate
        return self.linear(f"{prefix}.o", self.round(out))

    def mixer(self, index: int, layer: dict, h: np.ndarray, positions: np.ndarray) -> np.ndarray:
        prefix, sizes = f"l{index}.mix", layer["mixer"]
        if layer["type"] == "mamba2":
            return self.state_space_mixer(prefix, sizes, h)
        if layer["type"] == "parallel":
            return sizes["left_scale"] * self.attention_mixer(prefix + ".left", sizes["left"], h, positions) \
                + sizes["right_scale"] * self.time_mixer(prefix + ".right", sizes["right"], h)
        raise ValueError(f"unknown layer type {layer['type']!r}")

    def feed_forward(self, index: int, h: np.ndarray) -> np.ndarray:
        prefix = f"l{index}.mlp"
        p, q = self.w[f"{prefix}.act"]
        hidden = self.round(xielu(self.linear(f"{prefix}.up", h, bias=True), p, q))
        return self.linear(f"{prefix}.down", hidden, bias=True)

    # ------------------------------------------------------------------- layers

    def sublayer(self, x: np.ndarray, prefix: str, which: int, function) -> np.ndarray:
        norm, scale = self.w[f"{prefix}.norm{which}"], self.w[f"{prefix}.ls{which}"]
        if self.streams is None:
            return x + scale * function(self.round(rms_norm_one_plus(x, norm, self.eps)))
        read, write = self.w[f"{prefix}.hc{which}.in"], self.w[f"{prefix}.hc{which}.out"]
        mixing = self.w[f"{prefix}.hc{which}.mix"]
        u = np.einsum("s,stw->tw", read, x)
        y = scale * function(self.round(rms_norm_one_plus(u, norm, self.eps)))
        return np.einsum("sr,stw->rtw", mixing, x) + write[:, None, None] * y[None]

    def layer_order(self) -> List[int]:
        count, loop = len(self.config["layers"]), self.config.get("loop")
        if not loop:
            return list(range(count))
        return list(range(loop["start"])) \
            + list(range(loop["start"], loop["stop"])) * loop["times"] \
            + list(range(loop["stop"], count))

    def logits(self, tokens) -> np.ndarray:
        return self.forward(tokens).astype(np.float32)

    def hidden_states(self, tokens) -> List[np.ndarray]:
        """The residual (the sum of the streams) after every run of a layer."""
        states: List[np.ndarray] = []
        self.after_layer = lambda run, x: states.append(x.copy())
        try:
            self.forward(tokens)
        finally:
            self.after_layer = None
        return states

    def forward(self, tokens) -> np.ndarray:
        """Logits ``[T, vocab]`` of one whole sequence from position 0."""
        tokens = np.asarray(tokens, dtype=np.int64)
        positions = np.arange(len(tokens), dtype=np.float64)
        x = self.w["embed"][tokens]
        if self.streams is not None:
            x = np.tile(x[None], (self.streams, 1, 1))
        for run, index in enumerate(self.layer_order()):
            layer = self.config["layers"][index]
            x = self.sublayer(x, f"l{index}", 1, lambda h: self.mixer(index, layer, h, positions))
            if layer.get("mlp") is not None:
                x = self.sublayer(x, f"l{index}", 2, lambda h: self.feed_forward(index, h))
            if self.after_layer is not None:
                self.after_layer(run, x if self.streams is None else x.sum(axis=0))
        if self.streams is not None:
            x = x.sum(axis=0)
        final = self.round(rms_norm_one_plus(x, self.w["final.norm"], self.eps))
        return final @ self.w["head"].T
