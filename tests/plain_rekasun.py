"""Plain, slow implementation of the Rekasun decoder: whole sequences, no cache, NumPy in
double precision, one function per mechanism.  It shares no code with the engine (own
safetensors reader, own order of layers, own mask).

Notation.  ``x`` is the residual stream ``[T, W]``.  A layer computes ``h = LN(x)`` and
``x <- x + mixer(h) + ff(h)``.  The attention mixer: ``q, k, v = h Wq', h Wk', h Wv'``;
each channel is filtered along time, ``y[t] = sum_j f[:, j] u[t - (n - 1) + j]``; scores
``s[i, j] = scale * q_i . k_j`` over the keys ``j <= i`` with ``i - j < window`` or
``j < kept``; softmax; the concatenated heads times ``sigmoid(h Wg')``; times ``Wo'``.
Feed-forward: ``(gelu_tanh(h Wgate') * (h Wup')) Wdown'``.

``precision="bfloat16"`` rounds activations to bfloat16 at the places where a bfloat16 engine
stores them (norm output, projections, filtered rows, attention output, gated heads,
feed-forward activation); sums stay in double, the residual stream is never rounded.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence, Tuple

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
        else:
            raise ValueError(f"unsupported dtype {record['dtype']}")
        tensors[name] = value.reshape(tuple(record["shape"]))
    return tensors


def to_bfloat16(values: np.ndarray) -> np.ndarray:
    """Round to the nearest bfloat16 (ties to even), returned as float64."""
    bits = np.asarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) << 16
    return rounded.astype(np.uint32).view(np.float32).astype(np.float64).reshape(np.shape(values))


# ------------------------------------------------------------------- mechanisms

def layer_norm(x: np.ndarray, weight: np.ndarray, bias: Optional[np.ndarray], eps: float) -> np.ndarray:
    mean = x.mean(axis=-1, keepdims=True)
    variance = ((x - mean) ** 2).mean(axis=-1, keepdims=True)
    out = (x - mean) / np.sqrt(variance + eps) * weight
    return out if bias is None else out + bias


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def causal_filter(u: np.ndarray, taps: np.ndarray, history: Optional[np.ndarray] = None) -> np.ndarray:
    """``u [T, C]``, ``taps [C, n]``: ``y[t] = sum_j taps[:, j] * u[t - (n - 1) + j]``; what lies
    before the rows of ``u`` is ``history [n - 1, C]`` (zeros when the sequence starts here)."""
    n = taps.shape[1]
    if history is None:
        history = np.zeros((n - 1, u.shape[1]))
    padded = np.concatenate([history, u], axis=0)
    out = np.zeros_like(u, dtype=np.float64)
    for j in range(n):
        out += padded[j:j + u.shape[0]] * taps[:, j]
    return out


def visible(queries: Sequence[int], keys: int, window: Optional[int], kept: int = 0) -> np.ndarray:
    """``[len(queries), keys]`` booleans: may the query at that position see key j?"""
    i = np.asarray(queries)[:, None]
    j = np.arange(keys)[None, :]
    seen = j <= i
    if window:
        seen &= (i - j < window) | (j < kept)
    return seen


def attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, scale: float, window: Optional[int],
              kept: int = 0, query_offset: int = 0) -> np.ndarray:
    """``q [H, Tq, D]``, ``k [G, Tk, D]``, ``v [G, Tk, V]`` -> ``[H, Tq, V]``; query i sits at
    position ``query_offset + i``; head h reads key/value head ``h // (H / G)``."""
    heads, rows = q.shape[0], q.shape[1]
    group = heads // k.shape[0]
    mask = visible(range(query_offset, query_offset + rows), k.shape[1], window, kept)
    out = np.zeros((heads, rows, v.shape[2]))
    for head in range(heads):
        scores = (q[head] @ k[head // group].T) * scale
        scores = np.where(mask, scores, -np.inf)
        scores -= scores.max(axis=-1, keepdims=True)
        weights = np.exp(scores)
        weights /= weights.sum(axis=-1, keepdims=True)
        out[head] = weights @ v[head // group]
    return out


def gated_feed_forward(h: np.ndarray, gate: np.ndarray, up: np.ndarray, down: np.ndarray,
                       store=lambda a: a) -> np.ndarray:
    return store(gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def layer_runs(layers: int, loop: Optional[dict]) -> List[Tuple[int, bool]]:
    """``(layer, add the embedding first)`` in running order."""
    if not loop:
        return [(layer, False) for layer in range(layers)]
    runs = [(layer, False) for layer in range(loop["start"])]
    for turn in range(loop["times"]):
        for layer in range(loop["start"], loop["stop"]):
            runs.append((layer, turn > 0 and layer == loop["start"]))
    runs += [(layer, False) for layer in range(loop["stop"], layers)]
    return runs


# ------------------------------------------------------------------------ model

class PlainRekasun:
    def __init__(self, folder: str, precision: str = "float32") -> None:
        with open(os.path.join(folder, "config.json"), "r", encoding="utf-8") as source:
            self.config = json.load(source)
        self.weights = read_safetensors(os.path.join(folder, "model.safetensors"))
        self.store = to_bfloat16 if precision == "bfloat16" else (lambda a: a)
        if precision == "bfloat16":      # a bfloat16 engine holds its matrices in bfloat16
            self.weights = {name: (value if value.ndim == 1 or name.endswith(".conv")
                                   else to_bfloat16(value))
                            for name, value in self.weights.items()}

    def mixer(self, h: np.ndarray, prefix: str, sizes: dict) -> np.ndarray:
        w, store = self.weights, self.store
        heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
        rows = h.shape[0]
        q, k, v = (store(h @ w[f"{prefix}.{name}"].T) for name in ("q", "k", "v"))
        if sizes.get("conv", 1) > 1:
            q, k, v = (store(causal_filter(u, w[f"{prefix}.{name}.conv"]))
                       for u, name in ((q, "q"), (k, "k"), (v, "v")))
        mask = sizes["mask"]
        mixed = attention(q.reshape(rows, heads, dim).transpose(1, 0, 2),
                          k.reshape(rows, groups, dim).transpose(1, 0, 2),
                          v.reshape(rows, groups, vdim).transpose(1, 0, 2),
                          sizes["scale"], mask["size"], mask.get("keep_first", 0))
        mixed = store(mixed.transpose(1, 0, 2).reshape(rows, heads * vdim))
        mixed = store(mixed * sigmoid(store(h @ w[f"{prefix}.g"].T)))
        return mixed @ w[f"{prefix}.o"].T

    def hidden_states(self, tokens: Sequence[int]) -> List[np.ndarray]:
        """The residual stream after every run of a layer."""
        config, w = self.config, self.weights
        eps = config["norm"]["eps"]
        embedded = w["embed"][np.asarray(tokens)] * config.get("embedding", {}).get("scale", 1.0)
        x = embedded.copy()
        states = []
        for layer, again in layer_runs(len(config["layers"]), config.get("loop")):
            if again:
                x = x + embedded
            sizes = config["layers"][layer]
            h = self.store(layer_norm(x, w[f"l{layer}.norm1"], w[f"l{layer}.norm1.b"], eps))
            update = self.mixer(h, f"l{layer}.mix", sizes["mixer"])
            if sizes.get("mlp") is not None:
                update = update + gated_feed_forward(h, w[f"l{layer}.mlp.gate"],
                                                     w[f"l{layer}.mlp.up"],
                                                     w[f"l{layer}.mlp.down"], self.store)
            x = x + update
            states.append(x.copy())
        return states

    def logits(self, tokens: Sequence[int]) -> np.ndarray:
        config, w = self.config, self.weights
        x = self.hidden_states(tokens)[-1]
        x = self.store(layer_norm(x, w["final.norm"], w["final.norm.b"], config["norm"]["eps"]))
        return (x @ w["head"].T).astype(np.float32)

    def greedy(self, prompt: Sequence[int], new_tokens: int) -> List[int]:
        tokens = list(prompt)
        for _ in range(new_tokens):
            tokens.append(int(np.argmax(self.logits(tokens)[-1])))
        return tokens[len(prompt):]
