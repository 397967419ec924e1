"""Recurrent mixers: the selective state-space layer, the time-mixing layer with a decayed
outer-product state, and a mixer that runs several mixers side by side.

All three keep per-request state in ONE float32 row per schedule entry (``StateNeed`` of a flat
shape); a mixer cuts its row into the pieces it needs.  A step brings a portion of each
request's tokens (cut anywhere, one token when decoding); the kernels carry the state from
portion to portion, so the result does not depend on the cut.

:class:`StateSpaceMixer` (``state_space``).  Parameters ``heads``, ``head_width`` (``P``),
``state_size`` (``N``), ``groups`` (``G``), ``filter_taps``, ``norm_groups``, ``eps``.  With
``inner = heads * P``, the input projection's rows are ``[z: inner | x: inner | B: G N | C: G N |
dt: heads]``; ``x, B, C`` pass a causal per-channel filter with bias, then silu;
``d = softplus(dt + dt_bias)``; per head (head ``h`` reads group ``h // (heads / G)``)
``S_t = exp(-exp(A_log) d_t) S_(t-1) + d_t B_t x_t'``, ``y_t = S_t' C_t + D x_t``; ``y silu(z)``
is RMS-normed in ``norm_groups`` equal parts, times ``norm``, then the output projection.
State: the filter's last ``filter_taps - 1`` inputs and the matrices ``S`` (in the scan
kernel's own order, ``ops.scan_state_floats`` floats per head).

:class:`TimeMix` (``time_mix``).  Parameters ``heads``, ``head_dim``, ``decay_rank``, ``eps``.
With ``h'`` the previous token's input, each of r, k, v, g, w reads ``h + (h' - h) mu_s``;
``r, k, v`` are projections of their blends, ``gate = silu(W_g m_g)``,
``w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))``; per head ``o_t = (S_(t-1) + diag(u) k_t v_t')' r_t``
then ``S_t = diag(w_t) S_(t-1) + k_t v_t'``; each head's ``o`` over its root mean square, times
``norm``, times the gate, then the output projection.  State: ``h'`` and the
matrices ``S`` (``ops.scan_state_floats`` floats per head).

:class:`SideBySide` (``side_by_side``).  Parameters ``mixers`` (part specs) and ``scales``: every
mixer reads the same input and the result is ``sum_i scales[i] * mixer_i(x)``, summed in float32.
"""
from __future__ import annotations

import dataclasses
from typing import List, Mapping, Optional

import torch

from ..cache.manager import KvNeed, StateNeed
from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import LayerCache, Mixer, StepContext, build_part, register_part
from .linear import Weight, project


def _state_piece(cache: LayerCache, offset: int, size: int) -> torch.Tensor:
    """Columns ``[offset, offset + size)`` of the entry's state rows (a view; the kernels take
    its address and the stride between slots)."""
    return cache.state[:, offset:offset + size]


class StateSpaceMixer(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["heads"])
        self.head_width = int(spec["head_width"])
        self.state_size = int(spec["state_size"])
        self.groups = int(spec.get("groups", 1))
        self.taps = int(spec.get("filter_taps", 1))
        self.norm_groups = int(spec.get("norm_groups", 1))
        self.eps = float(spec["eps"])
        if self.heads % self.groups:
            raise ValueError("heads must be a multiple of groups")
        self.inner = self.heads * self.head_width
        if self.inner % self.norm_groups:
            raise ValueError("norm_groups must divide heads * head_width")
        if self.taps < 1:
            raise ValueError("filter_taps counts the filter's taps: at least 1")
        self.filtered = self.inner + 2 * self.groups * self.state_size
        self.projected = 2 * self.inner + 2 * self.groups * self.state_size + self.heads
        self.filter_state = (self.taps - 1) * self.filtered
        self.matrix_state = self.heads * ops.scan_state_floats(self.head_width, self.state_size)
        self.names = dict(spec.tensors)
        self.w_in: Optional[Weight] = None
        self.w_o: Optional[Weight] = None

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.filter_state + self.matrix_state,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        h = self.hidden_size
        return [TensorRequest(self.names["in"], (self.projected, h)),
                TensorRequest(self.names["filter"], (self.filtered, self.taps), role="scale"),
                TensorRequest(self.names["filter_bias"], (self.filtered,), role="scale"),
                TensorRequest(self.names["dt_bias"], (self.heads,), role="scale"),
                TensorRequest(self.names["a_log"], (self.heads,), role="scale"),
                TensorRequest(self.names["skip"], (self.heads,), role="scale"),
                TensorRequest(self.names["norm"], (self.inner,), role="scale"),
                TensorRequest(self.names["o"], (h, self.inner))]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        self.w_in = Weight(tensors[self.names["in"]].to(device=device, dtype=dtype).contiguous())
        self.w_o = Weight(tensors[self.names["o"]].to(device=device, dtype=dtype).contiguous())
        self.filter, self.filter_bias = scale("filter"), scale("filter_bias")
        self.dt_bias, self.a_log, self.skip = scale("dt_bias"), scale("a_log"), scale("skip")
        self.norm = scale("norm")

    def weight_bytes(self) -> int:
        return self.w_in.nbytes() + self.w_o.nbytes()

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n = ctx.n_tokens
        # a row width that keeps every row of the scratch 16-byte aligned for the products
        wide = -(-self.projected // 8) * 8
        rows = ctx.workspace.get(f"state_space.rows/{wide}", (ctx.capacity, wide), ctx.dtype)
        filtered = ctx.workspace.get(f"state_space.filtered/{self.filtered}",
                                     (ctx.capacity, self.filtered), ctx.dtype)
        y = ctx.workspace.get(f"state_space.y/{self.inner}", (ctx.capacity, self.inner),
                              torch.float32)
        gated = ctx.workspace.get(f"state_space.gated/{self.inner}", (ctx.capacity, self.inner),
                                  ctx.dtype)
        project(x, self.w_in, rows, n, ops.EPI_STORE, ctx.status)
        inner, bc = self.inner, self.groups * self.state_size
        ops.causal_filter(rows[:, inner:inner + self.filtered], filtered, self.filter,
                          self.filter_bias,
                          _state_piece(cache, 0, self.filter_state) if self.taps > 1 else None,
                          n, True, ctx.token_request, ctx.request_slot, ctx.request_start)
        ops.state_space_scan(filtered[:, :inner], filtered[:, inner:inner + bc],
                             filtered[:, inner + bc:inner + 2 * bc],
                             rows[:, inner + self.filtered:inner + self.filtered + self.heads],
                             self.dt_bias, self.a_log, self.skip,
                             _state_piece(cache, self.filter_state, self.matrix_state), y,
                             ctx.request_start, ctx.request_slot, ctx.n_requests, self.heads,
                             self.head_width, self.state_size, self.groups, tokens=n)
        ops.gated_group_norm(y, rows[:, :inner], self.norm, gated, n, self.norm_groups, self.eps,
                             gate_after=False)
        project(gated, self.w_o, residual, n, ops.EPI_ADD_F32, ctx.status, ctx.ordered_sums)


MIXES = ("r", "k", "v", "g", "w")


class TimeMix(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.heads = int(spec["heads"])
        self.head_dim = int(spec["head_dim"])
        self.decay_rank = int(spec["decay_rank"])
        self.eps = float(spec["eps"])
        self.width = self.heads * self.head_dim
        self.matrix_state = self.heads * ops.scan_state_floats(self.head_dim, self.head_dim)
        self.names = dict(spec.tensors)
        self.weights: dict = {}

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.hidden_size + self.matrix_state,), torch.float32)

    def tensor_requests(self) -> List[TensorRequest]:
        h, a = self.hidden_size, self.width
        requests = [TensorRequest(self.names[f"mu_{s}"], (h,), role="scale") for s in MIXES]
        requests += [TensorRequest(self.names[s], (a, h)) for s in ("r", "k", "v", "g")]
        requests += [TensorRequest(self.names["w1"], (self.decay_rank, h)),
                     TensorRequest(self.names["w2"], (a, self.decay_rank)),
                     TensorRequest(self.names["w0"], (a,), role="scale"),
                     TensorRequest(self.names["bonus"], (self.heads, self.head_dim), role="scale"),
                     TensorRequest(self.names["norm"], (a,), role="scale"),
                     TensorRequest(self.names["o"], (h, a))]
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def scale(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        for role in ("r", "k", "v", "g", "w1", "w2", "o"):
            self.weights[role] = Weight(tensors[self.names[role]].to(device=device, dtype=dtype)
                                        .contiguous())
        self.mu = torch.stack([scale(f"mu_{s}") for s in MIXES]).contiguous()
        self.w0, self.bonus, self.norm = scale("w0"), scale("bonus"), scale("norm")

    def weight_bytes(self) -> int:
        return sum(weight.nbytes() for weight in self.weights.values())

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        n, h, a, cap = ctx.n_tokens, self.hidden_size, self.width, ctx.capacity
        ws = ctx.workspace
        mixes = ws.get(f"time_mix.mixes/{h}", (len(MIXES), cap, h), ctx.dtype)
        projected = ws.get(f"time_mix.rkvg/{a}", (4, cap, a), ctx.dtype)
        rank = -(-self.decay_rank // 8) * 8
        low_sums = ws.get(f"time_mix.low_sums/{rank}", (cap, rank), torch.float32)
        low = ws.get(f"time_mix.low/{rank}", (cap, rank), ctx.dtype)
        decay_log = ws.get(f"time_mix.decay/{a}", (cap, a), torch.float32)
        o = ws.get(f"time_mix.o/{a}", (cap, a), torch.float32)
        normed = ws.get(f"time_mix.normed/{a}", (cap, a), ctx.dtype)
        ops.token_shift(x, self.mu, mixes, _state_piece(cache, 0, h), n, ctx.token_request,
                        ctx.request_slot, ctx.request_start)
        for index, role in enumerate(("r", "k", "v", "g")):
            project(mixes[index], self.weights[role], projected[index], n, ops.EPI_STORE, ctx.status)
        project(mixes[4], self.weights["w1"], low_sums, n, ops.EPI_STORE_F32, ctx.status)
        ops.biased_activation(low_sums[:, :self.decay_rank], None, low[:, :self.decay_rank], n,
                              ops.ACT_TANH)
        project(low[:, :self.decay_rank], self.weights["w2"], decay_log, n, ops.EPI_STORE_F32,
                ctx.status)
        ops.outer_product_scan(projected[0], projected[1], projected[2], decay_log, self.w0,
                               self.bonus, _state_piece(cache, h, self.matrix_state), o,
                               ctx.request_start, ctx.request_slot, ctx.n_requests, self.heads,
                               self.head_dim, tokens=n)
        ops.gated_group_norm(o, projected[3], self.norm, normed, n, self.heads, self.eps,
                             gate_after=True)
        project(normed, self.weights["o"], residual, n, ops.EPI_ADD_F32, ctx.status,
                ctx.ordered_sums)


class SideBySide(Mixer):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.mixers: List[Mixer] = [build_part("mixer", part, hidden_size)
                                    for part in spec["mixers"]]
        self.scales = [float(scale) for scale in spec["scales"]]
        if len(self.mixers) != len(self.scales) or not 1 <= len(self.mixers) <= 4:
            raise ValueError("side_by_side runs one to four mixers, each with its scale")
        needs = [mixer.kv_need() for mixer in self.mixers]
        if sum(need is not None for need in needs) > 1:
            raise ValueError("at most one of the mixers side by side may keep keys and values")
        self.offsets: List[Optional[int]] = []
        total = 0
        for mixer in self.mixers:
            need = mixer.state_need()
            if need is None:
                self.offsets.append(None)
                continue
            if need.dtype != torch.float32 or len(need.shape) != 1:
                raise ValueError("mixers side by side keep their state as one float32 row each")
            self.offsets.append(total)
            total += need.shape[0]
        self.state_size = total

    @property
    def graph_safe(self) -> bool:
        return all(mixer.graph_safe for mixer in self.mixers)

    def kv_need(self) -> Optional[KvNeed]:
        return next((need for need in (mixer.kv_need() for mixer in self.mixers)
                     if need is not None), None)

    def state_need(self) -> Optional[StateNeed]:
        return StateNeed((self.state_size,), torch.float32) if self.state_size else None

    def tensor_requests(self) -> List[TensorRequest]:
        return [request for mixer in self.mixers for request in mixer.tensor_requests()]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        for mixer in self.mixers:
            mixer.bind(tensors, dtype, device)

    def weight_bytes(self) -> int:
        return sum(mixer.weight_bytes() for mixer in self.mixers)

    def forward(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                residual: torch.Tensor) -> None:
        sources = []
        for index, (mixer, offset) in enumerate(zip(self.mixers, self.offsets)):
            # an all-zero float32 buffer per mixer: it sums its output in, the sum below reads
            # and clears it again
            output = ctx.workspace.accumulator(f"side_by_side.{index}/{self.hidden_size}",
                                               (ctx.capacity, self.hidden_size))
            view = cache
            if offset is not None:
                size = mixer.state_need().shape[0]
                view = dataclasses.replace(cache, state=cache.state[:, offset:offset + size])
            mixer.forward(ctx, view, x, output)
            sources.append(output)
        ops.scaled_sum(residual, sources, self.scales, ctx.n_tokens)


register_part("mixer", "state_space", StateSpaceMixer)
register_part("mixer", "time_mix", TimeMix)
register_part("mixer", "side_by_side", SideBySide)
