"""Position encodings.  Rotary position encoding with the cache append fused into the same
kernel, and :class:`NoPosition` (the append alone).

Parameters: ``theta``, ``head_dim``, ``rotary_dim`` (default: all of the head),
``row_dim`` (default ``head_dim``: the width a head has in the projected rows and in the
cache; the coordinates from ``head_dim`` on are carried along unrotated),
``pairing`` (``adjacent``: pairs ``(2p, 2p+1)`` as the reference rotates,
src/kernels/cpu/reference.cpp:519-531; ``half_split``: pairs ``(p, p + rotary_dim/2)``),
``max_positions``.  The cos/sin table ``[max_positions, rotary_dim/2]`` is built once
in double and cast to float32, as the reference builds its table
(src/model/llama_common.cpp:37-46); the kernel rotates in float32.
"""
from __future__ import annotations

from typing import Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from .base import LayerCache, PositionEncoding, StepContext, register_part
from .linear import Weight, uses_tensor_cores

PAIRINGS = {"adjacent": 0, "half_split": 1}


class RotaryEncoding(PositionEncoding):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.theta = float(spec["theta"])
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.row_dim = int(spec.get("row_dim", self.head_dim))
        if self.row_dim < self.head_dim:
            raise ValueError("row_dim must be at least head_dim")
        self.max_positions = int(spec["max_positions"])
        pairing = spec.get("pairing", "adjacent")
        if pairing not in PAIRINGS:
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.pairing = pairing
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if not self.theta > 0.0:
            raise ValueError("rotary theta must be positive")
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        half = max(self.rotary_dim // 2, 1)
        # the reference holds theta as a float32 value (include/helix/model/llama.hpp:22)
        theta = float(torch.tensor(self.theta, dtype=torch.float32).item())
        exponent = -2.0 * torch.arange(half, dtype=torch.float64) / float(max(self.rotary_dim, 1))
        frequency = torch.pow(torch.tensor(theta, dtype=torch.float64), exponent)
        angle = torch.arange(self.max_positions, dtype=torch.float64)[:, None] * frequency[None, :]
        self.cos = torch.cos(angle).to(torch.float32).to(device).contiguous()
        self.sin = torch.sin(angle).to(torch.float32).to(device).contiguous()

    def apply(self, ctx: StepContext, cache: LayerCache, qkv: torch.Tensor, heads: int,
              kv_heads: int, accum: Optional[torch.Tensor] = None) -> None:
        """Encode queries and keys of ``qkv[:n_tokens]`` in place; write keys and values into
        the pages when the entry owns its cache.  With ``accum`` the projection is taken from
        that float32 accumulator (and the accumulator cleared) instead of from ``qkv``."""
        write = cache.owns and cache.keys is not None
        ops.rope_append(qkv, ctx.positions, ctx.token_request, ctx.request_slot,
                        cache.block_tables, cache.keys if write else None,
                        cache.values if write else None, self.cos, self.sin, ctx.n_tokens, heads,
                        kv_heads, self.row_dim, self.rotary_dim, PAIRINGS[self.pairing],
                        cache.page_size, cache.num_pages, ctx.status, accum=accum)


    def project_and_apply(self, ctx: StepContext, cache: LayerCache, x: torch.Tensor,
                          weight: Weight, qkv: torch.Tensor, heads: int, kv_heads: int) -> bool:
        """Prompt portions in bfloat16: rotation and cache append are the epilogue of the
        tensor-core product, which saves a pass over the projected rows (read 3 heads' worth,
        write it again) per layer.  Needs adjacent pairs (a thread of the epilogue holds 16
        consecutive coordinates of one token) and heads in steps of 16."""
        n = ctx.n_tokens
        if (self.pairing != "adjacent" or self.row_dim % 16
                or weight.rows != (heads + 2 * kv_heads) * self.row_dim
                or n < ops.gemm_tc_rope_append_min_tokens() or not uses_tensor_cores(x, weight, n)
                or qkv.dtype != torch.bfloat16 or qkv.stride(0) % 8):
            return False
        write = cache.owns and cache.keys is not None
        held = weight.tiles if weight.tiles is not None else weight.matrix
        ops.gemm_tc_rope_append(x, held, qkv, n, ctx.positions, ctx.token_request,
                                ctx.request_slot, cache.block_tables if write else None,
                                cache.keys if write else None, cache.values if write else None,
                                self.cos, self.sin, heads, kv_heads, self.row_dim, self.rotary_dim,
                                cache.page_size, cache.num_pages, ctx.status,
                                weight_shape=weight.shape)
        return True


class NoPosition(PositionEncoding):
    """No position encoding: queries and keys go into the scores as projected, and ``apply``
    is the plain cache append.  Parameters: ``head_dim``, ``row_dim`` (default ``head_dim``)."""

    pairing = None

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.head_dim = int(spec["head_dim"])
        self.row_dim = int(spec.get("row_dim", self.head_dim))
        if self.row_dim < self.head_dim:
            raise ValueError("row_dim must be at least head_dim")
        self.rotary_dim = 0
        self._no_angles: Optional[torch.Tensor] = None

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self._no_angles = torch.zeros((1, 1), dtype=torch.float32, device=device)

    def apply(self, ctx: StepContext, cache: LayerCache, qkv: torch.Tensor, heads: int,
              kv_heads: int, accum: Optional[torch.Tensor] = None) -> None:
        write = cache.owns and cache.keys is not None
        ops.rope_append(qkv, ctx.positions, ctx.token_request, ctx.request_slot,
                        cache.block_tables, cache.keys if write else None,
                        cache.values if write else None, self._no_angles, self._no_angles,
                        ctx.n_tokens, heads, kv_heads, self.row_dim, 0, 0, cache.page_size,
                        cache.num_pages, ctx.status, accum=accum)


class ComputedRotary(PositionEncoding):
    """Rotary encoding whose angles are computed from the position (no table, so no bound on
    positions), with three optional companions in the same kernel.

    Parameters: ``theta``, ``head_dim``, ``rotary_dim`` (default: all of the head; 0: none),
    ``row_dim`` (default: the larger of ``head_dim`` and ``value_dim``), ``pairing``
    (``half_split``: ``(m, m + rotary_dim/2)``,
    the default; ``adjacent``: ``(2m, 2m + 1)``).  The angle of pair ``m`` at position ``p`` is
    the float32 product ``p * f[m]`` with ``f[m] = theta^(-2m / rotary_dim)`` rounded to float32
    once; sine and cosine are float32.

    * ``qk_norm`` (with ``eps``): before the rotation every query and key head is divided by
      its root mean square over ``head_dim`` and multiplied by the weight ``q_norm`` (keys:
      ``k_norm``) ``[head_dim]``, one weight for all heads.
    * ``rotate_values`` (with ``value_dim``; ``value_theta`` and ``value_pairing`` default to the
      keys'): the value of position ``j`` is turned by ``j`` over all ``value_dim`` coordinates,
      pair ``m`` by ``j * value_theta^(-2m / value_dim)``, and cached so; :meth:`restore_values`
      turns a head's attention output at position ``i`` back by ``-i``.
    """

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.theta = float(spec["theta"])
        self.head_dim = int(spec["head_dim"])
        self.rotary_dim = int(spec.get("rotary_dim", self.head_dim))
        self.value_dim = int(spec.get("value_dim", self.head_dim))
        self.row_dim = int(spec.get("row_dim", max(self.head_dim, self.value_dim)))
        if self.row_dim < max(self.head_dim, self.value_dim):
            raise ValueError("row_dim must hold the head and its values")
        pairing = spec.get("pairing", "half_split")
        if pairing not in PAIRINGS:
            raise ValueError(f"unknown rotary pairing {pairing!r}")
        self.pairing = pairing
        if self.rotary_dim % 2 or not 0 <= self.rotary_dim <= self.head_dim:
            raise ValueError("rotary_dim must be even and at most head_dim")
        if not self.theta > 0.0:
            raise ValueError("rotary theta must be positive")
        self.qk_norm = bool(spec.get("qk_norm", False))
        self.eps = float(spec.get("eps", 0.0))
        if self.qk_norm and not self.eps > 0.0:
            raise ValueError("the query and key norm needs a positive eps")
        self.rotate_values = bool(spec.get("rotate_values", False))
        self.value_theta = float(spec.get("value_theta", self.theta))
        value_pairing = spec.get("value_pairing", pairing)
        if value_pairing not in PAIRINGS:
            raise ValueError(f"unknown rotary pairing {value_pairing!r}")
        self.value_pairing = value_pairing
        if self.rotate_values and self.value_dim % 2:
            raise ValueError("rotated values need an even value_dim")
        self.names = dict(spec.tensors)
        self.freq: Optional[torch.Tensor] = None
        self.value_freq: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None

    @staticmethod
    def frequencies(theta: float, dims: int, device) -> torch.Tensor:
        half = max(dims // 2, 1)
        exponent = -2.0 * torch.arange(half, dtype=torch.float64) / float(max(dims, 1))
        return torch.pow(torch.tensor(theta, dtype=torch.float64), exponent) \
            .to(torch.float32).to(device).contiguous()

    def tensor_requests(self):
        if not self.qk_norm:
            return []
        from ..weights.loader import TensorRequest
        return [TensorRequest(self.names["q_norm"], (self.head_dim,), role="scale"),
                TensorRequest(self.names["k_norm"], (self.head_dim,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.freq = self.frequencies(self.theta, self.rotary_dim, device)
        if self.rotate_values:
            self.value_freq = self.frequencies(self.value_theta, self.value_dim, device)
        if self.qk_norm:
            self.q_norm = tensors[self.names["q_norm"]].to(device=device, dtype=torch.float32).contiguous()
            self.k_norm = tensors[self.names["k_norm"]].to(device=device, dtype=torch.float32).contiguous()

    def apply(self, ctx: StepContext, cache: LayerCache, qkv: torch.Tensor, heads: int,
              kv_heads: int, accum: Optional[torch.Tensor] = None) -> None:
        write = cache.owns and cache.keys is not None
        ops.norm_rotary_append(qkv, ctx.positions, ctx.token_request, ctx.request_slot,
                               cache.block_tables, cache.keys if write else None,
                               cache.values if write else None, self.freq, self.value_freq,
                               self.q_norm, self.k_norm, self.eps, ctx.n_tokens, heads, kv_heads,
                               self.head_dim, self.value_dim, self.row_dim, self.rotary_dim,
                               PAIRINGS[self.pairing], PAIRINGS[self.value_pairing],
                               cache.page_size, cache.num_pages, ctx.status, accum=accum)

    def restore_values(self, ctx: StepContext, context: torch.Tensor, heads: int) -> None:
        """Turn every head of the attention output back by its query's position (in place)."""
        if self.rotate_values:
            ops.rotate_back(context, ctx.positions, self.value_freq, ctx.n_tokens, heads,
                            self.row_dim, self.value_dim, PAIRINGS[self.value_pairing])


register_part("position", "rotary", RotaryEncoding)
register_part("position", "computed_rotary", ComputedRotary)
register_part("position", "none", NoPosition)
