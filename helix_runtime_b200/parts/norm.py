"""Norms.  RMSNorm: ``y = x / sqrt(mean(x^2) + eps) * w`` (src/kernels/cpu/reference.cpp:392-406);
LayerNorm: see :class:`LayerNorm`.

Reads the float32 residual stream, computes in float32, writes the compute dtype.
Parameters: ``eps``, ``one_plus`` (the weight is stored around zero and the row is multiplied
by ``1 + w``; the sum is taken in float32 at load); tensors: ``weight`` ``[hidden]``.
``forward_streams`` is the same norm on a weighted sum of several residual streams.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import Norm, StepContext, register_part


class RmsNorm(Norm):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.eps = float(spec["eps"])
        if not self.eps > 0.0:
            raise ValueError("RmsNorm eps must be positive")
        self.one_plus = bool(spec.get("one_plus", False))
        self.weight_name = spec.tensors["weight"]
        self.weight: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        return [TensorRequest(self.weight_name, (self.hidden_size,), role="scale")]

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        weight = tensors[self.weight_name].to(device=device, dtype=torch.float32)
        self.weight = (weight + 1.0 if self.one_plus else weight).contiguous()

    def weight_bytes(self) -> int:
        return self.hidden_size * 4

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
        count = ctx.n_tokens if n_rows is None else n_rows
        ops.rmsnorm(x, self.weight, out[:count], self.eps, rows)

    def forward_streams(self, ctx: StepContext, streams: torch.Tensor, count: int,
                        read: Optional[torch.Tensor], out: torch.Tensor,
                        clear: Optional[torch.Tensor] = None,
                        rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None,
                        initial: Optional[torch.Tensor] = None) -> None:
        """The norm of ``sum_s read[s] * streams[:, s]`` (``read`` None: the plain sum) for
        ``streams`` ``[rows, count * hidden]``; ``clear``: a float32 buffer whose rows are zeroed
        on the way (the sublayer sums its output into it), or set to ``initial`` ``[hidden]``."""
        ops.streams_read_norm(streams, read, count, self.weight, out, self.eps,
                              ctx.n_tokens if n_rows is None else n_rows, clear=clear, rows=rows,
                              initial=initial)


class LayerNorm(Norm):
    """``y = (x - mean) / sqrt(var + eps) * w + b``, ``var`` the mean of the squared deviations;
    float32 throughout, written in the compute dtype.  Parameters: ``eps``; tensors: ``weight``
    and (optional) ``bias``, both ``[hidden]``."""

    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.eps = float(spec["eps"])
        if not self.eps >= 0.0:
            raise ValueError("LayerNorm eps must not be negative")
        self.weight_name = spec.tensors["weight"]
        self.bias_name = spec.tensors.get("bias")
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        requests = [TensorRequest(self.weight_name, (self.hidden_size,), role="scale")]
        if self.bias_name is not None:
            requests.append(TensorRequest(self.bias_name, (self.hidden_size,), role="scale"))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        self.weight = tensors[self.weight_name].to(device=device, dtype=torch.float32).contiguous()
        if self.bias_name is not None:
            self.bias = tensors[self.bias_name].to(device=device, dtype=torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.hidden_size * 4 * (1 if self.bias_name is None else 2)

    def forward(self, ctx: StepContext, x: torch.Tensor, out: torch.Tensor,
                rows: Optional[torch.Tensor] = None, n_rows: Optional[int] = None) -> None:
        count = ctx.n_tokens if n_rows is None else n_rows
        ops.layernorm(x, self.weight, self.bias, out[:count], self.eps, rows)


register_part("norm", "rms", RmsNorm)
register_part("norm", "layer_norm", LayerNorm)
