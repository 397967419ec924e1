"""How a sublayer is joined to the residual: several residual streams (hyper-connections)
and a per-channel layer scale.

A model with ``streams`` residual streams ``X[s]`` (all equal to the embedding at the start)
joins a sublayer ``f`` with read weights ``a[s]``, write weights ``b[r]`` and a mixing matrix
``M[s, r]`` (indexed from, to):

    u = sum_s a[s] X[s];   y = f(norm(u));   X[r] <- sum_s M[s, r] X[s] + b[r] * scale * y

for all ``r`` at once from the old streams.  Parameters: ``streams`` (1: the ordinary residual
sum ``x <- x + scale * y``; no read, write or mixing tensors then unless ``weighted``),
``weighted`` (the tensors ``read`` ``[streams]``, ``write`` ``[streams]`` and ``mixing``
``[streams, streams]`` exist), ``layer_scale`` (the tensor ``scale`` ``[hidden]`` exists).
Everything is float32; the streams of a token lie next to each other, ``[rows, streams * hidden]``.
"""
from __future__ import annotations

from typing import List, Mapping, Optional

import torch

from ..config.spec import PartSpec
from ..ops import library as ops
from ..weights.loader import TensorRequest
from .base import Norm, Part, StepContext, register_part


class StreamConnection(Part):
    def __init__(self, spec: PartSpec, hidden_size: int) -> None:
        super().__init__(spec, hidden_size)
        self.streams = int(spec.get("streams", 1))
        if self.streams < 1:
            raise ValueError("a model has at least one residual stream")
        self.weighted = bool(spec.get("weighted", self.streams > 1))
        self.layer_scale = bool(spec.get("layer_scale", False))
        self.names = dict(spec.tensors)
        self.read: Optional[torch.Tensor] = None
        self.write: Optional[torch.Tensor] = None
        self.mixing: Optional[torch.Tensor] = None
        self.scale: Optional[torch.Tensor] = None

    def tensor_requests(self) -> List[TensorRequest]:
        s = self.streams
        requests = []
        if self.weighted:
            requests += [TensorRequest(self.names["read"], (s,), role="scale"),
                         TensorRequest(self.names["write"], (s,), role="scale"),
                         TensorRequest(self.names["mixing"], (s, s), role="scale")]
        if self.layer_scale:
            requests.append(TensorRequest(self.names["scale"], (self.hidden_size,), role="scale"))
        return requests

    def bind(self, tensors: Mapping[str, torch.Tensor], dtype, device) -> None:
        def held(role: str) -> torch.Tensor:
            return tensors[self.names[role]].to(device=device, dtype=torch.float32).contiguous()
        if self.weighted:
            self.read, self.write, self.mixing = held("read"), held("write"), held("mixing")
        if self.layer_scale:
            self.scale = held("scale")

    def weight_bytes(self) -> int:
        return 4 * ((self.streams * (self.streams + 2) if self.weighted else 0)
                    + (self.hidden_size if self.layer_scale else 0))

    def read_normed(self, ctx: StepContext, norm: Norm, streams: torch.Tensor, normed: torch.Tensor,
                    output: torch.Tensor, initial: Optional[torch.Tensor] = None) -> None:
        """``normed[:n] = norm(sum_s a[s] X[s])``; ``output[:n]`` is zeroed for the sublayer, or
        set to ``initial`` (a bias of the sublayer's output, ``[hidden]`` float32)."""
        norm.forward_streams(ctx, streams, self.streams, self.read, normed, clear=output,
                             initial=initial)

    def write_back(self, ctx: StepContext, streams: torch.Tensor, output: torch.Tensor) -> None:
        ops.streams_write(streams, output, self.mixing, self.write, self.scale, self.streams,
                          ctx.n_tokens)


register_part("connection", "streams", StreamConnection)
