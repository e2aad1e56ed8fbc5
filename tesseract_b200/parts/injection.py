"""Steps between blocks that bring the embedding output back into the stream.

``origin_mix``: ``x <- W [x; x0]`` with ``W`` ``[hidden, 2 * hidden]`` (the stream's columns first), ``x`` the stream with
its pending updates added and ``x0`` the embedding output.  A model that walks a run of layers several times starts
every walk with one.  The pending sum and the concatenation are one kernel (32-bit sum, rounded once to the run
dtype as the product's operand); the product's result is the new stream, in 32-bit.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import INJECTIONS, Injection, ResidualStream, Runtime, StepContext
from .linear import Linear


@INJECTIONS.register("origin_mix")
class OriginMix(Injection):
    """params: ``hidden_size``; weights: ``weight`` ``[hidden, 2 * hidden]``.  Takes and returns a 32-bit stream."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec.params["hidden_size"])
        self.proj = Linear(tensors["weight"], runtime)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        hidden = int(spec.params["hidden_size"])
        return {spec.weights["weight"]: ExpectedTensor((hidden, 2 * hidden))}

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        # near [I, 0] + noise: the stream keeps its size from walk to walk
        hidden = shape[0]
        noise = torch.randn(shape, generator=generator, dtype=torch.float32) * (0.3 * shape[-1] ** -0.5)
        return noise + torch.cat([torch.eye(hidden), torch.zeros(hidden, hidden)], dim=1) * 0.7

    def products(self):
        return [("stream + origin", self.proj, plan.F32)]

    def forward(self, stream: ResidualStream, origin: torch.Tensor, ctx: StepContext) -> ResidualStream:
        if stream.prepared is not None:
            raise NotImplementedError("origin_mix takes the stream as a residual and its pending updates")
        residual = stream.residual
        if residual.dtype != torch.float32 or origin.dtype != torch.float32:
            raise NotImplementedError("origin_mix mixes 32-bit streams")
        first, second = (stream.update, stream.update_b) if stream.update is not None else (stream.update_b, None)
        both = torch.empty((residual.shape[0], 2 * self.hidden_size), dtype=self.runtime.dtype, device=residual.device)
        kernels.sum_concat(residual, first, second, origin, both)
        return ResidualStream(self.proj.forward(both, float32_out=True))


@INJECTIONS.register("stream_bias")
class StreamBias(Injection):
    """``x <- x + table[row]``: a learned vector added to the 32-bit stream (every walk of a run of layers that is
    walked several times starts with one of its own).  params: ``hidden_size``, ``rows``, ``row``; weights: ``table``
    ``[rows, hidden]`` (one tensor for all walks; kept in 32-bit)."""

    graph_safe = True
    reads_origin = False

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec.params["hidden_size"])
        row, rows = int(spec.params["row"]), int(spec.params["rows"])
        if not 0 <= row < rows:
            raise ValueError(f"row {row} of a table of {rows}")
        self.vector = runtime.vector_f32(tensors["table"])[row].contiguous()

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        return {spec.weights["table"]: ExpectedTensor((int(spec.params["rows"]), int(spec.params["hidden_size"])))}

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.3

    def forward(self, stream: ResidualStream, origin, ctx: StepContext) -> ResidualStream:
        if stream.prepared is not None or stream.update is not None or stream.update_b is not None:
            raise NotImplementedError("stream_bias takes a stream without pending updates")
        if stream.residual.dtype != torch.float32:
            raise NotImplementedError("stream_bias adds to a 32-bit stream")
        kernels.add_bias(stream.residual, self.vector)
        return stream
