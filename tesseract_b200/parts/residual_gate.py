"""A learned scale per feature and a sigmoid gate per row and feature on a sublayer's way into the stream.

For each sublayer of a layer (the mixer, the feed-forward) with input rows ``h`` and result ``r``:

    stream += r * scale * sigmoid(G h + b)

``scale`` ``[hidden]``, ``G`` ``[hidden, hidden]`` and ``b`` ``[hidden]`` are the sublayer's own.  This part holds the
tensors and runs the gate's product (32-bit logits); the weighting itself, the addition and the following norm are the
block's fused kernel.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import RESIDUAL_GATES, ResidualGates, Runtime
from .linear import Linear

_SUBLAYERS = ("mixer", "feed_forward")


@RESIDUAL_GATES.register("scaled_sigmoid_gate")
class ScaledSigmoidGate(ResidualGates):
    """params: ``hidden_size``, ``feed_forward`` (bool: whether the layer has one); weights: ``mixer_scale, mixer_gate,
    mixer_gate_bias`` and, with a feed-forward, the same three under ``feed_forward_``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        self.hidden_size = int(spec.params["hidden_size"])
        self.sublayers = _SUBLAYERS if spec.params.get("feed_forward") else _SUBLAYERS[:1]
        self._gate = {w: Linear(tensors[w + "_gate"], runtime) for w in self.sublayers}
        self._bias = {w: runtime.vector_f32(tensors[w + "_gate_bias"]) for w in self.sublayers}
        self._scale = {w: runtime.vector_f32(tensors[w + "_scale"]) for w in self.sublayers}

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        hidden, w = int(spec.params["hidden_size"]), spec.weights
        out = {}
        for which in (_SUBLAYERS if spec.params.get("feed_forward") else _SUBLAYERS[:1]):
            out[w[which + "_scale"]] = ExpectedTensor((hidden,))
            out[w[which + "_gate"]] = ExpectedTensor((hidden, hidden))
            out[w[which + "_gate_bias"]] = ExpectedTensor((hidden,))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role.endswith("_scale"):
            return 1.0 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.2
        if role.endswith("_gate_bias"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.5
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the gates' products, for the printed kernel plan."""
        return [(which + " gate", self._gate[which], plan.F32) for which in self.sublayers]

    def logits(self, which: str, rows_in: torch.Tensor) -> torch.Tensor:
        return self._gate[which].forward(rows_in, float32_out=True)

    def bias(self, which: str) -> torch.Tensor:
        return self._bias[which]

    def scale(self, which: str) -> torch.Tensor:
        return self._scale[which]
