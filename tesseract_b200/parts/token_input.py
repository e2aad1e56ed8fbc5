"""Terms that a layer adds to the stream for the token itself, behind its sublayers.

``gated_token_slice``: a second embedding table holds, per token, one slice of ``dim`` numbers per layer.  With ``x``
the stream behind the layer's sublayers and ``e`` the layer's slice of the row's token,

    g = act(Wg x) * e            (``Wg`` ``[dim, hidden]``)
    y = Wp g                     (``Wp`` ``[hidden, dim]``)
    x <- x + y / sqrt(mean(y^2) + eps) * w

The gate product takes the stream rounded once to the run dtype and leaves 32-bit numbers; activation and gating are
one kernel in 32-bit; the second product leaves 32-bit rows whose norm and addition are one kernel.  One table serves
all layers (the parts name the same checkpoint tensor and share its device copy).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import TOKEN_INPUTS, Runtime, StepContext, TokenInput
from .linear import Linear

_ACTIVATIONS = {"silu": kernels.ACT_SILU, "gelu_tanh": kernels.ACT_GELU_TANH}


@TOKEN_INPUTS.register("gated_token_slice")
class GatedTokenSlice(TokenInput):
    """params: ``hidden_size, vocab_size, dim, slices`` (slices per table row), ``slice`` (this layer's), ``activation``,
    ``eps``; weights: ``table`` ``[vocab, slices * dim]``, ``gate`` ``[dim, hidden]``, ``proj`` ``[hidden, dim]``, ``norm``
    ``[hidden]``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.dim = int(p["dim"])
        self.slices = int(p["slices"])
        self.slice = int(p["slice"])
        if not 0 <= self.slice < self.slices:
            raise ValueError(f"slice {self.slice} of a table with {self.slices} slices a row")
        if p.get("activation") not in _ACTIVATIONS:
            raise ValueError(f"activation must be one of {sorted(_ACTIVATIONS)}, got {p.get('activation')!r}")
        self.activation = _ACTIVATIONS[p["activation"]]
        self.eps = float(p["eps"])
        self.table = runtime.matrix(tensors["table"])
        self.gate_proj = Linear(tensors["gate"], runtime)
        self.out_proj = Linear(tensors["proj"], runtime)
        self.norm_weight = runtime.vector_f32(tensors["norm"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, dim = int(p["hidden_size"]), int(p["dim"])
        return {w["table"]: ExpectedTensor((int(p["vocab_size"]), int(p["slices"]) * dim)),
                w["gate"]: ExpectedTensor((dim, hidden)), w["proj"]: ExpectedTensor((hidden, dim)),
                w["norm"]: ExpectedTensor((hidden,))}

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role == "norm":
            return 0.5 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.1
        if role == "table":
            return torch.randn(shape, generator=generator, dtype=torch.float32)
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        return [("token gate", self.gate_proj, plan.F32), ("token proj", self.out_proj, plan.F32)]

    def forward(self, residual: torch.Tensor, ctx: StepContext, rounded: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual`` (float32, in place) gains the layer's term; ``rounded``: the stream already rounded to the run
        dtype, if the caller has it."""
        rows = residual.shape[0]
        if rounded is None:
            rounded = residual if self.runtime.is_float32 else residual.to(self.runtime.dtype)
        z = self.gate_proj.forward(rounded, float32_out=True)
        g = torch.empty((rows, self.dim), dtype=self.runtime.dtype, device=residual.device)
        kernels.token_gate(z, ctx.token_ids, self.table, self.slice * self.dim, g, self.activation)
        y = self.out_proj.forward(g, float32_out=True)
        kernels.norm_add_norm(residual, y, (kernels.NORM_RMS, self.norm_weight, None), None, None, None, self.eps)
        return residual
