"""Gated feed-forward with the SiLU activation (SwiGLU).

``down( silu(x Wg^T) * (x Wu^T) )`` (src/cuda/dense_decoder.rs:737-774,
src/cuda/kernels.rs:191-208).  Gate and up weights are merged at load so that one product
feeds the activation; each output column equals the separate product's.  When the
intermediate size is a multiple of eight the merged rows alternate in blocks of eight
(eight gate rows, the eight matching up rows, ...), which lets the decode kernel apply
the activation to its own accumulators; otherwise the gate rows come first.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import FEED_FORWARDS, DeferredNorm, FeedForward, Runtime, StepContext
from .linear import Linear


@FEED_FORWARDS.register("swiglu")
class SwiGLU(FeedForward):
    """params: ``hidden_size, intermediate_size``; weights: ``gate, up, down``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.interleaved = self.intermediate_size % 8 == 0
        if self.interleaved:
            blocks = self.intermediate_size // 8
            merged = torch.stack([tensors["gate"].view(blocks, 8, self.hidden_size),
                                  tensors["up"].view(blocks, 8, self.hidden_size)], dim=1)
            merged = merged.reshape(2 * self.intermediate_size, self.hidden_size)
        else:
            merged = torch.cat([tensors["gate"], tensors["up"]], dim=0)
        self.gate_up_proj = Linear(merged, runtime)
        self.down_proj = Linear(tensors["down"], runtime)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        return {
            w["gate"]: ExpectedTensor((inter, hidden)),
            w["up"]: ExpectedTensor((inter, hidden)),
            w["down"]: ExpectedTensor((hidden, inter)),
        }

    accepts_deferred_norm = True
    accepts_follow_norm = True

    def forward(self, x, ctx: StepContext, follow=None):
        activated = None
        epilogue = plan.SWIGLU if self.interleaved else plan.BF16
        if isinstance(x, DeferredNorm):
            if self.interleaved:      # norm, both projections and the activation in one kernel, if the plan has one
                activated = self.gate_up_proj.forward_normed(x, epilogue=epilogue)
            if activated is None:
                x = x.materialize()
        if activated is None and self.interleaved:
            activated = self.gate_up_proj.forward(x, epilogue=epilogue)     # both projections + SwiGLU, if planned
        if activated is None:
            gate_up = self.gate_up_proj.forward(x)
            activated = torch.empty((x.shape[0], self.intermediate_size), dtype=x.dtype, device=x.device)
            kernels.silu_mul(gate_up, activated, interleaved=self.interleaved)
        return self.down_proj.forward(activated, follow=follow)


@FEED_FORWARDS.register("polynorm_mlp")
class PolyNormMLP(FeedForward):
    """A dense feed-forward ``down(act(up h))`` whose activation is a normalised polynomial:

        act(z) = a N(z) + b N(z^2) + c N(z^3) + e,      N(v) = v / sqrt(mean(v^2) + eps) over the row,

    with powers taken element by element and ``(a, b, c, e)`` a tensor of four numbers.  params: ``hidden_size,
    intermediate_size, eps``, optional ``stream``; weights: ``up, down, act``.  The activation is one kernel with
    32-bit statistics; the down product comes out in 32-bit for a residual stream kept in 32-bit."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        self.eps = float(p["eps"])
        self.stream_f32 = p.get("stream") == "float32"
        self.up_proj = Linear(tensors["up"], runtime)
        self.down_proj = Linear(tensors["down"], runtime)
        self.coefficients = runtime.vector_f32(tensors["act"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        return {w["up"]: ExpectedTensor((inter, hidden)), w["down"]: ExpectedTensor((hidden, inter)),
                w["act"]: ExpectedTensor((4,))}

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role == "act":
            return torch.tensor([0.6, 0.3, 0.2, 0.05]) + torch.randn(shape, generator=generator) * 0.05
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the feed-forward's matrix products, for the printed kernel plan."""
        return [("up", self.up_proj, plan.BF16), ("down", self.down_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def forward(self, x, ctx: StepContext, follow=None):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        z = self.up_proj.forward(x)
        kernels.polynorm(z, self.coefficients, self.eps, z)        # in place: a row is read whole before it is written
        return self.down_proj.forward(z, float32_out=self.stream_f32)


@FEED_FORWARDS.register("plain_mlp")
class PlainMLP(FeedForward):
    """A dense feed-forward without a gate: ``down(act(up h))``, ``act`` the squared ReLU ``max(z, 0)^2``.

    params: ``hidden_size, intermediate_size``, ``activation`` (``"squared_relu"``), optional ``stream``; weights:
    ``up, down``.  The activation is a kernel of its own behind the first product; the down product comes out in 32-bit
    for a residual stream kept in 32-bit."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        if p.get("activation") != "squared_relu":
            raise ValueError(f"activation must be 'squared_relu', got {p.get('activation')!r}")
        self.stream_f32 = p.get("stream") == "float32"
        self.up_proj = Linear(tensors["up"], runtime)
        self.down_proj = Linear(tensors["down"], runtime)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        return {w["up"]: ExpectedTensor((inter, hidden)), w["down"]: ExpectedTensor((hidden, inter))}

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the feed-forward's matrix products, for the printed kernel plan."""
        return [("up", self.up_proj, plan.BF16), ("down", self.down_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def forward(self, x, ctx: StepContext, follow=None):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        z = self.up_proj.forward(x)
        kernels.squared_relu(z, z)
        return self.down_proj.forward(z, float32_out=self.stream_f32)


_ACTIVATIONS = {"silu": kernels.ACT_SILU, "gelu_tanh": kernels.ACT_GELU_TANH}


@FEED_FORWARDS.register("gated_mlp")
class GatedMLP(FeedForward):
    """A gated feed-forward ``down(act(gate h + bg) * (up h + bu)) + bd`` with a choice of activation and optional biases.

    params: ``hidden_size, intermediate_size``, ``activation`` (``"silu"`` or ``"gelu_tanh"``: ``0.5 z (1 + tanh(sqrt(2/pi)
    (z + 0.044715 z^3)))``), ``bias`` (bool), optional ``stream``; weights: ``gate, up, down`` and, with ``bias``,
    ``gate_bias, up_bias, down_bias``.  Gate and up are one product; biases, activation and the gating are one kernel
    in 32-bit behind it; the down product comes out in 32-bit for a residual stream kept in 32-bit."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.intermediate_size = int(p["intermediate_size"])
        if p.get("activation") not in _ACTIVATIONS:
            raise ValueError(f"activation must be one of {sorted(_ACTIVATIONS)}, got {p.get('activation')!r}")
        self.activation = _ACTIVATIONS[p["activation"]]
        self.biased = bool(p.get("bias"))
        self.stream_f32 = p.get("stream") == "float32"
        self.gate_up_proj = Linear(torch.cat([tensors["gate"], tensors["up"]], dim=0), runtime)
        self.gate_up_bias = None
        if self.biased:
            self.gate_up_bias = torch.cat([tensors["gate_bias"], tensors["up_bias"]]).to(
                device=runtime.device, dtype=torch.float32).contiguous()
        self.down_proj = Linear(tensors["down"], runtime, bias=tensors["down_bias"] if self.biased else None)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, inter = int(p["hidden_size"]), int(p["intermediate_size"])
        out = {w["gate"]: ExpectedTensor((inter, hidden)), w["up"]: ExpectedTensor((inter, hidden)),
               w["down"]: ExpectedTensor((hidden, inter))}
        if p.get("bias"):
            out.update({w["gate_bias"]: ExpectedTensor((inter,)), w["up_bias"]: ExpectedTensor((inter,)),
                        w["down_bias"]: ExpectedTensor((hidden,))})
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role.endswith("_bias"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.3
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the feed-forward's matrix products, for the printed kernel plan."""
        return [("gate/up", self.gate_up_proj, plan.BF16),
                ("down", self.down_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def forward(self, x, ctx: StepContext, follow=None):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        gate_up = self.gate_up_proj.forward(x)
        activated = torch.empty((x.shape[0], self.intermediate_size), dtype=gate_up.dtype, device=gate_up.device)
        kernels.gated_activation(gate_up, self.gate_up_bias, activated, self.activation)
        return self.down_proj.forward(activated, float32_out=self.stream_f32)
