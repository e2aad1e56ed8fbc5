"""Root-mean-square normalisation, alone and fused with the residual addition.

``y = round(x * rsqrt(mean(x^2) + eps) * w)`` with 32-bit statistics and the weight
multiplied before the single rounding (src/cuda/kernels.rs:26-57); the fused form
adds first and takes the statistics of the unrounded sum (src/cuda/kernels.rs:59-103).
"""

from __future__ import annotations

from typing import Dict, Mapping, Optional, Tuple

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import NORMS, Norm, Runtime


@NORMS.register("rms_norm")
class RMSNorm(Norm):
    """params: ``size``, ``eps``; weights: ``weight`` ``[size]``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = runtime.vector_f32(tensors["weight"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        return {spec.weights["weight"]: ExpectedTensor((int(spec.params["size"]),))}

    @classmethod
    def random_tensor(cls, spec, role, shape: Tuple[int, ...], generator) -> torch.Tensor:
        return 1.0 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.02

    def rms_parameters(self) -> Tuple[torch.Tensor, float]:
        """``(weight, eps)``: what a product kernel needs to compute this norm in its own first phase.  A norm that
        has this method may be folded into the product behind it; one that has not runs its own kernel."""
        return self.weight, self.eps

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(x)
        return kernels.rms_norm(x, self.weight, self.eps, out)

    def forward_add(self, residual: torch.Tensor, update: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        if out is None:
            out = torch.empty_like(residual)
        kernels.add_rms_norm(residual, update, self.weight, self.eps, out, residual)
        return out


@NORMS.register("grouped_rms_norm")
class GroupedRMSNorm(Norm):
    """RMS norm over equal consecutive parts of the vector, for a residual stream kept in 32-bit.

    params: ``size``, ``groups``, ``eps``, optional ``offset``; weights: ``weight`` ``[size]``.  The row is cut into
    ``groups`` parts, each is divided by its own ``sqrt(mean(part^2) + eps)``, and the whole is multiplied by
    ``offset + weight`` (``offset`` 0 unless given: a checkpoint that stores its norm weights around zero has
    ``offset`` 1; the sum is taken once, in 32-bit, when the model is built); ``groups = 1`` is the plain norm.  The stream (``x`` / ``residual``) is float32 whatever the run dtype, an update may be float32
    or bfloat16, and the normalised rows come out in the run dtype, rounded once."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.size = int(params["size"])
        self.groups = int(params.get("groups") or 1)
        self.eps = float(params["eps"])
        if self.groups < 1 or self.size % self.groups:
            raise ValueError(f"a norm over {self.groups} groups needs a size that they divide, got {self.size}")
        self.offset = float(params.get("offset") or 0.0)
        self.weight = runtime.vector_f32(tensors["weight"])
        if self.offset:
            self.checkpoint_weight = self.weight          # as stored (what an upload check compares)
            self.weight = self.weight + self.offset

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        return {spec.weights["weight"]: ExpectedTensor((int(spec.params["size"]),))}

    @classmethod
    def random_tensor(cls, spec, role, shape: Tuple[int, ...], generator) -> torch.Tensor:
        centre = 1.0 - float(spec.params.get("offset") or 0.0)
        return centre + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.1

    def shared_statistic(self) -> Optional[Tuple[torch.Tensor, float]]:
        """``(weight, eps)`` if this is a plain RMS norm over the whole row of a 32-bit stream (one group): two such
        norms of the same row with the same ``eps`` differ in their weights only and may leave one kernel together."""
        return (self.weight, self.eps) if self.groups == 1 else None

    def forward_sum(self, residual: torch.Tensor, update_a: Optional[torch.Tensor], update_b: Optional[torch.Tensor],
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual += update_a + update_b`` (either may be None; 32-bit, in place), then the norm of the sum."""
        if self.groups == 1 and all(u is None or u.dtype == torch.float32 for u in (update_a, update_b)):
            first, second = (update_a, update_b) if update_a is not None else (update_b, None)
            out = self._out(residual, out)
            kernels.sum_norms(residual, first, second, self.weight, out, None, None, self.eps)
            return out
        return super().forward_sum(residual, update_a, update_b, out)

    def _out(self, x: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        return out if out is not None else torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return kernels.group_rms_norm(x, None, self.weight, self.groups, self.eps, self._out(x, out))

    def forward_add(self, residual: torch.Tensor, update: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        return kernels.group_rms_norm(residual, update, self.weight, self.groups, self.eps, self._out(residual, out))


@NORMS.register("layer_norm")
class LayerNorm(Norm):
    """Layer norm with weight and bias over a residual stream kept in 32-bit: ``(x - mean) / sqrt(var + eps) * weight +
    bias``, ``var`` the mean of the squared deviations.

    params: ``size``, ``eps``; weights: ``weight``, ``bias`` (``[size]`` each, kept in 32-bit).  The stream (``x`` /
    ``residual``) and an update are float32 whatever the run dtype; the normalised rows come out in the run dtype,
    rounded once.  ``norm_parameters()`` hands a block the kernel's description of this norm, so that the block may
    run it together with the addition in front (a sublayer whose result is normed before it joins the stream)."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.weight = runtime.vector_f32(tensors["weight"])
        self.bias = runtime.vector_f32(tensors["bias"])

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        size = int(spec.params["size"])
        return {spec.weights["weight"]: ExpectedTensor((size,)), spec.weights["bias"]: ExpectedTensor((size,))}

    @classmethod
    def random_tensor(cls, spec, role, shape: Tuple[int, ...], generator) -> torch.Tensor:
        noise = torch.randn(shape, generator=generator, dtype=torch.float32) * 0.1
        return noise if role == "bias" else 1.0 + noise

    def norm_parameters(self):
        """``(kind, weight, bias)`` as ``kernels.norm_add_norm`` takes a norm."""
        return (kernels.NORM_LAYER, self.weight, self.bias)

    def _out(self, x: torch.Tensor, out: Optional[torch.Tensor]) -> torch.Tensor:
        return out if out is not None else torch.empty(x.shape, dtype=self.runtime.dtype, device=x.device)

    def forward(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = self._out(x, out)
        kernels.norm_add_norm(x, None, None, self.norm_parameters(), out, None, self.eps)
        return out

    def forward_add(self, residual: torch.Tensor, update: torch.Tensor,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        out = self._out(residual, out)
        kernels.norm_add_norm(residual, update, None, self.norm_parameters(), out, None, self.eps)
        return out
