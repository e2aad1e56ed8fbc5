"""Linear attention with a fixed decay per head (fixed-size state per request instead of pages).

With ``h`` the mixer's input, per head (``dim`` query/key numbers, ``vdim`` value numbers, decay ``a``):

    q_t = silu(Wq h_t), k_t = silu(Wk h_t), v_t = silu(Wv h_t)
    S_t = a S_(t-1) + k_t v_t^T          S_(-1) = 0, ``[dim, vdim]``, 32-bit, in the request's state slot
    o_t = S_t^T q_t
    y_t = Wo (rms(o_t over all heads) * w * sigmoid(Wg h_t))

The four input projections are one product; activations, scores, decay powers and the state are 32-bit inside the
recurrence kernel, which walks a step's rows in chunks; the norm over the concatenated heads and the output gate are
one kernel; the output product leaves 32-bit rows for a stream kept in 32-bit.

The same recurrence with other surroundings (retention) is a matter of parameters: ``activation`` ``"none"`` takes q, k
and v as projected; a ``position`` child (``rotary_blend``, rotate-half layout) turns the first ``dims`` numbers of every
query and key head by the row's position; ``key_scale`` multiplies the keys afterwards; ``norm`` ``"per_head"`` divides
every head's ``o_t`` by its own root mean square, without a weight; ``gate`` ``"silu"`` multiplies by ``silu(Wg h_t)``
instead of the sigmoid.  Rotation and scaling happen in 32-bit in a kernel in front of the recurrence, which then reads
32-bit rows.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, POSITION_ENCODINGS, DeferredNorm, Mixer, Runtime, StateNeed, StepContext
from .linear import Linear


@MIXERS.register("lightning")
class Lightning(Mixer):
    """params: ``hidden_size, num_heads, key_dim, value_dim``, ``decay`` (one number per head), ``eps``, optional
    ``stream``, ``activation`` (``"silu"`` | ``"none"``), ``key_scale``, ``norm`` (``"all_heads"`` | ``"per_head"``), ``gate``
    (``"sigmoid"`` | ``"silu"``); weights: ``q, k, v, g, o`` and, with ``norm`` ``"all_heads"``, ``norm``; children:
    ``position`` (optional)."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.key_dim = int(p["key_dim"])
        self.value_dim = int(p["value_dim"])
        self.eps = float(p["eps"])
        self.stream_f32 = p.get("stream") == "float32"
        decay = [float(a) for a in p["decay"]]
        if len(decay) != self.num_heads or not all(0.0 <= a <= 1.0 for a in decay):
            raise ValueError("lightning takes one decay in [0, 1] per head")
        self.decay = torch.tensor(decay, dtype=torch.float64).to(torch.float32).to(runtime.device)
        self.o_width = self.num_heads * self.value_dim
        self.gate_offset = self.num_heads * (2 * self.key_dim + self.value_dim)
        self.in_proj = Linear(torch.cat([tensors["q"], tensors["k"], tensors["v"], tensors["g"]], dim=0), runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        self.activation = p.get("activation") or "silu"
        self.norm_kind = p.get("norm") or "all_heads"
        self.gate_kind = p.get("gate") or "sigmoid"
        if self.activation not in ("silu", "none") or self.norm_kind not in ("all_heads", "per_head") \
                or self.gate_kind not in ("sigmoid", "silu"):
            raise ValueError("lightning: activation is 'silu' or 'none', norm 'all_heads' or 'per_head', gate 'sigmoid' or 'silu'")
        if self.norm_kind == "all_heads" and self.gate_kind != "sigmoid":
            raise ValueError("lightning: the norm over all heads comes with a sigmoid gate")
        self.key_scale = float(p.get("key_scale") or 1.0)
        self.norm_weight = runtime.vector_f32(tensors["norm"]) if self.norm_kind == "all_heads" else None
        position_spec = spec.children.get("position") or PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if self.position.kind not in ("rotary_blend", "none"):
            raise ValueError(f"lightning rotates halves or not at all, got position encoding '{self.position.kind}'")
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.inv_freq = getattr(self.position, "half_inv_freq", None)
        self.amplitude = float(getattr(self.position, "amplitude", 1.0))
        if self.rot_dims > self.key_dim:
            raise ValueError("the rotation covers more numbers than a key has")
        # rows that the recurrence cannot read as projected go through a 32-bit copy first
        self.prepares = bool(self.rot_dims) or self.key_scale != 1.0
        if self.prepares and self.activation != "none":
            raise ValueError("lightning: rotation and key scaling apply to queries and keys as projected (activation 'none')")

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, heads, d, dv = int(p["hidden_size"]), int(p["num_heads"]), int(p["key_dim"]), int(p["value_dim"])
        out = {w["q"]: ExpectedTensor((heads * d, hidden)), w["k"]: ExpectedTensor((heads * d, hidden)),
               w["v"]: ExpectedTensor((heads * dv, hidden)), w["g"]: ExpectedTensor((heads * dv, hidden)),
               w["o"]: ExpectedTensor((hidden, heads * dv))}
        if (p.get("norm") or "all_heads") == "all_heads":
            out[w["norm"]] = ExpectedTensor((heads * dv,))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role == "norm":
            return 1.0 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.1
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's matrix products, for the printed kernel plan."""
        return [("q/k/v/gate", self.in_proj, plan.BF16), ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def cache_need(self) -> StateNeed:
        return StateNeed((self.num_heads, self.key_dim, self.value_dim), torch.float32)

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        if cache is None or cache.storage is None:
            raise RuntimeError("lightning needs a state binding")
        proj = self.in_proj.forward(x)
        rows = proj.shape[0]
        attended = torch.empty((rows, self.o_width), dtype=torch.float32, device=proj.device)
        recurrent_rows = proj
        if self.prepares:
            recurrent_rows = torch.empty((rows, self.gate_offset), dtype=torch.float32, device=proj.device)
            kernels.retention_prepare(proj, recurrent_rows, ctx.positions, self.inv_freq, heads=self.num_heads,
                                      dim=self.key_dim, vdim=self.value_dim, rot_dims=self.rot_dims,
                                      amplitude=self.amplitude, k_scale=self.key_scale)
        kernels.lightning(recurrent_rows, self.decay, cache.storage, attended, ctx.row_start, ctx.state_slots,
                          num_seqs=ctx.num_seqs, heads=self.num_heads, dim=self.key_dim, vdim=self.value_dim,
                          max_new=ctx.max_new, activation=self.activation == "silu")
        gated = torch.empty((rows, self.o_width), dtype=proj.dtype, device=proj.device)
        if self.norm_kind == "per_head":
            kernels.head_norm_gate(attended, proj[:, self.gate_offset:], gated, heads=self.num_heads, vdim=self.value_dim,
                                   eps=self.eps, gate_kind=kernels.GATE_SILU if self.gate_kind == "silu" else kernels.GATE_SIGMOID)
        else:
            kernels.gated_rms_norm(attended, self.norm_weight, proj[:, self.gate_offset:], gated, self.eps)
        return self.o_proj.forward(gated, float32_out=self.stream_f32)
