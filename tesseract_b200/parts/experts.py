"""A feed-forward of many small experts, of which a router gives every row a few.

Per row ``h`` (the feed-forward's input):

* router logits ``z = W_r h`` accumulated and kept in 32-bit; the ``top_k`` largest are chosen (largest first, the
  lowest index of equal logits) and weighted by the softmax over the chosen logits alone;
* an expert is ``down_e(act(up_e h))`` without biases, ``act`` the squared ReLU ``max(z, 0)^2``;
* the output is the weighted sum of the chosen experts' outputs, slots in order, plus, if the model has one, a
  shared expert of the same form (and a size of its own) that every row takes.

Other routers and experts are a matter of parameters.  ``scoring`` ``"softmax_all"``: the scores are the softmax over
all experts' logits; the experts form ``groups`` equal runs of neighbours, a group counts as much as its best score, and
only experts of the ``keep_groups`` best groups can be chosen; the ``top_k`` largest scores among those are chosen and
weighted by their scores over the chosen scores' sum (``+ 1e-20``), times ``weight_scale``.  ``expert_form``
``"gated_silu"``: an expert (and the shared one) is ``down_e(silu(gate_e h) * (up_e h))``; gate and up are one product.

The step's ``rows * top_k`` (row, slot) assignments are grouped by expert on the device; each of the experts' two
products then runs as one launch over all groups, whose grid is sized for the worst case, so the host never learns
(or waits for) how many rows an expert received and a step can be captured in a graph.  Router, assignment weights
and the sum are 32-bit; the experts' products take the run dtype's operands and accumulate in 32-bit.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import FEED_FORWARDS, DeferredNorm, FeedForward, Runtime, StepContext
from .linear import Linear


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """params: ``hidden_size, num_experts, top_k, expert_size``, ``shared_size`` (None: no shared expert), optional
    ``stream``, ``scoring`` (``"softmax_chosen"`` | ``"softmax_all"``, the latter with ``groups``, ``keep_groups``,
    ``weight_scale``), ``expert_form`` (``"squared_relu"`` | ``"gated_silu"``); weights: ``router`` ``[experts, hidden]``,
    ``up.<e>`` ``[expert_size, hidden]`` and ``down.<e>`` ``[hidden, expert_size]`` for every expert ``e``, and with a
    shared expert ``shared_up``, ``shared_down``; gated experts also ``gate.<e>`` and ``shared_gate``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_experts = int(p["num_experts"])
        self.top_k = int(p["top_k"])
        self.expert_size = int(p["expert_size"])
        self.shared_size = int(p["shared_size"]) if p.get("shared_size") else 0
        self.stream_f32 = p.get("stream") == "float32"
        if not 1 <= self.top_k <= self.num_experts:
            raise ValueError(f"top_k must lie between 1 and the {self.num_experts} experts, got {self.top_k}")
        # the router's product: the run dtype's operands (a bfloat16 weight and row multiply exactly in 32-bit),
        # 32-bit accumulation, 32-bit logits; in a float32 run the package's own 32-bit product
        self.router = Linear(tensors["router"], runtime)
        experts = range(self.num_experts)
        self.scoring = p.get("scoring") or "softmax_chosen"
        self.form = p.get("expert_form") or "squared_relu"
        if self.scoring not in ("softmax_chosen", "softmax_all") or self.form not in ("squared_relu", "gated_silu"):
            raise ValueError("routed_experts: scoring is 'softmax_chosen' or 'softmax_all', expert_form 'squared_relu' or 'gated_silu'")
        self.groups = int(p.get("groups") or 1)
        self.keep_groups = int(p.get("keep_groups") or self.groups)
        self.weight_scale = float(p.get("weight_scale") if p.get("weight_scale") is not None else 1.0)
        if self.num_experts % self.groups or not 1 <= self.keep_groups <= self.groups \
                or self.top_k > self.keep_groups * (self.num_experts // self.groups):
            raise ValueError("routed_experts: groups must divide the experts, keep_groups lie between 1 and groups, and the "
                             "kept groups hold at least top_k experts")
        self.gated = self.form == "gated_silu"
        if self.gated:      # an expert's gate rows, then its up rows: one product, then the gating
            tensors = dict(tensors)
            for e in experts:
                tensors[f"up.{e}"] = torch.cat([tensors[f"gate.{e}"], tensors[f"up.{e}"]], dim=0)
            if self.shared_size:
                tensors["shared_up"] = torch.cat([tensors["shared_gate"], tensors["shared_up"]], dim=0)
        self.up = torch.stack([tensors[f"up.{e}"] for e in experts]).to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.down = torch.stack([tensors[f"down.{e}"] for e in experts]).to(device=runtime.device, dtype=runtime.dtype).contiguous()
        self.shared_up = self.shared_down = None
        if self.shared_size:
            self.shared_up = Linear(tensors["shared_up"], runtime)
            self.shared_down = Linear(tensors["shared_down"], runtime)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, size = int(p["hidden_size"]), int(p["expert_size"])
        out = {w["router"]: ExpectedTensor((int(p["num_experts"]), hidden))}
        gated = p.get("expert_form") == "gated_silu"
        for e in range(int(p["num_experts"])):
            out[w[f"up.{e}"]] = ExpectedTensor((size, hidden))
            out[w[f"down.{e}"]] = ExpectedTensor((hidden, size))
            if gated:
                out[w[f"gate.{e}"]] = ExpectedTensor((size, hidden))
        if p.get("shared_size"):
            out[w["shared_up"]] = ExpectedTensor((int(p["shared_size"]), hidden))
            out[w["shared_down"]] = ExpectedTensor((hidden, int(p["shared_size"])))
            if gated:
                out[w["shared_gate"]] = ExpectedTensor((int(p["shared_size"]), hidden))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role == "router":
            return torch.randn(shape, generator=generator, dtype=torch.float32) * (4.0 * shape[-1] ** -0.5)
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the products that go through the kernel plan (the shared expert's)."""
        out = [("router", self.router, plan.F32)]
        if self.shared_size:
            out += [("shared up", self.shared_up, plan.BF16),
                    ("shared down", self.shared_down, plan.F32 if self.stream_f32 else plan.BF16)]
        return out

    def route(self, x: torch.Tensor):
        """``(ids int32 [rows, top_k], weights float32 [rows, top_k])`` of the rows of ``x``."""
        rows = x.shape[0]
        ids = torch.empty((rows, self.top_k), dtype=torch.int32, device=x.device)
        weights = torch.empty((rows, self.top_k), dtype=torch.float32, device=x.device)
        logits = self.router.forward(x, float32_out=True)
        if self.scoring == "softmax_all":
            kernels.choose_grouped(logits, ids, weights, groups=self.groups, keep=self.keep_groups,
                                   weight_scale=self.weight_scale)
        else:
            kernels.choose_topk(logits, ids, weights)
        return ids, weights

    def forward(self, x, ctx: StepContext, follow=None):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        rows, device = x.shape[0], x.device
        ids, weights = self.route(x)
        count = rows * self.top_k
        offsets = torch.empty(self.num_experts + 1, dtype=torch.int32, device=device)
        order = torch.empty(count, dtype=torch.int32, device=device)
        kernels.expert_plan(ids, self.num_experts, offsets, order)
        if self.gated:
            gate_up = torch.empty((count, 2 * self.expert_size), dtype=x.dtype, device=device)
            kernels.expert_linear(x, self.up, gate_up, offsets, order, source_div=self.top_k)
            hidden = torch.empty((count, self.expert_size), dtype=x.dtype, device=device)
            kernels.gated_activation(gate_up, None, hidden, kernels.ACT_SILU)
        else:
            hidden = torch.empty((count, self.expert_size), dtype=x.dtype, device=device)
            kernels.expert_linear(x, self.up, hidden, offsets, order, source_div=self.top_k,
                                  epilogue=kernels.EXPERT_SQUARED_RELU)
        parts = torch.empty((count, self.hidden_size), dtype=torch.float32, device=device)
        kernels.expert_linear(hidden, self.down, parts, offsets, order, source_div=1)
        base = None
        if self.shared_size:
            z = self.shared_up.forward(x)
            if self.gated:
                z = kernels.gated_activation(z, None, torch.empty((rows, self.shared_size), dtype=z.dtype, device=device),
                                             kernels.ACT_SILU)
            else:
                kernels.squared_relu(z, z)
            base = self.shared_down.forward(z, float32_out=True)
        out = base if base is not None else torch.empty((rows, self.hidden_size), dtype=torch.float32, device=device)
        kernels.expert_combine(parts, weights, base, out)
        if self.stream_f32 or self.runtime.is_float32:
            return out
        return out.to(self.runtime.dtype)
