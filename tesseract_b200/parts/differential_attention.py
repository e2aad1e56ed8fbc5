"""Grouped-query attention with two score maps per head over the same values.

Per row ``h`` (the mixer's input), with ``H`` heads, ``G`` kv heads, ``dim`` numbers per map and ``vdim`` per value:

* one fused product gives the queries (``H * 2 * dim``: per head its two maps side by side), keys (``G * 2 * dim``),
  values (``G * vdim``) and, with ``gate``, the output gate (``H * vdim``);
* the position encoding (``rotary_pairs``) turns every map of every query and key head; rotated keys and the values
  go into the request's pages;
* each map is a softmax attention of its own (scores ``(q . k) * scale``, causal or windowed mask) over the kv
  head's values; with ``a1``, ``a2`` the two outputs of a head, ``o = a1 - lambda a2`` is divided by
  ``sqrt(mean(o^2) + eps)`` over the head and multiplied by ``post_scale``;
* with ``gate`` the concatenated heads are multiplied by ``sigmoid(gate)``; then the output projection.

To the attention kernel the maps are query heads: the query rows of the weight are reordered once, at load, to
``[kv head][map][head within the group]``, so that a run of ``H / G`` query heads reads key head ``2 g + map``, and
both key heads of a group read value head ``g`` (``keys_per_value = 2``).  In bfloat16, with head sizes they are built
for, the tensor-core kernels take it (prompt portions in tiles, few rows a block each); the 32-bit row kernel otherwise.
The kernel leaves its weighted sums in 32-bit;
the subtraction, the norm and the gate are one kernel behind it, 32-bit up to the single rounding of its output.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, POSITION_ENCODINGS, DeferredNorm, Mixer, PagedKeyValueNeed, Runtime, StepContext
from .linear import Linear

_MASKS = {"causal": kernels.MASK_CAUSAL, "window": kernels.MASK_WINDOW}


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, key_dim`` (of one map)``, value_dim, scale``, ``lambda_offset``
    (``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_offset``), ``post_scale``, ``eps``, ``mask``, ``gate`` (bool),
    optional ``stream``.  weights: ``q, k, v, o, lq1, lk1, lq2, lk2`` and, with ``gate``, ``g``.  children: ``position``."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.key_dim = int(p["key_dim"])
        self.value_dim = int(p["value_dim"])
        self.scale = float(p["scale"])
        self.post_scale = float(p["post_scale"])
        self.eps = float(p["eps"])
        self.gated = bool(p.get("gate"))
        self.stream_f32 = p.get("stream") == "float32"
        mask = dict(p.get("mask") or {"kind": "causal"})
        if mask.get("kind") not in _MASKS:
            raise ValueError(f"mask kind must be one of {sorted(_MASKS)}, got {mask.get('kind')!r}")
        self.mask_kind = mask["kind"]
        self.mask_size = int(mask.get("size") or 0)
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (1 <= self.key_dim <= 1024 and 1 <= self.value_dim <= 512):
            raise ValueError("the attention kernel takes keys of up to 1024 and values of up to 512 numbers a head")
        H, G, d = self.num_heads, self.num_kv_heads, self.key_dim
        per = H // G
        # lambda: 32-bit sums and exponentials of the four vectors, once, at load
        vectors = [tensors[name].to(torch.float32) for name in ("lq1", "lk1", "lq2", "lk2")]
        first, second = (vectors[0] * vectors[1]).sum(), (vectors[2] * vectors[3]).sum()
        self.lam = float(torch.exp(first) - torch.exp(second) + torch.tensor(float(p["lambda_offset"]), dtype=torch.float32))
        # query rows [head][map][dim] -> [kv head][map][head within the group][dim]
        q = tensors["q"].view(G, per, 2, d, self.hidden_size).permute(0, 2, 1, 3, 4).reshape(H * 2 * d, self.hidden_size)
        rows = [q, tensors["k"], tensors["v"]] + ([tensors["g"]] if self.gated else [])
        self.in_proj = Linear(torch.cat(rows, dim=0), runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        self.q_width = H * 2 * d
        self.gate_offset = self.q_width + G * 2 * d + G * self.value_dim
        position_spec = spec.children.get("position") or PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if self.position.kind not in ("rotary_pairs", "none"):
            raise ValueError(f"differential_attention rotates pairs or not at all, got position encoding '{self.position.kind}'")
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.inv_freq = getattr(self.position, "pair_inv_freq", None)

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, d, dv = int(p["hidden_size"]), int(p["key_dim"]), int(p["value_dim"])
        heads, kv = int(p["num_heads"]), int(p["num_kv_heads"])
        out = {w["q"]: ExpectedTensor((heads * 2 * d, hidden)), w["k"]: ExpectedTensor((kv * 2 * d, hidden)),
               w["v"]: ExpectedTensor((kv * dv, hidden)), w["o"]: ExpectedTensor((hidden, heads * dv))}
        for name in ("lq1", "lk1", "lq2", "lk2"):
            out[w[name]] = ExpectedTensor((d,))
        if p.get("gate"):
            out[w["g"]] = ExpectedTensor((heads * dv, hidden))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role in ("lq1", "lk1", "lq2", "lk2"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.3
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's matrix products, for the printed kernel plan."""
        return [("q/k/v/gate", self.in_proj, plan.BF16), ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def attention_choice(self, rows: int) -> str:
        """The attention kernel of a step of ``rows`` rows (both maps of all heads in one launch)."""
        return plan.masked_attention(self.runtime.dtype, rows, self.key_dim, self.value_dim,
                                     heads_per_kv=self.num_heads // self.num_kv_heads)

    def cache_need(self):
        return PagedKeyValueNeed(num_kv_heads=2 * self.num_kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                                 window=self.mask_size if self.mask_kind == "window" else None,
                                 num_value_heads=self.num_kv_heads)

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        if cache is None or cache.storage is None:
            raise RuntimeError("differential_attention needs a paged key/value cache binding")
        if not cache.writes:
            raise NotImplementedError("differential_attention keeps a cache of its own")
        group = ctx.groups[cache.group]
        proj = self.in_proj.forward(x)
        rows = proj.shape[0]
        H, G = self.num_heads, self.num_kv_heads
        q = torch.empty((rows, self.q_width), dtype=proj.dtype, device=proj.device)
        kernels.pair_rope_cache(proj, q, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table, self.inv_freq,
                                q_heads=2 * H, key_heads=2 * G, value_heads=G, dim=self.key_dim, vdim=self.value_dim,
                                rot_dims=self.rot_dims, page_size=cache.page_size)
        maps = torch.empty((rows, 2 * H * self.value_dim), dtype=torch.float32, device=proj.device)
        choice = self.attention_choice(rows)
        common = dict(heads=2 * H, kv_heads=2 * G, dim=self.key_dim, vdim=self.value_dim, page_size=cache.page_size,
                      mask_kind=_MASKS[self.mask_kind], mask_size=self.mask_size, scale=self.scale, keys_per_value=2)
        if choice == "attention_rows_mma":
            kernels.attention_rows_mma(q, maps, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table, **common)
        elif choice == "attention_prompt_mma":
            kernels.attention_prompt_mma(q, maps, cache.storage, ctx.positions, ctx.row_start, group.block_table,
                                         num_seqs=ctx.num_seqs, **common)
        else:
            kernels.attention_masked(q, None, maps, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                     sink=False, **common)
        out = torch.empty((rows, H * self.value_dim), dtype=proj.dtype, device=proj.device)
        kernels.differential_combine(maps, proj[:, self.gate_offset:] if self.gated else None, out, heads=H, kv_heads=G,
                                     vdim=self.value_dim, lam=self.lam, post=self.post_scale, eps=self.eps)
        return self.o_proj.forward(out, float32_out=self.stream_f32)
