"""Attention whose keys and values are projections of one latent vector per token.

Per row ``h`` (the mixer's input), with ``H`` heads, per head ``dim`` plain and ``rot_width`` rotated query/key numbers,
values of ``vdim`` and a latent of ``rank``:

* ``q = Wq h`` is laid out head by head as ``[dim plain | rot_width rotated]``;
* ``Wd h`` gives ``rank + rot_width`` numbers: the first ``rank``, divided by their root mean square and weighted, are the
  latent ``c``; the rest is one rotated key part shared by all heads.  The page keeps ``[c | rotated part]`` per token;
* head ``i`` has plain keys ``Uk_i c`` and values ``Uv_i c``; its score is ``(q_plain . Uk_i c + q_rot . k_rot) * scale``;
  softmax over the keys the mask lets a row see (causal or a sliding window).

Scores and outputs are taken in the latent space, so nothing per head is ever kept per token:
``q_plain . (Uk_i c) = (Uk_i^T q_plain) . c`` and ``sum_j w_j Uv_i c_j = Uv_i (sum_j w_j c_j)``.  A batched product
turns every head's plain query into ``rank`` numbers, the attention kernel runs with one key head of
``rank + rot_width`` numbers whose first ``rank`` are also its value, and a second batched product takes every head's
output to ``vdim`` numbers; then the output projection.  In bfloat16, for the latent sizes it is built for, the
attention kernel is the tensor-core one over cached vectors (a block a row and sixteen heads), else the 32-bit row
kernel.  Scores, softmax, weights and the weighted sums are 32-bit in the attention kernel; rotation, the latent's norm and the cache write are one kernel in front of it.
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, POSITION_ENCODINGS, DeferredNorm, Mixer, PagedVectorNeed, Runtime, StepContext
from .linear import Linear

_MASKS = {"causal": kernels.MASK_CAUSAL, "window": kernels.MASK_WINDOW}


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: ``hidden_size, num_heads, key_dim`` (plain)``, rot_width, value_dim, rank, scale, eps``, ``mask``, optional
    ``stream``, ``gate`` (bool: the concatenated heads are multiplied by ``sigmoid(Wg h)`` in front of the output
    projection).  weights: ``q, down, down_norm, up_k, up_v, o`` and, with ``gate``, ``g``.  children: ``position`` (over
    ``rot_width``; its ``amplitude``, if it has one, multiplies cosine and sine)."""

    graph_safe = True

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.key_dim = int(p["key_dim"])
        self.rot_width = int(p["rot_width"])
        self.value_dim = int(p["value_dim"])
        self.rank = int(p["rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.stream_f32 = p.get("stream") == "float32"
        mask = dict(p.get("mask") or {"kind": "causal"})
        if mask.get("kind") not in _MASKS:
            raise ValueError(f"mask kind must be one of {sorted(_MASKS)}, got {mask.get('kind')!r}")
        self.mask_kind = mask["kind"]
        self.mask_size = int(mask.get("size") or 0)
        if self.mask_kind == "window" and self.mask_size < 1:
            raise ValueError("a 'window' mask needs a positive size")
        self.entry = self.rank + self.rot_width          # what a page keeps per token, and a query head's width
        if not (1 <= self.entry <= 1024 and 1 <= self.rank <= 512):
            raise ValueError("the attention kernel takes a latent of up to 512 numbers and entries of up to 1024")
        H = self.num_heads
        self.gated = bool(p.get("gate"))
        self.q_width = H * (self.key_dim + self.rot_width)
        # (queries and the gate's pre-activations leave one product)
        self.q_proj = Linear(torch.cat([tensors["q"], tensors["g"]], dim=0) if self.gated else tensors["q"], runtime)
        self.down_proj = Linear(tensors["down"], runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        self.down_norm = runtime.vector_f32(tensors["down_norm"])
        # per head: [rank, dim] (the key matrix transposed) and [vdim, rank], as the batched products read them
        self.up_k_t = runtime.matrix(tensors["up_k"]).view(H, self.key_dim, self.rank).transpose(1, 2).contiguous()
        self.up_v = runtime.matrix(tensors["up_v"]).view(H, self.value_dim, self.rank)
        position_spec = spec.children.get("position") or PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if self.position.kind not in ("rotary_pairs", "none"):
            raise ValueError(f"latent_attention rotates pairs or not at all, got position encoding '{self.position.kind}'")
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.inv_freq = getattr(self.position, "pair_inv_freq", None)
        self.amplitude = float(getattr(self.position, "amplitude", 1.0))
        if self.rot_dims > self.rot_width:
            raise ValueError("the rotation covers more numbers than the rotated part has")

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, heads, d, dr = int(p["hidden_size"]), int(p["num_heads"]), int(p["key_dim"]), int(p["rot_width"])
        dv, rank = int(p["value_dim"]), int(p["rank"])
        out = {w["q"]: ExpectedTensor((heads * (d + dr), hidden)), w["down"]: ExpectedTensor((rank + dr, hidden)),
               w["down_norm"]: ExpectedTensor((rank,)), w["up_k"]: ExpectedTensor((heads * d, rank)),
               w["up_v"]: ExpectedTensor((heads * dv, rank)), w["o"]: ExpectedTensor((hidden, heads * dv))}
        if p.get("gate"):
            out[w["g"]] = ExpectedTensor((heads * dv, hidden))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role == "down_norm":
            return 1.0 + torch.randn(shape, generator=generator, dtype=torch.float32) * 0.1
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's planned matrix products, for the printed kernel plan."""
        return [("q/gate" if self.gated else "q", self.q_proj, plan.BF16), ("down", self.down_proj, plan.F32),
                ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def attention_choice(self, rows: int) -> str:
        """The attention kernel of a step of ``rows`` rows: one key head as wide as the cached entry."""
        return plan.latent_attention(self.runtime.dtype, self.entry, self.rank)

    def cache_need(self):
        return PagedVectorNeed(width=self.entry, window=self.mask_size if self.mask_kind == "window" else None)

    def _per_head(self, rows_in: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
        """``out[:, i, :] = rows_in[:, i, :] @ weight[i]^T`` for every head ``i`` (views ``[rows, H, *]``)."""
        if self.runtime.is_float32:
            for head in range(self.num_heads):          # the package's own 32-bit product, a head at a time
                kernels.gemm_f32_nt(rows_in[:, head, :], weight[head], out[:, head, :])
        else:
            torch.bmm(rows_in.transpose(0, 1), weight.transpose(1, 2), out=out.transpose(0, 1))

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        if cache is None or cache.storage is None:
            raise RuntimeError("latent_attention needs a paged cache binding")
        if not cache.writes:
            raise NotImplementedError("latent_attention keeps a cache of its own")
        group = ctx.groups[cache.group]
        H, d, dr, rank, dv = self.num_heads, self.key_dim, self.rot_width, self.rank, self.value_dim
        q = self.q_proj.forward(x)
        gate = None
        if self.gated:
            q, gate = q[:, :self.q_width], q[:, self.q_width:]
        down = self.down_proj.forward(x, float32_out=True)       # the latent's norm reads 32-bit numbers
        rows = q.shape[0]
        q_full = torch.empty((rows, H * self.entry), dtype=q.dtype, device=q.device)
        self._per_head(q.view(rows, H, d + dr)[:, :, :d], self.up_k_t, q_full.view(rows, H, self.entry)[:, :, :rank])
        kernels.latent_rope_cache(down, q, q_full, cache.storage, self.down_norm, ctx.positions, ctx.seq_of_row,
                                  group.block_table, self.inv_freq, heads=H, dim=d, rank=rank, rot_width=dr,
                                  rot_dims=self.rot_dims, page_size=cache.page_size, eps=self.eps, amplitude=self.amplitude)
        mixed = torch.empty((rows, H * rank), dtype=q.dtype, device=q.device)
        if self.attention_choice(rows) == "attention_latent_mma":
            kernels.attention_latent_mma(q_full, mixed, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                         heads=H, dim=self.entry, vdim=rank, page_size=cache.page_size,
                                         mask_kind=_MASKS[self.mask_kind], mask_size=self.mask_size, scale=self.scale)
        else:
            kernels.attention_masked(q_full, None, mixed, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                     heads=H, kv_heads=1, dim=self.entry, vdim=rank, page_size=cache.page_size,
                                     mask_kind=_MASKS[self.mask_kind], mask_size=self.mask_size, sink=False,
                                     scale=self.scale, keys_per_value=0)
        out = torch.empty((rows, H * dv), dtype=q.dtype, device=q.device)
        self._per_head(mixed.view(rows, H, rank), self.up_v, out.view(rows, H, dv))
        if gate is not None:
            kernels.sigmoid_mul(out, gate, out)
        return self.o_proj.forward(out, float32_out=self.stream_f32)
