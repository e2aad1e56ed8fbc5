"""Grouped-query attention whose queries and keys are brought to unit root mean square after the rotation.

Per row ``h`` (the mixer's input):

* one fused product gives the queries (``num_heads * key_dim``), keys (``num_kv_heads * key_dim``) and values
  (``num_kv_heads * value_dim``); query head ``i`` reads kv head ``i // (num_heads / num_kv_heads)``;
* the position encoding (``rotary_blend``, rotate-half layout) turns the first ``dims`` numbers of every query and
  key head; with ``qk_norm_eps`` every query and key head is then divided by ``sqrt(mean(head^2) + qk_norm_eps)``
  (no weight); rotated, normalised keys and the values go into the request's pages;
* every row attends over the keys its mask lets it see: ``causal`` (all up to its own position), ``window`` (its own
  and the ``size - 1`` positions before it; older pages go back to the pool) or ``window_pooled``: the window and, for
  every block of ``pool`` positions that ends in front of it (blocks are counted from position 0; block ``b`` is seen
  from position ``p`` if ``(b + 1) * pool <= p - size + 1``), one key and one value that are the averages of the block's
  keys and values as the pages hold them; so for up to ``pool - 1`` steps a token is visible neither by itself nor through
  its block.  The averages live in pages of their own (an entry a block) and are written by the step that brings a
  block's last token.  Scores ``(q . k) * scale``, with ``softcap`` then ``softcap * tanh(score / softcap)``, the softmax
  and the weights are 32-bit; with ``sink`` the denominator also holds ``exp`` of a learned number per query head;
* with ``bias`` the three projections add a bias each;
* the output projection's result comes out in 32-bit for a residual stream kept in 32-bit (``stream`` = ``"float32"``).

Rotation, normalisation and the cache write are one kernel; the attention kernel is the one the other mixers with
keys and values of separate widths use, or, for bfloat16 steps of many rows and head sizes it is built for, the
tensor-core kernel with the same masks and 32-bit scores and weights (the kernel plan decides).
"""

from __future__ import annotations

from typing import Dict, Mapping

import torch

from .. import kernels, plan
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import (MIXERS, POSITION_ENCODINGS, DeferredNorm, Mixer, PagedKeyValueNeed, PooledBlocksNeed, Runtime,
                   StepContext)
from .linear import Linear

_MASKS = {"causal": kernels.MASK_CAUSAL, "window": kernels.MASK_WINDOW, "window_pooled": kernels.MASK_WINDOW_POOLED}


@MIXERS.register("normed_attention")
class NormedAttention(Mixer):
    """params: ``hidden_size, num_heads, num_kv_heads, key_dim, value_dim, scale``, ``mask`` (``{"kind": "causal" |
    "window" | "window_pooled", "size": n, "pool": P}``), ``qk_norm_eps`` (None: queries and keys stay as rotated),
    optional ``softcap``, ``sink`` (bool), ``bias`` (bool), ``stream``.  weights: ``q, k, v, o``, with ``bias`` also
    ``q_bias, k_bias, v_bias``, with ``sink`` also ``sink`` ``[num_heads]``.  children: ``position``."""

    graph_safe = True      # reads only device-side metadata of the step (and its shape)

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p = spec.params
        self.hidden_size = int(p["hidden_size"])
        self.num_heads = int(p["num_heads"])
        self.num_kv_heads = int(p["num_kv_heads"])
        self.key_dim = int(p["key_dim"])
        self.value_dim = int(p["value_dim"])
        self.scale = float(p["scale"])
        mask = dict(p.get("mask") or {"kind": "causal"})
        if mask.get("kind") not in _MASKS:
            raise ValueError(f"mask kind must be one of {sorted(_MASKS)}, got {mask.get('kind')!r}")
        self.mask_kind = mask["kind"]
        self.mask_size = int(mask.get("size") or 0)
        if self.mask_kind != "causal" and self.mask_size < 1:
            raise ValueError(f"a '{self.mask_kind}' mask needs a positive size")
        self.pool = int(mask.get("pool") or 0)
        if self.mask_kind == "window_pooled" and self.pool < 1:
            raise ValueError("a 'window_pooled' mask needs a positive pool")
        self.softcap = float(p.get("softcap") or 0.0)
        if self.softcap < 0.0:
            raise ValueError("softcap must not be negative")
        self.sinks = runtime.vector_f32(tensors["sink"]) if p.get("sink") else None
        self.biased = bool(p.get("bias"))
        eps = p.get("qk_norm_eps")
        self.unit_norm = eps is not None
        self.qk_norm_eps = float(eps) if eps is not None else 0.0
        self.stream_f32 = p.get("stream") == "float32"
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if not (1 <= self.key_dim <= 1024 and 1 <= self.value_dim <= 512):
            raise ValueError("the attention kernel takes keys of up to 1024 and values of up to 512 numbers a head")
        self.q_width = self.num_heads * self.key_dim
        self.o_width = self.num_heads * self.value_dim
        # (the biases are added by the kernel behind the product, in 32-bit, in front of its rotation)
        self.in_bias = None
        if self.biased:
            self.in_bias = torch.cat([tensors["q_bias"], tensors["k_bias"], tensors["v_bias"]]).to(
                device=runtime.device, dtype=torch.float32).contiguous()
        self.in_proj = Linear(torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0), runtime)
        self.o_proj = Linear(tensors["o"], runtime)
        position_spec = spec.children.get("position") or PartSpec.make("none")
        self.position = POSITION_ENCODINGS.get(position_spec.kind)(position_spec, {}, runtime)
        if self.position.kind not in ("rotary_blend", "none"):
            raise ValueError(f"normed_attention rotates halves or not at all, got position encoding '{self.position.kind}'")
        self.rot_dims = int(getattr(self.position, "dims", 0))
        self.inv_freq = getattr(self.position, "half_inv_freq", None)
        self.amplitude = float(getattr(self.position, "amplitude", 1.0))
        if self.rot_dims > self.key_dim:
            raise ValueError("the rotation covers more numbers than a key has")

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        p, w = spec.params, spec.weights
        hidden, d, dv = int(p["hidden_size"]), int(p["key_dim"]), int(p["value_dim"])
        heads, kv = int(p["num_heads"]), int(p["num_kv_heads"])
        out = {
            w["q"]: ExpectedTensor((heads * d, hidden)),
            w["k"]: ExpectedTensor((kv * d, hidden)),
            w["v"]: ExpectedTensor((kv * dv, hidden)),
            w["o"]: ExpectedTensor((hidden, heads * dv)),
        }
        if p.get("bias"):
            out.update({w["q_bias"]: ExpectedTensor((heads * d,)), w["k_bias"]: ExpectedTensor((kv * d,)),
                        w["v_bias"]: ExpectedTensor((kv * dv,))})
        if p.get("sink"):
            out[w["sink"]] = ExpectedTensor((heads,))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        if role.endswith("_bias"):
            return torch.randn(shape, generator=generator, dtype=torch.float32) * 0.3
        if role == "sink":
            return torch.randn(shape, generator=generator, dtype=torch.float32)
        return torch.randn(shape, generator=generator, dtype=torch.float32) * (shape[-1] ** -0.5)

    def products(self):
        """``(name, Linear, epilogue)`` of the mixer's matrix products, for the printed kernel plan."""
        from .. import plan

        return [("q/k/v", self.in_proj, plan.BF16), ("o", self.o_proj, plan.F32 if self.stream_f32 else plan.BF16)]

    def cache_need(self):
        if self.mask_kind == "window_pooled":
            # the tokens of a block stay until the block is averaged, although the window may have passed them
            return (PagedKeyValueNeed(num_kv_heads=self.num_kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                                      window=self.mask_size, hold=self.pool),
                    PooledBlocksNeed(num_kv_heads=self.num_kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                                     pool=self.pool))
        return PagedKeyValueNeed(num_kv_heads=self.num_kv_heads, key_dim=self.key_dim, value_dim=self.value_dim,
                                 window=self.mask_size if self.mask_kind == "window" else None)

    def attention_choice(self, rows: int) -> str:
        """The attention kernel of a step of ``rows`` rows (all three know the cap, the learned sink and pooled blocks)."""
        return plan.masked_attention(self.runtime.dtype, rows, self.key_dim, self.value_dim,
                                     heads_per_kv=self.num_heads // self.num_kv_heads)

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        pooled = None
        if self.mask_kind == "window_pooled":
            if not isinstance(cache, tuple) or len(cache) != 2:
                raise RuntimeError("a pooled window needs two cache bindings: the tokens' pages and the blocks'")
            cache, pooled = cache
        if cache is None or cache.storage is None:
            raise RuntimeError("normed_attention needs a paged key/value cache binding")
        if not cache.writes:
            raise NotImplementedError("normed_attention keeps a cache of its own: a run entry cannot read another entry's")
        group = ctx.groups[cache.group]
        proj = self.in_proj.forward(x)
        rows = proj.shape[0]
        q = torch.empty((rows, self.q_width), dtype=proj.dtype, device=proj.device)
        kernels.rope_norm_cache(proj, q, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table, self.inv_freq,
                                amplitude=self.amplitude, heads=self.num_heads, kv_heads=self.num_kv_heads,
                                dim=self.key_dim, vdim=self.value_dim, rot_dims=self.rot_dims,
                                unit_norm=self.unit_norm, eps=self.qk_norm_eps, page_size=cache.page_size,
                                bias=self.in_bias)
        extras = {"sinks": self.sinks, "softcap": self.softcap}
        if pooled is not None:
            pool_table = ctx.groups[pooled.group].block_table
            kernels.pool_blocks(cache.storage, pooled.storage, ctx.positions, ctx.seq_of_row, group.block_table, pool_table,
                                kv_heads=self.num_kv_heads, dim=self.key_dim, vdim=self.value_dim,
                                page_size=cache.page_size, pool=self.pool)
            extras["pooled"] = (pooled.storage, pool_table, self.pool)
        attended = torch.empty((rows, self.o_width), dtype=proj.dtype, device=proj.device)
        choice = self.attention_choice(rows)
        if choice == "attention_rows_mma":
            kernels.attention_rows_mma(q, attended, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                       heads=self.num_heads, kv_heads=self.num_kv_heads, dim=self.key_dim,
                                       vdim=self.value_dim, page_size=cache.page_size, mask_kind=_MASKS[self.mask_kind],
                                       mask_size=self.mask_size, scale=self.scale, **extras)
        elif choice == "attention_prompt_mma":
            kernels.attention_prompt_mma(q, attended, cache.storage, ctx.positions, ctx.row_start, group.block_table,
                                         num_seqs=ctx.num_seqs, heads=self.num_heads, kv_heads=self.num_kv_heads,
                                         dim=self.key_dim, vdim=self.value_dim, page_size=cache.page_size,
                                         mask_kind=_MASKS[self.mask_kind], mask_size=self.mask_size, scale=self.scale,
                                         **extras)
        else:
            kernels.attention_masked(q, None, attended, cache.storage, ctx.positions, ctx.seq_of_row, group.block_table,
                                     heads=self.num_heads, kv_heads=self.num_kv_heads, dim=self.key_dim,
                                     vdim=self.value_dim, page_size=cache.page_size, mask_kind=_MASKS[self.mask_kind],
                                     mask_size=self.mask_size, sink=False, scale=self.scale, **extras)
        return self.o_proj.forward(attended, float32_out=self.stream_f32)
