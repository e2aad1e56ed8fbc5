"""Arrangement of norms, mixer and feed-forward in a block.

``pre_norm`` is the Llama arrangement (src/cuda/dense_decoder.rs:658-782):

    x  = input_norm(residual [+ pending update])
    a  = mixer(x)
    m  = post_mixer_norm(residual + a)
    f  = feed_forward(m)            -> leaves (residual, f) for the next block's norm

A layer without a feed-forward (``feed_forward`` None) ends after the mixer: ``(residual, a)`` goes to the next
block's norm, and the role ``post_mixer`` needs no norm.

Each addition is fused into the norm that follows it; where the part in front can, its last product does that
norm's work on the way out (``FollowNorm`` -> ``PreparedNorm``), and the product behind only applies the scale.

``parallel`` lets the mixer and the feed-forward read the same stream, each through a norm of its own, and adds
both results:

    x  = residual [+ pending updates]
    a  = mixer(mixer_norm(x))
    f  = feed_forward(feed_forward_norm(x))     -> leaves (x, a, f): the stream is x + (a + f)

Two RMS norms of one row share the row's statistic, so where both norms say so (``shared_statistic``) the pending
sum and both norms are one kernel.  A layer without a feed-forward leaves (x, a).

``sandwich`` norms every sublayer on both sides, over a stream kept in 32-bit:

    x <- x + post_mixer(mixer(pre_mixer(x)))
    x <- x + post_feed_forward(feed_forward(pre_feed_forward(x)))       (absent without a feed-forward)
    x <- x + token_input(x, tokens)                                     (absent without a token input)

The norm of a sublayer's result, the addition and the norm in front of the next sublayer are one kernel
(``norm_add_norm``); it also leaves the rounded stream that the token input's first product reads.

``gated_pre_norm`` is the pre-norm arrangement over a 32-bit stream in which every sublayer's result is weighted, feature
by feature, by a learned scale and by a gate that reads the sublayer's own input:

    h  = input_norm(x);       x <- x + mixer(h) * scale_1 * sigmoid(G_1 h + b_1)
    m  = post_mixer_norm(x);  x <- x + feed_forward(m) * scale_2 * sigmoid(G_2 m + b_2)       (absent without one)

The weighting, the addition and the norm in front of the next sublayer (the next block's first norm, or the final norm)
are one kernel (``gated_add_norm``); the gate's product leaves 32-bit logits.
"""

from __future__ import annotations

from typing import Mapping, Optional, Tuple

from .base import (BLOCKS, Block, CacheBinding, DeferredNorm, FollowNorm, Norm, PreparedNorm, ResidualStream,
                   StepContext)


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    @classmethod
    def norm_roles(cls, with_feed_forward: bool = True) -> Tuple[str, ...]:
        return ("input", "post_mixer") if with_feed_forward else ("input",)

    accepts_next_norm = True

    def entry_norm(self) -> Optional[Norm]:
        return self.norms["input"]

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding],
                next_norm: Optional[Norm] = None) -> ResidualStream:
        # each norm is handed on unevaluated: a part that can fold it into its first kernel does so
        if stream.prepared is not None and stream.prepared.norm is self.norms["input"]:
            first = stream.prepared                       # the block in front already did this norm's work
        else:
            first = DeferredNorm(self.norms["input"], stream.residual, stream.update, stream.update_b)
        x = first if self.mixer.accepts_deferred_norm else first.materialize()
        if self.feed_forward is None:
            return ResidualStream(first.residual, self.mixer.forward(x, ctx, cache))
        if self.mixer.accepts_follow_norm:
            mixed = self.mixer.forward(x, ctx, cache, follow=FollowNorm(self.norms["post_mixer"], first))
        else:
            mixed = self.mixer.forward(x, ctx, cache)
        second = mixed if isinstance(mixed, PreparedNorm) else DeferredNorm(self.norms["post_mixer"], first.residual, mixed)
        m = second if self.feed_forward.accepts_deferred_norm else second.materialize()
        if self.feed_forward.accepts_follow_norm and next_norm is not None:
            update = self.feed_forward.forward(m, ctx, follow=FollowNorm(next_norm, second))
        else:
            update = self.feed_forward.forward(m, ctx)
        if isinstance(update, PreparedNorm):
            return ResidualStream(update.residual, None, prepared=update)
        return ResidualStream(second.residual, update)


@BLOCKS.register("parallel")
class ParallelBlock(Block):
    @classmethod
    def norm_roles(cls, with_feed_forward: bool = True) -> Tuple[str, ...]:
        return ("mixer", "feed_forward") if with_feed_forward else ("mixer",)

    def entry_norm(self) -> Optional[Norm]:
        return self.norms["mixer"]

    def _norms_of_sum(self, stream: ResidualStream):
        """``(x for the mixer, x for the feed-forward or None)``; afterwards ``stream.residual`` holds the sum."""
        import torch

        from .. import kernels

        first, second = self.norms["mixer"], self.norms.get("feed_forward") if self.feed_forward is not None else None
        residual = stream.residual
        one = getattr(first, "shared_statistic", lambda: None)()
        two = getattr(second, "shared_statistic", lambda: None)() if second is not None else None
        updates = [u for u in (stream.update, stream.update_b) if u is not None]
        shared = (one is not None and two is not None and one[1] == two[1] and residual.dtype == torch.float32
                  and residual.is_contiguous() and all(u.dtype == torch.float32 and u.is_contiguous() for u in updates))
        if shared:
            dtype = first.runtime.dtype
            x_mixer = torch.empty(residual.shape, dtype=dtype, device=residual.device)
            x_feed = torch.empty_like(x_mixer)
            kernels.sum_norms(residual, updates[0] if updates else None, updates[1] if len(updates) > 1 else None,
                              one[0], x_mixer, two[0], x_feed, one[1])
            return x_mixer, x_feed
        x_mixer = DeferredNorm(first, residual, stream.update, stream.update_b).materialize()
        return x_mixer, (second.forward(residual) if second is not None else None)

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding]) -> ResidualStream:
        if stream.prepared is not None:
            raise NotImplementedError("a parallel block takes the stream as a residual and its pending updates")
        x_mixer, x_feed = self._norms_of_sum(stream)
        mixed = self.mixer.forward(x_mixer, ctx, cache)
        if self.feed_forward is None:
            return ResidualStream(stream.residual, mixed)
        return ResidualStream(stream.residual, mixed, update_b=self.feed_forward.forward(x_feed, ctx))


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """Norm roles: ``pre_mixer``, ``post_mixer`` and, with a feed-forward, ``pre_feed_forward``, ``post_feed_forward``.
    Every norm offers ``norm_parameters()`` (what ``kernels.norm_add_norm`` takes) and ``eps``; all share one ``eps``."""

    accepts_token_input = True

    def __init__(self, norms, mixer, feed_forward, token_input=None):
        super().__init__(norms, mixer, feed_forward)
        self.token_input = token_input
        for role, norm in self.norms.items():
            if not hasattr(norm, "norm_parameters"):
                raise ValueError(f"a sandwich block's norms describe themselves to the fused kernel; '{norm.kind}' ({role}) does not")
        if len({norm.eps for norm in self.norms.values()}) != 1:
            raise ValueError("the norms of a sandwich block share one eps")
        self.eps = next(iter(self.norms.values())).eps

    @classmethod
    def norm_roles(cls, with_feed_forward: bool = True) -> Tuple[str, ...]:
        both = ("pre_mixer", "post_mixer", "pre_feed_forward", "post_feed_forward")
        return both if with_feed_forward else both[:2]

    def entry_norm(self) -> Optional[Norm]:
        return self.norms["pre_mixer"]

    def forward(self, stream: ResidualStream, ctx: StepContext, cache) -> ResidualStream:
        import torch

        from .. import kernels

        if stream.prepared is not None or stream.update_b is not None:
            raise NotImplementedError("a sandwich block takes the stream as a residual and at most one pending update")
        residual = stream.residual
        if residual.dtype != torch.float32:
            raise NotImplementedError("a sandwich block keeps its stream in 32-bit")
        dtype = self.mixer.runtime.dtype

        def rows_like():
            return torch.empty(residual.shape, dtype=dtype, device=residual.device)

        x = rows_like()
        kernels.norm_add_norm(residual, stream.update, None, self.norms["pre_mixer"].norm_parameters(), x, None, self.eps)
        mixed = self.mixer.forward(x, ctx, cache)
        wants_copy = self.token_input is not None and dtype != torch.float32
        if self.feed_forward is not None:
            x = rows_like()
            kernels.norm_add_norm(residual, mixed, self.norms["post_mixer"].norm_parameters(),
                                  self.norms["pre_feed_forward"].norm_parameters(), x, None, self.eps)
            update, post = self.feed_forward.forward(x, ctx), self.norms["post_feed_forward"]
        else:
            update, post = mixed, self.norms["post_mixer"]
        copy = rows_like() if wants_copy else None
        kernels.norm_add_norm(residual, update, post.norm_parameters(), None, None, copy, self.eps)
        if self.token_input is not None:
            self.token_input.forward(residual, ctx, rounded=copy if wants_copy else residual)
        return ResidualStream(residual, None)


class FinishedNorm(DeferredNorm):
    """``norm(residual)`` that the block in front has already computed together with its last addition: ``residual``
    is complete and ``materialize()`` hands out the rows."""

    def __init__(self, norm: Norm, residual, rows):
        super().__init__(norm, residual, None)
        self._value = rows
        self.done = True


@BLOCKS.register("gated_pre_norm")
class GatedPreNormBlock(Block):
    """Norm roles ``input`` and, with a feed-forward, ``post_mixer``: RMS norms over the whole row of a 32-bit stream
    that offer ``shared_statistic()`` (weight and eps).  ``extras``: per sublayer (``mixer``, ``feed_forward``) the
    scale vector ``scale`` and the gate's ``Linear`` ``gate`` with its bias ``gate_bias``, built by the model from the
    layer's ``residual_gates`` part."""

    accepts_next_norm = True
    accepts_residual_gates = True

    def __init__(self, norms, mixer, feed_forward, residual_gates=None):
        super().__init__(norms, mixer, feed_forward)
        if residual_gates is None:
            raise ValueError("a gated_pre_norm block needs its residual gates")
        self.gates = residual_gates
        for role, norm in self.norms.items():
            if getattr(norm, "shared_statistic", lambda: None)() is None:
                raise ValueError(f"a gated_pre_norm block takes RMS norms over the whole row; '{norm.kind}' ({role}) is not one")

    @classmethod
    def norm_roles(cls, with_feed_forward: bool = True) -> Tuple[str, ...]:
        return ("input", "post_mixer") if with_feed_forward else ("input",)

    def entry_norm(self) -> Optional[Norm]:
        return self.norms["input"]

    def _join(self, residual, update, rows_in, which: str, following: Optional[Norm]):
        """``residual += update * scale * sigmoid(gate(rows_in))``; the rows of ``following`` over the new residual, or None."""
        import torch

        from .. import kernels

        logits = self.gates.logits(which, rows_in)
        statistic = getattr(following, "shared_statistic", lambda: None)() if following is not None else None
        out = weight = None
        eps = 0.0
        if statistic is not None:
            weight, eps = statistic
            out = torch.empty(residual.shape, dtype=following.runtime.dtype, device=residual.device)
        kernels.gated_add_norm(residual, update, logits, self.gates.bias(which), self.gates.scale(which), weight, out, eps)
        return out

    def forward(self, stream: ResidualStream, ctx: StepContext, cache: Optional[CacheBinding],
                next_norm: Optional[Norm] = None) -> ResidualStream:
        import torch

        if stream.update_b is not None:
            raise NotImplementedError("a gated_pre_norm block takes the stream as a residual and at most one pending update")
        residual = stream.residual
        if residual.dtype != torch.float32:
            raise NotImplementedError("a gated_pre_norm block keeps its stream in 32-bit")
        if stream.prepared is not None and stream.prepared.norm is self.norms["input"]:
            h = stream.prepared.materialize()
        else:
            h = DeferredNorm(self.norms["input"], residual, stream.update).materialize()
        mixed = self.mixer.forward(h, ctx, cache)
        last = self.feed_forward is None
        rows = self._join(residual, mixed, h, "mixer", next_norm if last else self.norms["post_mixer"])
        if not last:
            if rows is None:
                rows = self.norms["post_mixer"].forward(residual)
            update = self.feed_forward.forward(rows, ctx)
            rows = self._join(residual, update, rows, "feed_forward", next_norm)
        if rows is not None:
            return ResidualStream(residual, None, prepared=FinishedNorm(next_norm, residual, rows))
        return ResidualStream(residual, None)
