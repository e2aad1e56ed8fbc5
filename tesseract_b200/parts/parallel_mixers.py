"""Two mixers side by side: both read the same rows, and the mixer's result is a weighted sum of theirs.

    y = left_scale * left(h) + right_scale * right(h)

``left`` and ``right`` are mixers of any registered kind, each with its own sizes, tensors and cache need (pages for
one, a state slot for the other, say); this part hands each its share of the run entry's cache bindings.  Both leave
32-bit rows (a residual stream kept in 32-bit) and the sum is taken in 32-bit.
"""

from __future__ import annotations

from typing import Dict, Mapping, Tuple

import torch

from .. import kernels
from ..config.spec import PartSpec
from ..weights.loader import ExpectedTensor
from .base import MIXERS, DeferredNorm, Mixer, Runtime, StepContext

_SIDES = ("left", "right")


def _needs_of(need) -> Tuple[object, ...]:
    if need is None:
        return ()
    return tuple(need) if isinstance(need, tuple) else (need,)


@MIXERS.register("parallel_mixers")
class ParallelMixers(Mixer):
    """params: ``hidden_size, left_scale, right_scale``; children: ``left``, ``right`` (mixer descriptions, each with its
    own ``weights``); weights: every tensor of a child under the child's role with ``left.`` or ``right.`` in front."""

    def __init__(self, spec: PartSpec, tensors: Mapping[str, torch.Tensor], runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        p, children = spec.params, spec.children
        self.hidden_size = int(p["hidden_size"])
        self.scales = (float(p["left_scale"]), float(p["right_scale"]))
        self.sides = []
        for side in _SIDES:
            child = children[side]
            mine = {role[len(side) + 1:]: t for role, t in tensors.items() if role.startswith(side + ".")}
            self.sides.append(MIXERS.get(child.kind)(child, mine, runtime))
        self.graph_safe = all(getattr(part, "graph_safe", False) for part in self.sides)
        self._counts = [len(_needs_of(part.cache_need())) for part in self.sides]

    @staticmethod
    def lifted_weights(children: Mapping[str, PartSpec]) -> Dict[str, str]:
        """The ``weights`` of a description whose children are ``children``: every child's roles with its side in front."""
        return {f"{side}.{role}": name for side in _SIDES for role, name in children[side].weights.items()}

    @classmethod
    def expected_tensors(cls, spec: PartSpec) -> Dict[str, ExpectedTensor]:
        out: Dict[str, ExpectedTensor] = {}
        for side in _SIDES:
            child = spec.children[side]
            out.update(MIXERS.get(child.kind).expected_tensors(child))
        return out

    @classmethod
    def random_tensor(cls, spec, role, shape, generator) -> torch.Tensor:
        side, _, inner = role.partition(".")
        child = spec.children[side]
        return MIXERS.get(child.kind).random_tensor(child, inner, shape, generator)

    def products(self):
        """``(name, Linear, epilogue)`` of both mixers' matrix products, for the printed kernel plan."""
        out = []
        for side, part in zip(_SIDES, self.sides):
            out += [(f"{side} {name}", linear, epilogue) for name, linear, epilogue in getattr(part, "products", lambda: [])()]
        return out

    def cache_need(self):
        needs = tuple(n for part in self.sides for n in _needs_of(part.cache_need()))
        return needs if needs else None

    def forward(self, x, ctx: StepContext, cache):
        if isinstance(x, DeferredNorm):
            x = x.materialize()
        bindings = tuple(cache) if isinstance(cache, tuple) else (() if cache is None else (cache,))
        if len(bindings) != sum(self._counts):
            raise RuntimeError(f"parallel_mixers: {sum(self._counts)} cache bindings expected, got {len(bindings)}")
        results, at = [], 0
        for part, count in zip(self.sides, self._counts):
            share = bindings[at:at + count]
            at += count
            results.append(part.forward(x, ctx, None if count == 0 else (share[0] if count == 1 else share)))
        left, right = results
        if left.dtype != torch.float32 or right.dtype != torch.float32:
            raise NotImplementedError("parallel_mixers adds 32-bit rows (its mixers leave them for a 32-bit stream)")
        return kernels.blend_rows(left, right, self.scales[0], self.scales[1])
