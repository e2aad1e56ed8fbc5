"""Rotary position encoding (rotate-half) with optional Llama-3 frequency scaling.

Inverse frequencies are computed on the host in 32-bit exactly as the reference does
(src/cuda/dense_decoder.rs:1516-1544): ``f = 1 / theta^(2i/d)``; wavelength ``2*pi/f``;
unchanged above the high-frequency cut, divided by ``factor`` below the low-frequency
cut, interpolated between.  The angle of position ``p`` is ``float32(p) * f'_i``
(src/cuda/dense_decoder.rs:1549-1556); the kernels take cos and sin of it in 32-bit
instead of reading a ``[max_position, d/2]`` table.
"""

from __future__ import annotations

import math
from typing import Mapping, Optional

import numpy as np
import torch

from .. import kernels
from ..config.spec import PartSpec
from .base import POSITION_ENCODINGS, PositionEncoding, Runtime


def rotary_inverse_frequencies(head_dim: int, theta: float, scaling: Optional[Mapping[str, float]]) -> np.ndarray:
    """float32 ``[head_dim/2]`` inverse frequencies, Llama-3 scaled when ``scaling`` is given."""
    f32 = np.float32
    half = head_dim // 2
    out = np.empty(half, dtype=np.float32)
    theta32 = f32(theta)
    for index in range(half):
        exponent = f32(2 * index) / f32(head_dim)
        base = f32(1.0) / np.power(theta32, exponent, dtype=np.float32)
        frequency = base
        if scaling is not None:
            original = f32(scaling["original_max_position_embeddings"])
            low_ff = f32(scaling["low_freq_factor"])
            high_ff = f32(scaling["high_freq_factor"])
            factor = f32(scaling["factor"])
            wavelength = f32(2.0 * math.pi) / base
            low_wavelength = original / low_ff
            high_wavelength = original / high_ff
            if wavelength < high_wavelength:
                frequency = base
            elif wavelength > low_wavelength:
                frequency = base / factor
            else:
                smooth = (original / wavelength - low_ff) / (high_ff - low_ff)
                frequency = (f32(1.0) - smooth) * base / factor + smooth * base
        out[index] = frequency
    return out


@POSITION_ENCODINGS.register("rotary")
class RotaryEncoding(PositionEncoding):
    """params: ``head_dim``, ``theta``, ``scaling`` (mapping or None)."""

    def __init__(self, spec: PartSpec, tensors, runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.head_dim = int(params["head_dim"])
        scaling = params.get("scaling")
        self.inv_freq_host = rotary_inverse_frequencies(self.head_dim, float(params["theta"]),
                                                        dict(scaling) if scaling else None)
        self.rotary_inv_freq = torch.from_numpy(self.inv_freq_host).to(runtime.device)

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError("rotary encoding is applied by the attention mixer's fused rotate-and-store kernel")


def banded_inverse_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]]) -> np.ndarray:
    """float64 ``[dims / 2]``: ``f_i = base^(-2i / dims)`` and, with ``scaling`` (``factor``, ``low``, ``high``,
    ``original``), three bands by wavelength ``l = 2 pi / f``: short ones (``l < original / high``) keep ``f``, long ones
    (``l > original / low``) take ``f / factor``, and between them ``(1 - s) f / factor + s f`` with
    ``s = (original / l - low) / (high - low)``."""
    out = np.asarray([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)
    if not scaling:
        return out
    factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
    original = float(scaling["original"])
    for i, f in enumerate(out):
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            continue
        if wavelength > original / low:
            out[i] = f / factor
        else:
            s = (original / wavelength - low) / (high - low)
            out[i] = (1.0 - s) * f / factor + s * f
    return out


@POSITION_ENCODINGS.register("rotary_pairs")
class RotaryPairs(PositionEncoding):
    """Rotation of neighbouring pairs: of every head's first ``dims`` numbers, numbers ``2i`` and ``2i + 1`` turn by
    ``position * base^(-2i / dims)``; the rest of the head passes unchanged.

    params: ``head_dim``, ``dims`` (even, at most ``head_dim``), ``base``, optional ``scaling``: a mapping with ``factor``,
    ``low``, ``high``, ``original`` (:func:`banded_inverse_frequencies`), or one with ``factor``, ``original``, ``fast``,
    ``slow`` (:func:`blended_inverse_frequencies`, which also raises ``amplitude``, the factor on cosine and sine, above
    1).  The frequencies are taken in 64-bit on
    the host and rounded once to 32-bit; the angle and its sine and cosine are 32-bit, in the kernel that applies
    them (the mixer's rotate-and-store kernel reads ``pair_inv_freq`` and ``dims``)."""

    def __init__(self, spec: PartSpec, tensors, runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.head_dim = int(params["head_dim"])
        self.dims = int(params["dims"])
        self.base = float(params["base"])
        if self.dims < 0 or self.dims % 2 or self.dims > self.head_dim:
            raise ValueError(f"rotation over pairs needs an even number of dimensions up to {self.head_dim}, got {self.dims}")
        if not self.base > 0.0:
            raise ValueError("the rotation's base must be positive")
        scaling = params.get("scaling")
        self.amplitude = 1.0
        if scaling and "fast" in dict(scaling):
            if self.base == 1.0:
                raise ValueError("blended frequencies need a base other than 1")
            frequencies, self.amplitude = blended_inverse_frequencies(self.dims, self.base, dict(scaling))
            self.inv_freq_host = frequencies.astype(np.float32)
        else:
            self.inv_freq_host = banded_inverse_frequencies(self.dims, self.base, dict(scaling) if scaling else None).astype(np.float32)
        self.pair_inv_freq = torch.from_numpy(self.inv_freq_host).to(runtime.device) if self.dims else None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError("the pair rotation is applied by the mixer's convolve-rotate-and-store kernel")


def blended_inverse_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]]):
    """``(float64 [dims / 2] frequencies, amplitude)`` of a rotation whose context was stretched by ``factor``.

    Plain frequencies are ``f_i = base^(-2i / dims)``.  With ``scaling`` (``factor``, ``original``, ``fast``, ``slow``)
    every frequency becomes ``f_i / factor * r_i + f_i * (1 - r_i)``: the index at which ``original`` positions make
    ``t`` full turns is ``n(t) = dims * ln(original / (2 pi t)) / (2 ln base)``; ``r`` rises linearly over the index
    from 0 at ``max(floor(n(fast)), 0)`` to 1 at ``min(ceil(n(slow)), dims - 1)`` (a span of at least 0.001) and is
    clamped outside.  Cosine and sine are both multiplied by the amplitude ``0.1 ln(factor) + 1``."""
    half = dims // 2
    plain = np.asarray([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return plain, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turns_index(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    low = max(math.floor(turns_index(float(scaling["fast"]))), 0)
    high = min(math.ceil(turns_index(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half, dtype=np.float64) - low) / max(high - low, 0.001), 0.0, 1.0)
    return plain / factor * ramp + plain * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


@POSITION_ENCODINGS.register("rotary_blend")
class RotaryBlend(PositionEncoding):
    """Rotate-half rotation of a head's first ``dims`` numbers (number ``i`` with number ``i + dims / 2``) by
    ``position * f_i``, the frequencies blended between plain and stretched ones and the amplitude raised with the
    stretch (:func:`blended_inverse_frequencies`); the rest of the head passes unchanged.

    params: ``head_dim``, ``dims`` (even, at most ``head_dim``), ``base``, ``scaling`` (mapping with ``factor``,
    ``original``, ``fast``, ``slow``, or None).  The frequencies are taken in 64-bit on the host and rounded once to
    32-bit; the angle and its sine and cosine are 32-bit, in the kernel that applies them (the mixer's
    rotate-normalise-and-store kernel reads ``half_inv_freq``, ``amplitude`` and ``dims``)."""

    def __init__(self, spec: PartSpec, tensors, runtime: Runtime):
        super().__init__(spec, tensors, runtime)
        params = spec.params
        self.head_dim = int(params["head_dim"])
        self.dims = int(params["dims"])
        self.base = float(params["base"])
        if self.dims < 0 or self.dims % 2 or self.dims > self.head_dim:
            raise ValueError(f"rotation of halves needs an even number of dimensions up to {self.head_dim}, got {self.dims}")
        if not self.base > 0.0 or self.base == 1.0:
            raise ValueError("the rotation's base must be positive and not 1")
        scaling = params.get("scaling")
        frequencies, self.amplitude = blended_inverse_frequencies(self.dims, self.base, dict(scaling) if scaling else None)
        self.inv_freq_host = frequencies.astype(np.float32)
        self.half_inv_freq = torch.from_numpy(self.inv_freq_host).to(runtime.device) if self.dims else None

    def apply(self, q: torch.Tensor, k: torch.Tensor, positions: torch.Tensor) -> None:
        raise NotImplementedError("the rotation of halves is applied by the mixer's rotate-normalise-and-store kernel")


@POSITION_ENCODINGS.register("none")
class NoPositionEncoding(PositionEncoding):
    """Leaves queries and keys as they are."""

    def apply(self, q, k, positions) -> None:
        return None
