"""Typed configuration of the ``Kazodra`` architecture, read from ``config.json``.

``config.json`` names the architecture under ``architecture`` and gives ``width`` (the residual stream), ``vocab``,
``norm.eps``, ``layers`` and, optionally, ``loop`` and ``token_side``.  A layer entry gives ``type`` (which mixer:
``latent_attention``, ``lightning`` or ``attention``), ``mixer`` (its sizes and constants) and ``mlp``: null or a dense
gated feed-forward (``{"kind": "dense", "ff": n}``).  ``loop`` (``start``, ``stop``, ``times``) makes layers ``start`` to
``stop - 1`` run ``times`` times in a row with the same weights.  ``token_side.dim`` is the width of the slice that every
layer reads from a second embedding table.  Layers may differ from one another in every number.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..config.reading import ConfigError, require as _require

_NUMBER = (int, float)


def _finite(value, what: str) -> float:
    value = float(value)
    if not math.isfinite(value):
        raise ConfigError(f"{what} must be finite")
    return value


def _positive_int(data: Mapping[str, Any], key: str, where: str) -> int:
    value = _require(data, key, int, where)
    if value <= 0:
        raise ConfigError(f"{where}: {key} must be positive")
    return value


@dataclass(frozen=True)
class KazodraRotation:
    dims: int
    base: float
    # (factor, high, low, original) of stretched long wavelengths, or None
    scaling: Optional[Tuple[Tuple[str, float], ...]]

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], dim: int, where: str) -> "KazodraRotation":
        dims = _require(data, "dims", int, where)
        base = _finite(_require(data, "base", _NUMBER, where), where + ".base")
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{where}: dims must be even and at most the rotated vector's size ({dim})")
        if not base > 0:
            raise ConfigError(f"{where}: base must be positive")
        scaling = data.get("scaling")
        frozen = None
        if scaling is not None:
            if not isinstance(scaling, dict):
                raise ConfigError(f"{where}.scaling must be an object or null")
            frozen = tuple((key, _finite(_require(scaling, key, _NUMBER, where + ".scaling"), f"{where}.scaling.{key}"))
                           for key in ("factor", "high", "low", "original"))
            values = dict(frozen)
            if not (values["factor"] > 0 and values["original"] > 0 and values["low"] > 0
                    and values["high"] > values["low"]):
                raise ConfigError(f"{where}.scaling: needs factor > 0, original > 0 and high > low > 0")
        return cls(dims, base, frozen)

    def params(self) -> Optional[Tuple[Tuple[str, float], ...]]:
        return self.scaling


def _window(data: Mapping[str, Any], where: str) -> Optional[int]:
    if data.get("mask") is None:
        return None
    size = _require(_require(data, "mask", dict, where), "size", int, where + ".mask")
    if size < 1:
        raise ConfigError(f"{where}: mask.size must be positive")
    return size


def _rotation(data: Mapping[str, Any], dim: int, where: str) -> Optional[KazodraRotation]:
    if data.get("rot") is None:
        return None
    return KazodraRotation.from_dict(_require(data, "rot", dict, where), dim, where + ".rot")


@dataclass(frozen=True)
class KazodraLatentAttention:
    """Attention whose keys and values come from a latent of ``kv_rank`` numbers per token; per head ``dim`` plain and
    ``rot_dim`` rotated query/key numbers (the rotated key part is shared by all heads)."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    window: Optional[int]
    rotation: Optional[KazodraRotation]
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "KazodraLatentAttention":
        rot_dim = _require(data, "rot_dim", int, where)
        if rot_dim < 0:
            raise ConfigError(f"{where}: rot_dim must not be negative")
        return cls(heads=_positive_int(data, "heads", where), dim=_positive_int(data, "dim", where), rot_dim=rot_dim,
                   vdim=_positive_int(data, "vdim", where), kv_rank=_positive_int(data, "kv_rank", where),
                   window=_window(data, where), rotation=_rotation(data, rot_dim, where),
                   scale=_finite(_require(data, "scale", _NUMBER, where), where + ".scale"))


@dataclass(frozen=True)
class KazodraLightning:
    """Linear attention with one fixed decay per head and a ``[dim, vdim]`` state per head."""

    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "KazodraLightning":
        heads = _positive_int(data, "heads", where)
        decay = _require(data, "decay", list, where)
        if len(decay) != heads or not all(isinstance(a, _NUMBER) and not isinstance(a, bool) and 0.0 <= a <= 1.0
                                          for a in decay):
            raise ConfigError(f"{where}: decay must list one number in [0, 1] per head")
        return cls(heads, _positive_int(data, "dim", where), _positive_int(data, "vdim", where),
                   tuple(float(a) for a in decay))


@dataclass(frozen=True)
class KazodraAttention:
    """Grouped-query attention with two score maps per head (``dim`` numbers each) over values of ``vdim``."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    diff: float
    window: Optional[int]
    rotation: Optional[KazodraRotation]
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "KazodraAttention":
        heads, kv_heads = _positive_int(data, "heads", where), _positive_int(data, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
        dim = _positive_int(data, "dim", where)
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive_int(data, "vdim", where),
                   diff=_finite(_require(data, "diff", _NUMBER, where), where + ".diff"), window=_window(data, where),
                   rotation=_rotation(data, dim, where),
                   scale=_finite(_require(data, "scale", _NUMBER, where), where + ".scale"))


KazodraMixer = Union[KazodraLatentAttention, KazodraLightning, KazodraAttention]
_MIXERS = {"latent_attention": KazodraLatentAttention, "lightning": KazodraLightning, "attention": KazodraAttention}


@dataclass(frozen=True)
class KazodraLayer:
    type: str
    mixer: KazodraMixer
    ff: Optional[int]            # the dense feed-forward's inner size; None: the layer has none


@dataclass(frozen=True)
class KazodraLoop:
    start: int
    stop: int
    times: int


def _read_ff(mlp: Any, where: str) -> Optional[int]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    kind = _require(mlp, "kind", str, where)
    if kind != "dense":
        raise ConfigError(f"{where}: unknown kind '{kind}' (known: dense)")
    return _positive_int(mlp, "ff", where)


@dataclass(frozen=True)
class KazodraConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: Tuple[KazodraLayer, ...]
    loop: Optional[KazodraLoop]
    side_dim: Optional[int]      # token_side.dim; None: layers add nothing for the token itself

    ARCHITECTURE = "Kazodra"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "KazodraConfig":
        norm = _require(data, "norm", dict)
        layers = []
        for index, entry in enumerate(_require(data, "layers", list)):
            where = f"layers[{index}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            kind = _require(entry, "type", str, where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}: unknown type '{kind}' (known: {sorted(_MIXERS)})")
            mixer = _MIXERS[kind].from_dict(_require(entry, "mixer", dict, where), where + ".mixer")
            layers.append(KazodraLayer(kind, mixer, _read_ff(entry.get("mlp"), where + ".mlp")))
        loop = None
        if data.get("loop") is not None:
            raw = _require(data, "loop", dict)
            loop = KazodraLoop(_require(raw, "start", int, "loop"), _require(raw, "stop", int, "loop"),
                               _require(raw, "times", int, "loop"))
            if not (0 <= loop.start <= loop.stop <= len(layers)) or loop.times < 1:
                raise ConfigError("loop: needs 0 <= start <= stop <= number of layers and times >= 1")
        side_dim = None
        if data.get("token_side") is not None:
            side_dim = _positive_int(_require(data, "token_side", dict), "dim", "token_side")
        cfg = cls(width=_require(data, "width", int), vocab=_require(data, "vocab", int),
                  norm_eps=float(_require(norm, "eps", _NUMBER, "norm")), layers=tuple(layers), loop=loop,
                  side_dim=side_dim)
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.layers:
            raise ConfigError("width and vocab must be positive and layers not empty")
        if not (cfg.norm_eps > 0 and math.isfinite(cfg.norm_eps)):
            raise ConfigError("norm.eps must be finite and positive")
        return cfg

    @property
    def loops(self) -> bool:
        return self.loop is not None and self.loop.stop > self.loop.start

    def run_order(self) -> Tuple[Tuple[int, Optional[int]], ...]:
        """``(layer, walk)`` in the order the layers run: the looped run ``times`` times; ``walk`` is the number of the
        walk at its first layer and None everywhere else."""
        count = len(self.layers)
        if not self.loops:
            return tuple((i, None) for i in range(count))
        order = [(i, None) for i in range(self.loop.start)]
        for walk in range(self.loop.times):
            order += [(i, walk if i == self.loop.start else None) for i in range(self.loop.start, self.loop.stop)]
        return tuple(order + [(i, None) for i in range(self.loop.stop, count)])
