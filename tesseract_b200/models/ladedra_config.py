"""Typed configuration of the ``Ladedra`` architecture, read from ``config.json``.

``config.json`` names the architecture under ``architecture`` and gives ``width`` (the residual stream), ``vocab``,
``norm.eps``, ``embedding.scale`` and ``layers``.  A layer entry gives ``type`` (which mixer: ``latent_attention`` or
``parallel``), ``mixer`` (its sizes and constants) and ``mlp``: null, a dense feed-forward (``{"kind": "dense", "ff": n}``)
or routed experts (``{"kind": "moe", "router": {"experts", "top", "scale", "groups": {"count", "keep"}}, "expert":
{"ff"}, "shared": {"ff"}}``; ``groups`` and ``shared`` may be absent).  Layers may differ from one another in every number.
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


def _number(data: Mapping[str, Any], key: str, where: str) -> float:
    return _finite(_require(data, key, _NUMBER, where), f"{where}.{key}")


def _positive_int(data: Mapping[str, Any], key: str, where: str) -> int:
    value = _require(data, key, int, where)
    if value <= 0:
        raise ConfigError(f"{where}: {key} must be positive")
    return value


@dataclass(frozen=True)
class LadedraRotation:
    dims: int
    base: float
    # (factor, fast, original, slow) of a stretched context, or None
    scaling: Optional[Tuple[Tuple[str, float], ...]]

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], dim: int, where: str) -> "LadedraRotation":
        dims = _require(data, "dims", int, where)
        base = _number(data, "base", where)
        if dims < 0 or dims % 2 or dims > dim:
            raise ConfigError(f"{where}: dims must be even and at most the rotated vector's size ({dim})")
        if not base > 0 or base == 1.0:
            raise ConfigError(f"{where}: base must be positive and not 1")
        frozen = None
        if data.get("scaling") is not None:
            scaling = _require(data, "scaling", dict, where)
            frozen = tuple((key, _number(scaling, key, where + ".scaling")) for key in ("factor", "fast", "original", "slow"))
            values = dict(frozen)
            if not (values["factor"] > 0 and values["original"] > 0 and values["fast"] > 0 and values["slow"] > 0):
                raise ConfigError(f"{where}.scaling: factor, original, fast and slow must be positive")
        return cls(dims, base, frozen)


def _rotation(data: Mapping[str, Any], dim: int, where: str) -> Optional[LadedraRotation]:
    if data.get("rot") is None:
        return None
    return LadedraRotation.from_dict(_require(data, "rot", dict, where), dim, where + ".rot")


@dataclass(frozen=True)
class LadedraLatentAttention:
    """Causal attention whose keys and values come from a latent of ``kv_rank`` numbers per token; per head ``dim`` plain
    and ``rot_dim`` rotated query/key numbers (the rotated key part is shared by all heads); an output gate."""

    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    rotation: Optional[LadedraRotation]
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LadedraLatentAttention":
        rot_dim = _require(data, "rot_dim", int, where)
        if rot_dim < 0:
            raise ConfigError(f"{where}: rot_dim must not be negative")
        return cls(heads=_positive_int(data, "heads", where), dim=_positive_int(data, "dim", where), rot_dim=rot_dim,
                   vdim=_positive_int(data, "vdim", where), kv_rank=_positive_int(data, "kv_rank", where),
                   rotation=_rotation(data, rot_dim, where), scale=_number(data, "scale", where))


@dataclass(frozen=True)
class LadedraWindowAttention:
    """Grouped-query attention over a sliding window and averaged blocks in front of it, with biases, unit-norm queries
    and keys, capped scores and a learned sink per head."""

    heads: int
    kv_heads: int
    dim: int
    vdim: int
    window: int
    pool: int
    softcap: Optional[float]
    rotation: Optional[LadedraRotation]
    scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LadedraWindowAttention":
        heads, kv_heads = _positive_int(data, "heads", where), _positive_int(data, "kv_heads", where)
        if heads % kv_heads:
            raise ConfigError(f"{where}: heads must be a multiple of kv_heads")
        mask = _require(data, "mask", dict, where)
        dim = _positive_int(data, "dim", where)
        softcap = None
        if data.get("softcap") is not None:
            softcap = _number(data, "softcap", where)
            if not softcap > 0:
                raise ConfigError(f"{where}: softcap must be positive")
        return cls(heads=heads, kv_heads=kv_heads, dim=dim, vdim=_positive_int(data, "vdim", where),
                   window=_positive_int(mask, "size", where + ".mask"), pool=_positive_int(mask, "pool", where + ".mask"),
                   softcap=softcap, rotation=_rotation(data, dim, where), scale=_number(data, "scale", where))


@dataclass(frozen=True)
class LadedraRetention:
    """Linear attention with one fixed decay per head, rotated queries and keys and a ``[dim, vdim]`` state per head."""

    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rotation: Optional[LadedraRotation]

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LadedraRetention":
        heads = _positive_int(data, "heads", where)
        decay = _require(data, "decay", list, where)
        if len(decay) != heads or not all(isinstance(a, _NUMBER) and not isinstance(a, bool) and 0.0 <= a <= 1.0
                                          for a in decay):
            raise ConfigError(f"{where}: decay must list one number in [0, 1] per head")
        dim = _positive_int(data, "dim", where)
        return cls(heads, dim, _positive_int(data, "vdim", where), tuple(float(a) for a in decay),
                   _rotation(data, dim, where))


@dataclass(frozen=True)
class LadedraParallel:
    left: LadedraWindowAttention
    right: LadedraRetention
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str) -> "LadedraParallel":
        return cls(LadedraWindowAttention.from_dict(_require(data, "left", dict, where), where + ".left"),
                   LadedraRetention.from_dict(_require(data, "right", dict, where), where + ".right"),
                   _number(data, "left_scale", where), _number(data, "right_scale", where))


@dataclass(frozen=True)
class LadedraDense:
    ff: int


@dataclass(frozen=True)
class LadedraExperts:
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]
    groups: int
    keep: int
    scale: float


LadedraMixer = Union[LadedraLatentAttention, LadedraParallel]
_MIXERS = {"latent_attention": LadedraLatentAttention, "parallel": LadedraParallel}


def _read_mlp(mlp: Any, where: str):
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        raise ConfigError(f"{where} must be an object or null")
    kind = _require(mlp, "kind", str, where)
    if kind == "dense":
        return LadedraDense(_positive_int(mlp, "ff", where))
    if kind != "moe":
        raise ConfigError(f"{where}: unknown kind '{kind}' (known: dense, moe)")
    router = _require(mlp, "router", dict, where)
    experts, top = _positive_int(router, "experts", where + ".router"), _positive_int(router, "top", where + ".router")
    groups, keep = 1, 1
    if router.get("groups") is not None:
        raw = _require(router, "groups", dict, where + ".router")
        groups = _positive_int(raw, "count", where + ".router.groups")
        keep = _positive_int(raw, "keep", where + ".router.groups")
    if experts % groups or keep > groups or top > keep * (experts // groups):
        raise ConfigError(f"{where}.router: groups.count must divide experts, groups.keep be at most groups.count, and the "
                          f"kept groups hold at least 'top' experts")
    shared = None
    if mlp.get("shared") is not None:
        shared = _positive_int(_require(mlp, "shared", dict, where), "ff", where + ".shared")
    return LadedraExperts(experts=experts, top=top, ff=_positive_int(_require(mlp, "expert", dict, where), "ff", where + ".expert"),
                          shared_ff=shared, groups=groups, keep=keep,
                          scale=_number(router, "scale", where + ".router") if router.get("scale") is not None else 1.0)


@dataclass(frozen=True)
class LadedraLayer:
    type: str
    mixer: LadedraMixer
    mlp: Union[None, LadedraDense, LadedraExperts]


@dataclass(frozen=True)
class LadedraConfig:
    width: int
    vocab: int
    norm_eps: float
    embedding_scale: float
    layers: Tuple[LadedraLayer, ...]

    ARCHITECTURE = "Ladedra"

    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "LadedraConfig":
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
            layers.append(LadedraLayer(kind, mixer, _read_mlp(entry.get("mlp"), where + ".mlp")))
        scale = 1.0
        if data.get("embedding") is not None:
            scale = _number(_require(data, "embedding", dict), "scale", "embedding")
        cfg = cls(width=_require(data, "width", int), vocab=_require(data, "vocab", int),
                  norm_eps=float(_require(norm, "eps", _NUMBER, "norm")), embedding_scale=scale, layers=tuple(layers))
        if cfg.width <= 0 or cfg.vocab <= 0 or not cfg.layers:
            raise ConfigError("width and vocab must be positive and layers not empty")
        if not (cfg.norm_eps > 0 and math.isfinite(cfg.norm_eps)):
            raise ConfigError("norm.eps must be finite and positive")
        return cfg
