"""Plain, slow Kazodra: whole sequences, no cache, one function per mechanism.

Kazodra is a decoder whose layers are listed in ``config.json``.  A layer has a token mixer and, optionally, a gated
feed-forward; each sublayer reads the stream through a layer norm (weight and bias) and its result passes a second
layer norm before it is added: ``x += post(sub(pre(x)))``.  After the sublayers a layer adds a term that depends on the
token itself: a slice of a second embedding table, gated by a small projection of the stream, projected back and
brought to unit root mean square.  Three mixers exist: attention over a latent vector per token with a shared rotated
key part and a sliding window; a linear-attention recurrence with a fixed decay per head, a norm over all heads and an
output gate; and grouped-query attention with two score maps per head whose outputs are subtracted, normed per head
and gated.  A run of layers may be walked several times with the same weights; every walk starts by adding a learned
vector of its own to the stream.  The logits come from the embedding table.

This module shares no code with ``tesseract_b200``: it reads the model folder itself and computes with torch on the
CPU in ``dtype`` (float64 by default).  Every function takes a whole sequence ``[T, ...]``; nothing is cached.
"""

from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping, Optional, Sequence

import torch
from safetensors import safe_open


def load_folder(model_dir: str):
    with open(os.path.join(model_dir, "config.json")) as handle:
        config = json.load(handle)
    tensors: Dict[str, torch.Tensor] = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as handle:
        for name in handle.keys():
            tensors[name] = handle.get_tensor(name)
    return config, tensors


# ----------------------------------------------------------------------------- mechanisms
# ``round_to`` (None or a torch dtype): where a serving path would store an activation in a 16-bit format (the
# operands of products, stored queries, keys, values and latents), the value is rounded to that format and widened
# again.  Sums that the design keeps in 32-bit (the stream, scores and weights, norms, the recurrent state) never are.


def rounded(x: torch.Tensor, round_to) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, eps: float) -> torch.Tensor:
    centred = x - x.mean(dim=-1, keepdim=True)
    return centred / torch.sqrt((centred * centred).mean(dim=-1, keepdim=True) + eps) * weight + bias


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z * z * z)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def pair_frequencies(dims: int, base: float, scaling: Optional[Mapping[str, float]] = None) -> List[float]:
    """``base^(-2i/dims)``; with ``scaling`` (``factor``, ``low``, ``high``, ``original``) a frequency whose wavelength
    is under ``original / high`` stays, one whose wavelength is over ``original / low`` is divided by ``factor``, and
    between the two the divided and the plain one are mixed linearly in ``original / wavelength``."""
    out = []
    for i in range(dims // 2):
        f = base ** (-2.0 * i / dims)
        if scaling:
            factor, low, high = float(scaling["factor"]), float(scaling["low"]), float(scaling["high"])
            original = float(scaling["original"])
            wavelength = 2.0 * math.pi / f
            if wavelength < original / high:
                pass
            elif wavelength > original / low:
                f = f / factor
            else:
                s = (original / wavelength - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, frequencies: Sequence[float]) -> torch.Tensor:
    """``x`` ``[T, heads, n]``: of the first ``2 * len(frequencies)`` numbers, neighbours ``(2i, 2i + 1)`` turn by
    ``position * f_i``; the rest passes."""
    out = x.clone()
    f = torch.tensor(list(frequencies), dtype=x.dtype)
    angle = positions.to(x.dtype)[:, None, None] * f[None, None, :]
    cos, sin = torch.cos(angle), torch.sin(angle)
    n = 2 * len(frequencies)
    u, v = x[..., 0:n:2], x[..., 1:n:2]
    out[..., 0:n:2] = u * cos - v * sin
    out[..., 1:n:2] = v * cos + u * sin
    return out


def softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float,
                      window: Optional[int]) -> torch.Tensor:
    """``q`` ``[T, H, d]``, ``k`` ``[T, H, d]``, ``v`` ``[T, H, dv]`` (already one key/value head per query head):
    row ``i`` sees ``j <= i`` and, with ``window``, ``i - j < window``."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window:
        seen = seen & (i - j < window)
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), v)


def latent_attention(h, t: Mapping[str, torch.Tensor], m: Mapping, eps: float, positions, round_to=None):
    """Attention whose keys and values are projections of a latent vector per token."""
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    q = rounded(h @ t["q"].T, round_to).view(T, H, d + dr)
    down = h @ t["dkv"].T
    latent = rounded(unit_rms(down[:, :rank], eps) * t["dkv.norm"], round_to)
    rot = m.get("rot")
    frequencies = pair_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else []
    shared = rounded(rotate_pairs(down[:, None, rank:], positions, frequencies), round_to)       # [T, 1, dr]
    q_rot = rounded(rotate_pairs(q[..., d:], positions, frequencies), round_to)
    k_plain = rounded(latent @ t["uk"].T, round_to).view(T, H, d)
    values = rounded(latent @ t["uv"].T, round_to).view(T, H, dv)
    keys = torch.cat([k_plain, shared.expand(T, H, dr)], dim=-1)
    queries = torch.cat([q[..., :d], q_rot], dim=-1)
    window = (m.get("mask") or {}).get("size")
    out = softmax_attention(queries, keys, values, m["scale"], window)
    return rounded(out.reshape(T, H * dv), round_to) @ t["o"].T


def lightning(h, t: Mapping[str, torch.Tensor], m: Mapping, eps: float, round_to=None, state=None):
    """Linear attention with a fixed decay per head, token by token.  Returns ``(output, final state)``."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rounded(silu(h @ t["q"].T), round_to).view(T, H, d)
    k = rounded(silu(h @ t["k"].T), round_to).view(T, H, d)
    v = rounded(silu(h @ t["v"].T), round_to).view(T, H, dv)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, dv, dtype=h.dtype) if state is None else state.clone()
    out = torch.empty(T, H, dv, dtype=h.dtype)
    for step in range(T):
        S = decay[:, None, None] * S + k[step][:, :, None] * v[step][:, None, :]
        out[step] = torch.einsum("hde,hd->he", S, q[step])
    flat = unit_rms(out.reshape(T, H * dv), eps) * t["norm"]
    gated = flat * torch.sigmoid(rounded(h @ t["g"].T, round_to))
    return rounded(gated, round_to) @ t["o"].T, S


def differential_lambda(t: Mapping[str, torch.Tensor], diff: float) -> float:
    return float(torch.exp((t["lq1"].double() * t["lk1"].double()).sum())
                 - torch.exp((t["lq2"].double() * t["lk2"].double()).sum()) + diff)


def differential_attention(h, t: Mapping[str, torch.Tensor], m: Mapping, eps: float, positions, round_to=None):
    """Grouped-query attention with two score maps per head over the same values: the second map's output, times
    ``lambda``, is subtracted from the first's; the difference is normed per head and gated."""
    H, G, d, dv, diff = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["diff"]
    T = h.shape[0]
    rot = m.get("rot")
    frequencies = pair_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot else []
    q = (h @ t["q"].T).view(T, H * 2, d)
    k = (h @ t["k"].T).view(T, G * 2, d)
    q = rounded(rotate_pairs(q, positions, frequencies), round_to).view(T, H, 2, d)
    k = rounded(rotate_pairs(k, positions, frequencies), round_to).view(T, G, 2, d)
    v = rounded(h @ t["v"].T, round_to).view(T, G, dv)
    group = H // G
    k = k.repeat_interleave(group, dim=1)
    v = v.repeat_interleave(group, dim=1)
    window = (m.get("mask") or {}).get("size")
    first = softmax_attention(q[:, :, 0], k[:, :, 0], v, m["scale"], window)
    second = softmax_attention(q[:, :, 1], k[:, :, 1], v, m["scale"], window)
    out = unit_rms(first - differential_lambda(t, diff) * second, eps) * (1.0 - diff)
    gated = out.reshape(T, H * dv) * torch.sigmoid(rounded(h @ t["g"].T, round_to))
    return rounded(gated, round_to) @ t["o"].T


def gated_feed_forward(h, t: Mapping[str, torch.Tensor], round_to=None):
    inner = silu(rounded(h @ t["gate"].T, round_to)) * rounded(h @ t["up"].T, round_to)
    return rounded(inner, round_to) @ t["down"].T


def token_side(x, tokens, table, layer: int, dim: int, t: Mapping[str, torch.Tensor], eps: float, round_to=None):
    """What a layer adds for the token itself: its slice of the second table, gated by a projection of the stream."""
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(rounded(x, round_to) @ t["gate"].T) * e
    y = rounded(g, round_to) @ t["proj"].T
    return unit_rms(y, eps) * t["norm"]


# ----------------------------------------------------------------------------- the model


def run_order(config) -> List[tuple]:
    """``(layer, pass number or None)``: the pass number stands at the first layer of every walk of the loop."""
    count = len(config["layers"])
    loop = config.get("loop")
    if not loop:
        return [(i, None) for i in range(count)]
    order = [(i, None) for i in range(loop["start"])]
    for walk in range(loop["times"]):
        order += [(i, walk if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], count)]


def sub(tensors: Mapping[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {name[len(prefix):]: value.to(dtype) for name, value in tensors.items() if name.startswith(prefix)}


def forward(config, tensors, tokens: Sequence[int], dtype=torch.float64, round_to=None, return_layers: bool = False):
    """Logits ``[T, vocab]`` of one whole sequence (and the stream after every layer run)."""
    eps = float(config["norm"]["eps"])
    ids = torch.tensor(list(tokens), dtype=torch.long)
    positions = torch.arange(len(ids))
    embed = tensors["embed"].to(dtype)
    x = embed[ids]
    side = config.get("token_side")
    after = []
    for index, walk in run_order(config):
        layer = config["layers"][index]
        p = f"l{index}."
        w = sub(tensors, p, dtype)
        if walk is not None:
            x = x + tensors["loop.step"].to(dtype)[walk]
        h = rounded(layer_norm(x, w["norm1"], w["norm1.b"], eps), round_to)
        mix = sub(tensors, p + "mix.", dtype)
        if layer["type"] == "latent_attention":
            y = latent_attention(h, mix, layer["mixer"], eps, positions, round_to)
        elif layer["type"] == "lightning":
            y, _ = lightning(h, mix, layer["mixer"], eps, round_to)
        elif layer["type"] == "attention":
            y = differential_attention(h, mix, layer["mixer"], eps, positions, round_to)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, w["norm1b"], w["norm1b.b"], eps)
        if layer.get("mlp") is not None:
            h = rounded(layer_norm(x, w["norm2"], w["norm2.b"], eps), round_to)
            x = x + layer_norm(gated_feed_forward(h, sub(tensors, p + "mlp.", dtype), round_to), w["norm2b"], w["norm2b.b"], eps)
        if side is not None:
            x = x + token_side(x, ids, tensors["side.embed"].to(dtype), index, int(side["dim"]),
                               sub(tensors, p + "side.", dtype), eps, round_to)
        after.append(x)
    final = layer_norm(x, tensors["final.norm"].to(dtype), tensors["final.norm.b"].to(dtype), eps)
    logits = rounded(final, round_to) @ embed.T
    return (logits, torch.stack(after)) if return_layers else logits
