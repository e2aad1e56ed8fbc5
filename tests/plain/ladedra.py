"""A plain, slow Ladedra in float64: whole sequences, one function per mechanism, nothing shared with the package.

``forward(config, tensors, tokens)`` takes the dictionary of ``config.json``, a mapping from tensor name to a numpy
array, and one sequence's token ids; it returns the logits of every position and the stream behind every layer.
``store`` is applied wherever a serving path may keep numbers in 16 bits between two of its kernels (normed rows,
projected rows, cached keys and values in front of pooling, what enters an output product); the default keeps float64,
and ``bfloat16`` measures what such rounding alone does to a result.
"""

from __future__ import annotations

import math

import numpy as np


def identity(x):
    return x


def bfloat16(x):
    """``x`` rounded to bfloat16 and widened again."""
    import torch

    return torch.from_numpy(np.ascontiguousarray(x, dtype=np.float64)).to(torch.bfloat16).to(torch.float64).numpy()


def load_folder(folder):
    """``(config, {name: float64 array})`` of a model folder, read with a parser of its own."""
    import json
    import os
    import struct

    import torch

    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    raw = open(os.path.join(folder, "model.safetensors"), "rb").read()
    (size,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + size])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16}
    tensors = {}
    for name, entry in header.items():
        if name == "__metadata__":
            continue
        first, last = entry["data_offsets"]
        flat = torch.frombuffer(bytearray(raw[8 + size + first:8 + size + last]), dtype=kinds[entry["dtype"]])
        tensors[name] = flat.to(torch.float64).numpy().reshape(entry["shape"])
    return config, tensors


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_divide(x, eps):
    """Every row of the last axis divided by ``sqrt(mean(row^2) + eps)``."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms_divide(x, eps) * weight


def plain_frequencies(dims, base):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=np.float64)


def stretched_frequencies(dims, base, scaling):
    """``(frequencies, amplitude)``: frequencies blended between plain and divided ones along a ramp over the pair
    index, and the factor on cosine and sine."""
    f = plain_frequencies(dims, base)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def index_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(index_of(float(scaling["slow"]))), dims - 1)
    ramp = np.array([min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0) for i in range(dims // 2)])
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, frequencies, amplitude, layout):
    """``x`` ``[T, heads, d]``: the first ``2 * len(frequencies)`` numbers of every head turn; ``layout`` ``"pairs"``
    couples ``2i`` with ``2i + 1``, ``"halves"`` couples ``i`` with ``i + dims / 2``."""
    out = x.copy()
    half = len(frequencies)
    if half == 0:
        return out
    angle = np.asarray(positions, dtype=np.float64)[:, None] * frequencies[None, :]          # [T, half]
    cos, sin = np.cos(angle)[:, None, :] * amplitude, np.sin(angle)[:, None, :] * amplitude
    if layout == "pairs":
        u, v = x[..., 0:2 * half:2], x[..., 1:2 * half:2]
        out[..., 0:2 * half:2] = u * cos - v * sin
        out[..., 1:2 * half:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:2 * half]
        out[..., :half] = u * cos - v * sin
        out[..., half:2 * half] = v * cos + u * sin
    return out


# ----------------------------------------------------------------------------- mixers


def latent_attention(m, w, h, eps, store=identity):
    """``m``: the mixer's entry of the configuration; ``w``: name -> array with the layer's ``mix.`` prefix removed."""
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    positions = np.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    freq, amp = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot["dims"] else (np.zeros(0), 1.0)
    q = store(h @ w["q"].T).reshape(T, H, d + dr)
    down = h @ w["dkv"].T
    c = store(rms_norm(down[:, :rank], w["dkv.norm"], eps))
    k_rot = store(rotate(down[:, None, rank:], positions, freq, amp, "pairs"))[:, 0]          # [T, dr], one for all heads
    q_rot = rotate(q[..., d:], positions, freq, amp, "pairs")
    k_plain = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    out = np.zeros((T, H, dv))
    for t in range(T):
        for head in range(H):
            scores = (k_plain[:t + 1, head] @ q[t, head, :d] + k_rot[:t + 1] @ q_rot[t, head]) * m["scale"]
            weights = np.exp(scores - scores.max())
            out[t, head] = (weights / weights.sum()) @ v[:t + 1, head]
    gated = store(out.reshape(T, H * dv) * sigmoid(store(h @ w["g"].T)))
    return gated @ w["o"].T


def pooled_window_attention(m, w, h, eps, store=identity):
    """Grouped-query attention over the last ``mask.size`` tokens and one averaged key and value per block of
    ``mask.pool`` tokens that ends in front of them; a learned number per head joins the denominator."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    size, P, cap = m["mask"]["size"], m["mask"]["pool"], m.get("softcap")
    positions = np.arange(T)
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    freq, amp = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot["dims"] else (np.zeros(0), 1.0)
    q = store(h @ w["q"].T + w["q.b"]).reshape(T, H, d)
    k = store(h @ w["k"].T + w["k.b"]).reshape(T, G, d)
    v = store((h @ w["v"].T + w["v.b"]).reshape(T, G, dv))
    q = store(rms_divide(rotate(q, positions, freq, amp, "halves"), eps))
    k = store(rms_divide(rotate(k, positions, freq, amp, "halves"), eps))
    blocks = T // P
    pooled_k = store(np.stack([k[b * P:(b + 1) * P].mean(axis=0) for b in range(blocks)]) if blocks else np.zeros((0, G, d)))
    pooled_v = store(np.stack([v[b * P:(b + 1) * P].mean(axis=0) for b in range(blocks)]) if blocks else np.zeros((0, G, dv)))
    out = np.zeros((T, H, dv))
    for t in range(T):
        first = max(0, t - size + 1)
        seen = [b for b in range(blocks) if (b + 1) * P <= t - size + 1]
        for head in range(H):
            g = head // (H // G)
            keys = np.concatenate([pooled_k[seen, g], k[first:t + 1, g]])
            values = np.concatenate([pooled_v[seen, g], v[first:t + 1, g]])
            scores = keys @ q[t, head] * m["scale"]
            if cap:
                scores = cap * np.tanh(scores / cap)
            sink = w["sink"][head]
            top = max(scores.max(), sink)
            weights = np.exp(scores - top)
            out[t, head] = (weights / (weights.sum() + math.exp(sink - top))) @ values
    return store(out.reshape(T, H * dv)) @ w["o"].T


def retention(m, w, h, eps, state=None, store=identity, first_position=0):
    """Linear attention with a fixed decay per head; returns ``(output, state behind the last row)``."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    positions = np.arange(T) + first_position
    rot = m.get("rot") or {"dims": 0, "base": 10000.0}
    freq, amp = stretched_frequencies(rot["dims"], rot["base"], rot.get("scaling")) if rot["dims"] else (np.zeros(0), 1.0)
    q = rotate(store(h @ w["q"].T).reshape(T, H, d), positions, freq, amp, "halves")
    k = rotate(store(h @ w["k"].T).reshape(T, H, d), positions, freq, amp, "halves") * d ** -0.5
    v = store(h @ w["v"].T).reshape(T, H, dv)
    S = np.zeros((H, d, dv)) if state is None else state.copy()
    out = np.zeros((T, H, dv))
    for t in range(T):
        for head in range(H):
            S[head] = m["decay"][head] * S[head] + np.outer(k[t, head], v[t, head])
            out[t, head] = S[head].T @ q[t, head]
    normed = rms_divide(out, eps).reshape(T, H * dv)
    return store(normed * silu(store(h @ w["g"].T))) @ w["o"].T, S


def parallel_mixer(m, w, h, eps, store=identity):
    left = pooled_window_attention(m["left"], {k[5:]: a for k, a in w.items() if k.startswith("left.")}, h, eps, store)
    right, _ = retention(m["right"], {k[6:]: a for k, a in w.items() if k.startswith("right.")}, h, eps, store=store)
    return m["left_scale"] * left + m["right_scale"] * right


# ----------------------------------------------------------------------------- feed-forwards


def dense_feed_forward(w, h, store=identity):
    z = np.maximum(store(h @ w["up"].T), 0.0)
    return store(z * z) @ w["down"].T


def gated_expert(w, prefix, h, store=identity):
    return store(silu(store(h @ w[prefix + "gate"].T)) * store(h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(mlp, logits, gaps=None):
    """``(chosen experts, weights)`` of one row from its router logits.  ``gaps`` (a list) receives how far, in scores,
    the closest decision was from going the other way: the last kept group against the first one left out, and the last
    chosen expert against the best one not chosen."""
    r = mlp["router"]
    experts, top = r["experts"], r["top"]
    scores = np.exp(logits - logits.max())
    scores /= scores.sum()
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = experts // groups["count"]
    best = [scores[g * per:(g + 1) * per].max() for g in range(groups["count"])]
    kept = sorted(range(groups["count"]), key=lambda g: (-best[g], g))[:groups["keep"]]
    allowed = [e for e in range(experts) if e // per in kept]
    ranked = sorted(allowed, key=lambda e: (-scores[e], e))
    chosen = ranked[:top]
    if gaps is not None:
        order = sorted(range(groups["count"]), key=lambda g: (-best[g], g))
        if groups["keep"] < groups["count"]:
            gaps.append(best[order[groups["keep"] - 1]] - best[order[groups["keep"]]])
        if top < len(ranked):
            gaps.append(scores[ranked[top - 1]] - scores[ranked[top]])
    weights = scores[chosen] / (scores[chosen].sum() + 1e-20) * r["scale"]
    return chosen, weights


def expert_feed_forward(mlp, w, h, store=identity, close_calls=None):
    """``close_calls`` (a dictionary) receives, per row, the smallest gap of its routing decisions (see :func:`route`)."""
    out = np.zeros((h.shape[0], w["e0.down"].shape[0]))
    logits = h @ w["router"].T
    for t in range(h.shape[0]):
        gaps = []
        chosen, weights = route(mlp, logits[t], gaps)
        if close_calls is not None and gaps:
            close_calls[t] = min(close_calls.get(t, 1.0), min(gaps))
        for e, weight in zip(chosen, weights):
            out[t] += weight * gated_expert(w, f"e{e}.", h[t:t + 1], store)[0]
    if mlp.get("shared"):
        out += gated_expert(w, "shared.", h, store)
    return out


# ----------------------------------------------------------------------------- the model


def layer_forward(config, tensors, index, x, store=identity, close_calls=None):
    layer, eps, prefix = config["layers"][index], config["norm"]["eps"], f"l{index}."
    w = {name[len(prefix):]: a for name, a in tensors.items() if name.startswith(prefix)}
    mix = {name[4:]: a for name, a in w.items() if name.startswith("mix.")}
    h = store(rms_norm(x, w["norm1"], eps))
    if layer["type"] == "latent_attention":
        mixed = latent_attention(layer["mixer"], mix, h, eps, store)
    elif layer["type"] == "parallel":
        mixed = parallel_mixer(layer["mixer"], mix, h, eps, store)
    else:
        raise ValueError(layer["type"])
    x = x + mixed * w["ls1"] * sigmoid(h @ w["rg1"].T + w["rg1.b"])
    mlp = layer.get("mlp")
    if mlp is None:
        return x
    h = store(rms_norm(x, w["norm2"], eps))
    feed = {name[4:]: a for name, a in w.items() if name.startswith("mlp.")}
    update = dense_feed_forward(feed, h, store) if mlp["kind"] == "dense" else expert_feed_forward(mlp, feed, h, store, close_calls)
    return x + update * w["ls2"] * sigmoid(h @ w["rg2"].T + w["rg2.b"])


def forward(config, tensors, tokens, store=identity, close_calls=None):
    """``(logits [T, vocab], [stream behind layer 0, 1, ...])``.  ``close_calls`` (a dictionary) receives, per position, the
    smallest gap by which a router of any layer decided."""
    x = tensors["embed"][np.asarray(tokens)] * config["embedding"]["scale"]
    streams = []
    for index in range(len(config["layers"])):
        x = layer_forward(config, tensors, index, x, store, close_calls)
        streams.append(x.copy())
    logits = store(rms_norm(x, tensors["final.norm"], config["norm"]["eps"])) @ tensors["head"].T
    return logits, streams
