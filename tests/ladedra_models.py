"""Tiny Ladedra configurations for the tests: every size differs between them and between their layers, and the values
that make two mechanisms coincide or vanish (a pool of one token, a window of one, a window shorter than a block or longer
than any prompt, one group of experts, every expert a group of its own, one chosen expert, kv heads as many as heads,
keys as wide as values, a rotation over the whole head or none, decays of 0 and 1, scales of 1) appear in one layer and
not in the next."""


def rot(dims, base, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling is not None:
        factor, original, fast, slow = scaling
        out["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return out


def latent(heads, dim, rot_dim, vdim, rank, rotation, scale):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if rotation is not None:
        mixer["rot"] = rotation
    return {"type": "latent_attention", "mixer": mixer}


def window_attention(heads, kv_heads, dim, vdim, size, pool, rotation, scale, softcap):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": size, "pool": pool},
             "scale": scale, "softcap": softcap}
    if rotation is not None:
        mixer["rot"] = rotation
    return mixer


def retention(heads, dim, vdim, decay, rotation):
    mixer = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rotation is not None:
        mixer["rot"] = rotation
    return mixer


def parallel(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared, groups, scale):
    router = {"experts": experts, "top": top, "scale": scale}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "router": router, "expert": {"ff": ff}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


TINY_LADEDRA = {
    # stretched pair rotation over the whole rotated part; a window of 21 with blocks of 4; three groups of two experts
    "a": {"architecture": "Ladedra", "width": 48, "vocab": 131, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
          "layers": [layer(latent(3, 12, 8, 10, 20, rot(8, 1000.0, (4.0, 32, 8.0, 1.0)), 0.25), dense(72)),
                     layer(parallel(window_attention(4, 2, 12, 20, 21, 4, rot(8, 500.0), 0.6, 15.0),
                                    retention(3, 8, 12, (0.5, 0.97, 1.0), rot(8, 100.0)), 1.3, 0.7),
                           moe(6, 2, 16, 24, (3, 2), 1.5)),
                     layer(latent(2, 16, 4, 24, 12, rot(4, 50.0), 0.2), None),
                     layer(parallel(window_attention(2, 1, 16, 8, 9, 3, rot(16, 20.0), 0.5, 30.0),
                                    retention(1, 20, 10, (0.9,), None), 1.0, 1.0), dense(40))]},
    # a parallel layer first; a window shorter than a block; blocks that no page holds whole (5 of 16); as many kv heads as
    # heads; no groups in the router, one chosen expert, no shared expert; a layer without a feed-forward
    "b": {"architecture": "Ladedra", "width": 64, "vocab": 256, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
          "layers": [layer(parallel(window_attention(2, 2, 16, 16, 3, 5, rot(8, 100.0), 0.4, 8.0),
                                    retention(4, 16, 8, (0.8, 0.8, 0.25, 0.999), rot(16, 1000.0)), 0.5, 2.0),
                           moe(5, 1, 24, None, None, 1.0)),
                     layer(parallel(window_attention(6, 3, 8, 12, 40, 7, None, 0.7, 50.0),
                                    retention(2, 8, 16, (0.0, 1.0), rot(4, 10.0)), 1.1, 0.9), None),
                     layer(latent(4, 8, 6, 4, 8, rot(6, 20.0, (16.0, 8, 4.0, 0.5)), 0.3), moe(8, 3, 8, 16, (4, 2), 1.25))]},
    # widths that are no multiple of four or eight; a pool of one token and a window of one; every expert its own group
    "c": {"architecture": "Ladedra", "width": 42, "vocab": 77, "norm": {"eps": 1e-4}, "embedding": {"scale": 6.5},
          "layers": [layer(latent(1, 10, 6, 14, 9, rot(6, 30.0, (2.0, 16, 2.0, 1.0)), 0.3), moe(4, 2, 10, 6, (4, 3), 0.5)),
                     layer(parallel(window_attention(3, 1, 6, 10, 1, 1, rot(2, 7.0), 0.9, 4.0),
                                    retention(2, 5, 7, (0.0, 0.6), None), 2.0, 0.25), dense(30)),
                     layer(parallel(window_attention(2, 2, 10, 6, 17, 16, rot(10, 300.0), 0.3, 100.0),
                                    retention(3, 6, 5, (1.0, 0.5, 0.99), rot(6, 50.0)), 0.8, 1.2), None)]},
    # a window longer than any prompt of the tests (no block is ever seen); a latent without a rotated part
    "d": {"architecture": "Ladedra", "width": 32, "vocab": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 0.5},
          "layers": [layer(parallel(window_attention(4, 1, 8, 8, 1000, 16, rot(8, 20.0), 0.35, 12.0),
                                    retention(2, 8, 8, (0.95, 0.5), rot(8, 20.0)), 1.0, 0.5), dense(16)),
                     layer(latent(4, 8, 0, 4, 8, None, 0.3), dense(24)),
                     layer(parallel(window_attention(2, 1, 24, 8, 16, 16, rot(12, 9.0), 0.2, 10.0),
                                    retention(1, 12, 24, (0.75,), rot(12, 9.0)), 0.3, 1.7), moe(2, 2, 12, 12, (1, 1), 3.0))]},
    # head sizes of real models' layers, with prompts long enough for the kernels that take prompt portions in tiles
    "e": {"architecture": "Ladedra", "width": 64, "vocab": 90, "norm": {"eps": 1e-6}, "embedding": {"scale": 8.0},
          "layers": [layer(latent(2, 64, 32, 128, 128, rot(32, 10000.0, (8.0, 128, 16.0, 1.0)), 0.1), dense(48)),
                     layer(parallel(window_attention(4, 1, 64, 64, 100, 32, rot(64, 10000.0), 0.125, 30.0),
                                    retention(2, 64, 64, (0.95, 0.99), rot(32, 1000.0)), 1.4, 0.8),
                           moe(8, 3, 32, 40, (4, 2), 2.0)),
                     layer(parallel(window_attention(2, 2, 128, 64, 64, 8, rot(64, 100.0), 0.09, 25.0),
                                    retention(2, 32, 128, (0.9, 1.0), None), 0.7, 1.4), None)]},
}

LENGTHS = {"a": [1, 23, 97, 150, 7], "b": [2, 40, 130, 61], "c": [1, 19, 88, 140], "d": [3, 50, 120], "e": [5, 70, 330, 140]}


def random_config(seed: int) -> dict:
    """A Ladedra configuration drawn from ``seed``: two to five layers of the two mixers in any order, with a dense
    feed-forward, experts or none, windows from 1 to 500 positions and blocks from 1 to 40."""
    import random

    r = random.Random(seed)
    width = r.choice([24, 40, 64, 66, 96, 136, 200])

    def rotation(size, stretched=False):
        if size < 2 or r.random() < 0.15:
            return None
        scaling = None
        if stretched and r.random() < 0.7:
            scaling = (r.choice([2.0, 4.0, 10.0]), r.choice([16, 64, 1024]), r.choice([4.0, 16.0, 32.0]), r.choice([0.5, 1.0]))
        return rot(r.choice(range(2, size + 1, 2)), r.choice([10.0, 1000.0, 500000.0]), scaling)

    layers = []
    for _ in range(r.randint(2, 5)):
        if r.random() < 0.45:
            dim, rot_dim = r.choice([4, 8, 12, 24, 40, 64]), r.choice([0, 2, 8, 16, 32])
            rotated = rotation(rot_dim, stretched=True)
            if rotated is not None:
                rotated["dims"] = rot_dim                     # the rotation covers the whole rotated part
            mixer = latent(r.choice([1, 2, 3, 5, 8]), dim, rot_dim, r.choice([4, 8, 10, 24, 48, 64]),
                           r.choice([6, 16, 20, 64, 96, 128, 128]), rotated, r.choice([(dim + rot_dim) ** -0.5, 0.3, 0.07]))
        else:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            kv_heads = r.choice([d for d in range(1, heads + 1) if heads % d == 0])
            dim = r.choice([6, 8, 12, 16, 24, 32, 64, 128])
            left = window_attention(heads, kv_heads, dim, r.choice([4, 8, 10, 16, 24, 48, 64, 128]),
                                    r.choice([1, 3, 16, 17, 50, 64, 120, 500]), r.choice([1, 2, 5, 8, 16, 33, 40]),
                                    rotation(dim), r.choice([0.9 * dim ** -0.5, 0.3, 0.07]), r.choice([5.0, 15.0, 50.0]))
            rheads = r.choice([1, 2, 3, 4, 6])
            rdim = r.choice([4, 8, 16, 24, 32, 64])
            right = retention(rheads, rdim, r.choice([4, 10, 16, 33, 48, 64, 80]),
                              [r.choice([0.0, 0.3, 0.9, 0.99, 0.9999, 1.0]) for _ in range(rheads)], rotation(rdim))
            mixer = parallel(left, right, r.choice([1.0, 1.3, 0.4]), r.choice([1.0, 0.8, 1.6]))
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = dense(r.choice([8, 40, 100, 256]))
        else:
            groups = r.choice([1, 2, 3, 4])
            per = r.choice([1, 2, 4])
            keep = r.randint(1, groups)
            mlp = moe(groups * per, r.randint(1, min(4, keep * per)), r.choice([8, 16, 40, 64]), r.choice([None, 8, 48]),
                      r.choice([None, (groups, keep)]) if (groups, keep) == (1, 1) else (groups, keep), r.choice([1.0, 1.75, 0.7]))
        layers.append(layer(mixer, mlp))
    return {"architecture": "Ladedra", "width": width, "vocab": r.randint(40, 700), "norm": {"eps": r.choice([1e-5, 1e-6])},
            "embedding": {"scale": r.choice([1.0, 4.0, 12.0])}, "layers": layers}
