"""Tiny Kazodra configurations for the tests: every size differs between them and between their layers, and the
values that make two mechanisms coincide (keys as wide as values, one kv head, a rotation over the whole head or the
whole rotated part, equal decays, a single walk of the loop, a loop over everything) appear in one layer and not in
the next."""


def rot(dims, base, scaling=None):
    out = {"dims": dims, "base": base}
    if scaling is not None:
        factor, low, high, original = scaling
        out["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return out


def latent(heads, dim, rot_dim, vdim, rank, window, rotation, scale):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        mixer["mask"] = {"size": window}
    if rotation is not None:
        mixer["rot"] = rotation
    return {"type": "latent_attention", "mixer": mixer}


def lightning(heads, dim, vdim, decay):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}}


def differential(heads, kv_heads, dim, vdim, diff, rotation, scale):
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale}
    if rotation is not None:
        mixer["rot"] = rotation
    return {"type": "attention", "mixer": mixer}


def layer(mixer, ff):
    return dict(mixer, mlp=None if ff is None else {"kind": "dense", "ff": ff})


TINY_KAZODRA = {
    # the loop in the middle and walked twice; a window of 21 and one of 5 (shorter than a page); stretched frequencies
    # over part of a map; decays from fast to none at all
    "a": {"architecture": "Kazodra", "width": 48, "vocab": 131, "norm": {"eps": 1e-6}, "token_side": {"dim": 6},
          "loop": {"start": 1, "stop": 4, "times": 2},
          "layers": [layer(latent(3, 12, 8, 10, 20, 21, rot(8, 1000.0), 0.25), 72),
                     layer(lightning(3, 8, 12, (0.5, 0.97, 1.0)), 40),
                     layer(differential(4, 2, 12, 20, 0.35, rot(8, 500.0, (3.0, 1.0, 8.0, 64)), 0.3), 56),
                     layer(latent(2, 16, 4, 24, 12, 5, rot(4, 50.0), 0.2), None),
                     layer(lightning(1, 20, 10, (0.9,)), 24)]},
    # the loop from the first layer to the last, three walks; a layer without a feed-forward; no token input
    "b": {"architecture": "Kazodra", "width": 64, "vocab": 256, "norm": {"eps": 1e-5},
          "loop": {"start": 0, "stop": 2, "times": 3},
          "layers": [layer(differential(2, 2, 16, 8, 0.8, rot(16, 100.0), 0.25), None),
                     layer(lightning(4, 16, 8, (0.8, 0.8, 0.25, 0.999)), 96)]},
    # no loop; widths that are no multiple of four or eight; a window wider than any prompt of the tests; no rotation
    # in the differential layer; the rotation over a part of the rotated part
    "c": {"architecture": "Kazodra", "width": 42, "vocab": 77, "norm": {"eps": 1e-4}, "token_side": {"dim": 3},
          "layers": [layer(latent(1, 10, 6, 14, 9, 1000, rot(4, 30.0, (4.0, 1.0, 32.0, 40)), 0.3), 30),
                     layer(differential(3, 1, 6, 10, 0.5, None, 0.4), 20),
                     layer(lightning(2, 5, 7, (0.0, 0.6)), None)]},
    # a single walk of a loop that is the last layer alone; a window of one position; a latent without a rotated part
    "d": {"architecture": "Kazodra", "width": 32, "vocab": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
          "loop": {"start": 2, "stop": 3, "times": 1},
          "layers": [layer(latent(2, 8, 8, 8, 16, 1, rot(8, 20.0), 0.35), 16),
                     layer(latent(4, 8, 0, 4, 8, 17, None, 0.3), 24),
                     layer(differential(6, 3, 8, 8, 0.2, rot(6, 7.0, (16.0, 0.25, 1.0, 8)), 0.35), 16)]},
    # head sizes of real models' layers, with prompts long enough for the kernels that take prompt portions in tiles
    "e": {"architecture": "Kazodra", "width": 64, "vocab": 90, "norm": {"eps": 1e-6}, "token_side": {"dim": 4},
          "loop": {"start": 0, "stop": 2, "times": 2},
          "layers": [layer(differential(2, 1, 64, 128, 0.7, rot(64, 10000.0, (8.0, 1.0, 4.0, 128)), 0.125), 48),
                     layer(latent(2, 64, 32, 128, 128, 100, rot(32, 100.0), 0.1), None),
                     layer(lightning(2, 64, 64, (0.95, 0.99)), 40),
                     layer(differential(4, 2, 128, 64, 0.4, rot(32, 100.0), 0.09), 32)]},
}


def random_config(seed: int) -> dict:
    """A Kazodra configuration drawn from ``seed``: two to five layers of the three mixers, with or without a
    feed-forward, a loop anywhere or none, a token input or none, windows from 1 to 500 positions."""
    import random

    r = random.Random(seed)
    width = r.choice([24, 40, 64, 66, 96, 136, 200])

    def rotation(size):
        if size < 2 or r.random() < 0.15:
            return None
        scaling = None
        if r.random() < 0.6:
            low = r.choice([1.0, 0.5])
            scaling = (r.choice([2.0, 4.0, 10.0]), low, low * r.choice([2.0, 4.0, 32.0]), r.choice([16, 64, 1024]))
        return rot(r.choice(range(2, size + 1, 2)), r.choice([10.0, 1000.0, 500000.0]), scaling)

    layers = []
    for _ in range(r.randint(2, 5)):
        kind = r.choice(["latent", "lightning", "differential"])
        if kind == "latent":
            dim, rot_dim = r.choice([4, 8, 12, 24, 40, 64]), r.choice([0, 2, 8, 16, 32])
            mixer = latent(r.choice([1, 2, 3, 5, 8]), dim, rot_dim, r.choice([4, 8, 10, 24, 48, 64]),
                           r.choice([6, 16, 20, 64, 96, 128, 128]), r.choice([None, 1, 3, 16, 17, 50, 64, 120, 500]),
                           rotation(rot_dim), r.choice([(dim + rot_dim) ** -0.5, 0.3, 0.07]))
        elif kind == "lightning":
            heads = r.choice([1, 2, 3, 4, 6])
            mixer = lightning(heads, r.choice([4, 7, 16, 24, 32, 64]), r.choice([4, 10, 16, 33, 48, 64, 80]),
                              [r.choice([0.0, 0.3, 0.9, 0.99, 0.9999, 1.0]) for _ in range(heads)])
        else:
            heads = r.choice([1, 2, 3, 4, 6, 8])
            kv_heads = r.choice([d for d in range(1, heads + 1) if heads % d == 0])
            dim = r.choice([6, 8, 12, 16, 24, 32, 64, 128])
            mixer = differential(heads, kv_heads, dim, r.choice([4, 8, 10, 16, 24, 48, 64, 128]),
                                 r.choice([0.2, 0.5, 0.8]), rotation(dim), r.choice([dim ** -0.5, 0.3, 0.07]))
        layers.append(layer(mixer, r.choice([None, 8, 40, 100, 256])))
    config = {"architecture": "Kazodra", "width": width, "vocab": r.randint(40, 700),
              "norm": {"eps": r.choice([1e-5, 1e-6])}, "layers": layers}
    if r.random() < 0.8:
        config["token_side"] = {"dim": r.choice([1, 4, 6, 16, 24])}
    if r.random() < 0.8:
        start = r.randint(0, len(layers) - 1)
        config["loop"] = {"start": start, "stop": r.randint(start + 1, len(layers)), "times": r.randint(1, 3)}
    return config
