"""Kazodra without a GPU: reading ``config.json``, the run order of a looped model, the model description, the
tensors it expects, and the plain implementation against itself (the recurrence
token by token against the same recurrence continued from a carried state; the stretched frequencies at their edges)."""

import copy
import math

import pytest
import torch

from tesseract_b200.cache.manager import CacheManager
from tesseract_b200.config import ConfigError, load_model_description, resolve_architecture
from tesseract_b200.models.decoder import expected_tensors
from tesseract_b200.parts import PagedKeyValueNeed
from tesseract_b200.weights.random_init import write_random_model
from tests.kazodra_models import TINY_KAZODRA, random_config
from tests.plain import kazodra as plain

MIXER_KINDS = {"latent_attention": "latent_attention", "lightning": "lightning", "attention": "differential_attention"}


def test_the_architecture_is_found_by_its_single_name():
    assert resolve_architecture({"architecture": "Kazodra"}).name == "Kazodra"


@pytest.mark.parametrize("name", sorted(TINY_KAZODRA))
def test_description_and_expected_tensors(tmp_path, name):
    config = TINY_KAZODRA[name]
    folder = write_random_model(str(tmp_path / name), config, seed=3)
    architecture, typed, spec = load_model_description(folder)
    assert architecture.name == "Kazodra" and spec.vocab_size == config["vocab"] and spec.hidden_size == config["width"]
    assert len(spec.layers) == len(config["layers"])
    expected = expected_tensors(spec)
    width = config["width"]
    side = config.get("token_side")
    for index, layer in enumerate(config["layers"]):
        assert spec.layers[index].block == "sandwich" and spec.layers[index].mixer.kind == MIXER_KINDS[layer["type"]]
        for norm in ("norm1", "norm1b"):
            assert expected[f"l{index}.{norm}"].shape == expected[f"l{index}.{norm}.b"].shape == (width,)
        assert (f"l{index}.norm2" in expected) == (f"l{index}.norm2b.b" in expected) == (layer["mlp"] is not None)
        m = layer["mixer"]
        mix = f"l{index}.mix."
        if layer["type"] == "latent_attention":
            assert expected[mix + "q"].shape == (m["heads"] * (m["dim"] + m["rot_dim"]), width)
            assert expected[mix + "dkv"].shape == (m["kv_rank"] + m["rot_dim"], width)
            assert expected[mix + "dkv.norm"].shape == (m["kv_rank"],)
            assert expected[mix + "uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
            assert expected[mix + "uv"].shape == (m["heads"] * m["vdim"], m["kv_rank"])
        elif layer["type"] == "lightning":
            assert expected[mix + "q"].shape == expected[mix + "k"].shape == (m["heads"] * m["dim"], width)
            assert expected[mix + "v"].shape == expected[mix + "g"].shape == (m["heads"] * m["vdim"], width)
            assert expected[mix + "norm"].shape == (m["heads"] * m["vdim"],)
        else:
            assert expected[mix + "q"].shape == (m["heads"] * 2 * m["dim"], width)
            assert expected[mix + "k"].shape == (m["kv_heads"] * 2 * m["dim"], width)
            assert expected[mix + "v"].shape == (m["kv_heads"] * m["vdim"], width)
            assert expected[mix + "g"].shape == (m["heads"] * m["vdim"], width)
            assert all(expected[mix + v].shape == (m["dim"],) for v in ("lq1", "lk1", "lq2", "lk2"))
        assert expected[mix + "o"].shape == (width, m["heads"] * m["vdim"])
        if layer["mlp"]:
            assert expected[f"l{index}.mlp.gate"].shape == expected[f"l{index}.mlp.up"].shape == (layer["mlp"]["ff"], width)
            assert expected[f"l{index}.mlp.down"].shape == (width, layer["mlp"]["ff"])
        assert (f"l{index}.side.gate" in expected) == (side is not None)
        if side:
            assert expected[f"l{index}.side.gate"].shape == (side["dim"], width)
            assert expected[f"l{index}.side.proj"].shape == (width, side["dim"])
            assert expected[f"l{index}.side.norm"].shape == (width,)
    if side:
        assert expected["side.embed"].shape == (config["vocab"], side["dim"] * len(config["layers"]))
    assert spec.head.weights["weight"] == spec.embedding.weights["table"] == "embed"
    assert "final.norm.b" in expected
    if "loop" in config:
        assert expected["loop.step"].shape == (config["loop"]["times"], width)
    # the run order of the description is the plain model's; every walk of the loop starts with its own vector
    assert [(e.layer, e.inject) for e in spec.run_order] == plain.run_order(config)
    assert all(e.cache_of is None for e in spec.run_order)           # a cache or state of its own for every run
    libraries = architecture.kernel_libraries(typed, "float32")
    assert "gemm_f32" in libraries and "decode_linear" not in libraries and "attention_tcgen05" not in libraries
    kinds = {layer["type"] for layer in config["layers"]}
    assert ("lightning" in libraries) == ("lightning" in kinds) and ("differential" in libraries) == ("attention" in kinds)


def test_the_loop_repeats_its_layers_in_a_row_and_numbers_its_walks():
    from tesseract_b200.models.kazodra_config import KazodraConfig

    config = copy.deepcopy(TINY_KAZODRA["a"])
    config["loop"] = {"start": 2, "stop": 4, "times": 3}
    order = KazodraConfig.from_dict(config).run_order()
    assert order == ((0, None), (1, None), (2, 0), (3, None), (2, 1), (3, None), (2, 2), (3, None), (4, None))
    config["loop"] = {"start": 0, "stop": 5, "times": 2}
    assert [i for i, _ in KazodraConfig.from_dict(config).run_order()] == [0, 1, 2, 3, 4, 0, 1, 2, 3, 4]
    config["loop"] = {"start": 4, "stop": 5, "times": 1}
    assert KazodraConfig.from_dict(config).run_order()[-1] == (4, 0)    # a single walk still gets its vector
    del config["loop"]
    assert KazodraConfig.from_dict(config).run_order() == tuple((i, None) for i in range(5))


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].__setitem__("type", "lstm"), "unknown type"),
    (lambda c: c["layers"][2]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 10), "dims"),        # more than the rotated part
    (lambda c: c["layers"][2]["mixer"]["rot"]["scaling"].pop("high"), "high"),
    (lambda c: c["layers"][0]["mixer"]["mask"].__setitem__("size", 0), "mask.size"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5, 0.5, 1.5]), "decay"),
    (lambda c: c["layers"][0].__setitem__("mlp", {"kind": "experts", "ff": 8}), "unknown kind"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop"),
    (lambda c: c["loop"].__setitem__("times", 0), "loop"),
    (lambda c: c["token_side"].__setitem__("dim", 0), "dim"),
    (lambda c: c.pop("vocab"), "vocab"),
])
def test_bad_configurations_are_refused(change, message):
    from tesseract_b200.models.kazodra_config import KazodraConfig

    config = copy.deepcopy(TINY_KAZODRA["a"])
    change(config)
    with pytest.raises(ConfigError, match=message):
        KazodraConfig.from_dict(config)


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations_describe_and_write(tmp_path, seed):
    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "m"), config, seed=seed)
    _, _, spec = load_model_description(folder)
    loaded, tensors = plain.load_folder(folder)
    assert set(tensors) == set(expected_tensors(spec))
    assert len(spec.run_order) == len(plain.run_order(loaded))
    logits = plain.forward(loaded, tensors, [1, 2, 3, 0, 5])
    assert logits.shape == (5, config["vocab"]) and bool(torch.isfinite(logits).all())


def test_stretched_frequencies_agree_with_the_plain_recipe():
    from tesseract_b200.parts.rotary import banded_inverse_frequencies

    cases = [(64, 20000.0, {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 4096}),
             (8, 500.0, {"factor": 3.0, "low": 1.0, "high": 8.0, "original": 64}),
             (6, 7.0, {"factor": 16.0, "low": 0.25, "high": 1.0, "original": 8}),
             (10, 30.0, None)]
    for dims, base, scaling in cases:
        got = banded_inverse_frequencies(dims, base, scaling)
        assert list(got) == pytest.approx(plain.pair_frequencies(dims, base, scaling), rel=1e-12)
    # a short wavelength stays, a long one is divided by the factor, and one between them lies between the two
    dims, base, scaling = cases[0]
    got = banded_inverse_frequencies(dims, base, scaling)
    plain_f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    assert got[0] == 1.0 and got[-1] == pytest.approx(plain_f[-1] / 8.0)
    between = [i for i, f in enumerate(plain_f) if 4096 / 4.0 <= 2 * math.pi / f <= 4096 / 1.0]
    assert between and all(plain_f[i] / 8.0 <= got[i] <= plain_f[i] for i in between)


def test_the_plain_recurrence_continues_from_a_carried_state():
    torch.manual_seed(0)
    m = {"heads": 3, "dim": 5, "vdim": 7, "decay": [0.0, 0.7, 1.0]}
    width = 12
    t = {name: torch.randn(rows, width, dtype=torch.float64) * 0.4
         for name, rows in (("q", 15), ("k", 15), ("v", 21), ("g", 21))}
    t["o"] = torch.randn(width, 21, dtype=torch.float64) * 0.3
    t["norm"] = torch.rand(21, dtype=torch.float64) + 0.5
    h = torch.randn(9, width, dtype=torch.float64)
    whole, last = plain.lightning(h, t, m, 1e-6)
    head, state = plain.lightning(h[:4], t, m, 1e-6)
    tail, end = plain.lightning(h[4:], t, m, 1e-6, state=state)
    assert torch.allclose(torch.cat([head, tail]), whole, atol=1e-12) and torch.allclose(end, last, atol=1e-12)
    # a decay of zero keeps the last token's product alone; a decay of one keeps the plain sum
    k = plain.silu(h @ t["k"].T).view(9, 3, 5)
    v = plain.silu(h @ t["v"].T).view(9, 3, 7)
    assert torch.allclose(last[0], k[-1, 0][:, None] * v[-1, 0][None, :], atol=1e-12)
    assert torch.allclose(last[2], torch.einsum("td,te->de", k[:, 2], v[:, 2]), atol=1e-12)


def test_a_window_gives_pages_back_while_the_request_lives():
    pages = PagedKeyValueNeed(num_kv_heads=2, key_dim=8, value_dim=4, window=21)
    manager = CacheManager([pages, pages], [None, None], num_pages=6, page_size=16, max_requests=2,
                           dtype=torch.float32, device="cpu", max_step_tokens=16)
    assert manager.admit("a")
    held = []
    for _ in range(20):                                          # 200 tokens, ten at a time
        manager.extend("a", 10)
        manager.commit("a", 10)
        held.append(manager.used_pages())
    assert max(held) <= 4
    manager.release("a")
    manager.check()
    assert manager.used_pages() == 0
