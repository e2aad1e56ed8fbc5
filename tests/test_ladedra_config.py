"""Ladedra without a GPU: reading ``config.json``, the model description, the tensors it expects, the cache manager's
handling of a pooled window (tokens held until their block is finished, an entry per block in pages of their own), and the
plain implementation against itself (the recurrence continued from a carried state; the stretched frequencies; the router
at its edges)."""

import copy

import numpy as np
import pytest
import torch

from tesseract_b200.cache.manager import CacheManager
from tesseract_b200.config import ConfigError, load_model_description, resolve_architecture
from tesseract_b200.models.decoder import expected_tensors
from tesseract_b200.parts import PagedKeyValueNeed, PooledBlocksNeed
from tesseract_b200.parts.rotary import blended_inverse_frequencies
from tesseract_b200.weights.random_init import write_random_model
from tests.ladedra_models import TINY_LADEDRA, random_config
from tests.plain import ladedra as plain


def test_the_architecture_is_found_by_its_single_name():
    assert resolve_architecture({"architecture": "Ladedra"}).name == "Ladedra"


@pytest.mark.parametrize("name", sorted(TINY_LADEDRA))
def test_description_and_expected_tensors(tmp_path, name):
    config = TINY_LADEDRA[name]
    folder = write_random_model(str(tmp_path / name), config, seed=3)
    architecture, typed, spec = load_model_description(folder)
    assert architecture.name == "Ladedra" and spec.vocab_size == config["vocab"] and spec.hidden_size == config["width"]
    assert len(spec.layers) == len(config["layers"]) == len(spec.run_order)
    expected = expected_tensors(spec)
    width = config["width"]
    assert expected["embed"].shape == expected["head"].shape == (config["vocab"], width)
    for index, layer in enumerate(config["layers"]):
        prefix, mix, m = f"l{index}.", f"l{index}.mix.", layer["mixer"]
        assert spec.layers[index].block == "gated_pre_norm" and spec.layers[index].residual_gates.kind == "scaled_sigmoid_gate"
        assert expected[prefix + "norm1"].shape == expected[prefix + "ls1"].shape == expected[prefix + "rg1.b"].shape == (width,)
        assert expected[prefix + "rg1"].shape == (width, width)
        has_mlp = layer["mlp"] is not None
        assert all((prefix + n in expected) == has_mlp for n in ("norm2", "ls2", "rg2", "rg2.b"))
        if layer["type"] == "latent_attention":
            assert spec.layers[index].mixer.kind == "latent_attention"
            assert expected[mix + "q"].shape == (m["heads"] * (m["dim"] + m["rot_dim"]), width)
            assert expected[mix + "dkv"].shape == (m["kv_rank"] + m["rot_dim"], width)
            assert expected[mix + "dkv.norm"].shape == (m["kv_rank"],)
            assert expected[mix + "uk"].shape == (m["heads"] * m["dim"], m["kv_rank"])
            assert expected[mix + "uv"].shape == (m["heads"] * m["vdim"], m["kv_rank"])
            assert expected[mix + "g"].shape == (m["heads"] * m["vdim"], width)
            assert expected[mix + "o"].shape == (width, m["heads"] * m["vdim"])
        else:
            assert spec.layers[index].mixer.kind == "parallel_mixers"
            left, right = m["left"], m["right"]
            assert expected[mix + "left.q"].shape == (left["heads"] * left["dim"], width)
            assert expected[mix + "left.q.b"].shape == (left["heads"] * left["dim"],)
            assert expected[mix + "left.k"].shape == (left["kv_heads"] * left["dim"], width)
            assert expected[mix + "left.v.b"].shape == (left["kv_heads"] * left["vdim"],)
            assert expected[mix + "left.sink"].shape == (left["heads"],)
            assert expected[mix + "left.o"].shape == (width, left["heads"] * left["vdim"])
            assert expected[mix + "right.q"].shape == expected[mix + "right.k"].shape == (right["heads"] * right["dim"], width)
            assert expected[mix + "right.v"].shape == expected[mix + "right.g"].shape == (right["heads"] * right["vdim"], width)
            assert expected[mix + "right.o"].shape == (width, right["heads"] * right["vdim"])
            assert mix + "right.norm" not in expected
        mlp = layer["mlp"]
        if mlp and mlp["kind"] == "dense":
            assert expected[prefix + "mlp.up"].shape == (mlp["ff"], width) and expected[prefix + "mlp.down"].shape == (width, mlp["ff"])
        elif mlp:
            assert expected[prefix + "mlp.router"].shape == (mlp["router"]["experts"], width)
            for e in range(mlp["router"]["experts"]):
                assert expected[f"{prefix}mlp.e{e}.gate"].shape == expected[f"{prefix}mlp.e{e}.up"].shape == (mlp["expert"]["ff"], width)
                assert expected[f"{prefix}mlp.e{e}.down"].shape == (width, mlp["expert"]["ff"])
            assert (prefix + "mlp.shared.gate" in expected) == ("shared" in mlp)
    # the plain model reads the same folder
    tokens = [1, 2, 3, 4, 5, 6, 7]
    logits, streams = plain.forward(*plain.load_folder(folder), tokens)
    assert logits.shape == (7, config["vocab"]) and len(streams) == len(config["layers"]) and np.isfinite(logits).all()


def changed(path, value):
    def apply(config):
        at = config
        for key in path[:-1]:
            at = at[key]
        if value is KeyError:
            del at[path[-1]]
        else:
            at[path[-1]] = value
    return apply


@pytest.mark.parametrize("change,message", [
    (changed(("layers", 1, "mixer", "left", "kv_heads"), 3), "multiple of kv_heads"),
    (changed(("layers", 1, "mixer", "left", "mask", "pool"), 0), "pool must be positive"),
    (changed(("layers", 1, "mixer", "left", "mask"), KeyError), "mask"),
    (changed(("layers", 1, "mixer", "right", "decay"), [0.5]), "one number in [0, 1] per head"),
    (changed(("layers", 1, "mixer", "left_scale"), KeyError), "left_scale"),
    (changed(("layers", 1, "mlp", "router", "groups", "count"), 4), "groups.count must divide"),
    (changed(("layers", 1, "mlp", "router", "groups", "keep"), 5), "groups.keep"),
    (changed(("layers", 1, "mlp", "router", "top"), 5), "kept groups hold"),
    (changed(("layers", 1, "mlp", "kind"), "sparse"), "unknown kind"),
    (changed(("layers", 0, "mixer", "rot", "dims"), 7), "dims must be even"),
    (changed(("layers", 0, "mixer", "rot", "scaling", "factor"), -1.0), "must be positive"),
    (changed(("layers", 0, "type"), "attention"), "unknown type"),
    (changed(("norm", "eps"), 0.0), "finite and positive"),
    (changed(("layers",), []), "layers not empty"),
])
def test_bad_configurations_are_refused(change, message):
    config = copy.deepcopy(TINY_LADEDRA["a"])
    change(config)
    with pytest.raises(ConfigError) as caught:
        resolve_architecture(config).read_config(config)
    assert message in str(caught.value)


@pytest.mark.parametrize("seed", range(1, 25))
def test_random_configurations_describe_and_write(tmp_path, seed):
    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "m"), config, seed=seed)
    _, _, spec = load_model_description(folder)
    assert len(spec.layers) == len(config["layers"])
    loaded_config, tensors = plain.load_folder(folder)
    assert set(tensors) == set(expected_tensors(spec))


@pytest.mark.parametrize("dims,base,scaling", [(8, 1000.0, (4.0, 32, 8.0, 1.0)), (32, 30000.0, (6.0, 1024, 16.0, 1.0)),
                                               (6, 30.0, (2.0, 16, 2.0, 1.0)), (64, 1e6, (40.0, 4096, 32.0, 0.5)), (4, 50.0, None)])
def test_stretched_frequencies_agree_with_the_plain_recipe(dims, base, scaling):
    named = dict(zip(("factor", "original", "fast", "slow"), scaling)) if scaling else None
    got, amplitude = blended_inverse_frequencies(dims, base, named)
    want, want_amplitude = plain.stretched_frequencies(dims, base, named)
    assert np.allclose(got, want, rtol=1e-12, atol=0) and amplitude == pytest.approx(want_amplitude, rel=1e-12)
    if scaling:
        plain_f = plain.plain_frequencies(dims, base)
        assert np.all(got <= plain_f * (1 + 1e-12)) and np.all(got >= plain_f / scaling[0] * (1 - 1e-12)) and amplitude > 1.0


def test_the_plain_recurrence_continues_from_a_carried_state():
    rng = np.random.default_rng(4)
    m = {"heads": 2, "dim": 6, "vdim": 5, "decay": [0.9, 1.0], "rot": {"dims": 4, "base": 10.0}}
    width = 12
    w = {"q": rng.normal(size=(12, width)), "k": rng.normal(size=(12, width)), "v": rng.normal(size=(10, width)),
         "g": rng.normal(size=(10, width)), "o": rng.normal(size=(width, 10))}
    h = rng.normal(size=(40, width))
    whole, state = plain.retention(m, w, h, 1e-6)
    first, carried = plain.retention(m, w, h[:17], 1e-6)
    second, final = plain.retention(m, w, h[17:], 1e-6, state=carried, first_position=17)
    assert np.allclose(np.concatenate([first, second]), whole, atol=1e-12) and np.allclose(final, state, atol=1e-12)


def test_the_plain_router_at_its_edges():
    mlp = {"router": {"experts": 6, "top": 2, "scale": 3.0, "groups": {"count": 3, "keep": 1}}}
    # the best expert's group is kept although the two next best experts sit together in another
    chosen, weights = plain.route(mlp, np.log(np.array([0.30, 0.02, 0.25, 0.26, 0.10, 0.07])))
    assert chosen == [0, 1] and weights.sum() == pytest.approx(3.0) and weights[0] > weights[1]
    # equal scores: the lowest indices win; one group of all experts is no restriction
    chosen, weights = plain.route({"router": {"experts": 4, "top": 3, "scale": 1.0}}, np.zeros(4))
    assert chosen == [0, 1, 2] and np.allclose(weights, 1.0 / 3.0)
    gaps = []
    plain.route(mlp, np.log(np.array([0.30, 0.02, 0.25, 0.26, 0.10, 0.07])), gaps)
    assert min(gaps) == pytest.approx(0.04, abs=1e-9)


def test_a_pooled_window_holds_unfinished_blocks_and_an_entry_per_block():
    """A window of 5 with blocks of 40 positions, pages of 16: the tokens of the block being filled stay although the
    window has passed them; the block's page of averages fills once per 16 blocks; everything returns at the end."""
    tokens_need = PagedKeyValueNeed(num_kv_heads=2, key_dim=8, value_dim=4, window=5, hold=40)
    blocks_need = PooledBlocksNeed(num_kv_heads=2, key_dim=8, value_dim=4, pool=40)
    assert tokens_need.first_needed_position(39) == 0 and tokens_need.first_needed_position(40) == 36
    assert tokens_need.first_needed_position(79) == 40 and tokens_need.first_needed_position(47) == 40
    assert blocks_need.entries_for(1) == 1 and blocks_need.entries_for(40) == 1 and blocks_need.entries_for(41) == 2
    cache = CacheManager([(tokens_need, blocks_need)], [None], num_pages=64, page_size=16, max_requests=2,
                         dtype=torch.float32, device="cpu", allocate_storage=False)
    assert [g.pool.num_pages for g in cache.groups] == [64, 64 // 40 + 1 + 2]
    assert isinstance(cache.bindings[0], tuple) and len(cache.bindings[0]) == 2
    assert cache.admit("r")
    most = 0
    for step in range(100):
        cache.extend("r", 10)
        cache.commit("r", 10)
        held = len(cache.pages_of("r", 0))
        most = max(most, held)
        length = cache.length("r")
        first_needed = min(max(0, length - 4), (length // 40) * 40)
        assert min(cache.pages_of("r", 0)) == first_needed // 16 or held == 0
        assert len(cache.pages_of("r", 1)) == -(-(-(-length // 40)) // 16)
    assert most <= 4 and cache.length("r") == 1000
    cache.release("r")
    cache.check()
    assert cache.used_pages() == 0
