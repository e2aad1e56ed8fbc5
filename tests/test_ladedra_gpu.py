"""Ladedra on the GPU against the plain implementation (``tests/plain/ladedra.py``).

First every mechanism alone (its kernel or part against the plain function, with inputs made so that a fault shows: one
key or one averaged block that dominates, placed at the window's first position and one before it, in the block that is
just seen and the one that is not yet, at position 0, at page borders and hundreds of positions back; a recurrence
carried over many steps with decays of zero and one), then whole tiny models with random weights under every way of
cutting the work: whole prompts, token-by-token decoding, portions down to two tokens, mixed batches with slots and pages
used again, long decoding while the windows move over decoded tokens, and greedy generation through the package's own
entry point and scheduler.
"""

import numpy as np
import pytest
import torch

from tests.helpers import (GREEDY_MARGIN, compare, max_live_tokens, random_tokens, replay, trace_mixed, trace_portions,
                           trace_tail, trace_whole)
from tests.ladedra_models import LENGTHS, TINY_LADEDRA, random_config
from tests.plain import ladedra as plain

pytestmark = pytest.mark.gpu

# (of a request's largest |logit|; the stream behind a scaled embedding and several gated additions is some thirty times
# larger than the logits it ends in, so 32-bit rounding of the stream shows in them at a few 1e-5)
REL = {"float32": 5e-5, "bfloat16": 3e-2}
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}
# In bfloat16 a result may also differ by this many times what rounding to bfloat16 alone moves in the plain computation
# (``store=plain.bfloat16``): the package rounds at other places than the plain functions do (it attends in the latent
# space, for one), so the two are two draws of that noise, and in these tiny models single positions amplify it tenfold.
NOISE = 5.0


def dev():
    return torch.device("cuda", 0)


def runtime(dtype):
    from tesseract_b200.parts import Runtime

    return Runtime(dtype, dev())


def close(got, want, tol, what="", noise=0.0):
    got = got.detach().cpu().double().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert np.isfinite(got).all(), what
    worst = float(np.abs(got - want).max())
    assert worst <= max(tol * max(1.0, float(np.abs(want).max())), NOISE * noise), f"{what}: {worst}"


def i32(values):
    return torch.tensor(list(values), dtype=torch.int32, device=dev())


def step_context(positions, tables, page, slot=0):
    """A step of one sequence whose rows stand at ``positions`` (consecutive); ``tables``: one block table per cache group."""
    from tesseract_b200.parts import GroupView, StepContext

    n = len(positions)
    return StepContext(num_rows=n, num_seqs=1, token_ids=i32([0] * n), positions=i32(positions), seq_of_row=i32([0] * n),
                       row_start=i32([0, n]), seq_begin=i32([positions[0]]), state_slots=i32([slot]),
                       groups=[GroupView(torch.tensor([t], dtype=torch.int32, device=dev()) if t is not None else None, page)
                               for t in tables],
                       host_new=[n], host_begin=[positions[0]], host_slots=[slot], max_new=n, max_context=positions[-1] + 1)


def bf16(t):
    return t.to(torch.bfloat16)


def as_plain(tensors):
    return {name: t.double().numpy() for name, t in tensors.items()}


# ----------------------------------------------------------------------------- mechanisms alone


@pytest.mark.parametrize("width", [5, 42, 66, 256, 4096, 12288])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16, None])
def test_scaled_gated_addition_with_the_following_norm(width, out_dtype):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    rows = 7
    residual, update, gate = (torch.randn(rows, width, generator=g) * s for s in (3.0, 1.0, 2.0))
    bias, scale, weight = torch.randn(width, generator=g), 1.0 + 0.3 * torch.randn(width, generator=g), torch.rand(width, generator=g) + 0.5
    new = residual.double() + update.double() * scale.double() * torch.sigmoid(gate.double() + bias.double())
    normed = plain.rms_norm(new.numpy(), weight.double().numpy(), 1e-5)
    on = residual.to(dev())
    out = torch.empty(rows, width, dtype=out_dtype, device=dev()) if out_dtype is not None else None
    kernels.gated_add_norm(on, update.to(dev()), gate.to(dev()), bias.to(dev()), scale.to(dev()),
                           weight.to(dev()) if out is not None else None, out, 1e-5)
    close(on, new.numpy(), 2e-6, "stream")
    if out is not None:
        close(out, normed, 2e-6 if out_dtype == torch.float32 else 1e-2, "normed rows")


@pytest.mark.parametrize("experts,top,groups,keep,scale", [(8, 3, 2, 1, 1.75), (6, 2, 3, 2, 1.5), (5, 1, 1, 1, 1.0), (4, 2, 4, 3, 0.5),
                                                          (64, 6, 8, 3, 1.0), (12, 4, 3, 3, 2.0), (3, 3, 1, 1, 1.0), (40, 5, 1, 1, 0.3)])
def test_router_over_groups_of_experts(experts, top, groups, keep, scale):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(experts * 7 + top)
    logits = torch.randn(300, experts, generator=g) * 2.0
    logits[5] = logits[5, 0]                       # all equal: the lowest indices win
    ids = torch.empty(300, top, dtype=torch.int32, device=dev())
    weights = torch.empty(300, top, dtype=torch.float32, device=dev())
    kernels.choose_grouped(logits.to(dev()), ids, weights, groups=groups, keep=keep, weight_scale=scale)
    mlp = {"router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}}}
    for t in range(300):
        chosen, want = plain.route(mlp, logits[t].double().numpy())
        assert ids[t].tolist() == list(chosen), f"row {t}"
        close(weights[t], want, 1e-5, f"row {t}")
    assert ids[5].tolist() == list(range(top))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,ff", [(48, 72), (42, 30), (256, 1000)])
def test_squared_relu_feed_forward(dtype, width, ff):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import FEED_FORWARDS

    g = torch.Generator().manual_seed(width + ff)
    tensors = {"up": bf16(torch.randn(ff, width, generator=g) * width ** -0.5), "down": bf16(torch.randn(width, ff, generator=g) * ff ** -0.5)}
    spec = PartSpec.make("plain_mlp", {"hidden_size": width, "intermediate_size": ff, "activation": "squared_relu", "stream": "float32"},
                         {"up": "up", "down": "down"})
    part = FEED_FORWARDS.get(spec.kind)(spec, tensors, runtime(dtype))
    h = bf16(torch.randn(37, width, generator=g)).float()
    want = plain.dense_feed_forward(as_plain(tensors), h.double().numpy())
    noise = float(np.abs(plain.dense_feed_forward(as_plain(tensors), h.double().numpy(), plain.bfloat16) - want).max())
    got = part.forward(h.to(dtype).to(dev()), None)
    assert got.dtype == torch.float32
    close(got, want, TOL[dtype], "squared ReLU feed-forward", noise if dtype == torch.bfloat16 else 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,experts,top,ff,shared,groups,scale", [(48, 6, 2, 16, 24, (3, 2), 1.5), (64, 5, 1, 24, None, None, 1.0),
                                                                    (42, 4, 2, 10, 6, (4, 3), 0.5), (128, 16, 4, 64, 96, (4, 2), 2.0)])
@pytest.mark.parametrize("rows", [2, 9, 300])
def test_gated_experts_routed_within_groups(dtype, width, experts, top, ff, shared, groups, scale, rows):
    """The routed feed-forward alone against the plain function, row by row, at the rows whose router does not decide by
    so little that a rounding could turn the choice."""
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import FEED_FORWARDS

    g = torch.Generator().manual_seed(width + experts + rows)
    named = {"router": torch.randn(experts, width, generator=g) * (1.5 * width ** -0.5)}
    weights = {"router": "router"}
    for e in range(experts):
        named.update({f"e{e}.gate": torch.randn(ff, width, generator=g) * width ** -0.5, f"e{e}.up": torch.randn(ff, width, generator=g) * width ** -0.5,
                      f"e{e}.down": torch.randn(width, ff, generator=g) * ff ** -0.5})
        weights.update({f"gate.{e}": f"e{e}.gate", f"up.{e}": f"e{e}.up", f"down.{e}": f"e{e}.down"})
    if shared:
        named.update({"shared.gate": torch.randn(shared, width, generator=g) * width ** -0.5,
                      "shared.up": torch.randn(shared, width, generator=g) * width ** -0.5,
                      "shared.down": torch.randn(width, shared, generator=g) * shared ** -0.5})
        weights.update({"shared_gate": "shared.gate", "shared_up": "shared.up", "shared_down": "shared.down"})
    named = {n: bf16(t) for n, t in named.items()}
    count, keep = groups if groups else (1, 1)
    spec = PartSpec.make("routed_experts", {"hidden_size": width, "num_experts": experts, "top_k": top, "expert_size": ff,
                                            "shared_size": shared, "scoring": "softmax_all", "groups": count, "keep_groups": keep,
                                            "weight_scale": scale, "expert_form": "gated_silu", "stream": "float32"}, weights)
    part = FEED_FORWARDS.get(spec.kind)(spec, {role: named[name] for role, name in weights.items()}, runtime(dtype))
    mlp = {"router": {"experts": experts, "top": top, "scale": scale}}
    if groups:
        mlp["router"]["groups"] = {"count": count, "keep": keep}
    if shared:
        mlp["shared"] = {"ff": shared}
    h = bf16(torch.randn(rows, width, generator=g)).float()
    gaps = {}
    want = plain.expert_feed_forward(mlp, as_plain(named), h.double().numpy(), close_calls=gaps)
    coarse = plain.expert_feed_forward(mlp, as_plain(named), h.double().numpy(), plain.bfloat16)
    steady = [t for t in range(rows) if gaps.get(t, 1.0) >= 0.01]
    assert len(steady) >= max(1, rows // 3)
    noise = float(np.abs(coarse - want)[steady].max()) if dtype == torch.bfloat16 else 0.0
    got = part.forward(h.to(dtype).to(dev()), step_context(range(rows), [None], 16))
    assert got.dtype == torch.float32 and torch.isfinite(got).all()
    close(got[steady], want[steady], TOL[dtype], "routed experts", noise)


def retention_part(dtype, width, m, tensors):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    children = {}
    if m.get("rot"):
        children["position"] = PartSpec.make("rotary_blend", {"head_dim": m["dim"], "dims": m["rot"]["dims"],
                                                              "base": m["rot"]["base"], "scaling": None})
    spec = PartSpec.make("lightning", {"hidden_size": width, "num_heads": m["heads"], "key_dim": m["dim"],
                                       "value_dim": m["vdim"], "decay": tuple(m["decay"]), "eps": 1e-6, "activation": "none",
                                       "key_scale": m["dim"] ** -0.5, "norm": "per_head", "gate": "silu", "stream": "float32"},
                         {n: n for n in tensors}, children)
    return MIXERS.get(spec.kind)(spec, tensors, runtime(dtype))


def retention_tensors(width, heads, d, dv, g):
    return {n: bf16(t) for n, t in {
        "q": torch.randn(heads * d, width, generator=g) * 0.3, "k": torch.randn(heads * d, width, generator=g) * 0.3,
        "v": torch.randn(heads * dv, width, generator=g) * 0.3, "g": torch.randn(heads * dv, width, generator=g) * 0.3,
        "o": torch.randn(width, heads * dv, generator=g) * (heads * dv) ** -0.5}.items()}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dv,decay,rot", [(3, 8, 12, (0.5, 0.97, 1.0), (8, 100.0)), (1, 20, 10, (0.9,), None),
                                                  (2, 5, 7, (0.0, 0.6), (4, 10.0)), (2, 64, 64, (0.999, 1.0), (32, 1e6)),
                                                  (2, 32, 80, (0.3, 0.9999), (32, 50.0)), (1, 128, 33, (0.99,), (2, 7.0))])
def test_retention_in_portions_against_token_by_token(dtype, heads, d, dv, decay, rot):
    """The part in portions of many sizes (one row, two rows, more than a chunk) against the plain recurrence, with a
    state slot that held another request's state before, and then a second request in the same slot."""
    from tesseract_b200.parts import CacheBinding

    T, width = 421, 24
    g = torch.Generator().manual_seed(heads * d + dv)
    tensors = retention_tensors(width, heads, d, dv, g)
    m = {"heads": heads, "dim": d, "vdim": dv, "decay": list(decay)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    part = retention_part(dtype, width, m, tensors)
    need = part.cache_need()
    assert tuple(need.shape) == (heads, d, dv) and need.dtype == torch.float32
    h = torch.randn(T, width, generator=g).to(dtype)
    want, want_state = plain.retention(m, as_plain(tensors), h.double().numpy(), 1e-6)
    noise = 0.0
    if dtype == torch.bfloat16:
        noise = float(np.abs(plain.retention(m, as_plain(tensors), h.double().numpy(), 1e-6, store=plain.bfloat16)[0] - want).max())
    state = torch.full((3,) + tuple(need.shape), 5.0, dtype=torch.float32, device=dev())     # stale states everywhere
    binding = CacheBinding(group=0, storage=state, writes=True, page_size=16)
    sizes = [1, 1, 2, 3, 64, 65, 1, 130, 7, 2, 31, 1, 1, 100]
    for attempt in range(2):                               # the second request finds the first one's state in the slot
        state[1].zero_()                                   # what admitting a request does to its slot
        got, at, k = [], 0, 0
        while at < T:
            n = min(sizes[k % len(sizes)], T - at)
            got.append(part.forward(h[at:at + n].to(dev()), step_context(range(at, at + n), [None], 16, slot=1), binding))
            at, k = at + n, k + 1
        close(torch.cat(got), want, TOL[dtype], f"request {attempt}", noise)
        close(state[1], want_state, 2e-5 if dtype == torch.float32 else 2e-2, "state")
        assert bool((state[0] == 5.0).all()) and bool((state[2] == 5.0).all())      # other requests' slots untouched


@pytest.mark.parametrize("decay", [1.0, 0.995])
def test_retention_keeps_a_product_from_hundreds_of_tokens_back(decay):
    """One early token's key is what the last row's query asks for (all other keys are orthogonal to it), 637 tokens
    later and decoded one by one: the answer is that token's value times the decay's power."""
    from tesseract_b200.parts import CacheBinding

    heads, d, dv, width, T = 1, 8, 8, 16, 640
    tensors = {"q": torch.zeros(d, width), "k": torch.zeros(d, width), "v": torch.zeros(dv, width), "g": torch.zeros(dv, width),
               "o": torch.zeros(width, dv)}
    tensors["q"][:, :d] = torch.eye(d)
    tensors["k"][:, :d] = torch.eye(d)
    tensors["v"][:, d:] = torch.eye(dv)
    tensors["g"][:, :] = 0.25
    tensors["o"][:dv, :] = torch.eye(dv)
    m = {"heads": heads, "dim": d, "vdim": dv, "decay": [decay]}
    part = retention_part(torch.float32, width, m, tensors)
    h = torch.zeros(T, width)
    h[:, 1] = 1.0                                    # every key and query points along dimension 1 ...
    h[2, :d] = 0.0
    h[2, 0] = 1.0                                    # ... but token 2's key, along dimension 0,
    h[2, d:] = torch.arange(1, dv + 1).float()
    h[T - 1, :d] = 0.0
    h[T - 1, 0] = 1.0                                # which only the last row's query asks for
    h[:, d:] += 0.01
    want, _ = plain.retention(m, as_plain(tensors), h.double().numpy(), 1e-6)
    lost, _ = plain.retention(m, as_plain(tensors), np.concatenate([h[:2], h[3:]]).astype(np.float64), 1e-6)
    assert np.abs(want[T - 1] - lost[T - 2]).max() > 0.05, "the case is not sharp"
    state = torch.zeros((2, heads, d, dv), dtype=torch.float32, device=dev())
    binding = CacheBinding(group=0, storage=state, writes=True, page_size=16)
    got = [part.forward(h[:5].to(dev()), step_context(range(5), [None], 16), binding)]
    for t in range(5, T):
        got.append(part.forward(h[t:t + 1].to(dev()), step_context([t], [None], 16), binding))
    close(torch.cat(got), want, 2e-5, "decoded")


def window_case(heads, kv_heads, d, dv, size, pool, rot, T, seed):
    """Tensors, input rows and marked (row, key) pairs of a pooled-window attention in which queries read one slice of the
    input and keys another, so that a marked row's query points along its key and nowhere else.  A key that lies in front
    of the row's window shares its direction with its whole block, so that the block's average points there too."""
    g = torch.Generator().manual_seed(seed)
    width = 2 * d + 8
    tensors = {"q": torch.zeros(heads * d, width), "k": torch.zeros(kv_heads * d, width),
               "v": torch.randn(kv_heads * dv, width, generator=g) * 0.5, "o": torch.randn(width, heads * dv, generator=g) * 0.2,
               "q.b": torch.randn(heads * d, generator=g) * 0.02, "k.b": torch.randn(kv_heads * d, generator=g) * 0.02,
               "v.b": torch.randn(kv_heads * dv, generator=g) * 0.1, "sink": torch.randn(heads, generator=g)}
    for head in range(heads):
        tensors["q"][head * d:(head + 1) * d, d:2 * d] = torch.eye(d)
    for head in range(kv_heads):
        tensors["k"][head * d:(head + 1) * d, :d] = torch.eye(d)
    tensors = {n: bf16(t) for n, t in tensors.items()}
    h = torch.randn(T, width, generator=g)
    rows = [T - 1, 300, 257, 256, 200, 150, 64, 48, size + 2 * pool + 3, size - 1, size]
    backs = [size - 1, size, size + pool - 1, size + pool, 0, 16, size - 1, size, size + pool, size - 1, size]
    pairs = []
    for row, back in zip(rows, backs):
        key = row - back
        if 0 <= key <= row < T and all(row != r for r, _ in pairs):
            pairs.append((row, key))
    pairs.append((T - 2, 1))                          # hundreds of positions back, through its block's average
    for row, key in pairs:
        if key <= row - size:                         # in front of the window: the whole block points one way
            first = (key // pool) * pool
            h[first:first + pool, :d] = h[key, :d].clone()
        h[row, d:2 * d] = h[key, :d].clone() * 1.5
    m = {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": dv, "mask": {"size": size, "pool": pool},
         "scale": 6.0 / d ** 0.5, "softcap": 30.0}
    if rot is not None:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return tensors, bf16(h).float(), m, pairs


def window_part(dtype, width, m, tensors):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    children = {}
    if m.get("rot"):
        children["position"] = PartSpec.make("rotary_blend", {"head_dim": m["dim"], "dims": m["rot"]["dims"],
                                                              "base": m["rot"]["base"], "scaling": None})
    spec = PartSpec.make(
        "normed_attention",
        {"hidden_size": width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"], "value_dim": m["vdim"],
         "scale": m["scale"], "qk_norm_eps": 1e-6, "softcap": m["softcap"], "sink": True, "bias": True, "stream": "float32",
         "mask": (("kind", "window_pooled"), ("pool", m["mask"]["pool"]), ("size", m["mask"]["size"]))},
        {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "sink": "sink"}, children)
    return MIXERS.get(spec.kind)(spec, {role: tensors[name] for role, name in spec.weights.items()}, runtime(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,dv", [(4, 2, 16, 24), (3, 1, 6, 10), (2, 2, 64, 128), (6, 3, 12, 8), (2, 1, 128, 64)])
@pytest.mark.parametrize("size,pool,rot", [(33, 4, None), (16, 16, (4, 50.0)), (5, 7, None), (1, 1, None), (40, 3, (2, 9.0)),
                                           (80, 12, None)])
def test_a_pooled_window_sees_exactly_its_tokens_and_blocks(dtype, heads, kv_heads, d, dv, size, pool, rot):
    """The part as a prompt, in portions and as decoded rows over scrambled pages full of stale data, against the plain
    function; and the case is sharp: a window one position longer or shorter, blocks one token longer or shorter, or a
    forgotten sink would change a marked row."""
    from tesseract_b200.parts import CacheBinding

    T, page = 330, 16
    if rot is not None and rot[0] > d:
        rot = (d - d % 2, rot[1])
    tensors, h, m, pairs = window_case(heads, kv_heads, d, dv, size, pool, rot, T, seed=heads * 100 + d + size)
    weights = as_plain(tensors)
    want = plain.pooled_window_attention(m, weights, h.double().numpy(), 1e-6)
    marked = [row for row, _ in pairs]
    noticed = []
    for other_mask in ({"size": size + 1, "pool": pool}, {"size": max(size - 1, 1), "pool": pool}, {"size": size, "pool": pool + 1}):
        if other_mask == m["mask"]:
            continue
        other = plain.pooled_window_attention(dict(m, mask=other_mask), weights, h.double().numpy(), 1e-6)
        noticed.append(float(np.abs(other[marked] - want[marked]).max()))
    # (a block of one token is its own average: there a window one longer changes nothing)
    assert max(noticed) > 0.05 and (pool == 1 or d < 12 or min(noticed) > 0.05), f"marked rows do not notice a reach one off: {noticed}"
    no_sink = plain.pooled_window_attention(m, dict(weights, sink=weights["sink"] - 50.0), h.double().numpy(), 1e-6)
    assert np.abs(no_sink - want).max() > 0.02, "no row notices the sink"
    noise = 0.0
    if dtype == torch.bfloat16:
        coarse = plain.pooled_window_attention(m, weights, h.double().numpy(), 1e-6, store=plain.bfloat16)
        noise = float(np.abs(coarse - want).max())
    part = window_part(dtype, h.shape[1], m, tensors)
    tokens_need, blocks_need = part.cache_need()
    assert tokens_need.window == size and tokens_need.hold == pool and blocks_need.positions_per_entry == pool
    count = -(-T // page)
    torch.manual_seed(3)
    order = [1 + i for i in torch.randperm(count).tolist()]              # pages taken in scrambled order
    block_order = [1 + i for i in torch.randperm(count).tolist()]
    for cut in ("prompt", "decode", "portions", "twos"):
        storage = torch.full((count + 1, tokens_need.page_shape(page)[0]), 7.0, dtype=dtype, device=dev())     # stale data
        averaged = torch.full((count + 1, blocks_need.page_shape(page)[0]), -9.0, dtype=dtype, device=dev())
        bindings = (CacheBinding(group=0, storage=storage, writes=True, page_size=page),
                    CacheBinding(group=1, storage=averaged, writes=True, page_size=page))
        if cut == "prompt":
            portions = [(0, T)]
        elif cut == "decode":
            portions = [(0, 10)] + [(p, p + 1) for p in range(10, T)]
        elif cut == "twos":
            portions = [(p, min(p + 2, T)) for p in range(0, T, 2)]
        else:
            edges = list(range(0, T, 37)) + [T]
            portions = list(zip(edges[:-1], edges[1:]))
        got = torch.cat([part.forward(h[lo:hi].to(dtype).to(dev()), step_context(range(lo, hi), [order, block_order], page), bindings)
                         for lo, hi in portions])
        close(got, want, TOL[dtype], cut, noise)


def latent_part(dtype, width, m, tensors):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    children = {}
    if m.get("rot"):
        scaling = m["rot"].get("scaling")
        children["position"] = PartSpec.make("rotary_pairs", {"head_dim": m["rot_dim"], "dims": m["rot"]["dims"], "base": m["rot"]["base"],
                                                              "scaling": tuple(scaling.items()) if scaling else None})
    spec = PartSpec.make(
        "latent_attention",
        {"hidden_size": width, "num_heads": m["heads"], "key_dim": m["dim"], "rot_width": m["rot_dim"], "value_dim": m["vdim"],
         "rank": m["kv_rank"], "scale": m["scale"], "eps": 1e-6, "mask": (("kind", "causal"),), "gate": True, "stream": "float32"},
        {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "g": "g", "o": "o"}, children)
    return MIXERS.get(spec.kind)(spec, {role: tensors[name] for role, name in spec.weights.items()}, runtime(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dr,dv,rank,scaling", [(3, 12, 8, 10, 20, (4.0, 32, 8.0, 1.0)), (2, 16, 4, 24, 12, None),
                                                        (1, 10, 6, 14, 9, (2.0, 16, 2.0, 1.0)), (4, 8, 0, 4, 8, None),
                                                        (2, 64, 32, 128, 128, (8.0, 128, 16.0, 1.0))])
def test_gated_latent_attention_with_stretched_rotation(dtype, heads, d, dr, dv, rank, scaling):
    """The causal latent attention with its output gate as a prompt, in portions and decoded, against the plain function;
    the last rows ask for the first token's key, hundreds of positions back (its latent and the queries are scaled so that
    this score stands out), and would notice its loss."""
    from tesseract_b200.parts import CacheBinding

    T, page, width = 300, 16, 40
    g = torch.Generator().manual_seed(heads * 31 + d)
    tensors = {"q": torch.randn(heads * (d + dr), width, generator=g) * width ** -0.5,
               "dkv": torch.randn(rank + dr, width, generator=g) * width ** -0.5, "dkv.norm": torch.rand(rank, generator=g) + 0.5,
               "uk": torch.randn(heads * d, rank, generator=g) * rank ** -0.5, "uv": torch.randn(heads * dv, rank, generator=g) * rank ** -0.5,
               "g": torch.randn(heads * dv, width, generator=g) * width ** -0.5,
               "o": torch.randn(width, heads * dv, generator=g) * (heads * dv) ** -0.5}
    # feature 0 of the input goes into number 0 of the latent alone, which number 0 of head 0's key alone reads; feature 1
    # goes into number 0 of head 0's query alone: token 0 carries the one, the last rows the other, nobody else either
    tensors["dkv"][:, :2] = 0.0
    tensors["dkv"][0, :] = 0.0
    tensors["dkv"][0, 0] = 1.0
    tensors["uk"][0, :] = 0.0
    tensors["uk"][:, 0] = 0.0
    tensors["uk"][0, 0] = 4.0
    tensors["q"][:, :2] = 0.0
    tensors["q"][0, :] = 0.0
    tensors["q"][0, 1] = 4.0
    tensors = {n: bf16(t) for n, t in tensors.items()}
    m = {"heads": heads, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": (d + dr) ** -0.5}
    if dr:
        m["rot"] = {"dims": dr, "base": 1000.0}
        if scaling:
            m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    h = bf16(torch.randn(T, width, generator=g)).float()
    h[:, :2] = 0.0
    h[0, 0] = 6.0
    h[T - 3:, 1] = 3.0
    weights = as_plain(tensors)
    want = plain.latent_attention(m, weights, h.double().numpy(), 1e-6)
    lost = plain.latent_attention(m, weights, h[1:].double().numpy(), 1e-6)
    assert np.abs(lost[-1] - want[-1]).max() > 0.02, "the last row does not notice the first token"
    noise = 0.0
    if dtype == torch.bfloat16:
        noise = float(np.abs(plain.latent_attention(m, weights, h.double().numpy(), 1e-6, store=plain.bfloat16) - want).max())
    part = latent_part(dtype, width, m, tensors)
    need = part.cache_need()
    count = -(-T // page)
    torch.manual_seed(4)
    order = [1 + i for i in torch.randperm(count).tolist()]
    for cut in ("prompt", "decode", "portions"):
        storage = torch.full((count + 1, need.page_shape(page)[0]), 7.0, dtype=dtype, device=dev())
        binding = CacheBinding(group=0, storage=storage, writes=True, page_size=page)
        if cut == "prompt":
            portions = [(0, T)]
        elif cut == "decode":
            portions = [(0, 10)] + [(p, p + 1) for p in range(10, T)]
        else:
            edges = list(range(0, T, 37)) + [T]
            portions = list(zip(edges[:-1], edges[1:]))
        got = torch.cat([part.forward(h[lo:hi].to(dtype).to(dev()), step_context(range(lo, hi), [order], page), binding)
                         for lo, hi in portions])
        close(got, want, TOL[dtype], cut, noise)


# ----------------------------------------------------------------------------- whole models


def make_requests(name):
    vocab = TINY_LADEDRA[name]["vocab"]
    return {f"{name}{i}": random_tokens(vocab, n, seed=500 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tesseract_b200.weights.random_init import write_random_model

    made = {}

    def get(name):
        if name not in made:
            made[name] = write_random_model(str(tmp_path_factory.mktemp(f"ladedra_{name}")), TINY_LADEDRA[name], seed=23)
        return made[name]

    return get


@pytest.fixture(scope="module")
def engines(folders):
    from tesseract_b200.engine import load_model, make_stepper

    models = {}

    def get(name, dtype, capacity_tokens=4096, max_requests=8):
        if (name, dtype) not in models:
            models[(name, dtype)] = load_model(folders(name), dtype=dtype)
        return make_stepper(models[(name, dtype)], capacity_tokens=capacity_tokens, max_requests=max_requests)

    return get


_PLAIN = {}
# A router that decides by less than this (in scores, which sum to one) may decide the other way after a rounding to
# bfloat16: such a position's own logits are not compared in bfloat16 (they are in float32).
CLOSE_CALL = 0.05
CLOSE = {}


def plain_rows(folder, requests, dtype):
    """Per request the plain model's logits and, for bfloat16, the most that rounding to bfloat16 alone changes in the
    plain model's logits of that request (at positions without a close routing call)."""
    want, noise = {}, {}
    config, tensors = plain.load_folder(folder)
    for rid, tokens in requests.items():
        key = (folder, tuple(tokens))
        if key not in _PLAIN:
            gaps = {}
            exact = plain.forward(config, tensors, tokens, close_calls=gaps)[0]
            coarse = plain.forward(config, tensors, tokens, store=plain.bfloat16)[0]
            close_rows = {t for t, gap in gaps.items() if gap < CLOSE_CALL}
            steady = [t for t in range(len(tokens)) if t not in close_rows] or [0]
            _PLAIN[key] = (exact, float(np.abs(coarse - exact)[steady].max()), close_rows)
        want[rid], noise[rid], CLOSE[rid] = _PLAIN[key]
    worst = max(noise.values())           # (one model, one noise: a short request is a small sample of it)
    return want, ({rid: worst for rid in noise} if dtype == "bfloat16" else None)


def replay_against_plain(stepper, steps, folder, requests, dtype, what):
    """Replay a trace and compare every wanted row with the plain model.  In bfloat16 a row may also differ by ``NOISE``
    times what rounding to bfloat16 alone changes in the plain model's logits of its request."""
    want, noise = plain_rows(folder, requests, dtype)
    got = replay(stepper, steps)
    if noise is None:
        return compare(got, want, REL[dtype], what)
    assert got, f"{what}: nothing was replayed"
    for (rid, position), row in sorted(got.items(), key=lambda kv: (str(kv[0][0]), kv[0][1])):
        limit = max(REL[dtype] * float(np.abs(want[rid]).max()), NOISE * noise[rid])
        err = float(np.abs(row.astype(np.float64) - want[rid][position]).max())
        if position in CLOSE[rid]:
            assert np.isfinite(row).all()
            continue
        assert np.isfinite(row).all() and err <= limit, (f"{what}: first wrong token is request {rid!r} position "
                                                         f"{position}: max |diff| {err:.3e} > {limit:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_every_layer_matches_plain(engines, folders, name, dtype):
    """The stream after every layer against the plain model's."""
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.parts.block import GatedPreNormBlock

    config, tensors = plain.load_folder(folders(name))
    tokens = random_tokens(config["vocab"], 37, seed=8)
    _, want = plain.forward(config, tensors, tokens)
    _, coarse = plain.forward(config, tensors, tokens, store=plain.bfloat16)
    seen = []
    original = GatedPreNormBlock.forward

    def recording(self, stream, ctx, cache, next_norm=None):
        out = original(self, stream, ctx, cache, next_norm=next_norm)
        assert out.update is None and out.residual.dtype == torch.float32
        seen.append(out.residual.double().cpu().numpy())
        return out

    stepper = engines(name, dtype)
    assert stepper.cache.admit("one")
    GatedPreNormBlock.forward = recording
    try:
        stepper.step([StepEntry("one", tokens, [len(tokens) - 1])])
    finally:
        GatedPreNormBlock.forward = original
        stepper.cache.release("one")
    assert len(seen) == len(want) == len(config["layers"])
    for index, got in enumerate(seen):
        limit = REL[dtype] * float(np.abs(want[index]).max())
        if dtype == "bfloat16":       # or what rounding to bfloat16 alone moves in the plain model, NOISE times
            limit = max(limit, NOISE * float(np.abs(coarse[index] - want[index]).max()))
        assert float(np.abs(got - want[index]).max()) <= limit, f"layer {index}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "twos"])
def test_cuts_match_plain(engines, folders, name, dtype, cut):
    """Whole prompts, prompts with a decoded tail (over which the windows move, blocks fill and the states are carried),
    portions of changing size, and portions of two and three tokens throughout."""
    requests = make_requests(name)
    if cut == "twos":
        steps = trace_portions(requests, sizes=(2, 3, 2, 2))
    elif cut == "tail":
        steps = trace_tail(requests, tail=60)
    else:
        steps = {"whole": trace_whole, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/{cut}")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_mixed_batches_with_slots_and_pages_used_again(engines, folders, name, dtype):
    requests = make_requests(name)
    requests.update({f"{name}x{i}": random_tokens(TINY_LADEDRA[name]["vocab"], n, seed=17 + i)
                     for i, n in enumerate([50, 21, 90, 34, 7])})
    steps = trace_mixed(requests, seed=5, live_max=3)
    assert max(len(e) for e, _ in steps) >= 3, "the trace should batch several requests"
    # three state slots for eight or more requests: every slot serves several requests one after the other
    stepper = engines(name, dtype, capacity_tokens=max_live_tokens(steps), max_requests=3)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/mixed")
    assert stepper.cache.pages_reused > 0, "the pool was sized so that pages must be used again"
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "e"])
def test_a_batch_gives_each_request_what_it_gets_alone(engines, name, dtype):
    """Unequal requests side by side against each alone, in portions that cut windows, blocks and pages."""
    from tesseract_b200.engine import StepEntry

    requests = make_requests(name)
    sizes = [9, 2, 30, 5]
    alone = replay(engines(name, dtype), trace_portions(requests, sizes=tuple(sizes)))
    together = {}
    stepper = engines(name, dtype)
    at = {rid: 0 for rid in requests}
    for rid in requests:
        assert stepper.cache.admit(rid)
    turn = 0
    while any(at[rid] < len(t) for rid, t in requests.items()):
        batch, meta = [], []
        for rid, tokens in requests.items():
            if at[rid] >= len(tokens):
                continue
            size = sizes[turn % 4]
            if len(tokens) - at[rid] - size == 1:
                size += 1
            part = tokens[at[rid]:at[rid] + size]
            batch.append(StepEntry(rid, part, list(range(len(part)))))
            meta.append((rid, at[rid], len(part)))
            at[rid] += len(part)
        rows = stepper.step(batch).float().cpu().numpy()
        r = 0
        for rid, base, n in meta:
            for place in range(n):
                together[(rid, base + place)] = rows[r]
                r += 1
        turn += 1
    worst = max(float(np.abs(together[key] - alone[key]).max()) for key in alone)
    scale = max(float(np.abs(row).max()) for row in alone.values())
    # the products of a batch take other kernels at other row counts: equal up to rounding, not bit for bit
    assert worst <= REL[dtype] * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "c", "e"])
def test_long_decoding_while_windows_move_and_blocks_fill(engines, folders, name, dtype):
    tokens = random_tokens(TINY_LADEDRA[name]["vocab"], 180, seed=77)
    requests = {"long": tokens}
    steps = trace_tail(requests, tail=170)          # ten tokens of prompt, then 170 decoded one by one
    stepper = engines(name, dtype, capacity_tokens=192)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/long decode")
    assert stepper.cache.used_pages() == 0


def test_pages_behind_window_and_unfinished_block_go_back_while_the_request_lives(engines):
    """Model "b" has a window of 3 with blocks of 5 and a window of 40 with blocks of 7 (pages of 16) beside one causal
    layer: the windowed groups of a request of 200 tokens never hold more than a few pages, the causal one holds its
    thirteen, and a group of averaged blocks holds a page per 16 blocks."""
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.parts import PagedKeyValueNeed, PagedVectorNeed, PooledBlocksNeed

    stepper = engines("b", "float32", capacity_tokens=208)
    assert stepper.cache.admit("one")
    tokens = random_tokens(TINY_LADEDRA["b"]["vocab"], 200, seed=5)
    for at in range(0, 200, 10):
        stepper.step([StepEntry("one", tokens[at:at + 10], [9])])
        for index, group in enumerate(stepper.cache.groups):
            if group.pool is None:
                continue
            held = len(stepper.cache.pages_of("one", index))
            if isinstance(group.need, PagedVectorNeed):
                assert held == -(-(at + 10) // 16)
            elif isinstance(group.need, PooledBlocksNeed):
                assert held == -(-(-(-(at + 10) // group.need.pool)) // 16)
            else:
                assert isinstance(group.need, PagedKeyValueNeed) and held <= 5
    stepper.cache.release("one")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("name", ["a", "b", "e"])
def test_greedy_generation_through_the_scheduler(folders, name, dtype, graphs):
    from tesseract_b200 import LLM, SamplingParams

    config, tensors = plain.load_folder(folders(name))
    prompts = [random_tokens(config["vocab"], n, seed=n) for n in (3, 19, 75, 1)]
    steps = 24
    llm = LLM(folders(name), dtype=dtype, kv_capacity_tokens=1024, max_running=3, prefill_chunk_tokens=32,
              cuda_graphs=graphs)
    outs = llm.generate(prompts, SamplingParams(max_tokens=steps, temperature=0.0, ignore_eos=True))
    for prompt, out in zip(prompts, outs):
        assert len(out.token_ids) == steps and out.finish_reason == "length"
        tokens = list(prompt)
        for k, got in enumerate(out.token_ids):
            logits = plain.forward(config, tensors, tokens)[0][-1]
            best = int(np.argmax(logits))
            margin = float(logits[best] - logits[got])
            limit = GREEDY_MARGIN[dtype] * float(np.abs(logits).max())
            if got != best and margin > limit and dtype == "bfloat16":
                # what rounding to bfloat16 alone does to this position's logits in the plain model bounds what the
                # engine's token may lose
                coarse = plain.forward(config, tensors, tokens, store=plain.bfloat16)[0][-1]
                limit = max(limit, 3.0 * float(np.abs(coarse - logits).max()))
            assert got == best or margin <= limit, f"{name}/{dtype}: token {k} is {got}, plain says {best}"
            tokens.append(got)
    assert llm.stepper.cache.used_pages() == 0
    if graphs:      # decode steps were replayed as graphs, not issued launch by launch
        assert llm.stepper.graphs.safe and llm.stepper.graphs.replays >= steps - 2
    del llm
    torch.cuda.empty_cache()


def test_replay_program_runs_a_ladedra_folder(folders, tmp_path):
    """``bin/trace_run`` picks the model class by ``config.json`` and writes the logits of the wanted places."""
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    config, tensors = plain.load_folder(folders("c"))
    tokens = random_tokens(config["vocab"], 30, seed=9)
    lines = [json.dumps({"step": 0, "entries": [{"id": "a", "tokens": tokens[:20], "want": [0, 19]}], "end": []}),
             json.dumps({"step": 1, "entries": [{"id": "a", "tokens": tokens[20:], "want": [9]}], "end": ["a"]})]
    out = tmp_path / "out"
    done = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders("c"), "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "64"], input="\n".join(lines) + "\n",
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert [l for l in done.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want = plain.forward(config, tensors, tokens)[0]
    first = np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1)
    second = np.fromfile(out / "1.f32", dtype="<f4").reshape(1, -1)
    scale = float(np.abs(want).max())
    assert np.abs(first - want[[0, 19]]).max() <= 2e-5 * scale
    assert np.abs(second - want[[29]]).max() <= 2e-5 * scale


def test_command_line_generates_and_prints_the_plan(folders):
    import json
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    folder = folders("a")
    common = [sys.executable, os.path.join(root, "bin", "tesseract"), "--model-path", folder, "--kv-capacity-tokens",
              "256", "--max-running", "2", "--dtype", "float32"]
    done = subprocess.run(common + ["--prompt-ids", "5,6,7,8", "--random-prompt", "11", "--max-tokens", "4",
                                    "--temperature", "0", "--ignore-eos", "--json", "--check-weights"],
                          capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    records = [json.loads(line) for line in done.stdout.strip().splitlines()]
    assert len(records) == 2 and all(len(r["token_ids"]) == 4 and r["finish_reason"] == "length" for r in records)
    config, tensors = plain.load_folder(folder)
    tokens = [5, 6, 7, 8]
    for got in records[0]["token_ids"]:
        logits = plain.forward(config, tensors, tokens)[0][-1]
        best = int(np.argmax(logits))
        assert got == best or float(logits[best] - logits[got]) <= GREEDY_MARGIN["float32"] * float(np.abs(logits).max())
        tokens.append(got)
    shown = subprocess.run(common + ["--print-plan"], capture_output=True, text=True, timeout=600)
    assert shown.returncode == 0, shown.stderr[-2000:]
    assert "kernel plan for Ladedra" in shown.stdout
    for kind in ("latent_attention", "parallel_mixers"):
        assert f"mixer '{kind}'" in shown.stdout


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34])
def test_random_configurations_match_plain_in_float32(tmp_path, seed):
    """Configurations drawn at random (layer order, every size and constant), each whole, with a decoded tail, in
    portions and in mixed batches."""
    import random

    from tesseract_b200.engine import load_model, make_stepper
    from tesseract_b200.weights.random_init import write_random_model

    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "model"), config, seed=seed)
    r = random.Random(seed + 1000)
    lengths = [1, r.randint(2, 40), r.randint(41, 140), r.randint(141, 300), r.randint(5, 90)]
    requests = {f"q{i}": random_tokens(config["vocab"], n, seed=seed * 10 + i) for i, n in enumerate(lengths)}
    model = load_model(folder, dtype="float32")
    for name, steps in (("whole", trace_whole(requests)), ("tail", trace_tail(requests, tail=20)),
                        ("portions", trace_portions(requests)), ("mixed", trace_mixed(requests, seed=seed, live_max=4))):
        stepper = make_stepper(model, capacity_tokens=max(1024, max_live_tokens(steps)), max_requests=4)
        # (drawn models hold ill-conditioned spots, a head whose output the norm per head divides by almost nothing, say:
        # 32-bit rounding shows there at up to 1e-4 of the largest logit; a lost key or a reach one off moves percents)
        compare(replay(stepper, steps), plain_rows(folder, requests, "float32")[0], 1e-4, f"seed {seed}/{name}")
        assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34])
def test_random_configurations_match_plain_in_bfloat16(tmp_path, seed):
    """The same configurations in bfloat16 (products of odd sizes, head sizes on and off the tensor-core kernels),
    whole, with a decoded tail and in mixed batches."""
    import random

    from tesseract_b200.engine import load_model, make_stepper
    from tesseract_b200.weights.random_init import write_random_model

    config = random_config(seed)
    folder = write_random_model(str(tmp_path / "model"), config, seed=seed)
    r = random.Random(seed + 2000)
    lengths = [1, r.randint(2, 40), r.randint(41, 140), r.randint(260, 330), r.randint(5, 90)]
    requests = {f"q{i}": random_tokens(config["vocab"], n, seed=seed * 10 + i) for i, n in enumerate(lengths)}
    model = load_model(folder, dtype="bfloat16")
    for name, steps in (("whole", trace_whole(requests)), ("tail", trace_tail(requests, tail=20)),
                        ("mixed", trace_mixed(requests, seed=seed, live_max=4))):
        stepper = make_stepper(model, capacity_tokens=max(1024, max_live_tokens(steps)), max_requests=4)
        replay_against_plain(stepper, steps, folder, requests, "bfloat16", f"seed {seed}/{name}")
        assert stepper.cache.used_pages() == 0
