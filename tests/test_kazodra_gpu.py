"""Kazodra on the GPU against the plain implementation (``tests/plain/kazodra.py``).

First every mechanism alone (its kernel or part against the plain function of the same name, with inputs made so that
a fault shows: one key that dominates, placed hundreds of positions back, at a page border, just inside and just
outside a window; a recurrence carried over many steps with decays of zero and one), then whole tiny models with
random weights under every way of cutting the work: whole prompts, token-by-token decoding, portions down to two
tokens, mixed batches with slots and pages used again, long decoding while the windows move over decoded tokens, and
greedy generation through the package's own entry point and scheduler.
"""

import numpy as np
import pytest
import torch

from tests.helpers import (GREEDY_MARGIN, compare, max_live_tokens, random_tokens, replay, trace_mixed, trace_portions,
                           trace_tail, trace_whole)
from tests.kazodra_models import TINY_KAZODRA, random_config
from tests.plain import kazodra as plain

pytestmark = pytest.mark.gpu

REL = {"float32": 2e-5, "bfloat16": 3e-2}
TOL = {torch.float32: 2e-5, torch.bfloat16: 3e-2}
# In bfloat16 a result may also differ by this many times what rounding to bfloat16 alone moves in the plain computation
# (``round_to``): the package rounds at other places than the plain functions do (it attends in the latent space, for
# one), so the two are two draws of that noise, and in these tiny models single positions amplify it tenfold.
NOISE = 5.0


def dev():
    return torch.device("cuda", 0)


def runtime(dtype):
    from tesseract_b200.parts import Runtime

    return Runtime(dtype, dev())


def close(got, want, tol, what="", noise=0.0):
    """``noise``: what rounding to bfloat16 alone moves in the plain computation; ``NOISE`` times that is allowed too."""
    got, want = got.detach().cpu().double(), want.detach().cpu().double()
    assert torch.isfinite(got).all(), what
    worst = (got - want).abs().max().item()
    assert worst <= max(tol * max(1.0, want.abs().max().item()), NOISE * noise), f"{what}: {worst}"


def _step_context(positions, page_order, page, tokens=None, slot=0):
    """A step of one sequence whose rows stand at ``positions`` (consecutive), with the given block table and slot."""
    from tesseract_b200.parts import GroupView, StepContext

    n = len(positions)
    as_i32 = lambda values: torch.tensor(values, dtype=torch.int32, device=dev())         # noqa: E731
    return StepContext(num_rows=n, num_seqs=1, token_ids=as_i32(list(tokens) if tokens is not None else [0] * n),
                       positions=as_i32(list(positions)), seq_of_row=as_i32([0] * n), row_start=as_i32([0, n]),
                       seq_begin=as_i32([positions[0]]), state_slots=as_i32([slot]),
                       groups=[GroupView(as_i32([page_order]), page)], host_new=[n], host_begin=[positions[0]],
                       host_slots=[slot], max_new=n, max_context=positions[-1] + 1)


# ----------------------------------------------------------------------------- mechanisms alone


@pytest.mark.parametrize("width", [5, 42, 66, 2048, 12288])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_norms_around_an_addition(width, out_dtype):
    """``x += post(update)``, then ``following(x)``, with layer norms (weight and bias) and with a weighted unit root
    mean square; 32-bit sums whatever the output's dtype."""
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    rows, eps = 13, 1e-5
    x = torch.randn(rows, width, generator=g) * 3.0 + 1.5          # a mean far from zero: the variance is of deviations
    update = torch.randn(rows, width, generator=g) * 20.0 - 4.0
    w1, b1, w2, b2 = (torch.randn(width, generator=g) for _ in range(4))
    want_x = x.double() + plain.layer_norm(update.double(), w1.double(), b1.double(), eps)
    want_y = plain.layer_norm(want_x, w2.double(), b2.double(), eps)
    stream = x.to(dev())
    out = torch.empty(rows, width, dtype=out_dtype, device=dev())
    copy = torch.empty_like(out)
    kernels.norm_add_norm(stream, update.to(dev()), (kernels.NORM_LAYER, w1.to(dev()), b1.to(dev())),
                          (kernels.NORM_LAYER, w2.to(dev()), b2.to(dev())), out, copy, eps)
    close(stream, want_x, 2e-5, "stream")
    close(out, want_y, TOL[out_dtype], "following norm")
    close(copy, want_x, TOL[out_dtype], "copy")
    # the update alone, at unit root mean square with a plain weight, and nothing behind it
    stream = x.to(dev())
    kernels.norm_add_norm(stream, update.to(dev()), (kernels.NORM_RMS, w1.to(dev()), None), None, None, None, eps)
    close(stream, x.double() + plain.unit_rms(update.double(), eps) * w1.double(), 2e-5, "rms update")
    # no update: the stream stays and is normed
    stream = x.to(dev())
    kernels.norm_add_norm(stream, None, None, (kernels.NORM_LAYER, w2.to(dev()), b2.to(dev())), out, None, eps)
    assert torch.equal(stream.cpu(), x)
    close(out, plain.layer_norm(x.double(), w2.double(), b2.double(), eps), TOL[out_dtype], "norm alone")


@pytest.mark.parametrize("width", [7, 64, 200, 4096])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_over_all_heads_with_a_gate(width, dtype):
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(width)
    v = torch.randn(9, width, generator=g) * 50.0
    weight = torch.randn(width, generator=g)
    gate = (torch.randn(9, width + 3, generator=g) * 2.0).to(dtype)
    out = torch.empty(9, width, dtype=dtype, device=dev())
    kernels.gated_rms_norm(v.to(dev()), weight.to(dev()), gate.to(dev())[:, 3:], out, 1e-6)
    want = plain.unit_rms(v.double(), 1e-6) * weight.double() * torch.sigmoid(gate[:, 3:].double())
    close(out, want, TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,dim,slices,which", [(48, 6, 5, 2), (42, 3, 3, 0), (64, 16, 4, 3), (40, 1, 2, 1)])
def test_the_token_input_reads_its_own_slice(dtype, width, dim, slices, which):
    """The layer's term for the token itself against the plain function; a neighbouring slice gives another result."""
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import TOKEN_INPUTS

    g = torch.Generator().manual_seed(width + which)
    vocab, rows, eps = 37, 11, 1e-5
    tensors = {"table": torch.randn(vocab, slices * dim, generator=g), "gate": torch.randn(dim, width, generator=g) * 0.3,
               "proj": torch.randn(width, dim, generator=g), "norm": torch.rand(width, generator=g) + 0.5}
    tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    spec = PartSpec.make("gated_token_slice", {"hidden_size": width, "vocab_size": vocab, "dim": dim, "slices": slices,
                                               "slice": which, "activation": "gelu_tanh", "eps": eps},
                         {n: n for n in tensors})
    part = TOKEN_INPUTS.get(spec.kind)(spec, tensors, runtime(dtype))
    x = torch.randn(rows, width, generator=g)
    tokens = random_tokens(vocab, rows, seed=4)
    stream = x.to(dev())
    part.forward(stream, _step_context(range(rows), [1], 16, tokens=tokens))
    t = {n: v.double() for n, v in tensors.items()}
    ids = torch.tensor(tokens)
    round_to = None if dtype == torch.float32 else dtype
    want = plain.token_side(x.double(), ids, t["table"], which, dim, t, eps, round_to)
    close(stream - x.to(dev()), want, TOL[dtype])
    if slices > 1:
        other = plain.token_side(x.double(), ids, t["table"], (which + 1) % slices, dim, t, eps, round_to)
        assert (other - want).abs().max() > 0.05


# ----------------------------------------------------------------------------- the recurrence


def _lightning_part(dtype, width, heads, d, dv, decay, tensors):
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    spec = PartSpec.make("lightning", {"hidden_size": width, "num_heads": heads, "key_dim": d, "value_dim": dv,
                                       "decay": tuple(decay), "eps": 1e-6, "stream": "float32"}, {n: n for n in tensors})
    return MIXERS.get(spec.kind)(spec, tensors, runtime(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dv,decay", [(3, 8, 12, (0.5, 0.97, 1.0)), (1, 20, 10, (0.9,)), (2, 5, 7, (0.0, 0.6)),
                                              (2, 64, 64, (0.999, 1.0)), (2, 32, 80, (0.3, 0.9999)), (1, 128, 33, (0.99,))])
def test_recurrence_in_portions_against_token_by_token(dtype, heads, d, dv, decay):
    """The part in portions of many sizes (one row, two rows, more than a chunk) against the plain recurrence, with a
    state slot that held another request's state before, and then a second request in the same slot."""
    from tesseract_b200.parts import CacheBinding

    T, width = 421, 24
    g = torch.Generator().manual_seed(heads * d + dv)
    tensors = {"q": torch.randn(heads * d, width, generator=g) * 0.3, "k": torch.randn(heads * d, width, generator=g) * 0.3,
               "v": torch.randn(heads * dv, width, generator=g) * 0.3, "g": torch.randn(heads * dv, width, generator=g) * 0.3,
               "o": torch.randn(width, heads * dv, generator=g) * (heads * dv) ** -0.5,
               "norm": torch.rand(heads * dv, generator=g) + 0.5}
    tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    part = _lightning_part(dtype, width, heads, d, dv, decay, tensors)
    need = part.cache_need()
    assert tuple(need.shape) == (heads, d, dv) and need.dtype == torch.float32
    h = torch.randn(T, width, generator=g).to(dtype)
    m = {"heads": heads, "dim": d, "vdim": dv, "decay": list(decay)}
    weights = {n: t.double() for n, t in tensors.items()}
    want, want_state = plain.lightning(h.double(), weights, m, 1e-6, None if dtype == torch.float32 else dtype)
    state = torch.full((3,) + tuple(need.shape), 5.0, dtype=torch.float32, device=dev())     # stale states everywhere
    binding = CacheBinding(group=0, storage=state, writes=True, page_size=16)
    sizes = [1, 1, 2, 3, 64, 65, 1, 130, 7, 2, 31, 1, 1, 100]
    for attempt in range(2):                               # the second request finds the first one's state in the slot
        state[1].zero_()                                   # what admitting a request does to its slot
        got, at, k = [], 0, 0
        while at < T:
            n = min(sizes[k % len(sizes)], T - at)
            got.append(part.forward(h[at:at + n].to(dev()), _step_context(range(at, at + n), [1], 16, slot=1), binding))
            at, k = at + n, k + 1
        close(torch.cat(got), want, TOL[dtype], f"request {attempt}")
        close(state[1], want_state, 2e-5 if dtype == torch.float32 else 2e-2, "state")
        assert bool((state[0] == 5.0).all()) and bool((state[2] == 5.0).all())      # other requests' slots untouched


@pytest.mark.parametrize("decay", [1.0, 0.995])
def test_recurrence_keeps_a_product_from_hundreds_of_tokens_back(decay):
    """One token's key and value are large and every later query points at that key; all else is small: what the rows
    return is that value times the decay's power, whether they come in a prompt portion or one by one."""
    from tesseract_b200 import kernels

    heads, d, dv, T, mark = 2, 16, 24, 640, 3
    g = torch.Generator().manual_seed(1)
    proj = torch.randn(T, heads * (2 * d + dv), generator=g) * 0.05 - 8.0        # silu(-8) is tiny
    direction = torch.randn(heads, d, generator=g).abs() + 1.0
    proj[mark, heads * d:2 * heads * d] = direction.reshape(-1) * 3.0
    proj[mark, 2 * heads * d:] = 6.0
    proj[mark + 1:, :heads * d] = direction.reshape(-1) * 3.0
    q, k = plain.silu(proj[:, :heads * d].double()).view(T, heads, d), plain.silu(proj[:, heads * d:2 * heads * d].double()).view(T, heads, d)
    v = plain.silu(proj[:, 2 * heads * d:].double()).view(T, heads, dv)
    S = torch.zeros(heads, d, dv, dtype=torch.float64)
    want = torch.empty(T, heads, dv, dtype=torch.float64)
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        want[t] = torch.einsum("hde,hd->he", S, q[t])
    marked = (q[-1] * k[mark]).sum(-1)[:, None] * v[mark] * decay ** (T - 1 - mark)
    assert (marked / want[-1]).min() > 0.5                   # the marked token is most of what the last row returns
    decays = torch.full((heads,), decay, dtype=torch.float32, device=dev())
    for portions in ([T], [10] + [1] * (T - 10), [2] * (T // 2)):
        state = torch.zeros(1, heads, d, dv, device=dev())
        got, at = [], 0
        for n in portions:
            out = torch.empty(n, heads * dv, device=dev())
            i32 = lambda values: torch.tensor(values, dtype=torch.int32, device=dev())     # noqa: E731
            kernels.lightning(proj[at:at + n].to(dev()), decays, state, out, i32([0, n]), i32([0]), num_seqs=1,
                              heads=heads, dim=d, vdim=dv, max_new=n)
            got.append(out)
            at += n
        close(torch.cat(got).view(T, heads, dv), want, 2e-5, f"portions of {portions[0]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dv", [(3, 8, 12), (2, 64, 64), (1, 128, 33), (2, 5, 40)])
def test_long_portions_side_by_side_continue_each_sequence_from_its_slot(dtype, heads, d, dv):
    """A step with prompt portions of several chunks (whose chunks run side by side and meet in a scan) beside a single
    row and a short portion, every sequence from a state of its own in a slot of its own; then a second step of the same
    sequences goes on from what the first left."""
    from tesseract_b200 import kernels

    g = torch.Generator().manual_seed(d + dv)
    decay = [0.0, 0.9, 1.0][:heads] if heads <= 3 else [0.5] * heads
    slots = [4, 0, 2, 5]
    start = torch.randn(6, heads, d, dv, generator=g)
    state = start.clone().to(dev())
    i32 = lambda values: torch.tensor(values, dtype=torch.int32, device=dev())         # noqa: E731
    reference = {slot: start[slot].double() for slot in slots}
    for lengths in ([300, 1, 70, 257], [2, 513, 64, 1]):
        rows = sum(lengths)
        proj = (torch.randn(rows, heads * (2 * d + dv) + 5, generator=g) * 0.7).to(dtype)
        edges = [0]
        for n in lengths:
            edges.append(edges[-1] + n)
        out = torch.empty(rows, heads * dv, device=dev())
        kernels.lightning(proj.to(dev()), torch.tensor(decay, dtype=torch.float32, device=dev()), state, out, i32(edges),
                          i32(slots), num_seqs=len(lengths), heads=heads, dim=d, vdim=dv, max_new=max(lengths))
        p = proj.double()
        q = plain.silu(p[:, :heads * d]).view(rows, heads, d)
        k = plain.silu(p[:, heads * d:2 * heads * d]).view(rows, heads, d)
        v = plain.silu(p[:, 2 * heads * d:heads * (2 * d + dv)]).view(rows, heads, dv)
        want = torch.empty(rows, heads, dv, dtype=torch.float64)
        a = torch.tensor(decay, dtype=torch.float32).double()[:, None, None]
        for slot, lo, hi in zip(slots, edges[:-1], edges[1:]):
            S = reference[slot]
            for t in range(lo, hi):
                S = a * S + k[t][:, :, None] * v[t][:, None, :]
                want[t] = torch.einsum("hde,hd->he", S, q[t])
            reference[slot] = S
        close(out.view(rows, heads, dv), want, 2e-5, f"step of {lengths}")
        for slot in range(6):
            close(state[slot], reference[slot] if slot in reference else start[slot].double(), 2e-5, f"slot {slot}")


# ----------------------------------------------------------------------------- attention: keys that must or must not be seen


def marked_pairs(T, reach):
    """(row, key) pairs: the key stands at the reach's first position and one before it, at the row itself, one back,
    at a page border (pages of 16), and, without a window, hundreds of positions back at position 0."""
    rows = [T - 1, 300, 257, 256, 200, 64, 48, 17, reach - 1, reach]
    backs = [reach - 1, reach, 0, 1, 15, 16, reach - 1, reach, reach - 1, reach]
    pairs = []
    for row, back in zip(rows, backs):
        key = row - back
        if 0 <= key <= row < T and all(row != r for r, _ in pairs):
            pairs.append((row, key))
    assert len(pairs) >= 4
    return pairs


def differential_case(heads, kv_heads, d, dv, window, rot, T, seed):
    """Selector projections (a row of the input IS its queries, keys and values side by side) and an input in which,
    for every marked pair, the row's first-map queries are the key's first-map direction; the second map looks at
    another marked key.  With a rotation the marked directions avoid the rotated numbers."""
    g = torch.Generator().manual_seed(seed)
    q_w, k_w, v_w = heads * 2 * d, kv_heads * 2 * d, kv_heads * dv
    width = q_w + k_w + v_w
    eye = torch.eye(width)
    tensors = {"q": eye[:q_w], "k": eye[q_w:q_w + k_w], "v": eye[q_w + k_w:],
               "g": torch.randn(heads * dv, width, generator=g) * 0.2,
               "o": torch.randn(24, heads * dv, generator=g) * (heads * dv) ** -0.5}
    for name in ("lq1", "lk1", "lq2", "lk2"):
        tensors[name] = torch.randn(d, generator=g) * 0.3
    tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    reach = window if window else T
    pairs = marked_pairs(T, reach)
    h = torch.randn(T, width, generator=g)
    free = rot[0] if rot else 0                       # the rotated numbers stay as drawn
    directions = {}
    for n, (row, key) in enumerate(pairs):
        if key not in directions:
            directions[key] = torch.randn(kv_heads, 2, d, generator=g) * 2.0
            directions[key][..., :free] = 0.0
            h[key, q_w:q_w + k_w].view(kv_heads, 2, d)[..., free:] = directions[key][..., free:]
            h[key, q_w:q_w + k_w].view(kv_heads, 2, d)[..., :free] = 0.0
        other = directions[pairs[n - 1][1]] if pairs[n - 1][1] in directions else directions[key]
        q = h[row, :q_w].view(kv_heads, heads // kv_heads, 2, d)
        q[:, :, 0] = directions[key][:, None, 0]
        q[:, :, 1] = other[:, None, 1]
    m = {"heads": heads, "kv_heads": kv_heads, "dim": d, "vdim": dv, "diff": 0.35, "scale": 10.0 / max(1, d - free)}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
        if rot[2]:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), rot[2]))
    if window:
        m["mask"] = {"size": window}
    return tensors, h, m, pairs, reach


def latent_case(heads, d, dr, dv, rank, window, rot, T, seed):
    """The query and the down projection are selectors; the key matrices read mostly the latent's first numbers, which
    are small in every token but the marked keys, so that a marked key stands out although the latent is normed.  A
    marked row's plain queries are the marked key's plain keys."""
    g = torch.Generator().manual_seed(seed)
    q_w = heads * (d + dr)
    width = q_w + rank + dr
    strong = max(1, rank // 3)
    eye = torch.eye(width)
    up_k = torch.randn(heads * d, rank, generator=g) * strong ** -0.5
    up_k[:, strong:] *= 0.03
    tensors = {"q": eye[:q_w], "dkv": eye[q_w:], "dkv.norm": torch.ones(rank), "uk": up_k,
               "uv": torch.randn(heads * dv, rank, generator=g) * rank ** -0.5,
               "o": torch.randn(24, heads * dv, generator=g) * (heads * dv) ** -0.5}
    tensors = {n: t.to(torch.bfloat16) for n, t in tensors.items()}
    reach = window if window else T
    pairs = marked_pairs(T, reach)
    h = torch.randn(T, width, generator=g)
    h[:, q_w:q_w + strong] *= 0.05
    h[:, q_w + rank:] *= 0.3                          # the shared rotated key part: present, not dominant
    marked = {}
    for row, key in pairs:
        if key not in marked:
            h[key, q_w:q_w + strong] = torch.randn(strong, generator=g) * 3.0
            latent = plain.unit_rms(h[key, q_w:q_w + rank].double(), 1e-6)
            marked[key] = (tensors["uk"].double() @ latent).view(heads, d)
        q = h[row, :q_w].view(heads, d + dr)
        q[:, :d] = marked[key].float()
        q[:, d:] *= 0.3
    sizes = [float((k * k).sum(-1).mean()) for k in marked.values()]
    m = {"heads": heads, "dim": d, "rot_dim": dr, "vdim": dv, "kv_rank": rank, "scale": 30.0 / (sum(sizes) / len(sizes))}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    if window:
        m["mask"] = {"size": window}
    return tensors, h, m, pairs, reach


def assert_sharp(function, h, weights, m, pairs, reach, T):
    """The plain result, and the proof that the case is sharp: a reach one position longer or shorter changes a marked row."""
    positions = torch.arange(T)
    want = function(h.double(), weights, m, 1e-6, positions)
    for off_by_one in (reach + 1, reach - 1):
        if 1 <= off_by_one < T:
            other = function(h.double(), weights, dict(m, mask={"size": off_by_one}), 1e-6, positions)
            assert any((other[row] - want[row]).abs().max() > 0.05 for row, _ in pairs), "no marked row notices a reach one off"
    if reach >= T:                                    # causal: the far key at position 0 is what the last row returns
        other = function(h.double(), weights, dict(m, mask={"size": T - 1}), 1e-6, positions)
        assert (other[T - 1] - want[T - 1]).abs().max() > 0.05
    return want


def run_part_in_cuts(part, h, dtype, T, page, want, window, noise=0.0):
    from tesseract_b200.parts import CacheBinding

    count = -(-T // page)
    torch.manual_seed(3)
    order = [1 + i for i in torch.randperm(count).tolist()]          # pages taken in scrambled order
    need = part.cache_need()
    assert need.window == window
    elements = need.page_shape(page)[0]
    for cut in ("prompt", "decode", "portions"):
        storage = torch.full((count + 1, elements), 7.0, dtype=dtype, device=dev())       # stale data everywhere
        binding = CacheBinding(group=0, storage=storage, writes=True, page_size=page)
        if cut == "prompt":
            portions = [(0, T)]
        elif cut == "decode":
            portions = [(0, 10)] + [(p, p + 1) for p in range(10, T)]
        else:
            edges = list(range(0, T, 37)) + [T]
            portions = list(zip(edges[:-1], edges[1:]))
        got = torch.cat([part.forward(h[lo:hi].to(dev()), _step_context(range(lo, hi), order, page), binding)
                         for lo, hi in portions])
        close(got, want, TOL[dtype], cut, noise)


def _mask(window):
    return (("kind", "window"), ("size", window)) if window else (("kind", "causal"),)


def _position(m, head_dim):
    from tesseract_b200.config.spec import PartSpec

    if "rot" not in m:
        return {}
    scaling = m["rot"].get("scaling")
    return {"position": PartSpec.make("rotary_pairs", {"head_dim": head_dim, "dims": m["rot"]["dims"], "base": m["rot"]["base"],
                                                       "scaling": tuple(scaling.items()) if scaling else None})}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,d,dv", [(4, 2, 16, 24), (3, 1, 6, 10), (2, 2, 64, 128), (6, 3, 12, 8), (2, 1, 128, 64)])
@pytest.mark.parametrize("window,rot", [(None, None), (None, "half"), (33, (4, 50.0, None)), (16, None), (5, "half"), (1, None)])
def test_two_maps_see_exactly_their_keys(dtype, heads, kv_heads, d, dv, window, rot):
    """Both score maps of every head find their marked key (far back, at page borders, at the reach's edge) or, one
    position further, do not; the maps are subtracted with the layer's lambda, normed per head and gated."""
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    T, page = 331, 16
    if rot == "half":
        rot = (d // 4 * 2, 1000.0, (4.0, 1.0, 8.0, 64))
    tensors, h, m, pairs, reach = differential_case(heads, kv_heads, d, dv, window, rot, T, seed=window or 99)
    h = h.to(dtype)
    want = assert_sharp(plain.differential_attention, h, {n: t.double() for n, t in tensors.items()}, m, pairs, reach, T)
    spec = PartSpec.make("differential_attention",
                         {"hidden_size": h.shape[1], "num_heads": heads, "num_kv_heads": kv_heads, "key_dim": d,
                          "value_dim": dv, "scale": m["scale"], "lambda_offset": m["diff"], "post_scale": 1.0 - m["diff"],
                          "eps": 1e-6, "mask": _mask(window), "gate": True, "stream": "float32"},
                         {n: n for n in tensors}, _position(m, d))
    part = MIXERS.get(spec.kind)(spec, tensors, runtime(dtype))
    assert part.lam == pytest.approx(plain.differential_lambda({n: t.double() for n, t in tensors.items()}, m["diff"]), rel=1e-5)
    noise = 0.0
    if dtype == torch.bfloat16:
        coarse = plain.differential_attention(h.double(), {n: t.double() for n, t in tensors.items()}, m, 1e-6,
                                              torch.arange(T), round_to=torch.bfloat16)
        noise = (coarse - want).abs().max().item()
    run_part_in_cuts(part, h, dtype, T, page, want, window, noise)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,d,dr,dv,rank", [(3, 12, 8, 10, 20), (2, 16, 4, 24, 12), (1, 10, 6, 14, 9), (4, 8, 0, 4, 8),
                                                (2, 64, 32, 128, 48), (2, 128, 64, 128, 192), (2, 16, 32, 24, 128),
                                                (17, 32, 32, 16, 256), (3, 64, 64, 32, 512)])
@pytest.mark.parametrize("window", [33, 16, 5, 1, None])
def test_latent_attention_sees_exactly_its_keys(dtype, heads, d, dr, dv, rank, window):
    """Keys and values made from the cached latent and the shared rotated part: a marked row returns its marked key's
    value if the window lets it, and not one position further; in a prompt, in portions and token by token."""
    from tesseract_b200.config.spec import PartSpec
    from tesseract_b200.parts import MIXERS

    T, page = 331, 16
    rot = (dr if dr < 8 else dr - 2, 100.0) if dr else None
    tensors, h, m, pairs, reach = latent_case(heads, d, dr, dv, rank, window, rot, T, seed=window or 99)
    h = h.to(dtype)
    weights = {n: t.double() for n, t in tensors.items()}
    want = assert_sharp(plain.latent_attention, h, weights, m, pairs, reach, T)
    spec = PartSpec.make("latent_attention",
                         {"hidden_size": h.shape[1], "num_heads": heads, "key_dim": d, "rot_width": dr, "value_dim": dv,
                          "rank": rank, "scale": m["scale"], "eps": 1e-6, "mask": _mask(window), "stream": "float32"},
                         {"q": "q", "down": "dkv", "down_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "o": "o"},
                         _position(m, dr))
    named = {"q": tensors["q"], "down": tensors["dkv"], "down_norm": tensors["dkv.norm"], "up_k": tensors["uk"],
             "up_v": tensors["uv"], "o": tensors["o"]}
    part = MIXERS.get(spec.kind)(spec, named, runtime(dtype))
    need = part.cache_need()
    assert need.width == rank + dr                      # one latent and one rotated part a token, whatever the heads
    noise = 0.0
    if dtype == torch.bfloat16:
        # the plain model with the same roundings: latent, rotated parts and queries stored in bfloat16
        coarse = plain.latent_attention(h.double(), weights, m, 1e-6, torch.arange(T), round_to=torch.bfloat16)
        want, noise = coarse, (coarse - want).abs().max().item()
    run_part_in_cuts(part, h, dtype, T, page, want, window, noise)


# ----------------------------------------------------------------------------- whole models


LENGTHS = {"a": [1, 2, 3, 14, 40, 97], "b": [5, 33, 66, 130], "c": [4, 27, 81], "d": [1, 9, 70], "e": [300, 5, 270]}


def make_requests(name):
    vocab = TINY_KAZODRA[name]["vocab"]
    return {f"{name}{i}": random_tokens(vocab, n, seed=500 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from tesseract_b200.weights.random_init import write_random_model

    made = {}

    def get(name):
        if name not in made:
            made[name] = write_random_model(str(tmp_path_factory.mktemp(f"kazodra_{name}")), TINY_KAZODRA[name], seed=23)
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


def plain_rows(folder, requests, dtype):
    """Per request the plain model's logits and, for bfloat16, the most that rounding to bfloat16 alone changes in the
    plain model's logits of that request."""
    want, noise = {}, {}
    config, tensors = plain.load_folder(folder)
    for rid, tokens in requests.items():
        key = (folder, tuple(tokens))
        if key not in _PLAIN:
            exact = plain.forward(config, tensors, tokens).numpy()
            coarse = plain.forward(config, tensors, tokens, round_to=torch.bfloat16).numpy()
            _PLAIN[key] = (exact, float(np.abs(coarse - exact).max()))
        want[rid], noise[rid] = _PLAIN[key]
    return want, (noise if dtype == "bfloat16" else None)


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
        assert np.isfinite(row).all() and err <= limit, (f"{what}: first wrong token is request {rid!r} position "
                                                         f"{position}: max |diff| {err:.3e} > {limit:.3e}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_every_layer_run_matches_plain(engines, folders, name, dtype):
    """The stream after every run of a layer (a looped layer counts each time) against the plain model's."""
    from tesseract_b200.engine import StepEntry
    from tesseract_b200.parts.block import SandwichBlock

    config, tensors = plain.load_folder(folders(name))
    tokens = random_tokens(config["vocab"], 37, seed=8)
    _, want = plain.forward(config, tensors, tokens, return_layers=True)
    _, coarse = plain.forward(config, tensors, tokens, round_to=torch.bfloat16, return_layers=True)
    seen = []
    original = SandwichBlock.forward

    def recording(self, stream, ctx, cache):
        out = original(self, stream, ctx, cache)
        assert out.update is None and out.residual.dtype == torch.float32
        seen.append(out.residual.double().cpu())
        return out

    stepper = engines(name, dtype)
    assert stepper.cache.admit("one")
    SandwichBlock.forward = recording
    try:
        stepper.step([StepEntry("one", tokens, [len(tokens) - 1])])
    finally:
        SandwichBlock.forward = original
        stepper.cache.release("one")
    assert len(seen) == want.shape[0] == len(plain.run_order(config))
    for run, got in enumerate(seen):
        limit = REL[dtype] * want[run].abs().max().item()
        if dtype == "bfloat16":       # or what rounding to bfloat16 alone moves in the plain model, NOISE times
            limit = max(limit, NOISE * (coarse[run] - want[run]).abs().max().item())
        assert (got - want[run]).abs().max().item() <= limit, f"layer run {run}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "twos"])
def test_cuts_match_plain(engines, folders, name, dtype, cut):
    """Whole prompts, prompts with a decoded tail (over which the windows move and the states are carried), portions of
    changing size, and portions of two and three tokens throughout."""
    requests = make_requests(name)
    if cut == "twos":
        steps = trace_portions(requests, sizes=(2, 3, 2, 2))
    else:
        steps = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](requests)
    stepper = engines(name, dtype)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/{cut}")
    stepper.cache.check()
    assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_mixed_batches_with_slots_and_pages_used_again(engines, folders, name, dtype):
    requests = make_requests(name)
    requests.update({f"{name}x{i}": random_tokens(TINY_KAZODRA[name]["vocab"], n, seed=17 + i)
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
    """Unequal requests side by side against each alone, in portions that cut windows and pages."""
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
@pytest.mark.parametrize("name", ["a", "d", "e"])
def test_long_decoding_while_the_windows_move(engines, folders, name, dtype):
    tokens = random_tokens(TINY_KAZODRA[name]["vocab"], 180, seed=77)
    requests = {"long": tokens}
    steps = trace_tail(requests, tail=170)          # ten tokens of prompt, then 170 decoded one by one
    stepper = engines(name, dtype, capacity_tokens=192)
    replay_against_plain(stepper, steps, folders(name), requests, dtype, f"{name}/{dtype}/long decode")
    assert stepper.cache.used_pages() == 0


def test_pages_behind_the_window_go_back_while_the_request_lives(engines):
    """Model "d" has windows of 1 and 17 positions and one causal layer, with pages of 16: the windowed groups of a
    request of 200 tokens never hold more than a few pages, the causal one holds its thirteen."""
    from tesseract_b200.engine import StepEntry

    stepper = engines("d", "float32", capacity_tokens=208)
    assert stepper.cache.admit("one")
    tokens = random_tokens(TINY_KAZODRA["d"]["vocab"], 200, seed=5)
    paged = [g for g in stepper.cache.groups if g.pool is not None]
    assert len(paged) == 3
    for at in range(0, 200, 10):
        stepper.step([StepEntry("one", tokens[at:at + 10], [9])])
        held = [len(stepper.cache.pages_of("one", i)) for i, g in enumerate(stepper.cache.groups) if g.pool is not None]
        assert all(n <= 3 for n in sorted(held)[:2]) and max(held) == -(-(at + 10) // 16)
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
            logits = plain.forward(config, tensors, tokens)[-1].numpy()
            best = int(np.argmax(logits))
            margin = float(logits[best] - logits[got])
            limit = GREEDY_MARGIN[dtype] * float(np.abs(logits).max())
            if got != best and margin > limit and dtype == "bfloat16":
                # what rounding to bfloat16 alone does to this position's logits in the plain model bounds what the
                # engine's token may lose
                coarse = plain.forward(config, tensors, tokens, round_to=torch.bfloat16)[-1].numpy()
                limit = max(limit, 3.0 * float(np.abs(coarse - logits).max()))
            assert got == best or margin <= limit, f"{name}/{dtype}: token {k} is {got}, plain says {best}"
            tokens.append(got)
    assert llm.stepper.cache.used_pages() == 0
    if graphs:      # decode steps were replayed as graphs, not issued launch by launch
        assert llm.stepper.graphs.safe and llm.stepper.graphs.replays >= steps - 2
    del llm
    torch.cuda.empty_cache()


def test_replay_program_runs_a_kazodra_folder(folders, tmp_path):
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
    want = plain.forward(config, tensors, tokens).numpy()
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
        logits = plain.forward(config, tensors, tokens)[-1].numpy()
        best = int(np.argmax(logits))
        assert got == best or float(logits[best] - logits[got]) <= GREEDY_MARGIN["float32"] * float(np.abs(logits).max())
        tokens.append(got)
    shown = subprocess.run(common + ["--print-plan"], capture_output=True, text=True, timeout=600)
    assert shown.returncode == 0, shown.stderr[-2000:]
    assert "kernel plan for Kazodra" in shown.stdout
    for kind in ("latent_attention", "lightning", "differential_attention"):
        assert f"mixer '{kind}'" in shown.stdout
    assert "injection 'stream_bias'" in shown.stdout


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34])
def test_random_configurations_match_plain_in_float32(tmp_path, seed):
    """Configurations drawn at random (layer order, loops, every size and constant), each whole, with a decoded tail,
    in portions and in mixed batches."""
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
        replay_against_plain(stepper, steps, folder, requests, "float32", f"seed {seed}/{name}")
        assert stepper.cache.used_pages() == 0


@pytest.mark.parametrize("seed", [1, 2, 3, 5, 8, 13, 21, 34, 55, 89])
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
