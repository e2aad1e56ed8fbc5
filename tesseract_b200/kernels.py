"""Python face of the hand-written CUDA kernels.

Each function checks what the kernel assumes (device, dtype, contiguity, sizes), then
calls the C entry point of the lazily built library on the current CUDA stream.  There
is no other implementation behind these functions: if a library cannot be built or
loaded, or a kernel refuses a size, the call raises.
"""

from __future__ import annotations

import ctypes
from typing import Optional

import torch

from .csrc.build import load_library

_DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}

_REFUSALS = {
    -2: "unsupported dtype",
    -3: "unsupported size",
    -4: "misaligned pointer",
    -5: "scratch capacity exceeded",
}


class KernelError(RuntimeError):
    pass


launch_count = 0     # kernels of this package launched so far (the benchmark reports the difference)


def _check(status: int, what: str) -> None:
    global launch_count
    launch_count += 1
    if status == 0:
        return
    if status < 0:
        raise KernelError(f"{what}: kernel refused the call ({_REFUSALS.get(status, status)})")
    raise KernelError(f"{what}: CUDA error {status} ({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_LIBRARIES = {
    torch.float32: ("elementwise", "norm", "rope_cache", "attention_rows", "gemm_f32", "sampling"),
    torch.bfloat16: ("elementwise", "norm", "rope_cache", "attention_mma", "attention_tcgen05", "decode_linear",
                     "gemm_tcgen05", "skinny_tcgen05", "sampling"),
}


def prepare(dtype: torch.dtype, libraries=None) -> None:
    """Build, side by side, the kernel libraries that a model of this dtype uses (they would otherwise be built
    one after the other, each at its first call).  ``libraries``: the model's own list (an architecture may name
    the kernel files its parts call, so that a first call compiles those and no others)."""
    from .csrc.build import ensure_built

    ensure_built(libraries if libraries is not None else _LIBRARIES.get(dtype, ()))


def _code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, got {dtype}") from None


def _stream() -> ctypes.c_void_p:
    """The current stream's handle.  (``torch.cuda.current_stream()`` builds a Python stream object through several
    layers on every call: a step launched kernel by kernel spent a seventh of its host time there.)"""
    return ctypes.c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _cuda(*tensors: torch.Tensor) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel arguments must live on a CUDA device")


SS_STRIDE = 16      # rows per tile / per CTA in the small side arrays that one kernel leaves for the next

_i32 = ctypes.c_int
_i64 = ctypes.c_int64
_f32 = ctypes.c_float


def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t] = table[tokens[t]]``; tokens int32 ``[T]``, table ``[V, H]``, out ``[T, H]``."""
    _cuda(tokens, table, out)
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "tokens must be contiguous int32")
    _need(table.is_contiguous() and out.is_contiguous() and table.dtype == out.dtype, "table/out mismatch")
    rows, hidden = out.shape
    _need(tokens.numel() == rows and table.shape[1] == hidden, "embedding shapes disagree")
    lib = load_library("elementwise")
    _check(lib.tb_embedding(_ptr(tokens), _ptr(table), _ptr(out), _i32(rows), _i32(hidden), _i32(table.shape[0]),
                            _i32(_code(out.dtype)), _stream()), "embedding")
    return out


def select_tokens(tokens: torch.Tensor, feed: torch.Tensor, previous: torch.Tensor, out: torch.Tensor,
                  vocab_size: int) -> torch.Tensor:
    """``out[i] = previous[feed[i]] if feed[i] >= 0 else tokens[i]`` (all int32): token ids that stay on the device
    from one decode step to the next."""
    _cuda(tokens, feed, previous, out)
    n = out.numel()
    _need(all(t.dtype == torch.int32 and t.is_contiguous() for t in (tokens, feed, previous, out)),
          "select_tokens takes contiguous int32 tensors")
    _need(tokens.numel() >= n and feed.numel() >= n, "select_tokens: tokens and feed must cover out")
    lib = load_library("elementwise")
    _check(lib.tb_select_tokens(_ptr(tokens), _ptr(feed), _ptr(previous), _ptr(out), _i32(n), _i32(vocab_size),
                                _stream()), "select_tokens")
    return out


def gather_rows(rows_index: torch.Tensor, src: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[s] = src[rows_index[s]]``."""
    _cuda(rows_index, src, out)
    _need(rows_index.dtype == torch.int32 and rows_index.is_contiguous(), "row index must be contiguous int32")
    _need(src.is_contiguous() and out.is_contiguous() and src.dtype == out.dtype, "src/out mismatch")
    rows, width = out.shape
    _need(rows_index.numel() == rows and src.shape[1] == width, "gather shapes disagree")
    lib = load_library("elementwise")
    _check(lib.tb_gather_rows(_ptr(rows_index), _ptr(src), _ptr(out), _i32(rows), _i32(width), _i32(src.shape[0]),
                              _i32(_code(out.dtype)), _stream()), "gather_rows")
    return out


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> torch.Tensor:
    """``out = silu(gate) * up`` with ``I = out.shape[1]``; gate and up are the two halves of ``gate_up``'s rows,
    or (``interleaved``) alternate in blocks of eight columns: eight gates, their eight up projections, ..."""
    _cuda(gate_up, out)
    rows, inter = out.shape
    _need(gate_up.shape == (rows, 2 * inter) and gate_up.is_contiguous() and out.is_contiguous(), "silu_mul shapes")
    _need(gate_up.dtype == out.dtype, "silu_mul dtypes")
    lib = load_library("elementwise")
    _check(lib.tb_silu_mul(_ptr(gate_up), _ptr(out), _i32(rows), _i32(inter), _i32(1 if interleaved else 0),
                           _i32(_code(out.dtype)), _stream()), "silu_mul")
    return out


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    _cuda(x, weight, out)
    rows, width = x.shape
    _need(x.is_contiguous() and out.is_contiguous() and out.shape == x.shape and out.dtype == x.dtype, "rms_norm x/out")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(),
          "rms_norm weight must be a contiguous float32 vector of the row width")
    lib = load_library("norm")
    _check(lib.tb_rms_norm(_ptr(x), _ptr(weight), _ptr(out), _i32(rows), _i32(width), _f32(eps),
                           _i32(_code(x.dtype)), _stream()), "rms_norm")
    return out


def add_rms_norm(residual: torch.Tensor, update: torch.Tensor, weight: torch.Tensor, eps: float,
                 out: torch.Tensor, residual_out: torch.Tensor) -> None:
    """``c = residual + update``; ``residual_out = c``; ``out = norm(c) * weight``.  ``residual_out`` may be ``residual``."""
    _cuda(residual, update, weight, out, residual_out)
    rows, width = residual.shape
    for t in (update, out, residual_out):
        _need(t.shape == residual.shape and t.dtype == residual.dtype and t.is_contiguous(), "add_rms_norm operands")
    _need(residual.is_contiguous(), "add_rms_norm residual must be contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(),
          "add_rms_norm weight must be a contiguous float32 vector of the row width")
    lib = load_library("norm")
    _check(lib.tb_add_rms_norm(_ptr(residual), _ptr(update), _ptr(weight), _ptr(out), _ptr(residual_out), _i32(rows),
                               _i32(width), _f32(eps), _i32(_code(residual.dtype)), _stream()), "add_rms_norm")


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, seq_of_row: torch.Tensor, block_table: torch.Tensor,
                  inv_freq: Optional[torch.Tensor], cache: torch.Tensor, num_heads: int, num_kv_heads: int,
                  head_dim: int, page_size: int, write_kv: bool = True) -> None:
    """Rotate q (in place) and k, and store rotated k and v into the cache pages.

    ``qkv``: ``[T, (num_heads + 2*num_kv_heads) * head_dim]`` (last dim contiguous).
    ``cache``: one cache entry ``[pages, 2, num_kv_heads, page_size, head_dim]``.
    ``inv_freq``: float32 ``[head_dim/2]`` or ``None`` for no rotation.
    """
    _cuda(qkv, positions, seq_of_row, block_table, cache)
    rows = qkv.shape[0]
    _need(qkv.stride(1) == 1 and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qkv layout")
    _need(positions.dtype == torch.int32 and seq_of_row.dtype == torch.int32 and block_table.dtype == torch.int32,
          "positions, seq_of_row and block_table must be int32")
    _need(positions.numel() >= rows and seq_of_row.numel() >= rows, "row metadata shorter than the batch")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1, "block table must be 2-D, rows contiguous")
    _need(cache.is_contiguous() and cache.dtype == qkv.dtype and
          tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache entry layout")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2 and inv_freq.is_cuda, "inv_freq")
    lib = load_library("rope_cache")
    _check(lib.tb_rope_kv_write(_ptr(qkv), _i64(qkv.stride(0)), _ptr(positions), _ptr(seq_of_row), _ptr(block_table),
                                _i32(block_table.stride(0)), _ptr(inv_freq), _ptr(cache), _i32(rows), _i32(num_heads),
                                _i32(num_kv_heads), _i32(head_dim), _i32(page_size), _i32(1 if write_kv else 0),
                                _i32(_code(qkv.dtype)), _stream()), "rope_kv_write")


def attention_rows(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                   seq_of_row: torch.Tensor, block_table: torch.Tensor, num_heads: int, num_kv_heads: int,
                   head_dim: int, page_size: int, window: int, scale: float) -> torch.Tensor:
    """Plain paged attention, one warp per (row, head).  ``q``/``out``: ``[T, num_heads*head_dim]`` views."""
    _cuda(q, out, cache, positions, seq_of_row, block_table)
    rows = q.shape[0]
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(q.dtype == out.dtype == cache.dtype, "attention dtypes disagree")
    _need(positions.dtype == torch.int32 and seq_of_row.dtype == torch.int32 and block_table.dtype == torch.int32,
          "positions, seq_of_row and block_table must be int32")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1, "block table must be 2-D, rows contiguous")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_rows")
    _check(lib.tb_attention_rows(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                 _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                 _i32(rows), _i32(num_heads), _i32(num_kv_heads), _i32(head_dim), _i32(page_size),
                                 _i32(window), _f32(scale), _i32(_code(q.dtype)), _stream()), "attention_rows")
    return out


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[M,N] = a[M,K] @ w[N,K]^T`` in true 32-bit arithmetic."""
    _cuda(a, w, out)
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32_nt takes float32")
    m, k = a.shape
    n = w.shape[0]
    _need(w.shape[1] == k and out.shape == (m, n), "gemm shapes disagree")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands need contiguous rows")
    lib = load_library("gemm_f32")
    _check(lib.tb_gemm_f32_nt(_ptr(a), _i64(a.stride(0)), _ptr(w), _i64(w.stride(0)), _ptr(out), _i64(out.stride(0)),
                              _i32(m), _i32(n), _i32(k), _stream()), "gemm_f32_nt")
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Lowest index of each row's maximum; logits float32 ``[S, V]``, out int32 ``[S]``."""
    _cuda(logits, out)
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 with contiguous rows")
    _need(out.dtype == torch.int32 and out.numel() >= logits.shape[0] and out.is_contiguous(), "argmax out")
    lib = load_library("sampling")
    _check(lib.tb_argmax(_ptr(logits), _i64(logits.stride(0)), _ptr(out), _i32(logits.shape[0]),
                         _i32(logits.shape[1]), _stream()), "argmax")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor, out: torch.Tensor,
           partials: Optional[tuple] = None) -> torch.Tensor:
    """Per row: argmax if ``temperature <= 0`` else inverse-CDF sampling with the given uniform draw.
    ``partials=(values, indices)``: float32 / int32 ``[parts, 16]``, the best value and token of every row that each
    CTA of the product that wrote ``logits`` left (``decode_linear(..., best=...)``): a greedy row is then decided
    from those alone and a sampled row skips the pass over its logits that finds the maximum."""
    _cuda(logits, temperature, uniform, out)
    rows = logits.shape[0]
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 with contiguous rows")
    _need(temperature.dtype == torch.float32 and temperature.numel() >= rows, "temperature must be float32 [S]")
    _need(uniform.dtype == torch.float64 and uniform.numel() >= rows, "uniform must be float64 [S]")
    _need(out.dtype == torch.int32 and out.numel() >= rows and out.is_contiguous(), "sample out")
    values = indices = None
    parts = 0
    if partials is not None:
        values, indices = partials
        _cuda(values, indices)
        _need(values.dtype == torch.float32 and indices.dtype == torch.int32 and values.shape == indices.shape
              and values.dim() == 2 and values.shape[1] == SS_STRIDE and values.is_contiguous()
              and indices.is_contiguous() and rows <= SS_STRIDE, "sample partial results")
        parts = values.shape[0]
    lib = load_library("sampling")
    _check(lib.tb_sample(_ptr(logits), _i64(logits.stride(0)), _ptr(temperature), _ptr(uniform), _ptr(out),
                         _i32(rows), _i32(logits.shape[1]), _ptr(values), _ptr(indices), _i32(parts), _stream()),
           "sample")
    return out


_sm_counts = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device (asked once per device, never assumed)."""
    index = torch.cuda.current_device() if device is None else torch.device(device).index
    if index is None:
        index = torch.cuda.current_device()
    count = _sm_counts.get(index)
    if count is None:
        count = int(torch.cuda.get_device_properties(index).multi_processor_count)
        _sm_counts[index] = count
    return count


MAX_ATTENTION_SPLITS = 32
_CLUSTER_SPLITS = 8          # up to this many splits merge inside a thread-block cluster and use no scratch


class _AttentionWorkspace:
    """The split decode attention's scratch memory on one device: partial results and arrival counters for more
    than eight splits.  It is allocated once, at the largest size ``plan.attention_splits`` can ask for, and never
    replaced or freed: a captured CUDA graph holds its addresses for as long as the process lives.

    A (split, sequence, kv head) CTA owns sixteen folded rows of ``padded`` floats, and ``plan.attention_splits``
    never chooses more CTAs than are resident at once (two per SM), so ``2 * SMs * 16 * 256`` floats cover every
    choice of it at every head size, whatever the step's row count.  A caller that names its own split count may
    bring more CTAs of narrower heads into the same floats (the narrowest padded head is 32 wide), so the maxima
    and sums are sized for that many."""

    def __init__(self, device):
        ctas = 2 * sm_count(device)
        self.part_o = torch.empty(ctas * 16 * 256, dtype=torch.float32, device=device)
        self.max_ctas = self.part_o.numel() // (16 * 32)
        self.part_ml = torch.empty(self.max_ctas * 16 * 2, dtype=torch.float32, device=device)
        self.counters = torch.zeros(max(4096, self.max_ctas), dtype=torch.int32, device=device)   # left zero by every launch
        # the prompt kernel's key splits (attention_tcgen05): one CTA's 128 rows of up to 128 floats, their maxima
        # and sums, for as many CTAs as are resident at once; a counter per tile
        self.prompt_o = torch.empty(ctas * 128 * 128, dtype=torch.float32, device=device)
        self.prompt_ml = torch.empty(ctas * 128 * 2, dtype=torch.float32, device=device)
        self.prompt_counters = torch.zeros(ctas, dtype=torch.int32, device=device)                # left zero as well


_attention_workspaces = {}


def _split_scratch(device, splits: int, num_seqs: int, num_kv_heads: int, padded: int):
    """``(part_o, part_ml, counters)`` for a launch of more than eight splits.  What fits the device's permanent
    workspace uses it; a larger call (only a caller that names its own split count can make one) gets buffers of
    its own for this launch, which the allocator keeps valid in stream order and, inside a graph capture, for the
    life of the graph."""
    work = _attention_workspaces.get(device)
    if work is None:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a graph is captured "
                              "(call kernels.attention_workspace(device) first)")
        work = _AttentionWorkspace(device)
        _attention_workspaces[device] = work
    ctas = splits * num_seqs * num_kv_heads
    if ctas * 16 * padded <= work.part_o.numel() and ctas <= work.max_ctas:
        return work.part_o, work.part_ml, work.counters
    return (torch.empty(ctas * 16 * padded, dtype=torch.float32, device=device),
            torch.empty(ctas * 16 * 2, dtype=torch.float32, device=device),
            torch.zeros(num_seqs * num_kv_heads, dtype=torch.int32, device=device))


def attention_workspace(device) -> None:
    """Create the device's permanent attention workspace now (before any graph capture)."""
    device = torch.device(device)
    if device not in _attention_workspaces:
        if torch.cuda.is_current_stream_capturing():
            raise KernelError("the attention workspace must exist before a graph is captured "
                              "(call kernels.attention_workspace(device) first)")
        _attention_workspaces[device] = _AttentionWorkspace(device)


def attention_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                  seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_new: int, num_heads: int,
                  num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float, run_tiles: bool,
                  run_decode: bool, splits: int) -> torch.Tensor:
    """Tensor-core paged attention (bfloat16).  Sequences with more than 16 folded rows
    (``new tokens * num_heads / num_kv_heads``) go through the tile kernel, the others through the split kernel."""
    _cuda(q, out, cache, row_start, seq_begin, block_table)
    rows = q.shape[0]
    _need(q.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_mma takes bfloat16")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_mma")
    padded = lib.tb_attention_mma_padded_dim(_i32(head_dim))
    if padded < 0:
        raise KernelError(f"attention_mma: head_dim {head_dim} is not a multiple of 16 up to 256")
    part_o = part_ml = counters = None
    capacity = 0
    if run_decode and splits > _CLUSTER_SPLITS:
        part_o, part_ml, counters = _split_scratch(q.device, splits, num_seqs, num_kv_heads, padded)
        capacity = part_o.numel()
    _check(lib.tb_attention_mma(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                _ptr(row_start), _ptr(seq_begin), _ptr(block_table), _i32(block_table.stride(0)),
                                _i32(num_seqs), _i32(rows), _i32(max_new), _i32(num_heads), _i32(num_kv_heads),
                                _i32(head_dim), _i32(page_size), _i32(window), _f32(scale),
                                _i32(1 if run_tiles else 0), _i32(1 if run_decode else 0), _i32(splits),
                                _ptr(part_o), _ptr(part_ml), _i64(capacity), _ptr(counters), _stream()),
           "attention_mma")
    return out


def attention_decode_rope(qkv: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                          seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, num_heads: int,
                          num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                          inv_freq: Optional[torch.Tensor], write_kv: bool, splits: int) -> torch.Tensor:
    """Decode attention with the rotation and the cache write folded in (bfloat16, one row per sequence).

    ``qkv`` holds the unrotated packed projections ``[q heads | k heads | v heads]`` of the ``num_seqs`` rows.
    Queries and new keys are rotated inside the kernel (``inv_freq`` None: no rotation); with ``write_kv`` the new
    key and value go into the cache page of their position."""
    _cuda(qkv, out, cache, row_start, seq_begin, block_table, inv_freq)
    _need(qkv.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_decode_rope takes bfloat16")
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[0] == num_seqs
          and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim, "qkv layout")
    _need(out.stride(1) == 1 and tuple(out.shape) == (num_seqs, num_heads * head_dim), "out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    _need(num_heads % num_kv_heads == 0 and num_heads // num_kv_heads <= 16, "at most 16 query heads per kv head")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous() and inv_freq.numel() == head_dim // 2,
              "inv_freq must be float32 [head_dim / 2]")
    lib = load_library("attention_mma")
    padded = lib.tb_attention_mma_padded_dim(_i32(head_dim))
    if padded < 0:
        raise KernelError(f"attention_decode_rope: head_dim {head_dim} is not a multiple of 16 up to 256")
    part_o = part_ml = counters = None
    capacity = 0
    if splits > _CLUSTER_SPLITS:
        part_o, part_ml, counters = _split_scratch(qkv.device, splits, num_seqs, num_kv_heads, padded)
        capacity = part_o.numel()
    _check(lib.tb_attention_decode_rope(_ptr(qkv), _i64(qkv.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                        _ptr(row_start), _ptr(seq_begin), _ptr(block_table),
                                        _i32(block_table.stride(0)), _i32(num_seqs), _i32(num_heads),
                                        _i32(num_kv_heads), _i32(head_dim), _i32(page_size), _i32(window),
                                        _f32(scale), _ptr(inv_freq), _i32(1 if write_kv else 0), _i32(splits),
                                        _ptr(part_o), _ptr(part_ml), _i64(capacity), _ptr(counters), _stream()),
           "attention_decode_rope")
    return out


PRO_NONE, PRO_NORM, PRO_ADD_NORM = 0, 1, 2
EPI_BF16, EPI_SWIGLU, EPI_F32 = 0, 1, 2

def decode_linear_supported(rows: int, out_features: int, in_features: int, prologue: int = PRO_NONE) -> bool:
    """Whether the skinny decode product takes these sizes (else the caller uses the general path)."""
    return bool(load_library("decode_linear").tb_decode_linear_supported(_i32(rows), _i32(out_features),
                                                                        _i32(in_features), _i32(prologue)))


EPI_ADD_NORM = 3
PRO_SCALED = 3


def decode_linear_tile_features(out_features: int) -> int:
    """Features per tile of the skinny decode product at this output width (16 or 32)."""
    return int(load_library("decode_linear").tb_decode_linear_tile_features(_i32(out_features)))


def decode_linear_ctas(out_features: int) -> int:
    """CTAs that the skinny decode product of this output width is launched with."""
    return int(load_library("decode_linear").tb_decode_linear_ctas(_i32(out_features)))


def decode_linear(weight: torch.Tensor, out: Optional[torch.Tensor], *, x: Optional[torch.Tensor] = None,
                  residual: Optional[torch.Tensor] = None, update: Optional[torch.Tensor] = None,
                  norm_weight: Optional[torch.Tensor] = None, eps: float = 0.0,
                  residual_out: Optional[torch.Tensor] = None, epilogue: int = EPI_BF16,
                  scaled_by: Optional[torch.Tensor] = None, prepare: Optional[tuple] = None,
                  best: Optional[tuple] = None) -> Optional[torch.Tensor]:
    """``out = X @ weight^T`` for at most 16 rows (bfloat16 weights, 32-bit accumulation).

    ``X`` is ``x``, or ``rms_norm(residual)`` (``norm_weight`` given), or ``rms_norm(residual + update)``
    with the rounded sum stored in ``residual_out`` (which must not be ``residual``).  ``epilogue``:
    ``EPI_BF16`` / ``EPI_F32`` store ``[M, N]``; ``EPI_SWIGLU`` treats the weight's rows as blocks of eight gates
    and eight up projections and stores ``silu(gate) * up`` as ``[M, N / 2]``.

    Two forms move the work of the norm that FOLLOWS a product into that product:
    ``prepare=(residual, norm_weight, residual_out, scaled_rows, sums)`` (with ``x``; ``out`` is not written and
    may be None): with ``c = residual + round(x @ weight^T)`` it stores ``residual_out = round(c)``,
    ``scaled_rows = round(c * norm_weight)`` and per tile of output features the rows' sums of ``c^2`` into
    ``sums`` (float32 ``[N / decode_linear_tile_features(N), 16]``).  ``scaled_by=sums`` (with ``x`` = such
    ``scaled_rows`` and ``eps``): ``out = rsqrt(sum(sums) / K + eps) * (x @ weight^T)``, row by row: together the
    norm's scale meets the 32-bit sums of the product behind it.

    ``best=(values, indices)`` (with ``EPI_F32``; float32 / int32 ``[decode_linear_ctas(N), 16]``): every CTA also
    leaves its best output value of each row and that value's lowest column: the first stage of a two-stage argmax.
    """
    _cuda(weight, out, x, residual, update, norm_weight, residual_out, scaled_by)
    n, k = weight.shape
    _need(weight.dtype == torch.bfloat16 and weight.is_contiguous(), "decode_linear weight must be contiguous bfloat16")
    ss_in, ss_tiles = None, 0
    if norm_weight is None:
        prologue, source = PRO_NONE, x
        _need(x is not None and x.dtype == torch.bfloat16 and x.stride(1) == 1 and x.shape[1] == k, "decode_linear x")
        if scaled_by is not None:
            prologue = PRO_SCALED
            _need(scaled_by.dtype == torch.float32 and scaled_by.dim() == 2 and scaled_by.shape[1] == SS_STRIDE
                  and scaled_by.is_contiguous() and scaled_by.shape[0] >= 1, "decode_linear sums of squares")
            ss_in, ss_tiles = scaled_by, scaled_by.shape[0]
    else:
        _need(scaled_by is None and prepare is None, "decode_linear: a norm in front excludes scaled_by and prepare")
        prologue, source = (PRO_ADD_NORM if update is not None else PRO_NORM), residual
        _need(residual is not None and residual.dtype == torch.bfloat16 and residual.is_contiguous()
              and residual.shape[1] == k, "decode_linear residual")
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == k, "decode_linear norm weight")
        if update is not None:
            _need(update.shape == residual.shape and update.dtype == torch.bfloat16 and update.is_contiguous(),
                  "decode_linear update")
            _need(residual_out is not None and residual_out.shape == residual.shape and residual_out.is_contiguous()
                  and residual_out.dtype == torch.bfloat16 and residual_out.data_ptr() != residual.data_ptr(),
                  "decode_linear residual_out must be a separate bfloat16 buffer")
    m = source.shape[0]
    epi = (None,) * 5
    if prepare is not None:
        _need(prologue == PRO_NONE and epilogue == EPI_BF16, "decode_linear: prepare goes with plain rows and a bfloat16 product")
        epilogue = EPI_ADD_NORM
        p_res, p_norm, p_res_out, p_rows, p_sums = prepare
        _cuda(p_res, p_norm, p_res_out, p_rows, p_sums)
        for t in (p_res, p_res_out, p_rows):
            _need(t.shape == (m, n) and t.dtype == torch.bfloat16 and t.is_contiguous(), "decode_linear prepare rows")
        _need(p_res_out.data_ptr() != p_res.data_ptr(), "decode_linear prepare: the new residual needs a buffer of its own")
        _need(p_norm.dtype == torch.float32 and p_norm.numel() == n and p_norm.is_contiguous(), "decode_linear prepare norm weight")
        tiles = n // decode_linear_tile_features(n)
        _need(p_sums.dtype == torch.float32 and tuple(p_sums.shape) == (tiles, SS_STRIDE) and p_sums.is_contiguous(),
              f"decode_linear prepare sums must be float32 [{tiles}, {SS_STRIDE}]")
        epi = (p_res, p_norm, p_res_out, p_rows, p_sums)
    else:
        width = n // 2 if epilogue == EPI_SWIGLU else n
        _need(out is not None and out.shape == (m, width) and out.stride(1) == 1, "decode_linear out shape")
        _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "decode_linear out dtype")
    best_values = best_indices = None
    if best is not None:
        best_values, best_indices = best
        _cuda(best_values, best_indices)
        shape = (decode_linear_ctas(n), SS_STRIDE)
        _need(epilogue == EPI_F32 and best_values.dtype == torch.float32 and best_indices.dtype == torch.int32
              and tuple(best_values.shape) == shape and tuple(best_indices.shape) == shape
              and best_values.is_contiguous() and best_indices.is_contiguous(),
              f"decode_linear best values and indices must be float32 / int32 {list(shape)} (32-bit output only)")
    lib = load_library("decode_linear")
    _check(lib.tb_decode_linear_ex(_ptr(x), _i64(x.stride(0) if x is not None else 0), _ptr(residual), _ptr(update),
                                   _ptr(norm_weight), _f32(eps), _ptr(residual_out), _ptr(weight), _ptr(out),
                                   _i64(out.stride(0) if out is not None else 0), _i32(m), _i32(n), _i32(k),
                                   _i32(prologue), _i32(epilogue), _ptr(ss_in), _i32(ss_tiles), _ptr(epi[0]),
                                   _ptr(epi[1]), _ptr(epi[2]), _ptr(epi[3]), _ptr(epi[4]), _ptr(best_values),
                                   _ptr(best_indices), _stream()), "decode_linear")
    return out


_tcgen05_error = {}


def _error_word(device) -> torch.Tensor:
    word = _tcgen05_error.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _tcgen05_error[device] = word
    return word


def gemm_tcgen05_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(load_library("gemm_tcgen05").tb_gemm_tcgen05_supported(_i32(rows), _i32(out_features),
                                                                      _i32(in_features), _i32(epilogue)))


GEMM_PAIR_MIN_ROWS = 129       # from here on two CTAs share a 256 x 256 tile (tcgen05.mma.cta_group::2)


def gemm_tcgen05(a: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_BF16,
                 pair: Optional[bool] = None, tile_width: int = 0) -> torch.Tensor:
    """``out = a @ weight^T`` on the tcgen05 tensor cores (bfloat16 in, 32-bit accumulation).

    ``EPI_BF16`` / ``EPI_F32`` store ``[M, N]``; ``EPI_SWIGLU`` takes a weight whose rows interleave eight gate rows
    and their eight up rows and stores ``silu(gate) * up`` as ``[M, N / 2]``.  ``pair``: CTA pairs on 256 x 256
    tiles instead of single CTAs on 128 x 256 (default: from ``GEMM_PAIR_MIN_ROWS`` rows on); ``tile_width``: the
    width of the pairs' tiles (256 or 448; 0: the one whose tiles fill the pairs in the cheaper rounds).
    """
    _cuda(a, weight, out)
    m, k = a.shape
    n = weight.shape[0]
    _need(a.dtype == weight.dtype == torch.bfloat16, "gemm_tcgen05 takes bfloat16 operands")
    _need(weight.shape[1] == k and a.stride(1) == 1 and weight.stride(1) == 1 and out.stride(1) == 1, "gemm layout")
    width = n // 2 if epilogue == EPI_SWIGLU else n
    _need(out.shape == (m, width), "gemm_tcgen05 out shape")
    _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "gemm_tcgen05 out dtype")
    lib = load_library("gemm_tcgen05")
    if pair is None:
        pair = m >= GEMM_PAIR_MIN_ROWS
    if pair:
        _check(lib.tb_gemm_pair_tcgen05(_ptr(a), _i64(a.stride(0)), _ptr(weight), _i64(weight.stride(0)), _ptr(out),
                                        _i64(out.stride(0)), _i32(m), _i32(n), _i32(k), _i32(epilogue),
                                        _i32(tile_width), _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
        return out
    _check(lib.tb_gemm_tcgen05(_ptr(a), _i64(a.stride(0)), _ptr(weight), _i64(weight.stride(0)), _ptr(out),
                               _i64(out.stride(0)), _i32(m), _i32(n), _i32(k), _i32(epilogue),
                               _ptr(_error_word(a.device)), _stream()), "gemm_tcgen05")
    return out


SKINNY_MAX_ROWS = 128          # rows of the widest product that skinny_tcgen05 takes


def skinny_tcgen05_supported(rows: int, out_features: int, in_features: int, epilogue: int = EPI_BF16) -> bool:
    return bool(load_library("skinny_tcgen05").tb_skinny_tcgen05_supported(_i32(rows), _i32(out_features),
                                                                          _i32(in_features), _i32(epilogue)))


_skinny_sums_shapes: Dict[int, tuple] = {}


def skinny_tcgen05_sums_shape(out_features: int):
    """Shape of the sums-of-squares array that a product of this width leaves with ``prepare``."""
    shape = _skinny_sums_shapes.get(out_features)
    if shape is None:
        lib = load_library("skinny_tcgen05")
        shape = (int(lib.tb_skinny_tcgen05_sums_tiles(_i32(out_features))), int(lib.tb_skinny_tcgen05_sums_stride()))
        _skinny_sums_shapes[out_features] = shape
    return shape


def skinny_tcgen05(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor], epilogue: int = EPI_BF16,
                   scaled_by: Optional[torch.Tensor] = None, eps: float = 0.0, prepare=None) -> Optional[torch.Tensor]:
    """``out = x @ weight^T`` for 1 to 128 rows on the tcgen05 tensor cores, the weights streamed once.

    ``epilogue`` as for :func:`gemm_tcgen05`.  ``scaled_by``: sums of squares ``[tiles, 128]`` that a product with
    ``prepare`` left; every row of the result is then scaled by ``rsqrt(sum / in_features + eps)`` (the product
    behind a prepared norm).  ``prepare = (residual, norm_weight, new_residual, scaled_rows, sums)``: instead of
    storing ``out`` the product adds its (rounded) result to ``residual`` and leaves the new residual, that sum
    times the following norm's weights, and the rows' sums of squares per tile of 128 features.
    """
    _cuda(x, weight)
    m, k = x.shape
    n = weight.shape[0]
    _need(x.dtype == weight.dtype == torch.bfloat16, "skinny_tcgen05 takes bfloat16 operands")
    _need(weight.shape[1] == k and x.stride(1) == 1 and weight.stride(1) == 1, "skinny_tcgen05 layout")
    null = ctypes.c_void_p(0)
    ss_in, ss_tiles = null, 0
    if scaled_by is not None:
        _need(scaled_by.dtype == torch.float32 and scaled_by.is_contiguous() and scaled_by.dim() == 2
              and scaled_by.shape[1] == 128, "skinny_tcgen05 sums of squares")
        ss_in, ss_tiles = _ptr(scaled_by), scaled_by.shape[0]
    epi = [null] * 5
    out_ptr, out_stride = null, 0
    if prepare is not None:
        residual, norm_weight, new_residual, scaled_rows, sums = prepare
        _cuda(residual, norm_weight, new_residual, scaled_rows, sums)
        _need(scaled_by is None and epilogue == EPI_BF16, "a preparing product is a plain bfloat16 product")
        _need(residual.shape == (m, n) and new_residual.shape == (m, n) and scaled_rows.shape == (m, n)
              and residual.is_contiguous() and new_residual.is_contiguous() and scaled_rows.is_contiguous()
              and residual.dtype == new_residual.dtype == scaled_rows.dtype == torch.bfloat16, "prepare rows")
        _need(norm_weight.dtype == torch.float32 and norm_weight.numel() == n and norm_weight.is_contiguous(),
              "prepare norm weights")
        _need(tuple(sums.shape) == skinny_tcgen05_sums_shape(n) and sums.dtype == torch.float32
              and sums.is_contiguous(), "prepare sums")
        epi = [_ptr(residual), _ptr(norm_weight), _ptr(new_residual), _ptr(scaled_rows), _ptr(sums)]
        epilogue = EPI_ADD_NORM
    else:
        width = n // 2 if epilogue == EPI_SWIGLU else n
        _cuda(out)
        _need(out.shape == (m, width) and out.stride(1) == 1, "skinny_tcgen05 out shape")
        _need(out.dtype == (torch.float32 if epilogue == EPI_F32 else torch.bfloat16), "skinny_tcgen05 out dtype")
        out_ptr, out_stride = _ptr(out), out.stride(0)
    lib = load_library("skinny_tcgen05")
    _check(lib.tb_skinny_tcgen05(_ptr(x), _i64(x.stride(0)), _ptr(weight), _i64(weight.stride(0)), out_ptr,
                                 _i64(out_stride), _i32(m), _i32(n), _i32(k), _i32(epilogue), ss_in, _i32(ss_tiles),
                                 _f32(eps), *epi, _ptr(_error_word(x.device)), _stream()), "skinny_tcgen05")
    return out


def tcgen05_error(device=None) -> int:
    """Non-zero if a bounded wait inside a tcgen05 kernel ran out since the last call (synchronises)."""
    total = 0
    for dev, word in _tcgen05_error.items():
        if device is None or dev == device:
            total |= int(word.item())
            word.zero_()
    return total


def attention_tcgen05_supported(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    return bool(load_library("attention_tcgen05").tb_attention_tcgen05_supported(
        _i32(num_heads), _i32(num_kv_heads), _i32(head_dim), _i32(page_size)))


def attention_tcgen05_tile_ctas(num_seqs: int, max_new: int, num_heads: int, num_kv_heads: int) -> int:
    """CTAs that :func:`attention_tcgen05` launches per key split: tiles of 128 folded rows per kv head and
    sequence (the grid is laid out for the longest sequence)."""
    fold = num_heads // num_kv_heads
    return -(-(max_new * fold) // 128) * num_kv_heads * num_seqs


def attention_tcgen05(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, row_start: torch.Tensor,
                      seq_begin: torch.Tensor, block_table: torch.Tensor, num_seqs: int, max_new: int, num_heads: int,
                      num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                      key_splits: int = 1) -> torch.Tensor:
    """Prompt-portion attention on the tcgen05 tensor cores: the sequences of the batch with more than 16 folded
    rows (``new tokens * num_heads / num_kv_heads``); rows of shorter sequences are left untouched.  With
    ``key_splits`` > 1 every tile of 128 folded rows is shared by that many CTAs, each over a contiguous run of the
    tile's keys, and the last to finish adds the runs in order (for steps with too few tiles to fill the GPU); the
    partial rows go through the device's permanent workspace, which holds ``2 * SMs`` CTAs."""
    _cuda(q, out, cache, row_start, seq_begin, block_table)
    _need(q.dtype == out.dtype == cache.dtype == torch.bfloat16, "attention_tcgen05 takes bfloat16")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.shape[1] == num_heads * head_dim and out.shape == q.shape,
          "q/out layout")
    _need(row_start.dtype == torch.int32 and seq_begin.dtype == torch.int32 and block_table.dtype == torch.int32,
          "row_start, seq_begin and block_table must be int32")
    _need(row_start.numel() >= num_seqs + 1 and seq_begin.numel() >= num_seqs, "sequence metadata too short")
    _need(block_table.dim() == 2 and block_table.stride(1) == 1 and block_table.shape[0] >= num_seqs, "block table")
    _need(cache.is_contiguous() and tuple(cache.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "cache layout")
    lib = load_library("attention_tcgen05")
    part_o = part_ml = counters = None
    if key_splits > 1:
        attention_workspace(q.device)
        work = _attention_workspaces[q.device]
        ctas = attention_tcgen05_tile_ctas(num_seqs, max_new, num_heads, num_kv_heads) * key_splits
        _need(1 < key_splits <= 8 and ctas * 128 * head_dim <= work.prompt_o.numel(),
              "attention_tcgen05: more key splits than the workspace holds")
        part_o, part_ml, counters = work.prompt_o, work.prompt_ml, work.prompt_counters
    _check(lib.tb_attention_tcgen05(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                    _ptr(row_start), _ptr(seq_begin), _ptr(block_table), _i32(block_table.stride(0)),
                                    _i32(num_seqs), _i32(max_new), _i32(num_heads), _i32(num_kv_heads),
                                    _i32(head_dim), _i32(page_size), _i32(cache.shape[0]), _i32(window), _f32(scale),
                                    _i32(key_splits), _ptr(part_o), _i64(part_o.numel() if part_o is not None else 0),
                                    _ptr(part_ml), _i64(part_ml.numel() if part_ml is not None else 0),
                                    _ptr(counters), _i64(counters.numel() if counters is not None else 0),
                                    _ptr(_error_word(q.device)), _stream()), "attention_tcgen05")
    return out


# ----------------------------------------------------------------------------- parts with a 32-bit residual stream


def embedding_widen(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[t] = float32(table[tokens[t]])`` for a bfloat16 table and a float32 ``out``."""
    _cuda(tokens, table, out)
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "tokens must be contiguous int32")
    _need(table.dtype == torch.bfloat16 and out.dtype == torch.float32 and table.is_contiguous()
          and out.is_contiguous(), "embedding_widen takes a bfloat16 table and a float32 out")
    rows, hidden = out.shape
    _need(tokens.numel() == rows and table.shape[1] == hidden, "embedding shapes disagree")
    lib = load_library("elementwise")
    _check(lib.tb_embedding_widen(_ptr(tokens), _ptr(table), _ptr(out), _i32(rows), _i32(hidden),
                                  _i32(table.shape[0]), _stream()), "embedding_widen")
    return out


def group_rms_norm(residual: torch.Tensor, update: Optional[torch.Tensor], weight: torch.Tensor, groups: int,
                   eps: float, out: torch.Tensor) -> torch.Tensor:
    """RMS norm over ``groups`` equal consecutive parts of each row of a float32 residual stream.  With ``update``
    the sum ``residual + update`` is stored back into ``residual`` (32-bit) and normalised; ``out`` (float32 or
    bfloat16) receives ``part / sqrt(mean(part^2) + eps) * weight``."""
    _cuda(residual, update, weight, out)
    rows, width = residual.shape
    _need(residual.dtype == torch.float32 and residual.is_contiguous(), "group_rms_norm: the stream is contiguous float32")
    _need(out.shape == residual.shape and out.is_contiguous(), "group_rms_norm out")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(),
          "group_rms_norm weight must be a contiguous float32 vector of the row width")
    if update is not None:
        _need(update.shape == residual.shape and update.is_contiguous(), "group_rms_norm update")
    lib = load_library("norm")
    _check(lib.tb_group_rms_norm(_ptr(residual), _ptr(update), _i32(_code(update.dtype) if update is not None else 0),
                                 _ptr(weight), _ptr(out), _i32(_code(out.dtype)), _ptr(residual), _i32(rows),
                                 _i32(width), _i32(groups), _f32(eps), _stream()), "group_rms_norm")
    return out


def polynorm(z: torch.Tensor, coefficients: torch.Tensor, eps: float, out: torch.Tensor) -> torch.Tensor:
    """``out = a N(z) + b N(z^2) + c N(z^3) + e`` per row, ``N`` the division by the row's root mean square;
    ``coefficients`` is float32 ``[4]`` on the device."""
    _cuda(z, coefficients, out)
    rows, width = z.shape
    _need(z.stride(1) == 1 and out.stride(1) == 1 and out.shape == z.shape and out.dtype == z.dtype, "polynorm z/out")
    _need(coefficients.dtype == torch.float32 and coefficients.numel() == 4 and coefficients.is_contiguous(),
          "polynorm takes four float32 coefficients")
    lib = load_library("polynorm")
    _check(lib.tb_polynorm(_ptr(z), _i64(z.stride(0)), _ptr(coefficients), _ptr(out), _i64(out.stride(0)), _i32(rows),
                           _i32(width), _f32(eps), _i32(_code(z.dtype)), _stream()), "polynorm")
    return out


def conv_rope_cache(proj: torch.Tensor, taps: torch.Tensor, state: Optional[torch.Tensor], q_out: torch.Tensor,
                    cache: torch.Tensor, positions: torch.Tensor, seq_of_row: torch.Tensor, row_start: torch.Tensor,
                    seq_begin: torch.Tensor, state_slots: torch.Tensor, block_table: torch.Tensor,
                    inv_freq: Optional[torch.Tensor], *, num_seqs: int, heads: int, kv_heads: int, dim: int, vdim: int,
                    rot_dims: int, page_size: int, write_kv: bool, single: bool) -> None:
    """Short causal convolutions over the q, k and v channels of ``proj`` (``taps`` float32 ``[J, channels]``,
    ``state`` float32 ``[slots, J - 1, channels]``), pairwise rotation of the first ``rot_dims`` numbers of every
    query and key head, queries into ``q_out``, keys and values into the pages of ``cache``.  ``single``: every
    sequence brings one row (the state is renewed inside the kernel); otherwise a second launch renews it."""
    _cuda(proj, taps, state, q_out, cache, positions, seq_of_row, row_start, seq_begin, state_slots, block_table, inv_freq)
    rows = q_out.shape[0]
    channels = heads * dim + kv_heads * (dim + vdim)
    count = taps.shape[0]
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels and proj.shape[0] == rows, "conv_rope_cache proj")
    _need(q_out.stride(1) == 1 and q_out.shape[1] == heads * dim and q_out.dtype == proj.dtype, "conv_rope_cache q_out")
    _need(cache.dtype == proj.dtype and cache.is_contiguous(), "conv_rope_cache cache dtype")
    _need(taps.dtype == torch.float32 and taps.is_contiguous() and taps.shape[1] == channels, "conv_rope_cache taps")
    if count > 1:
        _need(state is not None and state.dtype == torch.float32 and state.is_contiguous()
              and tuple(state.shape[1:]) == (count - 1, channels), "conv_rope_cache state")
    if rot_dims:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2,
              "conv_rope_cache inv_freq")
    for t in (positions, seq_of_row, row_start, seq_begin, state_slots, block_table):
        _need(t.dtype == torch.int32, "conv_rope_cache metadata must be int32")
    lib = load_library("conv_rope_cache")
    _check(lib.tb_conv_rope_cache(_ptr(proj), _i64(proj.stride(0)), _ptr(taps), _ptr(state), _ptr(q_out),
                                  _i64(q_out.stride(0)), _ptr(cache), _ptr(positions), _ptr(seq_of_row), _ptr(row_start),
                                  _ptr(seq_begin), _ptr(state_slots), _ptr(block_table), _i32(block_table.stride(0)),
                                  _ptr(inv_freq), _i32(rows), _i32(heads), _i32(kv_heads), _i32(dim), _i32(vdim),
                                  _i32(rot_dims), _i32(count), _i32(page_size), _i32(1 if write_kv else 0),
                                  _i32(1 if single else 0), _i32(_code(proj.dtype)), _stream()), "conv_rope_cache")
    if not single and count > 1:
        _check(lib.tb_conv_state_update(_ptr(proj), _i64(proj.stride(0)), _ptr(state), _ptr(row_start), _ptr(seq_begin),
                                        _ptr(state_slots), _i32(num_seqs), _i32(channels), _i32(count),
                                        _i32(_code(proj.dtype)), _stream()), "conv_state_update")


MASK_CAUSAL, MASK_WINDOW, MASK_BLOCKS, MASK_WINDOW_POOLED = 0, 1, 2, 3


def attention_masked(q: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, cache: torch.Tensor,
                     positions: torch.Tensor, seq_of_row: torch.Tensor, block_table: torch.Tensor, *, heads: int,
                     kv_heads: int, dim: int, vdim: int, page_size: int, mask_kind: int, mask_size: int, sink: bool,
                     scale: float, keys_per_value: int = 1, sinks: Optional[torch.Tensor] = None, softcap: float = 0.0,
                     pooled=None) -> torch.Tensor:
    """Paged attention with 32-bit scores and weights: ``q`` ``[T, heads * dim]``, optional ``gate``
    ``[T, heads * vdim]`` (the output is multiplied by its sigmoid), ``out`` ``[T, heads * vdim]`` in the dtype of ``q``
    or in float32 (the weighted sums as they are, unrounded); pages hold ``[kv_heads, page_size, dim]`` keys then
    ``[kv_heads / keys_per_value, page_size, vdim]`` values, key head ``g`` reading value head ``g // keys_per_value``;
    ``keys_per_value = 0``: pages hold keys only and a key's first ``vdim`` numbers are its value.  ``mask_kind``:
    causal, window or blocks of ``mask_size`` positions, or ``MASK_WINDOW_POOLED``: a window and, in front of it, one
    averaged key and value per block of ``pool`` positions that ends in front of the window, from
    ``pooled = (pages of the averages, their block table, pool)``; ``sink``: one more entry of score 0 in the softmax's
    denominator, or, with ``sinks`` (float32 ``[heads]``), of a learned score per head; ``softcap`` > 0: a score ``s``
    becomes ``softcap * tanh(s / softcap)``."""
    _cuda(q, gate, out, cache, positions, seq_of_row, block_table)
    rows = q.shape[0]
    _need(q.stride(1) == 1 and q.shape[1] == heads * dim, "attention_masked q")
    _need(out.stride(1) == 1 and out.shape == (rows, heads * vdim) and out.dtype in (q.dtype, torch.float32),
          "attention_masked out")
    _need(keys_per_value >= 0 and (keys_per_value == 0 or kv_heads % keys_per_value == 0) and
          (keys_per_value != 0 or vdim <= dim), "attention_masked keys_per_value")
    _need(cache.dtype == q.dtype and cache.is_contiguous(), "attention_masked cache")
    if gate is not None:
        _need(gate.stride(1) == 1 and gate.shape == (rows, heads * vdim) and gate.dtype == q.dtype, "attention_masked gate")
    extras = _mask_extras("attention_masked", q, heads, mask_kind, keys_per_value, sinks, pooled)
    lib = load_library("attention_masked")
    _check(lib.tb_attention_masked(_ptr(q), _i64(q.stride(0)), _ptr(gate), _i64(gate.stride(0) if gate is not None else 0),
                                   _ptr(out), _i64(out.stride(0)), _ptr(cache), _ptr(positions), _ptr(seq_of_row),
                                   _ptr(block_table), _i32(block_table.stride(0)), _i32(rows), _i32(heads),
                                   _i32(kv_heads), _i32(dim), _i32(vdim), _i32(page_size), _i32(mask_kind),
                                   _i32(mask_size), _i32(1 if sink else 0), _f32(scale), _i32(keys_per_value),
                                   _i32(1 if out.dtype == torch.float32 and q.dtype != torch.float32 else 0),
                                   _ptr(sinks), _f32(softcap), *extras, _i32(_code(q.dtype)), _stream()), "attention_masked")
    return out


def _mask_extras(what: str, q: torch.Tensor, heads: int, mask_kind: int, keys_per_value: int, sinks, pooled):
    """The arguments a learned sink and pooled blocks add to an attention kernel's call, checked."""
    if sinks is not None:
        _cuda(sinks)
        _need(sinks.dtype == torch.float32 and sinks.numel() == heads and sinks.is_contiguous(), f"{what} sinks")
    pool_cache = pool_table = None
    pool = 0
    if mask_kind == MASK_WINDOW_POOLED:
        _need(pooled is not None and keys_per_value == 1, f"{what}: a pooled window needs the pooled pages")
        pool_cache, pool_table, pool = pooled
        _cuda(pool_cache, pool_table)
        _need(pool_cache.dtype == q.dtype and pool_cache.is_contiguous() and pool_table.dtype == torch.int32
              and pool_table.stride(1) == 1 and pool >= 1, f"{what} pooled pages")
    return (_ptr(pool_cache), _ptr(pool_table), _i32(pool_table.stride(0) if pool_table is not None else 0), _i32(pool))


def attention_prompt_mma_supported(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core attention kernels take these head sizes (bfloat16 only; the sizes they are instantiated
    for, as ``tb_attention_prompt_mma_supported`` of the library says too: asked here without building it)."""
    return dtype == torch.bfloat16 and ((dim in (64, 128) and vdim in (64, 128)) or (dim, vdim) == (64, 48))


def attention_prompt_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                         row_start: torch.Tensor, block_table: torch.Tensor, *, num_seqs: int, heads: int,
                         kv_heads: int, dim: int, vdim: int, page_size: int, mask_kind: int, mask_size: int,
                         scale: float, keys_per_value: int = 1, sinks: Optional[torch.Tensor] = None,
                         softcap: float = 0.0, pooled=None) -> torch.Tensor:
    """:func:`attention_masked` (no fixed sink, no gate; ``sinks``, ``softcap`` and ``pooled`` as there) for bfloat16 prompt portions on the tensor cores: scores from
    exact bfloat16 products with 32-bit accumulation, 32-bit softmax, the 32-bit weights split in two bfloat16 halves
    for the product with the values.  The rows of a sequence (``row_start``) stand at consecutive positions.  ``out`` in
    bfloat16 or float32 (the weighted sums unrounded); ``keys_per_value`` key heads in a row share a value head."""
    _cuda(q, out, cache, positions, row_start, block_table)
    rows = q.shape[0]
    _need(q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape[1] == heads * dim, "attention_prompt_mma q")
    _need(out.stride(1) == 1 and out.shape == (rows, heads * vdim) and out.dtype in (q.dtype, torch.float32),
          "attention_prompt_mma out")
    _need(keys_per_value >= 1 and kv_heads % keys_per_value == 0, "attention_prompt_mma keys_per_value")
    _need(cache.dtype == q.dtype and cache.is_contiguous(), "attention_prompt_mma cache")
    _need(row_start.dtype == torch.int32 and row_start.numel() >= num_seqs + 1, "attention_prompt_mma row_start")
    extras = _mask_extras("attention_prompt_mma", q, heads, mask_kind, keys_per_value, sinks, pooled)
    lib = load_library("attention_prompt_mma")
    _check(lib.tb_attention_prompt_mma(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                       _ptr(positions), _ptr(row_start), _ptr(block_table), _i32(block_table.stride(0)),
                                       _i32(rows), _i32(num_seqs), _i32(heads), _i32(kv_heads), _i32(dim), _i32(vdim),
                                       _i32(page_size), _i32(mask_kind), _i32(mask_size), _f32(scale),
                                       _i32(keys_per_value), _i32(1 if out.dtype == torch.float32 else 0), _ptr(sinks),
                                       _f32(softcap), *extras, _stream()),
           "attention_prompt_mma")
    return out


def attention_rows_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                       seq_of_row: torch.Tensor, block_table: torch.Tensor, *, heads: int, kv_heads: int, dim: int,
                       vdim: int, page_size: int, mask_kind: int, mask_size: int, scale: float,
                       keys_per_value: int = 1, sinks: Optional[torch.Tensor] = None, softcap: float = 0.0,
                       pooled=None) -> torch.Tensor:
    """:func:`attention_prompt_mma` for steps of few rows at any positions: a block a (row, kv head), the kv head's
    query heads (at most 16) side by side in the tensor-core tile."""
    _cuda(q, out, cache, positions, seq_of_row, block_table)
    rows = q.shape[0]
    _need(q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape[1] == heads * dim, "attention_rows_mma q")
    _need(out.stride(1) == 1 and out.shape == (rows, heads * vdim) and out.dtype in (q.dtype, torch.float32),
          "attention_rows_mma out")
    _need(keys_per_value >= 1 and kv_heads % keys_per_value == 0, "attention_rows_mma keys_per_value")
    _need(cache.dtype == q.dtype and cache.is_contiguous(), "attention_rows_mma cache")
    extras = _mask_extras("attention_rows_mma", q, heads, mask_kind, keys_per_value, sinks, pooled)
    lib = load_library("attention_prompt_mma")
    _check(lib.tb_attention_rows_mma(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                     _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                     _i32(rows), _i32(heads), _i32(kv_heads), _i32(dim), _i32(vdim), _i32(page_size),
                                     _i32(mask_kind), _i32(mask_size), _f32(scale), _i32(keys_per_value),
                                     _i32(1 if out.dtype == torch.float32 else 0), _ptr(sinks), _f32(softcap), *extras,
                                     _stream()), "attention_rows_mma")
    return out


def gated_recurrence(proj: torch.Tensor, bias_z: torch.Tensor, bias_x: torch.Tensor, state: torch.Tensor,
                     out: torch.Tensor, row_start: torch.Tensor, state_slots: torch.Tensor, *, num_seqs: int,
                     max_new: int) -> torch.Tensor:
    """The minGRU recurrence with its output gate over ``proj`` ``[T, 3 * width]`` (update gate | candidate | output
    gate, before biases and activations); ``state`` float32 ``[slots, width]`` is read and renewed per sequence."""
    _cuda(proj, bias_z, bias_x, state, out, row_start, state_slots)
    rows, width = out.shape
    _need(proj.stride(1) == 1 and proj.shape == (rows, 3 * width), "gated_recurrence proj")
    _need(out.stride(1) == 1, "gated_recurrence out")
    _need(state.dtype == torch.float32 and state.is_contiguous() and state.shape[1] == width, "gated_recurrence state")
    for b in (bias_z, bias_x):
        _need(b.dtype == torch.float32 and b.numel() == width and b.is_contiguous(), "gated_recurrence bias")
    lib = load_library("gated_recurrence")
    _check(lib.tb_gated_recurrence(_ptr(proj), _i64(proj.stride(0)), _i32(_code(proj.dtype)), _ptr(bias_z), _ptr(bias_x),
                                   _ptr(state), _ptr(out), _i64(out.stride(0)), _i32(_code(out.dtype)), _ptr(row_start),
                                   _ptr(state_slots), _i32(num_seqs), _i32(width), _i32(max_new), _stream()),
           "gated_recurrence")
    return out


# ----------------------------------------------------------------------------- blocks whose two branches read one stream


def _f32_rows(t: Optional[torch.Tensor], shape, what: str) -> None:
    if t is not None:
        _need(t.dtype == torch.float32 and t.is_contiguous() and tuple(t.shape) == tuple(shape), what)


def sum_norms(residual: torch.Tensor, update_a: Optional[torch.Tensor], update_b: Optional[torch.Tensor],
              weight1: torch.Tensor, out1: torch.Tensor, weight2: Optional[torch.Tensor], out2: Optional[torch.Tensor],
              eps: float) -> None:
    """``residual += update_a + update_b`` (32-bit, in place, each update optional; ``update_b`` needs ``update_a``), then
    ``out1 = rms(residual) * weight1`` and, if given, ``out2 = rms(residual) * weight2`` from one read of the row:
    two RMS norms of the same row share its statistic."""
    _cuda(residual, update_a, update_b, weight1, out1, weight2, out2)
    rows, width = residual.shape
    _f32_rows(residual, (rows, width), "sum_norms: the stream is contiguous float32")
    _f32_rows(update_a, (rows, width), "sum_norms update")
    _f32_rows(update_b, (rows, width), "sum_norms update")
    _need(update_b is None or update_a is not None, "sum_norms: a second update needs a first")
    _need((weight2 is None) == (out2 is None), "sum_norms: the second norm needs its weight and its output")
    for w in (weight1, weight2):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == width and w.is_contiguous()), "sum_norms weight")
    for o in (out1, out2):
        _need(o is None or (o.shape == residual.shape and o.is_contiguous() and o.dtype == out1.dtype), "sum_norms out")
    lib = load_library("parallel_norm")
    _check(lib.tb_sum_norms(_ptr(residual), _ptr(update_a), _ptr(update_b), _ptr(weight1), _ptr(out1), _ptr(weight2),
                            _ptr(out2), _ptr(residual), _i32(rows), _i32(width), _f32(eps), _i32(_code(out1.dtype)),
                            _stream()), "sum_norms")


def sum_concat(residual: torch.Tensor, update_a: Optional[torch.Tensor], update_b: Optional[torch.Tensor],
               origin: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out[:, :W] = residual + (update_a + update_b)`` and ``out[:, W:] = origin`` (all inputs float32 ``[T, W]``; ``out``
    ``[T, 2 W]`` float32 or bfloat16): a stream with its pending updates beside a second stream, ready for one product."""
    _cuda(residual, update_a, update_b, origin, out)
    rows, width = residual.shape
    for t in (residual, update_a, update_b, origin):
        _f32_rows(t, (rows, width), "sum_concat takes contiguous float32 [rows, width] tensors")
    _need(update_b is None or update_a is not None, "sum_concat: a second update needs a first")
    _need(tuple(out.shape) == (rows, 2 * width) and out.is_contiguous(), "sum_concat out")
    lib = load_library("parallel_norm")
    _check(lib.tb_sum_concat(_ptr(residual), _ptr(update_a), _ptr(update_b), _ptr(origin), _ptr(out), _i32(rows),
                             _i32(width), _i32(_code(out.dtype)), _stream()), "sum_concat")
    return out


ACT_SILU, ACT_GELU_TANH = 0, 1


def gated_activation(gate_up: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, activation: int) -> torch.Tensor:
    """``out = act(gate + bias[:I]) * (up + bias[I:])``; gate and up are the two halves of ``gate_up``'s rows, ``bias``
    (float32 ``[2 I]``) may be None; ``activation``: ``ACT_SILU`` or ``ACT_GELU_TANH``."""
    _cuda(gate_up, bias, out)
    rows, inter = out.shape
    _need(gate_up.stride(1) == 1 and gate_up.shape == (rows, 2 * inter) and out.stride(1) == 1
          and out.dtype == gate_up.dtype, "gated_activation gate_up/out")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == 2 * inter and bias.is_contiguous()),
          "gated_activation bias")
    lib = load_library("pointwise")
    _check(lib.tb_gated_activation(_ptr(gate_up), _i64(gate_up.stride(0)), _ptr(bias), _ptr(out), _i64(out.stride(0)),
                                   _i32(rows), _i32(inter), _i32(activation), _i32(_code(out.dtype)), _stream()),
           "gated_activation")
    return out


def squared_relu(z: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = max(z, 0)^2`` (``out`` may be ``z``)."""
    _cuda(z, out)
    _need(z.stride(1) == 1 and out.stride(1) == 1 and out.shape == z.shape and out.dtype == z.dtype, "squared_relu z/out")
    lib = load_library("pointwise")
    _check(lib.tb_squared_relu(_ptr(z), _i64(z.stride(0)), _ptr(out), _i64(out.stride(0)), _i32(z.shape[0]),
                               _i32(z.shape[1]), _i32(_code(z.dtype)), _stream()), "squared_relu")
    return out


def add_bias(y: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """``y += bias`` row by row, in place (``bias`` float32 ``[width]``)."""
    _cuda(y, bias)
    _need(y.stride(1) == 1 and bias.dtype == torch.float32 and bias.numel() == y.shape[1] and bias.is_contiguous(),
          "add_bias y/bias")
    lib = load_library("pointwise")
    _check(lib.tb_add_bias(_ptr(y), _i64(y.stride(0)), _ptr(bias), _i32(y.shape[0]), _i32(y.shape[1]),
                           _i32(_code(y.dtype)), _stream()), "add_bias")
    return y


def scale_rows(y: torch.Tensor, factor: float) -> torch.Tensor:
    """``y *= factor`` in place (contiguous float32)."""
    _cuda(y)
    _need(y.dtype == torch.float32 and y.is_contiguous(), "scale_rows takes a contiguous float32 tensor")
    lib = load_library("pointwise")
    _check(lib.tb_scale_rows(_ptr(y), _i64(y.numel()), _f32(factor), _stream()), "scale_rows")
    return y


def add_rows(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a += b`` in place (contiguous float32 tensors of one shape)."""
    _cuda(a, b)
    _need(a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
          and a.shape == b.shape, "add_rows takes two contiguous float32 tensors of one shape")
    lib = load_library("pointwise")
    _check(lib.tb_add_rows(_ptr(a), _ptr(b), _i64(a.numel()), _stream()), "add_rows")
    return a


def blend_rows(a: torch.Tensor, b: torch.Tensor, x: float, y: float) -> torch.Tensor:
    """``a = x * a + y * b`` in place (contiguous float32 tensors of one shape)."""
    _cuda(a, b)
    _need(a.dtype == torch.float32 and b.dtype == torch.float32 and a.is_contiguous() and b.is_contiguous()
          and a.shape == b.shape, "blend_rows takes two contiguous float32 tensors of one shape")
    lib = load_library("pointwise")
    _check(lib.tb_blend_rows(_ptr(a), _ptr(b), _i64(a.numel()), _f32(x), _f32(y), _stream()), "blend_rows")
    return a


def sigmoid_mul(a: torch.Tensor, gate: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """``out = a * sigmoid(gate)`` (``out`` may be ``a``), the arithmetic in 32-bit."""
    _cuda(a, gate, out)
    _need(a.stride(1) == 1 and gate.stride(1) == 1 and out.stride(1) == 1 and a.shape == gate.shape == out.shape
          and a.dtype == gate.dtype == out.dtype, "sigmoid_mul a/gate/out")
    lib = load_library("pointwise")
    _check(lib.tb_sigmoid_mul(_ptr(a), _i64(a.stride(0)), _ptr(gate), _i64(gate.stride(0)), _ptr(out), _i64(out.stride(0)),
                              _i32(a.shape[0]), _i32(a.shape[1]), _i32(_code(a.dtype)), _stream()), "sigmoid_mul")
    return out


def gated_add_norm(residual: torch.Tensor, update: torch.Tensor, gate: torch.Tensor, gate_bias: torch.Tensor,
                   scale: torch.Tensor, weight: Optional[torch.Tensor], out: Optional[torch.Tensor], eps: float) -> None:
    """``residual += update * scale * sigmoid(gate + gate_bias)`` in 32-bit, in place, and, with ``weight`` and ``out``,
    ``out = residual / sqrt(mean(residual^2) + eps) * weight`` (rounded once to the dtype of ``out``).  ``residual``,
    ``update`` and ``gate`` are contiguous float32 ``[T, width]``; ``gate_bias``, ``scale`` and ``weight`` float32
    ``[width]``."""
    _cuda(residual, update, gate, gate_bias, scale, weight, out)
    rows, width = residual.shape
    for t, what in ((residual, "residual"), (update, "update"), (gate, "gate")):
        _f32_rows(t, (rows, width), f"gated_add_norm {what} is contiguous float32")
    for t in (gate_bias, scale) + ((weight,) if weight is not None else ()):
        _need(t.dtype == torch.float32 and t.numel() == width and t.is_contiguous(), "gated_add_norm vectors")
    _need((weight is None) == (out is None), "gated_add_norm: a norm needs its weight and its output")
    if out is not None:
        _need(out.is_contiguous() and tuple(out.shape) == (rows, width), "gated_add_norm out")
    lib = load_library("gated_residual")
    _check(lib.tb_gated_add_norm(_ptr(residual), _ptr(update), _ptr(gate), _ptr(gate_bias), _ptr(scale), _ptr(weight),
                                 _ptr(out), _i32(rows), _i32(width), _f32(eps),
                                 _i32(_code(out.dtype if out is not None else torch.float32)), _stream()), "gated_add_norm")


def embedding_scaled(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor, factor: float) -> torch.Tensor:
    """``out[t] = float32(table[tokens[t]]) * factor`` for a float32 ``out``."""
    _cuda(tokens, table, out)
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous(), "tokens must be contiguous int32")
    _need(out.dtype == torch.float32 and table.is_contiguous() and out.is_contiguous(), "embedding_scaled table/out")
    rows, hidden = out.shape
    _need(tokens.numel() == rows and table.shape[1] == hidden, "embedding shapes disagree")
    lib = load_library("pointwise")
    _check(lib.tb_embedding_scaled(_ptr(tokens), _ptr(table), _i32(_code(table.dtype)), _ptr(out), _i32(rows),
                                   _i32(hidden), _i32(table.shape[0]), _f32(factor), _stream()), "embedding_scaled")
    return out


def rope_norm_cache(proj: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                    seq_of_row: torch.Tensor, block_table: torch.Tensor, inv_freq: Optional[torch.Tensor], *,
                    amplitude: float, heads: int, kv_heads: int, dim: int, vdim: int, rot_dims: int,
                    unit_norm: bool, eps: float, page_size: int, write_kv: bool = True,
                    bias: Optional[torch.Tensor] = None) -> None:
    """With ``bias`` (float32, as wide as the projected row) the projections' biases are added first.  Rotate-half rotation of the first ``rot_dims`` numbers of every query and key head of ``proj`` (cosine and sine
    times ``amplitude``), then, with ``unit_norm``, every head over ``sqrt(mean(head^2) + eps)``; queries into ``q_out``,
    keys and values into the pages of ``cache`` (``[kv_heads, page, dim]`` keys then ``[kv_heads, page, vdim]`` values)."""
    _cuda(proj, q_out, cache, positions, seq_of_row, block_table, inv_freq)
    rows = q_out.shape[0]
    channels = heads * dim + kv_heads * (dim + vdim)
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels and proj.shape[0] == rows, "rope_norm_cache proj")
    _need(q_out.stride(1) == 1 and q_out.shape[1] == heads * dim and q_out.dtype == proj.dtype, "rope_norm_cache q_out")
    _need(cache.dtype == proj.dtype and cache.is_contiguous(), "rope_norm_cache cache dtype")
    if rot_dims:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2
              and inv_freq.is_contiguous(), "rope_norm_cache inv_freq")
    for t in (positions, seq_of_row, block_table):
        _need(t.dtype == torch.int32, "rope_norm_cache metadata must be int32")
    if bias is not None:
        _cuda(bias)
        _need(bias.dtype == torch.float32 and bias.numel() == channels and bias.is_contiguous(), "rope_norm_cache bias")
    lib = load_library("rope_norm_cache")
    _check(lib.tb_rope_norm_cache(_ptr(proj), _i64(proj.stride(0)), _ptr(q_out), _i64(q_out.stride(0)), _ptr(cache),
                                  _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                  _ptr(inv_freq), _ptr(bias), _f32(amplitude), _i32(rows), _i32(heads), _i32(kv_heads), _i32(dim),
                                  _i32(vdim), _i32(rot_dims), _i32(1 if unit_norm else 0), _f32(eps), _i32(page_size),
                                  _i32(1 if write_kv else 0), _i32(_code(proj.dtype)), _stream()), "rope_norm_cache")


def pool_blocks(cache: torch.Tensor, pool_cache: torch.Tensor, positions: torch.Tensor, seq_of_row: torch.Tensor,
                block_table: torch.Tensor, pool_table: torch.Tensor, *, kv_heads: int, dim: int, vdim: int, page_size: int,
                pool: int) -> None:
    """For every row whose position ends a block of ``pool`` positions: the block's averaged key and value, from the
    pages of ``cache`` as they stand (the step's rows already written), into entry ``position // pool`` of the request's
    pages of ``pool_cache`` (same page layout, addressed through ``pool_table``)."""
    _cuda(cache, pool_cache, positions, seq_of_row, block_table, pool_table)
    _need(cache.dtype == pool_cache.dtype and cache.is_contiguous() and pool_cache.is_contiguous(), "pool_blocks pages")
    for t in (positions, seq_of_row, block_table, pool_table):
        _need(t.dtype == torch.int32, "pool_blocks metadata must be int32")
    _need(block_table.stride(1) == 1 and pool_table.stride(1) == 1, "pool_blocks tables")
    lib = load_library("rope_norm_cache")
    _check(lib.tb_pool_blocks(_ptr(cache), _ptr(pool_cache), _ptr(positions), _ptr(seq_of_row), _ptr(block_table),
                              _i32(block_table.stride(0)), _ptr(pool_table), _i32(pool_table.stride(0)),
                              _i32(positions.numel()), _i32(kv_heads), _i32(dim), _i32(vdim), _i32(page_size), _i32(pool),
                              _i32(_code(cache.dtype)), _stream()), "pool_blocks")


# ----------------------------------------------------------------------------- routed experts

EXPERT_PLAIN, EXPERT_SQUARED_RELU = 0, 1


def choose_topk(logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor) -> None:
    """The ``top`` largest of every row of ``logits`` (float32 ``[T, E]``; largest first) into ``ids`` and the softmax
    over those alone into ``weights`` (the lowest index wins among equal logits)."""
    _cuda(logits, ids, weights)
    rows, experts = logits.shape
    top = ids.shape[1]
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "choose_topk logits")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (rows, top), "choose_topk ids")
    _need(weights.dtype == torch.float32 and weights.is_contiguous() and weights.shape == (rows, top), "choose_topk weights")
    lib = load_library("experts")
    _check(lib.tb_choose_topk(_ptr(logits), _ptr(ids), _ptr(weights), _i32(rows), _i32(experts), _i32(top), _stream()),
           "choose_topk")


def choose_grouped(logits: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, *, groups: int, keep: int,
                   weight_scale: float) -> None:
    """Scores are the softmax over all of a row's ``logits`` (float32 ``[T, E]``).  The experts form ``groups`` equal runs
    of neighbours; only experts of the ``keep`` groups with the largest best score can be chosen; of those the ``top``
    largest scores (largest first, the lowest index among equals) go into ``ids``, and into ``weights`` their scores
    over the chosen scores' sum, times ``weight_scale``."""
    _cuda(logits, ids, weights)
    rows, experts = logits.shape
    top = ids.shape[1]
    _need(logits.dtype == torch.float32 and logits.is_contiguous(), "choose_grouped logits")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and weights.dtype == torch.float32 and weights.is_contiguous()
          and tuple(ids.shape) == (rows, top) and tuple(weights.shape) == (rows, top), "choose_grouped ids/weights")
    lib = load_library("experts")
    _check(lib.tb_choose_grouped(_ptr(logits), _ptr(ids), _ptr(weights), _i32(rows), _i32(experts), _i32(top), _i32(groups),
                                 _i32(keep), _f32(weight_scale), _stream()), "choose_grouped")


def expert_plan(ids: torch.Tensor, experts: int, offsets: torch.Tensor, order: torch.Tensor) -> None:
    """Group the assignments ``ids.flatten()`` by expert: ``order[offsets[e] : offsets[e + 1]]`` are expert ``e``'s."""
    _cuda(ids, offsets, order)
    count = ids.numel()
    _need(ids.dtype == torch.int32 and ids.is_contiguous(), "expert_plan ids")
    _need(offsets.dtype == torch.int32 and offsets.numel() == experts + 1 and offsets.is_contiguous(), "expert_plan offsets")
    _need(order.dtype == torch.int32 and order.numel() == count and order.is_contiguous(), "expert_plan order")
    lib = load_library("experts")
    _check(lib.tb_expert_plan(_ptr(ids), _i32(count), _i32(experts), _ptr(offsets), _ptr(order), _stream()), "expert_plan")


def expert_linear_tensor_cores(dtype: torch.dtype, in_features: int) -> bool:
    """Whether the experts' product of these sizes runs on the tensor cores (bfloat16, K a multiple of 32)."""
    return dtype == torch.bfloat16 and in_features % 32 == 0


def expert_linear(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, offsets: torch.Tensor, order: torch.Tensor,
                  *, source_div: int, epilogue: int = EXPERT_PLAIN) -> torch.Tensor:
    """``out[a] = act(weight[expert(a)] @ x[a // source_div])`` for every assignment ``a`` (``weight`` ``[E, N, K]``,
    ``out`` ``[assignments, N]`` in ``x``'s dtype or float32), grouped as ``expert_plan`` left them."""
    _cuda(x, weight, out, offsets, order)
    experts, n, k = weight.shape
    count = out.shape[0]
    _need(x.stride(1) == 1 and x.shape[1] == k and weight.is_contiguous() and weight.dtype == x.dtype, "expert_linear x/weight")
    _need(out.stride(1) == 1 and out.shape[1] == n and out.dtype in (x.dtype, torch.float32), "expert_linear out")
    _need(order.numel() == count and offsets.numel() == experts + 1, "expert_linear plan")
    _need(x.shape[0] * source_div >= count, "expert_linear: sources do not cover the assignments")
    tensor_cores = (expert_linear_tensor_cores(x.dtype, k) and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
                    and weight.data_ptr() % 16 == 0)
    lib = load_library("experts")
    _check(lib.tb_expert_linear(_ptr(x), _i64(x.stride(0)), _ptr(weight), _ptr(out), _i64(out.stride(0)), _ptr(offsets),
                                _ptr(order), _i32(count), _i32(experts), _i32(source_div), _i32(n), _i32(k),
                                _i32(epilogue), _i32(_code(x.dtype)), _i32(_code(out.dtype)),
                                _i32(1 if tensor_cores else 0), _stream()), "expert_linear")
    return out


def expert_combine(y: torch.Tensor, weights: torch.Tensor, base: Optional[torch.Tensor], out: torch.Tensor) -> torch.Tensor:
    """``out[t] = (base[t] if base is given else 0) + sum_s weights[t, s] * y[t * top + s]``, all float32."""
    _cuda(y, weights, base, out)
    rows, width = out.shape
    top = weights.shape[1]
    _f32_rows(y, (rows * top, width), "expert_combine y")
    _f32_rows(weights, (rows, top), "expert_combine weights")
    _f32_rows(base, (rows, width), "expert_combine base")
    _f32_rows(out, (rows, width), "expert_combine out")
    lib = load_library("experts")
    _check(lib.tb_expert_combine(_ptr(y), _ptr(weights), _ptr(base), _ptr(out), _i32(rows), _i32(width), _i32(top),
                                 _stream()), "expert_combine")
    return out


# ----------------------------------------------------------------------------- sublayers normed on both sides

NORM_NONE, NORM_LAYER, NORM_RMS = 0, 1, 2


def norm_add_norm(residual: torch.Tensor, update: Optional[torch.Tensor], post, following,
                  out: Optional[torch.Tensor], copy: Optional[torch.Tensor], eps: float) -> None:
    """``residual += post(update)`` (32-bit, in place; without ``update`` the stream stays), then ``out =
    following(residual)`` and ``copy = residual``, both rounded once to their dtype.  ``post`` and ``following`` are
    ``None`` or ``(kind, weight, bias)`` with kind ``NORM_LAYER`` (``(v - mean) / sqrt(var + eps) * weight + bias``) or
    ``NORM_RMS`` (``v / sqrt(mean(v^2) + eps) * weight``, bias None); both use ``eps``."""
    _cuda(residual, update, out, copy)
    rows, width = residual.shape
    _f32_rows(residual, (rows, width), "norm_add_norm: the stream is contiguous float32")
    _f32_rows(update, (rows, width), "norm_add_norm update")
    _need(post is None or update is not None, "norm_add_norm: a norm of the update needs an update")
    _need((following is None) == (out is None), "norm_add_norm: the following norm needs its output")
    dtype = None
    for o in (out, copy):
        if o is not None:
            _need(tuple(o.shape) == (rows, width) and o.is_contiguous() and dtype in (None, o.dtype), "norm_add_norm out/copy")
            dtype = o.dtype

    def parts(norm):
        if norm is None:
            return NORM_NONE, None, None
        kind, weight, bias = norm
        _need(kind in (NORM_LAYER, NORM_RMS), "norm_add_norm: unknown norm kind")
        for v in (weight, bias):
            _need(v is None or (v.is_cuda and v.dtype == torch.float32 and v.numel() == width and v.is_contiguous()),
                  "norm_add_norm weight/bias")
        _need(weight is not None and (kind != NORM_LAYER or bias is not None), "norm_add_norm: a norm needs its vectors")
        return kind, weight, bias

    post_kind, post_w, post_b = parts(post)
    next_kind, next_w, next_b = parts(following)
    lib = load_library("sandwich_norm")
    _check(lib.tb_norm_add_norm(_ptr(residual), _ptr(update), _i32(post_kind), _ptr(post_w), _ptr(post_b), _i32(next_kind),
                                _ptr(next_w), _ptr(next_b), _ptr(out), _ptr(copy), _i32(rows), _i32(width), _f32(eps),
                                _i32(_code(dtype) if dtype is not None else 0), _stream()), "norm_add_norm")


def gated_rms_norm(v: torch.Tensor, weight: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, eps: float) -> torch.Tensor:
    """``out = v / sqrt(mean(v^2) + eps) * weight * sigmoid(gate)`` over rows of float32 ``v``; ``gate`` and ``out`` in
    the run dtype."""
    _cuda(v, weight, gate, out)
    rows, width = v.shape
    _f32_rows(v, (rows, width), "gated_rms_norm takes contiguous float32 rows")
    _need(weight.dtype == torch.float32 and weight.numel() == width and weight.is_contiguous(), "gated_rms_norm weight")
    _need(gate.stride(1) == 1 and tuple(gate.shape) == (rows, width) and out.is_contiguous()
          and tuple(out.shape) == (rows, width) and out.dtype == gate.dtype, "gated_rms_norm gate/out")
    lib = load_library("sandwich_norm")
    _check(lib.tb_gated_rms_norm(_ptr(v), _ptr(weight), _ptr(gate), _i64(gate.stride(0)), _ptr(out), _i32(rows), _i32(width),
                                 _f32(eps), _i32(_code(out.dtype)), _stream()), "gated_rms_norm")
    return out


def token_gate(z: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, offset: int, out: torch.Tensor,
               activation: int) -> torch.Tensor:
    """``out[t] = act(z[t]) * table[tokens[t], offset : offset + width]``: ``z`` float32 ``[T, width]``, ``table`` and
    ``out`` in the run dtype."""
    _cuda(z, tokens, table, out)
    rows, width = z.shape
    _f32_rows(z, (rows, width), "token_gate takes contiguous float32 rows")
    _need(tokens.dtype == torch.int32 and tokens.is_contiguous() and tokens.numel() >= rows, "token_gate tokens")
    _need(table.stride(1) == 1 and 0 <= offset and offset + width <= table.shape[1], "token_gate table")
    _need(out.is_contiguous() and tuple(out.shape) == (rows, width) and out.dtype == table.dtype, "token_gate out")
    lib = load_library("pointwise")
    _check(lib.tb_token_gate(_ptr(z), _ptr(tokens), _ptr(table), _i64(table.stride(0)), _i32(offset), _ptr(out), _i32(rows),
                             _i32(width), _i32(table.shape[0]), _i32(activation), _i32(_code(out.dtype)), _stream()),
           "token_gate")
    return out


# ----------------------------------------------------------------------------- linear attention with a decay


def lightning(proj: torch.Tensor, decay: torch.Tensor, state: torch.Tensor, out: torch.Tensor, row_start: torch.Tensor,
              state_slots: torch.Tensor, *, num_seqs: int, heads: int, dim: int, vdim: int, max_new: int,
              activation: bool = True) -> torch.Tensor:
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head with ``q, k, v = silu`` of the columns
    ``[heads * dim | heads * dim | heads * vdim]`` of ``proj`` (``activation`` False: the columns as they are); ``state`` float32 ``[slots, heads, dim, vdim]`` is read and
    renewed per sequence; ``out`` float32 ``[T, heads * vdim]``."""
    _cuda(proj, decay, state, out, row_start, state_slots)
    rows = out.shape[0]
    _need(proj.stride(1) == 1 and proj.shape[0] == rows and proj.shape[1] >= heads * (2 * dim + vdim), "lightning proj")
    _f32_rows(out, (rows, heads * vdim), "lightning out is contiguous float32")
    _need(state.dtype == torch.float32 and state.is_contiguous() and tuple(state.shape[1:]) == (heads, dim, vdim),
          "lightning state")
    _need(decay.dtype == torch.float32 and decay.numel() == heads and decay.is_contiguous(), "lightning decay")
    _need(row_start.dtype == torch.int32 and state_slots.dtype == torch.int32, "lightning metadata must be int32")
    lib = load_library("lightning")
    # long prompt portions: the chunks of a sequence run side by side and meet through this scratch
    tiles = lib.tb_lightning_tiles(_i32(rows), _i32(num_seqs), _i32(dim), _i32(max(1, max_new)))
    scratch = torch.empty((tiles, heads, dim, vdim), dtype=torch.float32, device=out.device) if tiles else None
    _check(lib.tb_lightning(_ptr(proj), _i64(proj.stride(0)), _i32(0), _i32(heads * dim), _i32(2 * heads * dim), _ptr(decay),
                            _ptr(state), _ptr(out), _ptr(row_start), _ptr(state_slots), _i32(rows), _i32(num_seqs),
                            _i32(heads), _i32(dim), _i32(vdim), _i32(max(1, max_new)), _ptr(scratch),
                            _i32(1 if activation else 0), _i32(_code(proj.dtype)), _stream()), "lightning")
    if tiles:
        global launch_count
        launch_count += 2          # (the tiles' sums and the scan in front of the outputs)
    return out


GATE_SIGMOID, GATE_SILU = 0, 1


def retention_prepare(proj: torch.Tensor, out: torch.Tensor, positions: torch.Tensor, inv_freq: Optional[torch.Tensor], *,
                      heads: int, dim: int, vdim: int, rot_dims: int, amplitude: float, k_scale: float) -> torch.Tensor:
    """The columns ``[heads * dim q | heads * dim k | heads * vdim v]`` of ``proj`` widened into ``out`` (float32
    ``[T, heads * (2 dim + vdim)]``): of every q and k head's first ``rot_dims`` numbers, number ``i`` and number
    ``i + rot_dims / 2`` turn by ``position * inv_freq[i]`` (cosine and sine times ``amplitude``), k is multiplied by
    ``k_scale`` afterwards, v is copied."""
    _cuda(proj, out, positions, inv_freq)
    rows = out.shape[0]
    _need(proj.stride(1) == 1 and proj.shape[0] == rows and proj.shape[1] >= heads * (2 * dim + vdim), "retention_prepare proj")
    _f32_rows(out, (rows, heads * (2 * dim + vdim)), "retention_prepare out is contiguous float32")
    _need(positions.dtype == torch.int32, "retention_prepare positions must be int32")
    if rot_dims:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2
              and inv_freq.is_contiguous(), "retention_prepare inv_freq")
    lib = load_library("lightning")
    _check(lib.tb_retention_prepare(_ptr(proj), _i64(proj.stride(0)), _i32(0), _i32(heads * dim), _i32(2 * heads * dim),
                                    _ptr(out), _ptr(positions), _ptr(inv_freq), _i32(rows), _i32(heads), _i32(dim),
                                    _i32(vdim), _i32(rot_dims), _f32(amplitude), _f32(k_scale), _i32(_code(proj.dtype)),
                                    _stream()), "retention_prepare")
    return out


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, out: torch.Tensor, *, heads: int, vdim: int, eps: float,
                   gate_kind: int) -> torch.Tensor:
    """``out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * act(gate[t, h, :])`` with ``o`` float32
    ``[T, heads * vdim]`` and ``act`` the sigmoid (``GATE_SIGMOID``) or SiLU (``GATE_SILU``)."""
    _cuda(o, gate, out)
    rows = o.shape[0]
    _f32_rows(o, (rows, heads * vdim), "head_norm_gate o is contiguous float32")
    _need(gate.stride(1) == 1 and gate.shape == (rows, heads * vdim) and out.stride(1) == 1
          and out.shape == (rows, heads * vdim) and out.dtype == gate.dtype, "head_norm_gate gate/out")
    lib = load_library("lightning")
    _check(lib.tb_head_norm_gate(_ptr(o), _ptr(gate), _i64(gate.stride(0)), _ptr(out), _i64(out.stride(0)), _i32(rows),
                                 _i32(heads), _i32(vdim), _f32(eps), _i32(gate_kind), _i32(_code(out.dtype)), _stream()),
           "head_norm_gate")
    return out


# ----------------------------------------------------------------------------- two score maps over one set of values


def pair_rope_cache(proj: torch.Tensor, q_out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                    seq_of_row: torch.Tensor, block_table: torch.Tensor, inv_freq: Optional[torch.Tensor], *,
                    q_heads: int, key_heads: int, value_heads: int, dim: int, vdim: int, rot_dims: int,
                    page_size: int) -> None:
    """Rotation of neighbouring pairs of the first ``rot_dims`` numbers of every query and key head of ``proj``
    (``[q_heads * dim | key_heads * dim | value_heads * vdim | ...]``); queries into ``q_out``, keys and values into the
    pages of ``cache`` (``[key_heads, page, dim]`` keys then ``[value_heads, page, vdim]`` values)."""
    _cuda(proj, q_out, cache, positions, seq_of_row, block_table, inv_freq)
    rows = q_out.shape[0]
    channels = (q_heads + key_heads) * dim + value_heads * vdim
    _need(proj.stride(1) == 1 and proj.shape[1] >= channels and proj.shape[0] == rows, "pair_rope_cache proj")
    _need(q_out.stride(1) == 1 and q_out.shape[1] == q_heads * dim and q_out.dtype == proj.dtype, "pair_rope_cache q_out")
    _need(cache.dtype == proj.dtype and cache.is_contiguous(), "pair_rope_cache cache dtype")
    if rot_dims:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2
              and inv_freq.is_contiguous(), "pair_rope_cache inv_freq")
    for t in (positions, seq_of_row, block_table):
        _need(t.dtype == torch.int32, "pair_rope_cache metadata must be int32")
    lib = load_library("differential")
    _check(lib.tb_pair_rope_cache(_ptr(proj), _i64(proj.stride(0)), _ptr(q_out), _i64(q_out.stride(0)), _ptr(cache),
                                  _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                  _ptr(inv_freq), _i32(rows), _i32(q_heads), _i32(key_heads), _i32(value_heads), _i32(dim),
                                  _i32(vdim), _i32(rot_dims), _i32(page_size), _i32(_code(proj.dtype)), _stream()),
           "pair_rope_cache")


def differential_combine(maps: torch.Tensor, gate: Optional[torch.Tensor], out: torch.Tensor, *, heads: int,
                         kv_heads: int, vdim: int, lam: float, post: float, eps: float) -> torch.Tensor:
    """``o = a1 - lam * a2`` per head, over ``sqrt(mean(o^2) + eps)``, times ``post`` and ``sigmoid(gate)``.  ``maps``
    float32 ``[T, 2 * heads * vdim]`` holds the two maps' outputs as query heads laid out ``[kv head][map][head within
    the group]``; ``gate`` (or None) and ``out`` ``[T, heads * vdim]`` in the run dtype, laid out by head."""
    _cuda(maps, gate, out)
    rows = out.shape[0]
    _f32_rows(maps, (rows, 2 * heads * vdim), "differential_combine maps are contiguous float32")
    _need(out.is_contiguous() and tuple(out.shape) == (rows, heads * vdim), "differential_combine out")
    _need(gate is None or (gate.stride(1) == 1 and tuple(gate.shape) == (rows, heads * vdim) and gate.dtype == out.dtype),
          "differential_combine gate")
    lib = load_library("differential")
    _check(lib.tb_differential_combine(_ptr(maps), _ptr(gate), _i64(gate.stride(0) if gate is not None else 0), _ptr(out),
                                       _i32(rows), _i32(heads), _i32(kv_heads), _i32(vdim), _f32(lam), _f32(post),
                                       _f32(eps), _i32(_code(out.dtype)), _stream()), "differential_combine")
    return out


# ----------------------------------------------------------------------------- attention over a latent vector per token


def latent_rope_cache(down: torch.Tensor, q: torch.Tensor, q_full: torch.Tensor, cache: torch.Tensor,
                      weight: torch.Tensor, positions: torch.Tensor, seq_of_row: torch.Tensor, block_table: torch.Tensor,
                      inv_freq: Optional[torch.Tensor], *, heads: int, dim: int, rank: int, rot_width: int,
                      rot_dims: int, page_size: int, eps: float, amplitude: float = 1.0) -> None:
    """``down`` float32 ``[T, rank + rot_width]``: the first ``rank`` numbers over their root mean square times
    ``weight`` and the rotated rest go into the row's page (``[page, rank + rot_width]`` a page); the rotated parts of the
    query heads (``q`` ``[T, heads * (dim + rot_width)]``) go into ``q_full`` ``[T, heads * (rank + rot_width)]`` behind
    each head's first ``rank`` numbers, which this kernel leaves alone."""
    _cuda(down, q, q_full, cache, weight, positions, seq_of_row, block_table, inv_freq)
    rows = q.shape[0]
    _need(down.dtype == torch.float32 and down.stride(1) == 1 and tuple(down.shape) == (rows, rank + rot_width),
          "latent_rope_cache down")
    _need(q.stride(1) == 1 and q.shape[1] == heads * (dim + rot_width), "latent_rope_cache q")
    _need(q_full.stride(1) == 1 and tuple(q_full.shape) == (rows, heads * (rank + rot_width)) and q_full.dtype == q.dtype,
          "latent_rope_cache q_full")
    _need(cache.dtype == q.dtype and cache.is_contiguous(), "latent_rope_cache cache dtype")
    _need(weight.dtype == torch.float32 and weight.numel() == rank and weight.is_contiguous(), "latent_rope_cache weight")
    if rot_dims:
        _need(inv_freq is not None and inv_freq.dtype == torch.float32 and inv_freq.numel() == rot_dims // 2
              and inv_freq.is_contiguous(), "latent_rope_cache inv_freq")
    for t in (positions, seq_of_row, block_table):
        _need(t.dtype == torch.int32, "latent_rope_cache metadata must be int32")
    lib = load_library("latent_rope_cache")
    _check(lib.tb_latent_rope_cache(_ptr(down), _i64(down.stride(0)), _ptr(q), _i64(q.stride(0)), _ptr(q_full),
                                    _i64(q_full.stride(0)), _ptr(cache), _ptr(weight), _ptr(positions), _ptr(seq_of_row),
                                    _ptr(block_table), _i32(block_table.stride(0)), _ptr(inv_freq), _i32(rows), _i32(heads),
                                    _i32(dim), _i32(rank), _i32(rot_width), _i32(rot_dims), _i32(page_size), _f32(eps),
                                    _f32(amplitude), _i32(_code(q.dtype)), _stream()), "latent_rope_cache")


def attention_latent_mma_supported(dtype: torch.dtype, dim: int, vdim: int) -> bool:
    """Whether the tensor-core attention over cached latent vectors takes these sizes (bfloat16 only; the sizes it is
    instantiated for, as ``tb_attention_latent_mma_supported`` of the library says too: asked here without building it)."""
    return dtype == torch.bfloat16 and (dim, vdim) in ((576, 512), (288, 256), (160, 128))


def attention_latent_mma(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor,
                         seq_of_row: torch.Tensor, block_table: torch.Tensor, *, heads: int, dim: int, vdim: int,
                         page_size: int, mask_kind: int, mask_size: int, scale: float) -> torch.Tensor:
    """:func:`attention_masked` with ``kv_heads = 1`` and ``keys_per_value = 0`` (pages of ``[page_size, dim]`` vectors
    whose first ``vdim`` numbers are the value) on the tensor cores, for bfloat16: a block a row and sixteen query heads;
    exact bfloat16 products with 32-bit accumulation for the scores, 32-bit softmax, the weights as two bfloat16 halves.
    In a step of few rows every row's keys are shared out among several blocks, and a second kernel adds their results."""
    _cuda(q, out, cache, positions, seq_of_row, block_table)
    rows = q.shape[0]
    _need(q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.shape[1] == heads * dim, "attention_latent_mma q")
    _need(out.stride(1) == 1 and out.shape == (rows, heads * vdim) and out.dtype == q.dtype, "attention_latent_mma out")
    _need(cache.dtype == q.dtype and cache.is_contiguous(), "attention_latent_mma cache")
    _need(mask_kind in (MASK_CAUSAL, MASK_WINDOW), "attention_latent_mma mask")
    lib = load_library("attention_latent_mma")
    # a step of few rows gives every row several blocks, each over a run of its keys; they meet through this scratch
    splits = lib.tb_attention_latent_mma_splits(_i32(rows), _i32(heads))
    parts = torch.empty((rows, splits, heads, vdim + 2), dtype=torch.float32, device=q.device) if splits > 1 else None
    _check(lib.tb_attention_latent_mma(_ptr(q), _i64(q.stride(0)), _ptr(out), _i64(out.stride(0)), _ptr(cache),
                                       _ptr(positions), _ptr(seq_of_row), _ptr(block_table), _i32(block_table.stride(0)),
                                       _i32(rows), _i32(heads), _i32(dim), _i32(vdim), _i32(page_size), _i32(mask_kind),
                                       _i32(mask_size), _f32(scale), _ptr(parts), _stream()), "attention_latent_mma")
    if splits > 1:
        global launch_count
        launch_count += 1          # (the kernel that adds the runs up)
    return out
