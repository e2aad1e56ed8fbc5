// Rotation in the rotate-half layout, division of every query and key head by its root mean square, and the write
// of keys and values into the request's cache pages: what stands between an attention mixer's input projection
// and its attention kernel, in one pass over the projected rows.
//
// A projected row holds, side by side, H query heads of d numbers, G key heads of d numbers and G value heads of
// dv numbers; with `bias` (32-bit, as wide as that row) the projections' biases are added first, in 32-bit.  For queries and keys, of every head's first `rot_dims` numbers, number i and number i + rot_dims / 2
// turn together by the angle position * inv_freq[i] (32-bit angle, sincosf), cosine and sine both multiplied by
// `amplitude`; the rest of the head passes.  Then, with `unit_norm`, the head is divided by
// sqrt(mean(head^2) + eps), the mean over all d numbers of the rotated head.  Queries go to q_out, keys and values
// into the pages: a page is [G][page_size][d] keys followed by [G][page_size][dv] values.
//
// One warp per (row, head of q, k or v).  All arithmetic is 32-bit; each stored value is rounded once; the order
// of a head's sum of squares depends on d alone.
//
// tb_pool_blocks, for a mixer that also attends to averaged blocks of old tokens, runs behind it: every row that ends a
// block of `pool` positions leaves the block's averaged key and value in pages of their own.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;

struct HeadGeometry {
    int heads, kv_heads, dim, vdim;      // H, G, d, dv
    int rot_dims;                        // even, <= dim; 0: no rotation
    int page_size;
    int unit_norm;
    float amplitude, eps;
};

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
rope_norm_cache_kernel(const T* __restrict__ proj, int64_t proj_stride, T* __restrict__ q_out, int64_t q_stride,
                       T* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                       const int* __restrict__ block_table, int bt_stride, const float* __restrict__ inv_freq,
                       const float* __restrict__ bias, HeadGeometry g, int write_kv) {
    extern __shared__ float head_cache[];             // kWarps * dim
    pdl_trigger();
    pdl_wait();                                       // the projected rows and the step's metadata come from kernels in front
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int slot = blockIdx.y * kWarps + warp;      // which head of the row: queries, then keys, then values
    const int slots = g.heads + 2 * g.kv_heads;
    if (slot >= slots) return;                        // the whole warp leaves; no block-wide barrier below
    const int pos = positions[row];
    const T* prow = proj + (int64_t)row * proj_stride;

    T* dst;
    if (slot >= g.heads) {
        if (!write_kv) return;
        const int seq = seq_of_row[row];
        const int page = block_table[(int64_t)seq * bt_stride + pos / g.page_size];
        const int in_page = pos % g.page_size;
        const int64_t page_elems = (int64_t)g.kv_heads * g.page_size * (g.dim + g.vdim);
        dst = cache + (int64_t)page * page_elems;
        if (slot < g.heads + g.kv_heads) {
            dst += ((int64_t)(slot - g.heads) * g.page_size + in_page) * g.dim;
        } else {
            // a value head: copied as it is
            const int head = slot - g.heads - g.kv_heads;
            dst += (int64_t)g.kv_heads * g.page_size * g.dim + ((int64_t)head * g.page_size + in_page) * g.vdim;
            const int64_t at = (int64_t)(g.heads + g.kv_heads) * g.dim + (int64_t)head * g.vdim;
            const T* src = prow + at;
            if (bias == nullptr) {
                for (int i = lane; i < g.vdim; i += 32) dst[i] = src[i];
            } else {
                for (int i = lane; i < g.vdim; i += 32) Elem<T>::store(dst + i, Elem<T>::load(src + i) + bias[at + i]);
            }
            return;
        }
    } else {
        dst = q_out + (int64_t)row * q_stride + (int64_t)slot * g.dim;
    }
    const T* src = prow + (int64_t)slot * g.dim;      // query heads and key heads lie side by side in the row
    const float* add = bias == nullptr ? nullptr : bias + (int64_t)slot * g.dim;
    float* mine = head_cache + warp * g.dim;
    const int half = g.rot_dims >> 1;
    float ss = 0.0f;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf((float)pos * inv_freq[i], &sn, &cs);
        sn *= g.amplitude;
        cs *= g.amplitude;
        float u = Elem<T>::load(src + i), v = Elem<T>::load(src + i + half);
        if (add != nullptr) {
            u += add[i];
            v += add[i + half];
        }
        const float r0 = u * cs - v * sn;
        const float r1 = v * cs + u * sn;
        mine[i] = r0;
        mine[i + half] = r1;
        ss = fmaf(r0, r0, ss);
        ss = fmaf(r1, r1, ss);
    }
    for (int i = g.rot_dims + lane; i < g.dim; i += 32) {
        const float v = Elem<T>::load(src + i) + (add != nullptr ? add[i] : 0.0f);
        mine[i] = v;
        ss = fmaf(v, v, ss);
    }
    float inv = 1.0f;
    if (g.unit_norm) inv = 1.0f / sqrtf(warp_sum(ss) / (float)g.dim + g.eps);
    __syncwarp();
    for (int i = lane; i < g.dim; i += 32) Elem<T>::store(dst + i, mine[i] * inv);
}


// For every row of the step that ends a block of `pool` positions ((position + 1) % pool == 0): the averages of the block's
// keys and of its values, as the pages hold them, into entry position / pool of the request's pooled pages (same page
// layout).  A block of threads per (row, kv head), a thread a column, the block's tokens added in order in 32-bit.
template <typename T>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(const T* __restrict__ cache, T* __restrict__ pool_cache, const int* __restrict__ positions,
                   const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride,
                   const int* __restrict__ pool_table, int pool_bt_stride, int kv_heads, int dim, int vdim, int page_size,
                   int pool) {
    pdl_trigger();
    pdl_wait();                                       // the pages were written by the kernel in front
    const int row = blockIdx.x, g = blockIdx.y;
    const int pos = positions[row];
    if ((pos + 1) % pool != 0) return;
    const int seq = seq_of_row[row];
    const int entry = pos / pool, first = pos - pool + 1;
    const int64_t page_elems = (int64_t)kv_heads * page_size * (dim + vdim);
    const int* table = block_table + (int64_t)seq * bt_stride;
    const int64_t to_page = (int64_t)pool_table[(int64_t)seq * pool_bt_stride + entry / page_size] * page_elems;
    const int to_in_page = entry % page_size;
    for (int col = threadIdx.x; col < dim + vdim; col += blockDim.x) {
        const bool is_key = col < dim;
        const int width = is_key ? dim : vdim, c = is_key ? col : col - dim;
        const int64_t part = is_key ? 0 : (int64_t)kv_heads * page_size * dim;
        float sum = 0.0f;
        for (int j0 = 0; j0 < pool; j0 += 8) {         // eight loads in flight, then their sum in position order
            float v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const int key = first + min(j0 + u, pool - 1);
                const int64_t page = (int64_t)table[key / page_size] * page_elems;
                v[u] = Elem<T>::load(cache + page + part + ((int64_t)g * page_size + key % page_size) * width + c);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (j0 + u < pool) sum += v[u];
        }
        Elem<T>::store(pool_cache + to_page + part + ((int64_t)g * page_size + to_in_page) * width + c, sum / (float)pool);
    }
}

}  // namespace

// proj: [rows, >= (H + G) * d + G * dv] with row stride proj_stride (elements); q_out: [rows, H * d] with row
// stride q_stride; cache: this layer's pages; inv_freq: 32-bit [rot_dims / 2] (may be null when rot_dims is 0); bias:
// null or 32-bit [(H + G) * d + G * dv].
TB_EXPORT int tb_rope_norm_cache(const void* proj, int64_t proj_stride, void* q_out, int64_t q_stride, void* cache,
                                 const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
                                 const float* inv_freq, const float* bias, float amplitude, int rows, int heads, int kv_heads, int dim,
                                 int vdim, int rot_dims, int unit_norm, float eps, int page_size, int write_kv,
                                 int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (heads < 1 || kv_heads < 1 || dim < 1 || vdim < 1 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (rot_dims < 0 || rot_dims > dim || rot_dims % 2 != 0) return TB_ERR_BAD_SIZE;
    if (rot_dims > 0 && inv_freq == nullptr) return TB_ERR_BAD_SIZE;
    const size_t smem = (size_t)kWarps * dim * sizeof(float);
    if (smem > 40 * 1024) return TB_ERR_BAD_SIZE;
    HeadGeometry g;
    g.heads = heads; g.kv_heads = kv_heads; g.dim = dim; g.vdim = vdim; g.rot_dims = rot_dims; g.page_size = page_size;
    g.unit_norm = unit_norm; g.amplitude = amplitude; g.eps = eps;
    const int slots = heads + 2 * kv_heads;
    const dim3 grid(rows, (slots + kWarps - 1) / kWarps);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(rope_norm_cache_kernel<float>, grid, dim3(kWarps * 32), smem, stream, (const float*)proj,
                                 proj_stride, (float*)q_out, q_stride, (float*)cache, positions, seq_of_row, block_table,
                                 bt_stride, inv_freq, bias, g, write_kv);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(rope_norm_cache_kernel<__nv_bfloat16>, grid, dim3(kWarps * 32), smem, stream,
                                 (const __nv_bfloat16*)proj, proj_stride, (__nv_bfloat16*)q_out, q_stride,
                                 (__nv_bfloat16*)cache, positions, seq_of_row, block_table, bt_stride, inv_freq, bias, g,
                                 write_kv);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// cache: the layer's pages of keys and values ([G][page_size][d] keys then [G][page_size][dv] values a page), already
// holding the step's rows; pool_cache: its pages of averaged blocks, same layout, entry b of a request's pooled pages
// being block b; pool_table: the requests' tables of those pages.
TB_EXPORT int tb_pool_blocks(const void* cache, void* pool_cache, const int* positions, const int* seq_of_row,
                             const int* block_table, int bt_stride, const int* pool_table, int pool_bt_stride, int rows,
                             int kv_heads, int dim, int vdim, int page_size, int pool, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (kv_heads < 1 || kv_heads > 65535 || dim < 1 || vdim < 1 || page_size < 1 || pool < 1) return TB_ERR_BAD_SIZE;
    const dim3 grid(rows, kv_heads);
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(pool_blocks_kernel<float>, grid, dim3(128), (size_t)0, stream, (const float*)cache,
                                 (float*)pool_cache, positions, seq_of_row, block_table, bt_stride, pool_table,
                                 pool_bt_stride, kv_heads, dim, vdim, page_size, pool);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(pool_blocks_kernel<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream,
                                 (const __nv_bfloat16*)cache, (__nv_bfloat16*)pool_cache, positions, seq_of_row,
                                 block_table, bt_stride, pool_table, pool_bt_stride, kv_heads, dim, vdim, page_size, pool);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
