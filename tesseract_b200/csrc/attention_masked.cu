// Paged attention with 32-bit scores and weights, for mixers whose keys and values have widths of their own and
// whose mask, denominator and output are parameters:
//
//   mask     causal (every key up to the row's position), a sliding window of `mask_size` keys, blocks (the
//            positions of a sequence are cut into consecutive blocks of `mask_size`, counted from position 0, and
//            a row sees the keys of its own block up to its own position), or a window with pooled blocks: beside
//            the window's keys a row at position p sees one averaged key and value for every block of `pool`
//            positions that ends in front of the window (block b if (b + 1) * pool <= p - mask_size + 1);
//            the averages live in pages of their own (entry b of the request's pooled pages, same page layout), are
//            walked first, and share the softmax with the window's keys;
//   sink     the softmax denominator has one more entry that carries no value, of score 0
//            (w_j = exp(s_j) / (1 + sum_j exp(s_j))) or, with `sinks`, of a learned score per query head;
//   softcap  with softcap > 0 a score s becomes softcap * tanh(s / softcap) (the sink's score is not touched);
//   gate     the output is multiplied, element by element, by sigmoid(gate[row, head, :]).
//
// One warp per (query row, query head).  Keys are walked from the first visible one in blocks of 32, a lane a key:
// s_j = (q . k_j) * scale in 32-bit, a streaming softmax (running maximum m, sum l, accumulator acc; the sink is the
// start m = 0, l = 1), weights kept in 32-bit for the product with the values, lanes over the value's columns.  The
// order of every sum depends only on the row's position and the mask: not on the batch, on how the prompt was cut,
// or on the page ids.  A page is [G][page_size][d] keys followed by [G][page_size][dv] values.
//
// With block or window masks a row reads at most `mask_size` keys, so the work is linear in the rows of a step and
// the same kernel serves prompt portions and single decoded rows.
//
// Two kernels.  The packet kernel takes head sizes that are multiples of a 16-byte packet (8 bfloat16, 4 floats):
// a warp takes one row and up to four query heads of one kv head together, so that a key or value packet is
// loaded and widened once for all of them; a block is eight neighbouring rows of the same heads, which read all
// but a few of the same keys and meet in L1.  Scores: a lane a key, the key's packets against the queries in
// shared memory (read four numbers at a time).  Values: the warp is cut into groups of lanes that share a value
// row, a lane a packet of columns, the weights passed through shared memory; the groups' partial sums meet at the
// end in a fixed butterfly.  In a step of few rows (decoded ones) a block is one row instead, and its four or eight warps
// share the row's keys; which of the two runs depends on the number of rows of the step, so a row's values are the
// same in every batch up to the order of a few sums.  The element kernel takes every other size, a number at a time.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
enum MaskKind : int { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_BLOCKS = 2, MASK_WINDOW_POOLED = 3 };

// What only some mixers use: a learned sink score per query head (null: none, or the fixed 0 of `sink`), a cap on the
// scores (0: none), and the pooled blocks of MASK_WINDOW_POOLED (their pages, the requests' tables of those pages and
// the tokens a block holds).
struct MaskExtras {
    const float* sinks;
    float softcap;
    const void* pool_cache;
    const int* pool_table;
    int pool_bt_stride, pool;
};

__device__ __forceinline__ float capped(float s, float softcap) {
    return softcap > 0.0f ? softcap * tanhf(s / softcap) : s;
}

// The keys of a row in the order they are walked: `pooled` averaged blocks, then the positions first_key .. pos.
struct Reach {
    int first_key, pooled, total;
    __device__ Reach(int pos, int mask_kind, int mask_size, int pool) {
        first_key = 0;
        pooled = 0;
        if (mask_kind == MASK_WINDOW || mask_kind == MASK_WINDOW_POOLED) first_key = pos - mask_size + 1 > 0 ? pos - mask_size + 1 : 0;
        else if (mask_kind == MASK_BLOCKS) first_key = (pos / mask_size) * mask_size;
        if (mask_kind == MASK_WINDOW_POOLED) pooled = first_key / pool;       // blocks that end in front of the window
        total = pooled + pos - first_key + 1;
    }
};

// Where a page keeps what.  keys_per_value >= 1: [kv_heads][page][dim] keys, then [kv_heads / keys_per_value][page][vdim]
// values, key head g reading value head g / keys_per_value (1: the usual layout; 2: two score maps over one set of
// values).  keys_per_value == 0: the page holds keys only, and a key's first vdim numbers are its value (attention in a
// latent space).
struct PageLayout {
    int64_t page_elems, value_base;
    int value_row;
    __device__ PageLayout(int kv_heads, int kv_head, int page_size, int dim, int vdim, int keys_per_value) {
        if (keys_per_value == 0) {
            page_elems = (int64_t)kv_heads * page_size * dim;
            value_base = (int64_t)kv_head * page_size * dim;
            value_row = dim;
        } else {
            const int value_heads = kv_heads / keys_per_value;
            page_elems = (int64_t)page_size * ((int64_t)kv_heads * dim + (int64_t)value_heads * vdim);
            value_base = (int64_t)kv_heads * page_size * dim + (int64_t)(kv_head / keys_per_value) * page_size * vdim;
            value_row = vdim;
        }
    }
};

template <typename T, int NCV, bool VEC>
__global__ void __launch_bounds__(kWarps * 32)
attention_masked_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate, int64_t gate_stride,
                        T* __restrict__ out, int64_t out_stride, const T* __restrict__ cache,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                        const int* __restrict__ block_table, int bt_stride, int heads, int kv_heads, int dim, int vdim,
                        int page_size, int mask_kind, int mask_size, int sink, float scale, int keys_per_value,
                        int out_f32, MaskExtras extras) {
    extern __shared__ float q_smem[];                 // kWarps * dim
    pdl_trigger();
    pdl_wait();                                       // queries, pages and the step's metadata come from kernels in front
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x;
    const int head = blockIdx.y * kWarps + warp;
    if (head >= heads) return;                        // the whole warp leaves; no block-wide barrier below
    const int kv_head = head / (heads / kv_heads);
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    const Reach reach(pos, mask_kind, mask_size, extras.pool);

    float* qs = q_smem + warp * dim;
    const T* qrow = q + (int64_t)row * q_stride + (int64_t)head * dim;
    for (int i = lane; i < dim; i += 32) qs[i] = Elem<T>::load(qrow + i);
    __syncwarp();

    const PageLayout layout(kv_heads, kv_head, page_size, dim, vdim, keys_per_value);
    const int64_t page_elems = layout.page_elems;
    const int vrow = layout.value_row;
    const int64_t key_base = (int64_t)kv_head * page_size * dim;
    const int* table = block_table + (int64_t)seq * bt_stride;
    const int* pool_table = extras.pool_table == nullptr ? nullptr : extras.pool_table + (int64_t)seq * extras.pool_bt_stride;
    const T* pool_cache = reinterpret_cast<const T*>(extras.pool_cache);

    const bool starts = sink || extras.sinks != nullptr;
    float m = starts ? (extras.sinks != nullptr ? extras.sinks[head] : 0.0f) : -1.0e30f;
    float l = starts ? 1.0f : 0.0f;
    float acc[NCV];
#pragma unroll
    for (int c = 0; c < NCV; ++c) acc[c] = 0.0f;

    for (int v0 = 0; v0 < reach.total; v0 += 32) {
        const int at = v0 + lane;
        const bool valid = at < reach.total;
        int64_t v_row = 0;                            // the address of the key's value row
        float s = -1.0e30f;
        if (valid) {
            const bool averaged = at < reach.pooled;
            const int key = averaged ? at : reach.first_key + at - reach.pooled;
            const T* from = averaged ? pool_cache : cache;
            const int64_t page = (averaged ? pool_table : table)[key / page_size];
            const int in_page = key % page_size;
            v_row = (int64_t)(from + layout.value_base + page * page_elems + (int64_t)in_page * vrow);
            const T* kp = from + key_base + page * page_elems + (int64_t)in_page * dim;
            float dot = 0.0f;
            if (VEC) {
                constexpr int N = Packet<T>::N;
                float kv[N];
                for (int i = 0; i < dim; i += N) {
                    Packet<T>::load(kp + i, kv);
#pragma unroll
                    for (int e = 0; e < N; ++e) dot = fmaf(qs[i + e], kv[e], dot);
                }
            } else {
                for (int i = 0; i < dim; ++i) dot = fmaf(qs[i], Elem<T>::load(kp + i), dot);
            }
            s = capped(dot * scale, extras.softcap);
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float p = valid ? expf(s - m_new) : 0.0f;
        const float corr = expf(m - m_new);
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < NCV; ++c) acc[c] *= corr;
        const int keys_here = min(32, reach.total - v0);
        for (int j = 0; j < keys_here; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const T* vp = reinterpret_cast<const T*>(__shfl_sync(0xffffffffu, v_row, j));
#pragma unroll
            for (int c = 0; c < NCV; ++c) {
                const int col = c * 32 + lane;
                if (col < vdim) acc[c] = fmaf(pj, Elem<T>::load(vp + col), acc[c]);
            }
        }
        m = m_new;
    }
    const float denom = fmaxf(l, 1.0e-30f);
    const int64_t oat = (int64_t)row * out_stride + (int64_t)head * vdim;
    const T* grow = gate == nullptr ? nullptr : gate + (int64_t)row * gate_stride + (int64_t)head * vdim;
#pragma unroll
    for (int c = 0; c < NCV; ++c) {
        const int col = c * 32 + lane;
        if (col < vdim) {
            float value = acc[c] / denom;
            if (grow != nullptr) value *= 1.0f / (1.0f + expf(-Elem<T>::load(grow + col)));
            if (out_f32) reinterpret_cast<float*>(out)[oat + col] = value;
            else Elem<T>::store(out + oat + col, value);
        }
    }
}


constexpr int kRowsPerBlock = 8;      // warps of a block: neighbouring rows of the same heads
constexpr int kSplitWarps = 4;        // warps of a block that share one row's keys (steps of few rows)
constexpr int kSplitWarpsLong = 8;    // the same where few rows each see many keys (2.55 -> 1.49 ms a decode step of
                                      // eight rows under windows of 512; at 64 rows, or with at most 256 keys a row,
                                      // eight warps lose 3 to 9 %)
constexpr int kLongSpan = 256, kLongMaxRows = 32;

// HPW: query heads of one kv head that a warp takes together (1 to 4, a divisor of the heads per kv head); NP: packets of value columns per lane;
// lv: lanes that share a value row in the value phase (a power of two).
// SPLITW > 0: a block is ONE row (a step of few rows, decoded ones for instance): its SPLITW warps take every
// SPLITW-th block of 32 keys each and their partial results (running maximum, sum, accumulator) meet in shared memory.
template <typename T, int HPW, int NP, int SPLITW>
__global__ void __launch_bounds__(kRowsPerBlock * 32, 3)
attention_masked_packets_kernel(const T* __restrict__ q, int64_t q_stride, const T* __restrict__ gate,
                                int64_t gate_stride, T* __restrict__ out, int64_t out_stride,
                                const T* __restrict__ cache, const int* __restrict__ positions,
                                const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride,
                                int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind,
                                int mask_size, int sink, float scale, int lv, int keys_per_value, int out_f32,
                                MaskExtras extras) {
    constexpr int N = Packet<T>::N;
    constexpr bool SPLIT = SPLITW > 0;
    constexpr int WARPS = SPLIT ? SPLITW : kRowsPerBlock;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_trigger();
    pdl_wait();                                       // queries, pages and the step's metadata come from kernels in front
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = SPLIT ? blockIdx.x : blockIdx.x * WARPS + warp;
    const int head0 = blockIdx.y * HPW;
    if (!SPLIT && row >= rows) return;                // the whole warp leaves; no block-wide barrier on this path
    const size_t per_warp = 32 * sizeof(int64_t) + (size_t)HPW * (32 + dim) * sizeof(float);
    int64_t* voffs = reinterpret_cast<int64_t*>(smem_raw + warp * per_warp);      // addresses of the keys' value rows
    float* ps = reinterpret_cast<float*>(voffs + 32);         // [HPW][32]
    float* qs = ps + HPW * 32;                                // [HPW][dim]
    const int kv_head = head0 / (heads / kv_heads);
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    const Reach reach(pos, mask_kind, mask_size, extras.pool);

    const T* qrow = q + (int64_t)row * q_stride + (int64_t)head0 * dim;       // the HPW heads lie side by side
    for (int i = lane * N; i < HPW * dim; i += 32 * N) Packet<T>::load(qrow + i, qs + i);
    __syncwarp();

    const PageLayout layout(kv_heads, kv_head, page_size, dim, vdim, keys_per_value);
    const int64_t page_elems = layout.page_elems;
    const int vrow = layout.value_row;
    const int64_t key_base = (int64_t)kv_head * page_size * dim;
    const int* table = block_table + (int64_t)seq * bt_stride;
    const int* pool_table = extras.pool_table == nullptr ? nullptr : extras.pool_table + (int64_t)seq * extras.pool_bt_stride;
    const T* pool_cache = reinterpret_cast<const T*>(extras.pool_cache);
    const int vg = lane / lv, vs = lane % lv;         // value phase: group vg owns keys vg, vg + 32 / lv, ...
    const int value_step = 32 / lv;

    float m[HPW], l[HPW], acc[HPW][NP][N];
    const bool starts = (sink || extras.sinks != nullptr) && (!SPLIT || warp == 0);       // the sink is the start of one running softmax
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
        m[h] = starts ? (extras.sinks != nullptr ? extras.sinks[head0 + h] : 0.0f) : -1.0e30f;
        l[h] = starts ? 1.0f : 0.0f;
#pragma unroll
        for (int pk = 0; pk < NP; ++pk)
#pragma unroll
            for (int e = 0; e < N; ++e) acc[h][pk][e] = 0.0f;
    }

    for (int v0 = SPLIT ? 32 * warp : 0; v0 < reach.total; v0 += SPLIT ? 32 * WARPS : 32) {
        const bool valid = v0 + lane < reach.total;
        const int at = valid ? v0 + lane : reach.total - 1;       // (a lane behind the last key points at the last key)
        const bool averaged = at < reach.pooled;
        const int k = averaged ? at : reach.first_key + at - reach.pooled;
        const T* from = averaged ? pool_cache : cache;
        const int64_t base = (int64_t)(averaged ? pool_table : table)[k / page_size] * page_elems;
        const int in_page = k % page_size;
        const T* kp = from + key_base + base + (int64_t)in_page * dim;
        __syncwarp();                                 // the value phase of the block before has read voffs and ps
        voffs[lane] = (int64_t)(from + layout.value_base + base + (int64_t)in_page * vrow);
        // scores: a lane a key, the key's packets against the HPW queries in shared memory
        float dot[HPW];
#pragma unroll
        for (int h = 0; h < HPW; ++h) dot[h] = 0.0f;
#pragma unroll 2
        for (int i = 0; i < dim; i += N) {
            float kv[N];
            Packet<T>::load(kp + i, kv);
#pragma unroll
            for (int h = 0; h < HPW; ++h) {
#pragma unroll
                for (int e = 0; e < N; e += 4) {
                    const float4 qv = *reinterpret_cast<const float4*>(qs + h * dim + i + e);
                    dot[h] = fmaf(qv.x, kv[e], dot[h]);
                    dot[h] = fmaf(qv.y, kv[e + 1], dot[h]);
                    dot[h] = fmaf(qv.z, kv[e + 2], dot[h]);
                    dot[h] = fmaf(qv.w, kv[e + 3], dot[h]);
                }
            }
        }
        float corr[HPW];
#pragma unroll
        for (int h = 0; h < HPW; ++h) {
            const float s = valid ? capped(dot[h] * scale, extras.softcap) : -1.0e30f;
            const float m_new = fmaxf(m[h], warp_max(s));
            const float p = valid ? __expf(s - m_new) : 0.0f;
            corr[h] = __expf(m[h] - m_new);
            l[h] = l[h] * corr[h] + warp_sum(p);
            m[h] = m_new;
            ps[h * 32 + lane] = p;
        }
        __syncwarp();
#pragma unroll
        for (int h = 0; h < HPW; ++h)
#pragma unroll
            for (int pk = 0; pk < NP; ++pk)
#pragma unroll
                for (int e = 0; e < N; ++e) acc[h][pk][e] *= corr[h];
        // values: group vg takes keys vg, vg + value_step, ...; a key behind the last one has weight 0
        const int keys_here = min(32, reach.total - v0);
#pragma unroll 2
        for (int j0 = 0; j0 < keys_here; j0 += value_step) {
            const int j = j0 + vg;                    // (j < 32 always)
            const T* vp = reinterpret_cast<const T*>(voffs[j]);
            float pj[HPW];
#pragma unroll
            for (int h = 0; h < HPW; ++h) pj[h] = ps[h * 32 + j];
#pragma unroll
            for (int pk = 0; pk < NP; ++pk) {
                const int col = (pk * lv + vs) * N;
                if (col < vdim) {
                    float vv[N];
                    Packet<T>::load(vp + col, vv);
#pragma unroll
                    for (int h = 0; h < HPW; ++h)
#pragma unroll
                        for (int e = 0; e < N; ++e) acc[h][pk][e] = fmaf(pj[h], vv[e], acc[h][pk][e]);
                }
            }
        }
    }
    // the groups' partial sums, in a fixed butterfly
    for (int o = lv; o < 32; o <<= 1)
#pragma unroll
        for (int h = 0; h < HPW; ++h)
#pragma unroll
            for (int pk = 0; pk < NP; ++pk)
#pragma unroll
                for (int e = 0; e < N; ++e) acc[h][pk][e] += __shfl_xor_sync(0xffffffffu, acc[h][pk][e], o);
    if (SPLIT) {
        // every warp leaves (maximum, sum, accumulator) of its share of the keys; warp 0 adds them up in warp order
        float* parts = reinterpret_cast<float*>(smem_raw + WARPS * per_warp);     // [warps][HPW][vdim + 2]
        const int stride = vdim + 2;
        if (vg == 0) {
#pragma unroll
            for (int h = 0; h < HPW; ++h) {
                float* mine = parts + ((size_t)warp * HPW + h) * stride;
                if (vs == 0) {
                    mine[vdim] = m[h];
                    mine[vdim + 1] = l[h];
                }
#pragma unroll
                for (int pk = 0; pk < NP; ++pk) {
                    const int col = (pk * lv + vs) * N;
                    if (col < vdim) {
#pragma unroll
                        for (int e = 0; e < N; ++e) mine[col + e] = acc[h][pk][e];
                    }
                }
            }
        }
        __syncthreads();
        if (warp != 0 || vg != 0) return;
#pragma unroll
        for (int h = 0; h < HPW; ++h) {
            float top = -1.0e30f;
            for (int w = 0; w < WARPS; ++w) top = fmaxf(top, parts[((size_t)w * HPW + h) * stride + vdim]);
            float total = 0.0f;
#pragma unroll
            for (int pk = 0; pk < NP; ++pk)
#pragma unroll
                for (int e = 0; e < N; ++e) acc[h][pk][e] = 0.0f;
            for (int w = 0; w < WARPS; ++w) {
                const float* theirs = parts + ((size_t)w * HPW + h) * stride;
                const float weight = __expf(theirs[vdim] - top);
                total = fmaf(theirs[vdim + 1], weight, total);
#pragma unroll
                for (int pk = 0; pk < NP; ++pk) {
                    const int col = (pk * lv + vs) * N;
                    if (col < vdim) {
#pragma unroll
                        for (int e = 0; e < N; ++e) acc[h][pk][e] = fmaf(theirs[col + e], weight, acc[h][pk][e]);
                    }
                }
            }
            l[h] = total;
        }
    }
    if (vg != 0) return;
#pragma unroll
    for (int h = 0; h < HPW; ++h) {
        const float inv = 1.0f / fmaxf(l[h], 1.0e-30f);
        const int64_t oat = (int64_t)row * out_stride + (int64_t)(head0 + h) * vdim;
        const T* grow = gate == nullptr ? nullptr : gate + (int64_t)row * gate_stride + (int64_t)(head0 + h) * vdim;
#pragma unroll
        for (int pk = 0; pk < NP; ++pk) {
            const int col = (pk * lv + vs) * N;
            if (col < vdim) {
                float value[N];
#pragma unroll
                for (int e = 0; e < N; ++e) value[e] = acc[h][pk][e] * inv;
                if (grow != nullptr) {
                    float gv[N];
                    Packet<T>::load(grow + col, gv);
#pragma unroll
                    for (int e = 0; e < N; ++e) value[e] *= __fdividef(1.0f, 1.0f + __expf(-gv[e]));
                }
                if (out_f32) {
#pragma unroll
                    for (int e = 0; e < N; e += 4) Packet<float>::store(reinterpret_cast<float*>(out) + oat + col + e, value + e);
                } else {
                    Packet<T>::store(out + oat + col, value);
                }
            }
        }
    }
}

constexpr int kSplitMaxRows = 256;     // steps of at most this many rows give every row a block of its own

template <typename T, int HPW, int NP, int SPLITW>
int launch_packets_as(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out,
                      int64_t out_stride, const void* cache, const int* positions, const int* seq_of_row,
                      const int* block_table, int bt_stride, int rows, int heads, int kv_heads, int dim, int vdim,
                      int page_size, int mask_kind, int mask_size, int sink, float scale, int keys_per_value, int out_f32, MaskExtras extras, cudaStream_t stream) {
    constexpr int N = Packet<T>::N;
    int lv = 1;
    while (lv < 32 && lv * NP < vdim / N) lv <<= 1;
    constexpr bool SPLIT = SPLITW > 0;
    constexpr int WARPS = SPLIT ? SPLITW : kRowsPerBlock;
    const dim3 grid(SPLIT ? rows : (rows + WARPS - 1) / WARPS, heads / HPW);
    const size_t smem = WARPS * (32 * sizeof(int64_t) + (size_t)HPW * (32 + dim) * sizeof(float)) +
                        (SPLIT ? (size_t)WARPS * HPW * (vdim + 2) * sizeof(float) : 0);
    auto kernel = attention_masked_packets_kernel<T, HPW, NP, SPLITW>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    cudaError_t launched = tb_launch_pdl(kernel, grid, dim3(WARPS * 32), smem, stream, (const T*)q, q_stride,
                                         (const T*)gate, gate_stride, (T*)out, out_stride, (const T*)cache, positions,
                                         seq_of_row, block_table, bt_stride, rows, heads, kv_heads, dim, vdim,
                                         page_size, mask_kind, mask_size, sink, scale, lv, keys_per_value, out_f32, extras);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename T>
int launch_packets(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
                   const void* cache, const int* positions, const int* seq_of_row, const int* block_table,
                   int bt_stride, int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind,
                   int mask_size, int sink, float scale, int keys_per_value, int out_f32, MaskExtras extras, cudaStream_t stream) {
    const int per = heads / kv_heads;
    const bool two = vdim / Packet<T>::N > 32;        // more value packets than lanes: two a lane
    // (which form runs depends on the step's row count and the mask alone)
    const bool long_span = rows <= kLongMaxRows && (mask_kind == MASK_CAUSAL || mask_kind == MASK_WINDOW_POOLED || mask_size > kLongSpan);
#define TB_PACKETS_AS(HPW, NP, SPLITW)                                                                               \
    launch_packets_as<T, HPW, NP, SPLITW>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions,         \
                                          seq_of_row, block_table, bt_stride, rows, heads, kv_heads, dim, vdim,      \
                                          page_size, mask_kind, mask_size, sink, scale, keys_per_value, out_f32, extras, stream)
#define TB_PACKETS(HPW, NP)                                                                                          \
    return rows > kSplitMaxRows ? TB_PACKETS_AS(HPW, NP, 0)                                                          \
                                : (long_span ? TB_PACKETS_AS(HPW, NP, kSplitWarpsLong) : TB_PACKETS_AS(HPW, NP, kSplitWarps))
    if (per % 4 == 0 && !two) TB_PACKETS(4, 1);
    if (per % 3 == 0 && !two) TB_PACKETS(3, 1);
    if (per % 2 == 0) { if (two) TB_PACKETS(2, 2); else TB_PACKETS(2, 1); }
    if (two) TB_PACKETS(1, 2);
    TB_PACKETS(1, 1);
#undef TB_PACKETS
#undef TB_PACKETS_AS
}

template <typename T, bool VEC>
int launch_vec(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
               const void* cache, const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
               int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind, int mask_size,
               int sink, float scale, int keys_per_value, int out_f32, MaskExtras extras, cudaStream_t stream) {
    const dim3 grid(rows, (heads + kWarps - 1) / kWarps);
    const size_t smem = (size_t)kWarps * dim * sizeof(float);
#define TB_LAUNCH(NCV)                                                                                              \
    tb_launch_pdl(attention_masked_kernel<T, NCV, VEC>, grid, dim3(kWarps * 32), smem, stream, (const T*)q, q_stride,   \
                  (const T*)gate, gate_stride, (T*)out, out_stride, (const T*)cache, positions, seq_of_row,         \
                  block_table, bt_stride, heads, kv_heads, dim, vdim, page_size, mask_kind, mask_size, sink, scale, keys_per_value, \
                  out_f32, extras)
    if (vdim <= 32) TB_LAUNCH(1);
    else if (vdim <= 64) TB_LAUNCH(2);
    else if (vdim <= 96) TB_LAUNCH(3);
    else if (vdim <= 128) TB_LAUNCH(4);
    else if (vdim <= 192) TB_LAUNCH(6);
    else if (vdim <= 256) TB_LAUNCH(8);
    else TB_LAUNCH(16);
#undef TB_LAUNCH
    return tb_launch_status();
}

template <typename T>
int launch(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
           const void* cache, const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
           int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind, int mask_size, int sink,
           float scale, int keys_per_value, int out_f32, MaskExtras extras, cudaStream_t stream) {
    // 16-byte key loads need every key row to start on a 16-byte boundary
    const bool vec = dim % Packet<T>::N == 0 && vdim % Packet<T>::N == 0 && (uintptr_t)cache % 16 == 0;
    const uintptr_t bits = (uintptr_t)q | (uintptr_t)gate | (uintptr_t)out;
    const bool rows_in_packets = bits % 16 == 0 && q_stride % Packet<T>::N == 0 && out_stride % Packet<T>::N == 0 &&
                                 (gate == nullptr || gate_stride % Packet<T>::N == 0);
    if (vec && rows_in_packets && vdim <= 64 * Packet<T>::N && dim <= 64 * Packet<T>::N)
        return launch_packets<T>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                 block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                 mask_size, sink, scale, keys_per_value, out_f32, extras, stream);
    if (vec)
        return launch_vec<T, true>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                   block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                   mask_size, sink, scale, keys_per_value, out_f32, extras, stream);
    return launch_vec<T, false>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                mask_size, sink, scale, keys_per_value, out_f32, extras, stream);
}

}  // namespace

// q: [rows, heads * dim] (row stride q_stride, elements); gate: null or [rows, heads * vdim] (row stride
// gate_stride); out: [rows, heads * vdim], float32 if out_f32 (out_stride then counts floats) and else the dtype of q;
// cache: this layer's pages, laid out as keys_per_value says (PageLayout).  mask_kind: 0 causal, 1 window, 2 blocks,
// 3 window with pooled blocks (pool_cache: the layer's pages of averaged keys and values, pool_table: the requests'
// tables of those pages with row stride pool_bt_stride, pool: tokens a block).  sinks: null or float32 [heads];
// softcap: 0 for none.
TB_EXPORT int tb_attention_masked(const void* q, int64_t q_stride, const void* gate, int64_t gate_stride, void* out,
                                  int64_t out_stride, const void* cache, const int* positions, const int* seq_of_row,
                                  const int* block_table, int bt_stride, int rows, int heads, int kv_heads, int dim,
                                  int vdim, int page_size, int mask_kind, int mask_size, int sink, float scale,
                                  int keys_per_value, int out_f32, const float* sinks, float softcap,
                                  const void* pool_cache, const int* pool_table, int pool_bt_stride, int pool, int dtype,
                                  cudaStream_t stream) {
    if (rows == 0) return 0;
    if (mask_kind == MASK_WINDOW_POOLED && (pool < 1 || pool_cache == nullptr || pool_table == nullptr || keys_per_value != 1))
        return TB_ERR_BAD_SIZE;
    if (softcap < 0.0f) return TB_ERR_BAD_SIZE;
    MaskExtras extras;
    extras.sinks = sinks; extras.softcap = softcap; extras.pool_cache = pool_cache; extras.pool_table = pool_table;
    extras.pool_bt_stride = pool_bt_stride; extras.pool = pool;
    if (dim < 1 || dim > 1024 || vdim < 1 || vdim > 512) return TB_ERR_BAD_SIZE;
    if (kv_heads < 1 || heads < 1 || heads % kv_heads != 0 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (mask_kind < MASK_CAUSAL || mask_kind > MASK_WINDOW_POOLED) return TB_ERR_BAD_SIZE;
    if (mask_kind != MASK_CAUSAL && mask_size < 1) return TB_ERR_BAD_SIZE;
    if ((heads + kWarps - 1) / kWarps > 65535) return TB_ERR_BAD_SIZE;
    if (keys_per_value < 0 || (keys_per_value > 0 && kv_heads % keys_per_value != 0)) return TB_ERR_BAD_SIZE;
    if (keys_per_value == 0 && vdim > dim) return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32)
        return launch<float>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row, block_table,
                             bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind, mask_size, sink, scale,
                             keys_per_value, out_f32, extras, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(q, q_stride, gate, gate_stride, out, out_stride, cache, positions, seq_of_row,
                                     block_table, bt_stride, rows, heads, kv_heads, dim, vdim, page_size, mask_kind,
                                     mask_size, sink, scale, keys_per_value, out_f32, extras, stream);
    return TB_ERR_BAD_DTYPE;
}
