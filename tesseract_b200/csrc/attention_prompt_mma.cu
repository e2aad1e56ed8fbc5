// Paged attention on the tensor cores, for prompt portions and (second kernel) for steps of few rows, with 32-bit
// scores and weights kept to 32-bit accuracy: the masks and page layout of attention_masked.cu (keys and values of separate widths; causal, sliding window or
// blocks of positions, or a window with averaged blocks in front of it, which are walked first, from pages of their
// own), its learned sink per query head and its cap on the scores, for bfloat16 queries, keys and values.
//
//   S = Q K^T      mma.sync m16n8k16 on bfloat16 operands with 32-bit accumulators: the products of two bfloat16
//                  numbers are exact in 32-bit, so these are the 32-bit scores of the stored queries and keys;
//   softmax        32-bit, streaming over tiles of 64 keys (running maximum, sum and accumulator per row);
//   O += P V       the 32-bit weights are not rounded to bfloat16: P = hi + lo with hi = bf16(P) and
//                  lo = bf16(P - hi) (together 16 bits of mantissa or more), and O += hi V + lo V, two products with
//                  32-bit accumulators on the same value fragments.
//
// A block is 64 neighbouring rows of one sequence and one query head (four warps of 16 rows); it walks the keys that
// its rows' masks allow, from the first row's first key to the last row's position, in tiles of 64 keys that cp.async
// brings from the pages into a ring of two stages (rows of shared memory padded by 16 bytes, so that ldmatrix meets
// no bank conflicts).  Which block takes which rows follows from the step's row_start alone: a grid of
// ceil(rows / 64) + sequences blocks a head, of which those without rows leave at once.
#include "common.cuh"

namespace {

constexpr int QT = 64, KT = 64;
enum MaskKind : int { MASK_CAUSAL = 0, MASK_WINDOW = 1, MASK_BLOCKS = 2, MASK_WINDOW_POOLED = 3 };
typedef __nv_bfloat16 bf16;

// What only some mixers use: a learned sink score per query head (null: none), a cap on the scores (0: none), and the
// averaged blocks of MASK_WINDOW_POOLED: their pages (laid out like the tokens' with one value head a key head), the
// requests' tables of those pages and the tokens a block holds.  A row at position p sees the blocks
// 0 .. first_key(p) / pool - 1, then the tokens first_key(p) .. p.
struct Extras {
    const float* sinks;
    float softcap, cap_k;                 // cap_k = 2 log2(e) / softcap (0 without a cap)
    const bf16* pool_cache;
    const int* pool_table;
    int pool_bt_stride, pool;
};

// softcap * tanh(s / softcap) as softcap - 2 softcap / (2^(s k) + 1) with k = 2 log2(e) / softcap: one exponential and
// one reciprocal of the fast kind, good to some 1e-6 of softcap, which is far below what the bfloat16 queries and keys
// of these kernels leave.  (2^(s k) = inf gives softcap, 0 gives -softcap.)
__device__ __forceinline__ float capped(float s, float softcap, float k) {
    if (softcap <= 0.0f) return s;
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(s * k));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
    return fmaf(-2.0f * softcap, r, softcap);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t* r, uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
// (hi, lo) of two 32-bit weights: hi their bfloat16 rounding, lo the rounding of what hi leaves
__device__ __forceinline__ void split_bf16(float a, float b, uint32_t& hi, uint32_t& lo) {
    const __nv_bfloat16 ha = __float2bfloat16_rn(a), hb = __float2bfloat16_rn(b);
    hi = pack_bf16(a, b);
    lo = pack_bf16(a - __bfloat162float(ha), b - __bfloat162float(hb));
}

__device__ __forceinline__ int first_key_of(int pos, int mask_kind, int mask_size) {
    if (mask_kind == MASK_WINDOW || mask_kind == MASK_WINDOW_POOLED) return pos - mask_size + 1 > 0 ? pos - mask_size + 1 : 0;
    if (mask_kind == MASK_BLOCKS) return (pos / mask_size) * mask_size;
    return 0;
}

template <int D, int DV>
__global__ void __launch_bounds__(128)
attention_prompt_kernel(const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ out, int64_t out_stride,
                        const bf16* __restrict__ cache, const int* __restrict__ positions,
                        const int* __restrict__ row_start, const int* __restrict__ block_table, int bt_stride,
                        int num_seqs, int heads, int kv_heads, int page_size, int mask_kind, int mask_size, float scale,
                        int keys_per_value, int out_f32, Extras x) {
    constexpr int KS = D * 2 + 16, VS = DV * 2 + 16;              // bytes of a key row and a value row in shared memory
    constexpr int STAGE = KT * (KS + VS);
    extern __shared__ __align__(128) unsigned char tile_smem[];   // two stages of keys then values
    __shared__ int tile_info[3];
    pdl_trigger();
    pdl_wait();                                                   // queries, pages and the step's metadata come from kernels in front
    if (threadIdx.x == 0) {
        int tile = blockIdx.x, seq = -1, r0 = 0, n = 0;
        for (int s = 0; s < num_seqs; ++s) {
            const int begin = row_start[s], rows = row_start[s + 1] - begin;
            const int tiles = (rows + QT - 1) / QT;
            if (tile < tiles) {
                seq = s; r0 = begin + tile * QT; n = min(QT, rows - tile * QT);
                break;
            }
            tile -= tiles;
        }
        tile_info[0] = seq; tile_info[1] = r0; tile_info[2] = n;
    }
    __syncthreads();
    const int seq = tile_info[0], r0 = tile_info[1], n = tile_info[2];
    if (seq < 0) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int head = blockIdx.y, kv_head = head / (heads / kv_heads);
    const int pos_first = positions[r0], pos_last = pos_first + n - 1;        // a sequence's rows stand at consecutive positions
    const int key_lo = first_key_of(pos_first, mask_kind, mask_size);
    // the keys the block walks: the averaged blocks its last row sees, then the tokens key_lo .. pos_last
    const int blocks_last = mask_kind == MASK_WINDOW_POOLED ? first_key_of(pos_last, mask_kind, mask_size) / x.pool : 0;
    const int span = blocks_last + pos_last - key_lo + 1;
    const int tiles = (span - 1) / KT + 1;
    // keys_per_value key heads in a row read one value head: the page holds kv_heads / keys_per_value of those
    const int64_t page_elems = (int64_t)kv_heads * page_size * D + (int64_t)(kv_heads / keys_per_value) * page_size * DV;
    const int64_t k_off = (int64_t)kv_head * page_size * D;
    const int64_t v_off = (int64_t)kv_heads * page_size * D + (int64_t)(kv_head / keys_per_value) * page_size * DV;
    const int* table = block_table + (int64_t)seq * bt_stride;
    const int* pool_table = x.pool_table == nullptr ? nullptr : x.pool_table + (int64_t)seq * x.pool_bt_stride;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(tile_smem);

    // a tile's copy: two threads a key; one takes the first half of the key's and of the value's 16-byte chunks, the
    // other the second half
    const int copy_row = tid >> 1, copy_half = tid & 1;
    auto fill = [&](int tile) {
        const uint32_t stage = smem_base + (uint32_t)(tile & 1) * STAGE;
        const int at = tile * KT + copy_row;
        const bool there = at < span;
        const int a = there ? at : span - 1;
        const bool averaged = a < blocks_last;
        const int k = averaged ? a : key_lo + a - blocks_last;
        const bf16* from = averaged ? x.pool_cache : cache;
        const int64_t base = (int64_t)(averaged ? pool_table : table)[k / page_size] * page_elems;
        const int in_page = k % page_size;
        const bf16* kp = from + k_off + base + (int64_t)in_page * D;
        const bf16* vp = from + v_off + base + (int64_t)in_page * DV;
        const int bytes = there ? 16 : 0;                         // (a key behind the last one is zero-filled)
        constexpr int KC = D / 8, VC = DV / 8;
#pragma unroll
        for (int c = 0; c < (KC + 1) / 2; ++c) {
            const int chunk = copy_half * ((KC + 1) / 2) + c;
            if (chunk < KC) cp_async16(stage + copy_row * KS + chunk * 16, kp + chunk * 8, bytes);
        }
#pragma unroll
        for (int c = 0; c < (VC + 1) / 2; ++c) {
            const int chunk = copy_half * ((VC + 1) / 2) + c;
            if (chunk < VC) cp_async16(stage + KT * KS + copy_row * VS + chunk * 16, vp + chunk * 8, bytes);
        }
    };
    fill(0);
    cp_async_commit();

    // the warp's 16 query rows as the first operand: rows g and g + 8 of the warp's part, all of D
    const int i0 = warp * 16;
    uint32_t qa[D / 16][4];
    {
        const bool top_there = i0 + g < n, bottom_there = i0 + g + 8 < n;
        const bf16* top = q + (int64_t)(r0 + i0 + g) * q_stride + (int64_t)head * D;
        const bf16* bottom = top + 8 * q_stride;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = top_there ? *reinterpret_cast<const uint32_t*>(top + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = bottom_there ? *reinterpret_cast<const uint32_t*>(bottom + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = top_there ? *reinterpret_cast<const uint32_t*>(top + ks * 16 + 2 * t + 8) : 0u;
            qa[ks][3] = bottom_there ? *reinterpret_cast<const uint32_t*>(bottom + ks * 16 + 2 * t + 8) : 0u;
        }
    }
    int pos[2], first_key[2], blocks[2];
    bool there[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        pos[r] = pos_first + i0 + g + r * 8;
        there[r] = i0 + g + r * 8 < n;
        first_key[r] = first_key_of(pos[r], mask_kind, mask_size);
        blocks[r] = mask_kind == MASK_WINDOW_POOLED ? first_key[r] / x.pool : 0;
    }
    float m[2] = {-1.0e30f, -1.0e30f}, l[2] = {0.0f, 0.0f};
    if (x.sinks != nullptr) {                                     // the sink is the start of the running softmax
        m[0] = m[1] = x.sinks[head];
        l[0] = l[1] = t == 0 ? 1.0f : 0.0f;                       // (a row's four lanes add their sums at the end)
    }
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.0f;

    for (int tile = 0; tile < tiles; ++tile) {
        if (tile + 1 < tiles) {
            fill(tile + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                          // this tile's keys and values are in shared memory
        const uint32_t kstage = smem_base + (uint32_t)(tile & 1) * STAGE, vstage = kstage + KT * KS;
        const int at0 = tile * KT;
        const int key0 = key_lo + at0 - blocks_last;              // the token at the tile's first place, were it one
        // a warp whose rows see none of the tile's keys skips it (the rows' positions bound what they see)
        const int warp_first = first_key_of(pos_first + i0, mask_kind, mask_size);
        const int warp_last = pos_first + min(i0 + 15, n - 1);
        const bool any = i0 < n && (at0 < blocks_last || (key0 <= warp_last && key0 + KT - 1 >= warp_first));
        if (any) {
            float s[KT / 8][4];
#pragma unroll
            for (int j = 0; j < KT / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
                for (int jp = 0; jp < KT / 16; ++jp) {            // two tiles of eight keys a load
                    uint32_t b[4];
                    ldmatrix_x4(b, kstage + (jp * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + (ks * 2 + ((lane >> 3) & 1)) * 16);
                    mma_bf16_16816(s[2 * jp], qa[ks], b);
                    mma_bf16_16816(s[2 * jp + 1], qa[ks], b + 2);
                }
            }
            // scale, mask, and the tile's share of the streaming softmax
            float top[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
            for (int j = 0; j < KT / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1, place = j * 8 + 2 * t + (e & 1), key = key0 + place;
                    const bool seen = there[r] && (at0 + place < blocks_last ? at0 + place < blocks[r]
                                                                             : key <= pos[r] && key >= first_key[r]);
                    s[j][e] = seen ? capped(s[j][e] * scale, x.softcap, x.cap_k) : -1.0e30f;
                    top[r] = fmaxf(top[r], s[j][e]);
                }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
                top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
                const float m_new = fmaxf(m[r], top[r]);
                corr[r] = __expf(m[r] - m_new);
                m[r] = m_new;
                l[r] *= corr[r];
            }
#pragma unroll
            for (int j = 0; j < KT / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = e >> 1;
                    const float p = s[j][e] > -1.0e29f ? __expf(s[j][e] - m[r]) : 0.0f;
                    s[j][e] = p;
                    l[r] += p;                                    // (a lane's share; the four lanes of a row meet at the end)
                }
#pragma unroll
            for (int j = 0; j < DV / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
#pragma unroll
            for (int kk = 0; kk < KT / 16; ++kk) {
                uint32_t hi[4], lo[4];
                split_bf16(s[2 * kk][0], s[2 * kk][1], hi[0], lo[0]);
                split_bf16(s[2 * kk][2], s[2 * kk][3], hi[1], lo[1]);
                split_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1], hi[2], lo[2]);
                split_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3], hi[3], lo[3]);
#pragma unroll
                for (int jp = 0; jp < DV / 16; ++jp) {            // two tiles of eight value columns a load
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, vstage + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * VS + (jp * 2 + (lane >> 4)) * 16);
                    mma_bf16_16816(o[2 * jp], hi, b);
                    mma_bf16_16816(o[2 * jp], lo, b);
                    mma_bf16_16816(o[2 * jp + 1], hi, b + 2);
                    mma_bf16_16816(o[2 * jp + 1], lo, b + 2);
                }
            }
        }
        __syncthreads();                                          // the stage may be filled again
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (!there[r]) continue;
        const float inv = 1.0f / fmaxf(l[r], 1.0e-30f);
        if (out_f32) {                                            // the weighted sums as they are, unrounded
            float* orow = reinterpret_cast<float*>(out) + (int64_t)(r0 + i0 + g + r * 8) * out_stride + (int64_t)head * DV;
#pragma unroll
            for (int j = 0; j < DV / 8; ++j)
                *reinterpret_cast<float2*>(orow + j * 8 + 2 * t) = make_float2(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
            continue;
        }
        bf16* orow = out + (int64_t)(r0 + i0 + g + r * 8) * out_stride + (int64_t)head * DV;
#pragma unroll
        for (int j = 0; j < DV / 8; ++j)
            *reinterpret_cast<uint32_t*>(orow + j * 8 + 2 * t) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
}

// Steps of few rows (decoded ones): a block is ONE row and one kv head.  The query heads of that kv head (at most 16)
// are the 16 rows of the first operand, so a key or value is fetched once for all of them; the block's four warps
// share every tile of 64 keys, 16 keys a warp, each with a streaming softmax of its own, and their partial results
// (maximum, sum, accumulator) meet in shared memory in warp order.
template <int D, int DV>
__global__ void __launch_bounds__(128)
attention_rows_kernel(const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ out, int64_t out_stride,
                      const bf16* __restrict__ cache, const int* __restrict__ positions,
                      const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride, int heads,
                      int kv_heads, int page_size, int mask_kind, int mask_size, float scale, int keys_per_value,
                      int out_f32, Extras x) {
    constexpr int KS = D * 2 + 16, VS = DV * 2 + 16;
    constexpr int STAGE = KT * (KS + VS);
    constexpr int PART = DV + 2;                                  // a row's accumulator, maximum and sum
    extern __shared__ __align__(128) unsigned char tile_smem[];   // two stages, then [4 warps][16 rows][PART] floats
    pdl_trigger();
    pdl_wait();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row = blockIdx.x, kv_head = blockIdx.y, per = heads / kv_heads;
    const int pos = positions[row], seq = seq_of_row[row];
    const int key_lo = first_key_of(pos, mask_kind, mask_size);
    // the keys the row sees, in the order they are walked: its averaged blocks, then the tokens key_lo .. pos
    const int blocks = mask_kind == MASK_WINDOW_POOLED ? key_lo / x.pool : 0;
    const int span = blocks + pos - key_lo + 1;
    const int tiles = (span - 1) / KT + 1;
    // keys_per_value key heads in a row read one value head: the page holds kv_heads / keys_per_value of those
    const int64_t page_elems = (int64_t)kv_heads * page_size * D + (int64_t)(kv_heads / keys_per_value) * page_size * DV;
    const int64_t k_off = (int64_t)kv_head * page_size * D;
    const int64_t v_off = (int64_t)kv_heads * page_size * D + (int64_t)(kv_head / keys_per_value) * page_size * DV;
    const int* table = block_table + (int64_t)seq * bt_stride;
    const int* pool_table = x.pool_table == nullptr ? nullptr : x.pool_table + (int64_t)seq * x.pool_bt_stride;
    const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(tile_smem);
    const int copy_row = tid >> 1, copy_half = tid & 1;
    auto fill = [&](int tile) {
        const uint32_t stage = smem_base + (uint32_t)(tile & 1) * STAGE;
        const int at = tile * KT + copy_row;
        const bool there = at < span;
        const int a = there ? at : span - 1;
        const bool averaged = a < blocks;
        const int k = averaged ? a : key_lo + a - blocks;
        const bf16* from = averaged ? x.pool_cache : cache;
        const int64_t base = (int64_t)(averaged ? pool_table : table)[k / page_size] * page_elems;
        const int in_page = k % page_size;
        const bf16* kp = from + k_off + base + (int64_t)in_page * D;
        const bf16* vp = from + v_off + base + (int64_t)in_page * DV;
        const int bytes = there ? 16 : 0;
        constexpr int KC = D / 8, VC = DV / 8;
#pragma unroll
        for (int c = 0; c < (KC + 1) / 2; ++c) {
            const int chunk = copy_half * ((KC + 1) / 2) + c;
            if (chunk < KC) cp_async16(stage + copy_row * KS + chunk * 16, kp + chunk * 8, bytes);
        }
#pragma unroll
        for (int c = 0; c < (VC + 1) / 2; ++c) {
            const int chunk = copy_half * ((VC + 1) / 2) + c;
            if (chunk < VC) cp_async16(stage + KT * KS + copy_row * VS + chunk * 16, vp + chunk * 8, bytes);
        }
    };
    fill(0);
    cp_async_commit();
    uint32_t qa[D / 16][4];
    {
        const bool top_there = g < per, bottom_there = g + 8 < per;
        const bf16* top = q + (int64_t)row * q_stride + (int64_t)(kv_head * per + g) * D;
        const bf16* bottom = top + 8 * D;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            qa[ks][0] = top_there ? *reinterpret_cast<const uint32_t*>(top + ks * 16 + 2 * t) : 0u;
            qa[ks][1] = bottom_there ? *reinterpret_cast<const uint32_t*>(bottom + ks * 16 + 2 * t) : 0u;
            qa[ks][2] = top_there ? *reinterpret_cast<const uint32_t*>(top + ks * 16 + 2 * t + 8) : 0u;
            qa[ks][3] = bottom_there ? *reinterpret_cast<const uint32_t*>(bottom + ks * 16 + 2 * t + 8) : 0u;
        }
    }
    float m[2] = {-1.0e30f, -1.0e30f}, l[2] = {0.0f, 0.0f};
    if (x.sinks != nullptr && warp == 0) {                        // the sink is the start of ONE of the four running softmaxes
#pragma unroll
        for (int r = 0; r < 2; ++r)
            if (g + r * 8 < per) {
                m[r] = x.sinks[kv_head * per + g + r * 8];
                l[r] = t == 0 ? 1.0f : 0.0f;
            }
    }
    float o[DV / 8][4];
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.0f;
    for (int tile = 0; tile < tiles; ++tile) {
        if (tile + 1 < tiles) {
            fill(tile + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const uint32_t kstage = smem_base + (uint32_t)(tile & 1) * STAGE, vstage = kstage + KT * KS;
        const int at0 = tile * KT + warp * 16;                    // the warp's 16 keys of the tile
        if (at0 < span) {
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t b[4];
                ldmatrix_x4(b, kstage + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + (ks * 2 + ((lane >> 3) & 1)) * 16);
                mma_bf16_16816(s[0], qa[ks], b);
                mma_bf16_16816(s[1], qa[ks], b + 2);
            }
            float top[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int at = at0 + j * 8 + 2 * t + (e & 1);
                    s[j][e] = at < span ? capped(s[j][e] * scale, x.softcap, x.cap_k) : -1.0e30f;     // (all of the span is inside the mask)
                    top[e >> 1] = fmaxf(top[e >> 1], s[j][e]);
                }
            float corr[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
                top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
                const float m_new = fmaxf(m[r], top[r]);
                corr[r] = __expf(m[r] - m_new);
                m[r] = m_new;
                l[r] *= corr[r];
            }
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float p = s[j][e] > -1.0e29f ? __expf(s[j][e] - m[e >> 1]) : 0.0f;
                    s[j][e] = p;
                    l[e >> 1] += p;
                }
#pragma unroll
            for (int j = 0; j < DV / 8; ++j) {
                o[j][0] *= corr[0]; o[j][1] *= corr[0];
                o[j][2] *= corr[1]; o[j][3] *= corr[1];
            }
            uint32_t hi[4], lo[4];
            split_bf16(s[0][0], s[0][1], hi[0], lo[0]);
            split_bf16(s[0][2], s[0][3], hi[1], lo[1]);
            split_bf16(s[1][0], s[1][1], hi[2], lo[2]);
            split_bf16(s[1][2], s[1][3], hi[3], lo[3]);
#pragma unroll
            for (int jp = 0; jp < DV / 16; ++jp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, vstage + (warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * VS + (jp * 2 + (lane >> 4)) * 16);
                mma_bf16_16816(o[2 * jp], hi, b);
                mma_bf16_16816(o[2 * jp], lo, b);
                mma_bf16_16816(o[2 * jp + 1], hi, b + 2);
                mma_bf16_16816(o[2 * jp + 1], lo, b + 2);
            }
        }
        __syncthreads();
    }
    // the warps' partial results, then their sum in warp order
    float* parts = reinterpret_cast<float*>(tile_smem + 2 * STAGE);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        float* mine = parts + ((size_t)warp * 16 + g + r * 8) * PART;
#pragma unroll
        for (int j = 0; j < DV / 8; ++j) {
            mine[j * 8 + 2 * t] = o[j][2 * r];
            mine[j * 8 + 2 * t + 1] = o[j][2 * r + 1];
        }
        if (t == 0) {
            mine[DV] = m[r];
            mine[DV + 1] = l[r];
        }
    }
    __syncthreads();
    for (int index = tid; index < per * DV; index += 128) {
        const int head_row = index / DV, col = index % DV;
        float top = -1.0e30f;
#pragma unroll
        for (int w = 0; w < 4; ++w) top = fmaxf(top, parts[((size_t)w * 16 + head_row) * PART + DV]);
        float total = 0.0f, value = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float* theirs = parts + ((size_t)w * 16 + head_row) * PART;
            const float weight = __expf(theirs[DV] - top);
            total = fmaf(theirs[DV + 1], weight, total);
            value = fmaf(theirs[col], weight, value);
        }
        const int64_t at = (int64_t)row * out_stride + (int64_t)(kv_head * per + head_row) * DV + col;
        if (out_f32) reinterpret_cast<float*>(out)[at] = value / fmaxf(total, 1.0e-30f);
        else out[at] = __float2bfloat16_rn(value / fmaxf(total, 1.0e-30f));
    }
}

template <int D, int DV>
int launch_rows(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache, const int* positions,
                const int* seq_of_row, const int* block_table, int bt_stride, int rows, int heads, int kv_heads,
                int page_size, int mask_kind, int mask_size, float scale, int keys_per_value, int out_f32, Extras x,
                cudaStream_t stream) {
    constexpr int smem = 2 * KT * (D * 2 + 16 + DV * 2 + 16) + 4 * 16 * (DV + 2) * 4;
    auto kernel = attention_rows_kernel<D, DV>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return (int)err;
    }
    cudaError_t launched = tb_launch_pdl(kernel, dim3(rows, kv_heads), dim3(128), (size_t)smem, stream, (const bf16*)q,
                                         q_stride, (bf16*)out, out_stride, (const bf16*)cache, positions, seq_of_row,
                                         block_table, bt_stride, heads, kv_heads, page_size, mask_kind, mask_size, scale,
                                         keys_per_value, out_f32, x);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <int D, int DV>
int launch(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache, const int* positions,
           const int* row_start, const int* block_table, int bt_stride, int rows, int num_seqs, int heads, int kv_heads,
           int page_size, int mask_kind, int mask_size, float scale, int keys_per_value, int out_f32, Extras x,
           cudaStream_t stream) {
    constexpr int smem = 2 * KT * (D * 2 + 16 + DV * 2 + 16);
    auto kernel = attention_prompt_kernel<D, DV>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (err != cudaSuccess) return (int)err;
    }
    const dim3 grid((rows + QT - 1) / QT + num_seqs, heads);
    cudaError_t launched = tb_launch_pdl(kernel, grid, dim3(128), (size_t)smem, stream, (const bf16*)q, q_stride,
                                         (bf16*)out, out_stride, (const bf16*)cache, positions, row_start, block_table,
                                         bt_stride, num_seqs, heads, kv_heads, page_size, mask_kind, mask_size, scale,
                                         keys_per_value, out_f32, x);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

}  // namespace

// Whether tb_attention_prompt_mma takes these head sizes.
TB_EXPORT int tb_attention_prompt_mma_supported(int dim, int vdim) {
    return ((dim == 64 || dim == 128) && (vdim == 64 || vdim == 128)) || (dim == 64 && vdim == 48) ? 1 : 0;
}

// q: bfloat16 [rows, heads * dim] (row stride q_stride, elements); out: bfloat16, or with out_f32 float32 (the sums
// unrounded), [rows, heads * vdim], row stride out_stride in its own elements; cache: this layer's pages
// ([kv_heads][page_size][dim] keys then [kv_heads / keys_per_value][page_size][vdim] values a page, key head g reading
// value head g / keys_per_value); row_start: int32 [num_seqs + 1]; the rows of a sequence stand at consecutive
// positions.  mask_kind: 0 causal, 1 window, 2 blocks, 3 window with averaged blocks (pool_cache: the layer's pages of
// averages, pool_table: the requests' tables of those pages with row stride pool_bt_stride, pool: tokens a block).
// sinks: null or float32 [heads]; softcap: 0 for none.
TB_EXPORT int tb_attention_prompt_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                      const int* positions, const int* row_start, const int* block_table, int bt_stride,
                                      int rows, int num_seqs, int heads, int kv_heads, int dim, int vdim, int page_size,
                                      int mask_kind, int mask_size, float scale, int keys_per_value, int out_f32,
                                      const float* sinks, float softcap, const void* pool_cache, const int* pool_table,
                                      int pool_bt_stride, int pool, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (mask_kind == MASK_WINDOW_POOLED && (pool < 1 || pool_cache == nullptr || pool_table == nullptr || keys_per_value != 1 ||
                                            (uintptr_t)pool_cache % 16 != 0))
        return TB_ERR_BAD_SIZE;
    if (softcap < 0.0f) return TB_ERR_BAD_SIZE;
    Extras x;
    x.sinks = sinks; x.softcap = softcap; x.cap_k = softcap > 0.0f ? 2.8853900817779268f / softcap : 0.0f; x.pool_cache = (const bf16*)pool_cache; x.pool_table = pool_table;
    x.pool_bt_stride = pool_bt_stride; x.pool = pool;
    if (!tb_attention_prompt_mma_supported(dim, vdim)) return TB_ERR_BAD_SIZE;
    if (kv_heads < 1 || heads < 1 || heads % kv_heads != 0 || page_size < 1 || num_seqs < 1) return TB_ERR_BAD_SIZE;
    if (keys_per_value < 1 || kv_heads % keys_per_value != 0) return TB_ERR_BAD_SIZE;
    if (heads > 65535) return TB_ERR_BAD_SIZE;
    if (mask_kind < MASK_CAUSAL || mask_kind > MASK_WINDOW_POOLED) return TB_ERR_BAD_SIZE;
    if (mask_kind != MASK_CAUSAL && mask_size < 1) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 != 0 || q_stride % 2 != 0 || out_stride % 2 != 0)
        return TB_ERR_BAD_ALIGN;
#define TB_ATTEND(D, DV)                                                                                            \
    return launch<D, DV>(q, q_stride, out, out_stride, cache, positions, row_start, block_table, bt_stride, rows,    \
                         num_seqs, heads, kv_heads, page_size, mask_kind, mask_size, scale, keys_per_value, out_f32, x, stream)
    if (dim == 64 && vdim == 48) TB_ATTEND(64, 48);
    if (dim == 64 && vdim == 64) TB_ATTEND(64, 64);
    if (dim == 64 && vdim == 128) TB_ATTEND(64, 128);
    if (dim == 128 && vdim == 64) TB_ATTEND(128, 64);
    TB_ATTEND(128, 128);
#undef TB_ATTEND
}

// The same attention for steps of few rows: one block a (row, kv head), any positions.  At most 16 query heads a kv
// head; seq_of_row: int32 [rows].
TB_EXPORT int tb_attention_rows_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                    const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
                                    int rows, int heads, int kv_heads, int dim, int vdim, int page_size, int mask_kind,
                                    int mask_size, float scale, int keys_per_value, int out_f32, const float* sinks,
                                    float softcap, const void* pool_cache, const int* pool_table, int pool_bt_stride,
                                    int pool, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (mask_kind == MASK_WINDOW_POOLED && (pool < 1 || pool_cache == nullptr || pool_table == nullptr || keys_per_value != 1 ||
                                            (uintptr_t)pool_cache % 16 != 0))
        return TB_ERR_BAD_SIZE;
    if (softcap < 0.0f) return TB_ERR_BAD_SIZE;
    Extras x;
    x.sinks = sinks; x.softcap = softcap; x.cap_k = softcap > 0.0f ? 2.8853900817779268f / softcap : 0.0f; x.pool_cache = (const bf16*)pool_cache; x.pool_table = pool_table;
    x.pool_bt_stride = pool_bt_stride; x.pool = pool;
    if (!tb_attention_prompt_mma_supported(dim, vdim)) return TB_ERR_BAD_SIZE;
    if (kv_heads < 1 || heads < 1 || heads % kv_heads != 0 || heads / kv_heads > 16 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (keys_per_value < 1 || kv_heads % keys_per_value != 0) return TB_ERR_BAD_SIZE;
    if (kv_heads > 65535) return TB_ERR_BAD_SIZE;
    if (mask_kind < MASK_CAUSAL || mask_kind > MASK_WINDOW_POOLED) return TB_ERR_BAD_SIZE;
    if (mask_kind != MASK_CAUSAL && mask_size < 1) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 != 0 || q_stride % 2 != 0) return TB_ERR_BAD_ALIGN;
#define TB_ROWS(D, DV)                                                                                              \
    return launch_rows<D, DV>(q, q_stride, out, out_stride, cache, positions, seq_of_row, block_table, bt_stride,   \
                              rows, heads, kv_heads, page_size, mask_kind, mask_size, scale, keys_per_value, out_f32, x, stream)
    if (dim == 64 && vdim == 48) TB_ROWS(64, 48);
    if (dim == 64 && vdim == 64) TB_ROWS(64, 64);
    if (dim == 64 && vdim == 128) TB_ROWS(64, 128);
    if (dim == 128 && vdim == 64) TB_ROWS(128, 64);
    TB_ROWS(128, 128);
#undef TB_ROWS
}
