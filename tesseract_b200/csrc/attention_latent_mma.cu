// Paged attention in a latent space on the tensor cores: every query head reads the same cached vectors, a key is the
// whole vector ([D] numbers) and its value is the vector's first DV numbers, so a key tile in shared memory serves both
// products.  bfloat16 queries and pages; scores, softmax and weights kept to 32-bit accuracy as in
// attention_prompt_mma.cu:
//
//   S = Q K^T      mma.sync m16n8k16 on bfloat16 operands with 32-bit accumulators (exact products);
//   softmax        32-bit, streaming over tiles of 64 keys;
//   O += P V       P = hi + lo in bfloat16 halves, two products with 32-bit accumulators.
//
// A block is ONE row and sixteen query heads: the heads are the 16 rows of the first operand, so a cached vector is
// fetched once for all of them.  Per tile of 64 keys (cp.async into a ring of two stages, rows padded by 16 bytes) the
// four warps take 16 keys each for the scores, agree on the tile's maximum through shared memory, leave their weights
// (both halves) in shared memory, and then take a quarter of the value columns each for the second product, over all
// 64 keys.  The order of every sum follows from the row's position and the mask alone.  Prompt portions and decoded
// rows take the same kernel: the rows of a portion read nearly the same keys and meet in L2.
//
// A step of few rows (decoded ones) gives every row several blocks, each over a run of the row's key tiles (how many
// follows from the step's row count alone); they leave their running maximum, sum and unnormalised accumulator in
// scratch memory, and a second small kernel adds the runs up in order.
#include "common.cuh"

namespace {

constexpr int KT = 64;
enum MaskKind : int { MASK_CAUSAL = 0, MASK_WINDOW = 1 };
typedef __nv_bfloat16 bf16;

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

template <int D, int DV>
struct Layout {
    static constexpr int KS = D * 2 + 16;                 // bytes of a key row (and of a query row) in shared memory
    static constexpr int PS = KT * 2 + 16;                // bytes of a row of weights
    static constexpr int STAGE = KT * KS;
    static constexpr int Q_AT = 2 * STAGE;
    static constexpr int P_AT = Q_AT + 16 * KS;           // hi, then lo
    static constexpr int STAT_AT = P_AT + 2 * 16 * PS;    // [4 warps][16 rows] floats
    static constexpr int BYTES = STAT_AT + 4 * 16 * 4;
};

template <int D, int DV>
__global__ void __launch_bounds__(128)
attention_latent_kernel(const bf16* __restrict__ q, int64_t q_stride, bf16* __restrict__ out, int64_t out_stride,
                        const bf16* __restrict__ cache, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride, int heads,
                        int page_size, int mask_kind, int mask_size, float scale, float* __restrict__ parts) {
    typedef Layout<D, DV> L;
    constexpr int KS = L::KS, PS = L::PS;
    constexpr int COLS = DV / 4;                                  // value columns a warp owns
    extern __shared__ __align__(128) unsigned char smem[];
    pdl_trigger();
    pdl_wait();                                                   // queries, pages and the step's metadata come from kernels in front
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int row = blockIdx.x, head0 = blockIdx.y * 16;
    const int pos = positions[row], seq = seq_of_row[row];
    const int key_lo = (mask_kind == MASK_WINDOW && pos - mask_size + 1 > 0) ? pos - mask_size + 1 : 0;
    const int tiles = (pos - key_lo) / KT + 1;
    // with `parts` the row's tiles are shared out among gridDim.z blocks, a run of neighbouring tiles each
    const int per_split = (tiles + (int)gridDim.z - 1) / (int)gridDim.z;
    const int tile_first = parts == nullptr ? 0 : min(tiles, (int)blockIdx.z * per_split);
    const int tile_end = parts == nullptr ? tiles : min(tiles, tile_first + per_split);
    const int64_t page_elems = (int64_t)page_size * D;
    const int* table = block_table + (int64_t)seq * bt_stride;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(smem);
    float* stats = reinterpret_cast<float*>(smem + L::STAT_AT);

    const int copy_row = tid >> 1, copy_half = tid & 1;
    auto fill = [&](int tile) {
        const uint32_t stage = base + (uint32_t)(tile & 1) * L::STAGE;
        const int key = key_lo + tile * KT + copy_row;
        const bool there = key <= pos;
        const int k = there ? key : pos;
        const bf16* kp = cache + (int64_t)table[k / page_size] * page_elems + (int64_t)(k % page_size) * D;
        const int bytes = there ? 16 : 0;                         // (a key behind the last one is zero-filled)
        constexpr int KC = D / 8;
#pragma unroll 4
        for (int c = 0; c < KC / 2; ++c) {
            const int chunk = copy_half * (KC / 2) + c;
            cp_async16(stage + copy_row * KS + chunk * 16, kp + chunk * 8, bytes);
        }
    };
    // the sixteen heads' queries (heads the model does not have are rows of zeros)
    for (int index = tid; index < 16 * (D / 8); index += 128) {
        const int h = index / (D / 8), chunk = index % (D / 8);
        const bool there = head0 + h < heads;
        const bf16* src = q + (int64_t)row * q_stride + (int64_t)(there ? head0 + h : head0) * D + chunk * 8;
        cp_async16(base + L::Q_AT + h * KS + chunk * 16, src, there ? 16 : 0);
    }
    if (tile_first < tile_end) fill(tile_first);
    cp_async_commit();

    float m[2] = {-1.0e30f, -1.0e30f}, l[2] = {0.0f, 0.0f};
    float o[COLS / 8][4];
#pragma unroll
    for (int j = 0; j < COLS / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[j][e] = 0.0f;

    for (int tile = tile_first; tile < tile_end; ++tile) {
        if (tile + 1 < tile_end) {
            fill(tile + 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                                          // this tile's keys (and the queries) are in shared memory
        const uint32_t stage = base + (uint32_t)(tile & 1) * L::STAGE;
        const int key0 = key_lo + tile * KT + warp * 16;          // the warp's 16 keys of the tile
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) s[j][e] = 0.0f;
        if (key0 <= pos) {
#pragma unroll 4
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4], b[4];
                ldmatrix_x4(a, base + L::Q_AT + (lane & 15) * KS + (ks * 2 + (lane >> 4)) * 16);
                ldmatrix_x4(b, stage + (warp * 16 + (lane & 7) + ((lane >> 4) << 3)) * KS + (ks * 2 + ((lane >> 3) & 1)) * 16);
                mma_bf16_16816(s[0], a, b);
                mma_bf16_16816(s[1], a, b + 2);
            }
        }
        float top[2] = {-1.0e30f, -1.0e30f};
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int key = key0 + j * 8 + 2 * t + (e & 1);
                s[j][e] = key <= pos ? s[j][e] * scale : -1.0e30f;       // (every key from key_lo on is inside the mask)
                top[e >> 1] = fmaxf(top[e >> 1], s[j][e]);
            }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 1));
            top[r] = fmaxf(top[r], __shfl_xor_sync(0xffffffffu, top[r], 2));
            if (t == 0) stats[warp * 16 + g + r * 8] = top[r];
        }
        __syncthreads();                                          // the four warps' maxima of the tile
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float all = stats[g + r * 8];
#pragma unroll
            for (int w = 1; w < 4; ++w) all = fmaxf(all, stats[w * 16 + g + r * 8]);
            const float m_new = fmaxf(m[r], all);
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
                l[e >> 1] += p;                                   // (a warp sums the weights of its own keys)
            }
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                uint32_t hi, lo;
                split_bf16(s[j][2 * r], s[j][2 * r + 1], hi, lo);
                const uint32_t at = (g + r * 8) * PS + (warp * 16 + j * 8 + 2 * t) * 2;
                *reinterpret_cast<uint32_t*>(smem + L::P_AT + at) = hi;
                *reinterpret_cast<uint32_t*>(smem + L::P_AT + 16 * PS + at) = lo;
            }
#pragma unroll
        for (int j = 0; j < COLS / 8; ++j) {
            o[j][0] *= corr[0]; o[j][1] *= corr[0];
            o[j][2] *= corr[1]; o[j][3] *= corr[1];
        }
        __syncthreads();                                          // all 64 keys' weights are in shared memory
#pragma unroll
        for (int kk = 0; kk < KT / 16; ++kk) {
            if (key_lo + tile * KT + kk * 16 > pos) break;        // (keys behind the row's position: weights of zero)
            uint32_t hi[4], lo[4];
            const uint32_t p_at = base + L::P_AT + (lane & 15) * PS + (kk * 2 + (lane >> 4)) * 16;
            ldmatrix_x4(hi, p_at);
            ldmatrix_x4(lo, p_at + 16 * PS);
#pragma unroll
            for (int jp = 0; jp < COLS / 16; ++jp) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, stage + (kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3)) * KS +
                                         (warp * (COLS / 8) + jp * 2 + (lane >> 4)) * 16);
                mma_bf16_16816(o[2 * jp], hi, b);
                mma_bf16_16816(o[2 * jp], lo, b);
                mma_bf16_16816(o[2 * jp + 1], hi, b + 2);
                mma_bf16_16816(o[2 * jp + 1], lo, b + 2);
            }
        }
        __syncthreads();                                          // the stage and the weights may be written again
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
        if (t == 0) stats[warp * 16 + g + r * 8] = l[r];
    }
    __syncthreads();
    if (parts != nullptr) {                                       // this run's share: accumulator, maximum and sum
        cp_async_wait<0>();                                       // (a block without tiles still waits for its queries' copy)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int head = head0 + g + r * 8;
            if (head >= heads) continue;
            float* mine = parts + (((int64_t)row * gridDim.z + blockIdx.z) * heads + head) * (DV + 2);
#pragma unroll
            for (int j = 0; j < COLS / 8; ++j)
                *reinterpret_cast<float2*>(mine + warp * COLS + j * 8 + 2 * t) = make_float2(o[j][2 * r], o[j][2 * r + 1]);
            if (warp == 0 && t == 0) {
                float total = 0.0f;
#pragma unroll
                for (int w = 0; w < 4; ++w) total += stats[w * 16 + g + r * 8];
                mine[DV] = m[r];
                mine[DV + 1] = total;
            }
        }
        return;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int head = head0 + g + r * 8;
        if (head >= heads) continue;
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) total += stats[w * 16 + g + r * 8];
        const float inv = 1.0f / fmaxf(total, 1.0e-30f);
        bf16* orow = out + (int64_t)row * out_stride + (int64_t)head * DV + warp * COLS;
#pragma unroll
        for (int j = 0; j < COLS / 8; ++j)
            *reinterpret_cast<uint32_t*>(orow + j * 8 + 2 * t) = pack_bf16(o[j][2 * r] * inv, o[j][2 * r + 1] * inv);
    }
}

// The runs of a row and head, added in order: out = sum_z o_z e^(m_z - M) / sum_z l_z e^(m_z - M), M the largest m_z.
template <int DV>
__global__ void __launch_bounds__(128)
latent_merge_kernel(const float* __restrict__ parts, bf16* __restrict__ out, int64_t out_stride, int heads, int splits) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x, head = blockIdx.y;
    const float* mine = parts + ((int64_t)row * splits * heads + head) * (DV + 2);
    const int64_t step = (int64_t)heads * (DV + 2);
    float top = -1.0e30f;
    for (int z = 0; z < splits; ++z) top = fmaxf(top, mine[z * step + DV]);
    float total = 0.0f;
    for (int z = 0; z < splits; ++z) total = fmaf(mine[z * step + DV + 1], __expf(mine[z * step + DV] - top), total);
    const float inv = 1.0f / fmaxf(total, 1.0e-30f);
    for (int col = threadIdx.x; col < DV; col += 128) {
        float value = 0.0f;
        for (int z = 0; z < splits; ++z) value = fmaf(mine[z * step + col], __expf(mine[z * step + DV] - top), value);
        out[(int64_t)row * out_stride + (int64_t)head * DV + col] = __float2bfloat16_rn(value * inv);
    }
}

// Blocks a row in a step of `rows` rows: one where the rows alone fill the GPU, else as many runs of key tiles as bring
// the grid to about two blocks a multiprocessor (at most 16).
int splits_for(int rows, int heads) {
    const int blocks = rows * ((heads + 15) / 16);
    if (blocks >= 148) return 1;
    const int splits = 296 / blocks;
    return splits > 16 ? 16 : (splits < 1 ? 1 : splits);
}

template <int D, int DV>
int launch(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache, const int* positions,
           const int* seq_of_row, const int* block_table, int bt_stride, int rows, int heads, int page_size, int mask_kind,
           int mask_size, float scale, float* parts, cudaStream_t stream) {
    constexpr int smem = Layout<D, DV>::BYTES;
    auto kernel = attention_latent_kernel<D, DV>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return (int)err;
    const int splits = splits_for(rows, heads);
    if (splits > 1 && parts == nullptr) return TB_ERR_BAD_SIZE;
    cudaError_t launched = tb_launch_pdl(kernel, dim3(rows, (heads + 15) / 16, splits), dim3(128), (size_t)smem, stream,
                                         (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)cache, positions,
                                         seq_of_row, block_table, bt_stride, heads, page_size, mask_kind, mask_size, scale,
                                         splits > 1 ? parts : (float*)nullptr);
    if (launched != cudaSuccess) return (int)launched;
    if (splits > 1) {
        launched = tb_launch_pdl(latent_merge_kernel<DV>, dim3(rows, heads), dim3(128), (size_t)0, stream, (const float*)parts,
                                 (bf16*)out, out_stride, heads, splits);
        if (launched != cudaSuccess) return (int)launched;
    }
    return tb_launch_status();
}

}  // namespace

// Whether tb_attention_latent_mma takes a cached vector of `dim` numbers whose first `vdim` are its value.
TB_EXPORT int tb_attention_latent_mma_supported(int dim, int vdim) {
    return (dim == 576 && vdim == 512) || (dim == 288 && vdim == 256) || (dim == 160 && vdim == 128) ? 1 : 0;
}

// Blocks a row of a step of `rows` rows (1: no scratch is needed).
TB_EXPORT int tb_attention_latent_mma_splits(int rows, int heads) {
    return rows < 1 || heads < 1 ? 1 : splits_for(rows, heads);
}

// q: bfloat16 [rows, heads * dim] (row stride q_stride, elements); out: bfloat16 [rows, heads * vdim]; cache: this
// layer's pages ([page_size][dim] a page); positions, seq_of_row: int32 [rows]; mask_kind: 0 causal, 1 window; parts:
// float32 [rows, splits, heads, vdim + 2] of scratch where tb_attention_latent_mma_splits says more than 1.
TB_EXPORT int tb_attention_latent_mma(const void* q, int64_t q_stride, void* out, int64_t out_stride, const void* cache,
                                      const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
                                      int rows, int heads, int dim, int vdim, int page_size, int mask_kind, int mask_size,
                                      float scale, float* parts, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (!tb_attention_latent_mma_supported(dim, vdim)) return TB_ERR_BAD_SIZE;
    if (heads < 1 || (heads + 15) / 16 > 65535 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (mask_kind < MASK_CAUSAL || mask_kind > MASK_WINDOW) return TB_ERR_BAD_SIZE;
    if (mask_kind == MASK_WINDOW && mask_size < 1) return TB_ERR_BAD_SIZE;
    if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)cache) % 16 != 0 || q_stride % 8 != 0 || out_stride % 2 != 0)
        return TB_ERR_BAD_ALIGN;
#define TB_ATTEND(D, DV)                                                                                             \
    return launch<D, DV>(q, q_stride, out, out_stride, cache, positions, seq_of_row, block_table, bt_stride, rows,   \
                         heads, page_size, mask_kind, mask_size, scale, parts, stream)
    if (dim == 576) TB_ATTEND(576, 512);
    if (dim == 288) TB_ATTEND(288, 256);
    TB_ATTEND(160, 128);
#undef TB_ATTEND
}
