// A feed-forward made of many small experts of which every row takes a few: the router, the grouping of rows by
// expert, the experts' products, and the weighted sum.
//
//   tb_choose_topk     from the router's 32-bit logits (a product kernel left them): the `top` largest of a row,
//                      largest first (the lowest index wins a tie), and the softmax over those alone.
//   tb_choose_grouped  the softmax over all of a row's logits; the experts form `groups` equal runs of neighbours, a
//                      group counts as much as its best expert, only experts of the `keep` best groups can be chosen;
//                      of those the `top` with the largest scores, largest first (the lowest index wins a tie), weighted
//                      by their scores over the chosen scores' sum (+ 1e-20), times `weight_scale`.
//   tb_expert_plan     rows * top assignments (row t, slot s -> assignment t * top + s) are grouped by their expert:
//                      offsets[e] .. offsets[e + 1] of `order` name the assignments of expert e.
//   tb_expert_linear   out[a, :] = act(W[expert(a)] in[source(a), :]) for every assignment a, a tile of one expert's
//                      assignments per block; source(a) is a / top (the row itself: the first product of an expert)
//                      or a (the second).  Every output number is one chain over K that does not depend on which
//                      other assignments share its tile.
//   tb_expert_combine  out[t, :] = [base[t, :] +] sum_s weight[t, s] * y[t * top + s, :], slots in order, 32-bit.
//
// Nothing here needs the host to know how many rows an expert received: grids are sized for the worst case and
// blocks without work leave at once, so a step's launches depend on its row count alone.
#include "common.cuh"


namespace {

// ----------------------------------------------------------------------------- router

constexpr int kRouteWarps = 4;

// The `top` largest of a row's logits `z` (the warp's own copy in shared memory, consumed here), largest first, the
// lowest index winning a tie, and the softmax over those alone.
__device__ __forceinline__ void choose_top(float* z, int experts, int top, int* __restrict__ ids,
                                           float* __restrict__ weights, int lane) {
    float first = 0.0f, total = 0.0f;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int where = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = z[e];
            if (v > best) { best = v; where = e; }              // (ascending e: the lowest index of equal values stays)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, where, o);
            if (ob > best || (ob == best && ow < where)) { best = ob; where = ow; }
        }
        if (where == 0x7fffffff) where = 0;                      // (only if every logit is NaN or -inf)
        if (s == 0) first = best;
        const float p = expf(best - first);
        total += p;
        if (lane == 0) {
            ids[s] = where;
            weights[s] = p;
            z[where] = -INFINITY;
        }
        __syncwarp();
    }
    const float inv = 1.0f / total;
    for (int s = lane; s < top; s += 32) weights[s] *= inv;      // (lane 0's stores above are visible: same warp, synced)
}

// A warp a row; logits 32-bit [rows, experts].
__global__ void __launch_bounds__(kRouteWarps * 32)
choose_topk_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights, int rows,
                   int experts, int top) {
    extern __shared__ __align__(16) float route_smem[];          // per warp: its row's logits
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kRouteWarps + warp;
    if (row >= rows) return;
    float* zs = route_smem + (size_t)warp * experts;
    for (int e = lane; e < experts; e += 32) zs[e] = logits[(int64_t)row * experts + e];
    __syncwarp();
    choose_top(zs, experts, top, ids + (int64_t)row * top, weights + (int64_t)row * top, lane);
}


// A warp a row; logits 32-bit [rows, experts].  Shared memory per warp: the row's scores, then one flag per group.
__global__ void __launch_bounds__(kRouteWarps * 32)
choose_grouped_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ weights, int rows,
                      int experts, int top, int groups, int keep, float weight_scale) {
    extern __shared__ __align__(16) float route_smem[];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * kRouteWarps + warp;
    if (row >= rows) return;
    float* zs = route_smem + (size_t)warp * (experts + groups);
    float* best_of = zs + experts;                               // a group's best score; -inf once the group is kept
    const int per = experts / groups;
    float top_logit = -INFINITY;
    for (int e = lane; e < experts; e += 32) top_logit = fmaxf(top_logit, logits[(int64_t)row * experts + e]);
    top_logit = warp_max(top_logit);
    float total = 0.0f;
    for (int e = lane; e < experts; e += 32) {
        const float p = expf(logits[(int64_t)row * experts + e] - top_logit);
        zs[e] = p;
        total += p;
    }
    total = warp_sum(total);
    __syncwarp();
    const float inv_total = 1.0f / total;
    for (int e = lane; e < experts; e += 32) zs[e] *= inv_total;
    __syncwarp();
    for (int g = lane; g < groups; g += 32) {
        float best = -INFINITY;
        for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, zs[e]);
        best_of[g] = best;
    }
    __syncwarp();
    // the `keep` best groups, one after the other (the lowest index among equals); the experts of all others leave
    for (int k = 0; k < keep; ++k) {
        float best = -INFINITY;
        int where = 0x7fffffff;
        for (int g = lane; g < groups; g += 32) {
            const float v = best_of[g];
            if (v > best) { best = v; where = g; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, where, o);
            if (ob > best || (ob == best && ow < where)) { best = ob; where = ow; }
        }
        if (lane == 0 && where != 0x7fffffff) best_of[where] = -INFINITY;
        __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
        if (best_of[e / per] != -INFINITY) zs[e] = -INFINITY;       // (a kept group's entry was set to -inf above)
    __syncwarp();
    int* my_ids = ids + (int64_t)row * top;
    float* my_weights = weights + (int64_t)row * top;
    float chosen_sum = 0.0f;
    for (int s = 0; s < top; ++s) {
        float best = -INFINITY;
        int where = 0x7fffffff;
        for (int e = lane; e < experts; e += 32) {
            const float v = zs[e];
            if (v > best) { best = v; where = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int ow = __shfl_xor_sync(0xffffffffu, where, o);
            if (ob > best || (ob == best && ow < where)) { best = ob; where = ow; }
        }
        if (where == 0x7fffffff) { where = 0; best = 0.0f; }     // (fewer allowed experts than `top`, or NaN logits)
        chosen_sum += best;
        if (lane == 0) {
            my_ids[s] = where;
            my_weights[s] = best;
            zs[where] = -INFINITY;
        }
        __syncwarp();
    }
    const float factor = weight_scale / (chosen_sum + 1e-20f);
    for (int s = lane; s < top; s += 32) my_weights[s] *= factor;
}

// ----------------------------------------------------------------------------- grouping

__global__ void __launch_bounds__(1024)
expert_plan_kernel(const int* __restrict__ ids, int assignments, int experts, int* __restrict__ offsets,
                   int* __restrict__ order) {
    extern __shared__ int plan_smem[];                           // counts[experts], cursor[experts]
    pdl_trigger();
    pdl_wait();
    int* counts = plan_smem;
    int* cursor = plan_smem + experts;
    for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
        const int e = ids[a];
        if (e >= 0 && e < experts) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < experts; ++e) {
            offsets[e] = run;
            cursor[e] = run;
            run += counts[e];
        }
        offsets[experts] = run;
    }
    __syncthreads();
    // (which of an expert's assignments comes first is left to the atomics: no result depends on it)
    for (int a = threadIdx.x; a < assignments; a += blockDim.x) {
        const int e = ids[a];
        if (e >= 0 && e < experts) order[atomicAdd(&cursor[e], 1)] = a;
    }
}

// ----------------------------------------------------------------------------- the experts' products

enum ExpertEpilogue : int { EXP_PLAIN = 0, EXP_SQUARED_RELU = 1 };

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// The tile of this block: which expert, and the first of its assignments.  Returns false when the block has none.
__device__ __forceinline__ bool find_tile(const int* __restrict__ offsets, int experts, int tile, int tile_rows,
                                          int& expert, int& first, int& count) {
    for (int e = 0; e < experts; ++e) {
        const int begin = offsets[e], n = offsets[e + 1] - begin;
        const int tiles = (n + tile_rows - 1) / tile_rows;
        if (tile < tiles) {
            expert = e;
            first = begin + tile * tile_rows;
            count = min(tile_rows, n - tile * tile_rows);
            return true;
        }
        tile -= tiles;
    }
    return false;
}

// Plain multiply-adds, operands widened to 32-bit: the true 32-bit product, and the fallback for sizes the tensor-core
// kernel does not take.  Every output element is one K-ordered chain k = 0, 1, ..., K - 1.
template <typename T, typename O, int EPI>
__global__ void __launch_bounds__(256)
expert_linear_kernel(const T* __restrict__ in, int64_t in_stride, const T* __restrict__ W, O* __restrict__ out,
                     int64_t out_stride, const int* __restrict__ offsets, const int* __restrict__ order, int experts,
                     int top_div, int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    __shared__ int rows_of[BM];
    pdl_trigger();
    pdl_wait();
    int expert, first, count;
    if (!find_tile(offsets, experts, blockIdx.y, BM, expert, first, count)) return;
    const int tid = threadIdx.x;
    if (tid < BM) rows_of[tid] = tid < count ? order[first + tid] : -1;
    __syncthreads();
    const T* We = W + (int64_t)expert * N * K;
    const int n0 = blockIdx.x * BN;
    const int tx = tid % 16, ty = tid / 16;
    const int load_row = tid / 4;
    const int load_k = (tid % 4) * 4;
    const int a_assign = rows_of[load_row];
    const T* a_src = a_assign < 0 ? nullptr : in + (int64_t)(a_assign / top_div) * in_stride;
    const int wn = n0 + load_row;

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
        const int kk = k0 + load_k;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (a_src != nullptr && kk + e < K) a[e] = Elem<T>::load(a_src + kk + e);
            if (wn < N && kk + e < K) w[e] = Elem<T>::load(We + (int64_t)wn * K + kk + e);
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            As[load_k + e][load_row] = a[e];
            Ws[load_k + e][load_row] = w[e];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float ar[TM], wr[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ar[i] = As[k][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wr[j] = Ws[k][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int a = rows_of[ty * TM + i];
        if (a < 0) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (EPI == EXP_SQUARED_RELU) {
                v = fmaxf(v, 0.0f);
                v *= v;
            }
            Elem<O>::store(out + (int64_t)a * out_stride + n, v);
        }
    }
}

// bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulators): a block is 64 assignments of one expert by
// 64 features, a warp 16 assignments by 64 features; K in steps of 32 through shared memory.  K a multiple of 32.
constexpr int MK = 32, MPAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, const uint32_t* b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <typename O, int EPI>
__global__ void __launch_bounds__(128)
expert_linear_mma_kernel(const __nv_bfloat16* __restrict__ in, int64_t in_stride, const __nv_bfloat16* __restrict__ W,
                         O* __restrict__ out, int64_t out_stride, const int* __restrict__ offsets,
                         const int* __restrict__ order, int experts, int top_div, int N, int K) {
    __shared__ __align__(16) __nv_bfloat16 As[BM][MK + MPAD];
    __shared__ __align__(16) __nv_bfloat16 Ws[BN][MK + MPAD];
    __shared__ int rows_of[BM];
    pdl_trigger();
    pdl_wait();
    int expert, first, count;
    if (!find_tile(offsets, experts, blockIdx.y, BM, expert, first, count)) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < BM) rows_of[tid] = tid < count ? order[first + tid] : -1;
    __syncthreads();
    const __nv_bfloat16* We = W + (int64_t)expert * N * K;
    const int n0 = blockIdx.x * BN;
    // loads: 64 rows x 32 elements = 256 packets of 8; a thread two packets of A and two of W
    const int g = lane >> 2, t = lane & 3;
    float acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.0f;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int k0 = 0; k0 < K; k0 += MK) {
        uint4 av[2], wv[2];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int packet = tid + p * 128;
            const int r = packet >> 2, c = (packet & 3) * 8;
            const int a = rows_of[r];
            av[p] = a < 0 ? zero : *reinterpret_cast<const uint4*>(in + (int64_t)(a / top_div) * in_stride + k0 + c);
            const int n = n0 + r;
            wv[p] = n < N ? *reinterpret_cast<const uint4*>(We + (int64_t)n * K + k0 + c) : zero;
        }
        __syncthreads();
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            const int packet = tid + p * 128;
            const int r = packet >> 2, c = (packet & 3) * 8;
            *reinterpret_cast<uint4*>(&As[r][c]) = av[p];
            *reinterpret_cast<uint4*>(&Ws[r][c]) = wv[p];
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < MK; ks += 16) {
            uint32_t a[4];
            const int r = warp * 16 + g;
            a[0] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * t]);
            a[1] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * t]);
            a[2] = *reinterpret_cast<const uint32_t*>(&As[r][ks + 2 * t + 8]);
            a[3] = *reinterpret_cast<const uint32_t*>(&As[r + 8][ks + 2 * t + 8]);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t b[2];
                b[0] = *reinterpret_cast<const uint32_t*>(&Ws[j * 8 + g][ks + 2 * t]);
                b[1] = *reinterpret_cast<const uint32_t*>(&Ws[j * 8 + g][ks + 2 * t + 8]);
                mma_bf16_16816(acc[j], a, b);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int a = rows_of[warp * 16 + g + half * 8];
        if (a < 0) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int n = n0 + j * 8 + 2 * t + e;
                if (n >= N) continue;
                float v = acc[j][half * 2 + e];
                if (EPI == EXP_SQUARED_RELU) {
                    v = fmaxf(v, 0.0f);
                    v *= v;
                }
                Elem<O>::store(out + (int64_t)a * out_stride + n, v);
            }
        }
    }
}

// The same product for K a multiple of 64: a block of eight warps takes 64 assignments by 128 features (a warp 32 by
// 32); K runs in steps of 64 through a ring of three stages that cp.async fills two steps ahead (rows of absent
// assignments and features are zero-filled), fragments come from shared memory by ldmatrix, 16-byte chunks of a row
// XOR-swizzled by the row so that neither the copies nor ldmatrix meet bank conflicts.
constexpr int PM = 64, PN = 128, PK = 64, PSTAGES = 3;
constexpr int kPipeSmem = PSTAGES * (PM + PN) * PK * 2;

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
// byte offset of 16-byte chunk `chunk` (0..7) of row `row` in a tile whose rows are 128 bytes
__device__ __forceinline__ uint32_t swizzled(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

template <typename O, int EPI>
__global__ void __launch_bounds__(256)
expert_linear_pipe_kernel(const __nv_bfloat16* __restrict__ in, int64_t in_stride, const __nv_bfloat16* __restrict__ W,
                          O* __restrict__ out, int64_t out_stride, const int* __restrict__ offsets,
                          const int* __restrict__ order, int experts, int top_div, int N, int K) {
    extern __shared__ __align__(128) unsigned char pipe_smem[];
    __shared__ int rows_of[PM];
    pdl_trigger();
    pdl_wait();
    int expert, first, count;
    if (!find_tile(offsets, experts, blockIdx.y, PM, expert, first, count)) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid < PM) rows_of[tid] = tid < count ? order[first + tid] : -1;
    __syncthreads();
    const __nv_bfloat16* We = W + (int64_t)expert * N * K;
    const int n0 = blockIdx.x * PN;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(pipe_smem);
    // what this thread copies every step: two chunks of A (64 rows x 8 chunks) and four of W (128 rows x 8 chunks)
    const __nv_bfloat16* a_src[2];
    uint32_t a_dst[2];
    int a_bytes[2];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int c = tid + p * 256, r = c >> 3, chunk = c & 7;
        const int a = rows_of[r];
        a_bytes[p] = a < 0 ? 0 : 16;
        a_src[p] = in + (a < 0 ? 0 : (int64_t)(a / top_div) * in_stride) + chunk * 8;
        a_dst[p] = swizzled(r, chunk);
    }
    const __nv_bfloat16* w_src[4];
    uint32_t w_dst[4];
    int w_bytes[4];
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const int c = tid + p * 256, r = c >> 3, chunk = c & 7;
        const int n = n0 + r;
        w_bytes[p] = n < N ? 16 : 0;
        w_src[p] = We + (n < N ? (int64_t)n * K : 0) + chunk * 8;
        w_dst[p] = PM * 128 + swizzled(r, chunk);
    }
    const int steps = K / PK;
    auto fill = [&](int step) {
        const uint32_t stage = base + (uint32_t)(step % PSTAGES) * (PM + PN) * 128;
        const int k0 = step * PK;
#pragma unroll
        for (int p = 0; p < 2; ++p) cp_async16(stage + a_dst[p], a_src[p] + k0, a_bytes[p]);
#pragma unroll
        for (int p = 0; p < 4; ++p) cp_async16(stage + w_dst[p], w_src[p] + k0, w_bytes[p]);
    };
    for (int s = 0; s < PSTAGES - 1; ++s) {
        if (s < steps) fill(s);
        cp_async_commit();
    }
    const int wm = warp >> 2, wn = warp & 3;          // the warp's 32 x 32 part of the tile
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
    for (int step = 0; step < steps; ++step) {
        cp_async_wait<PSTAGES - 2>();
        __syncthreads();                               // the stage is complete, and the stage filled next is free
        if (step + PSTAGES - 1 < steps) fill(step + PSTAGES - 1);
        cp_async_commit();
        const uint32_t stage = base + (uint32_t)(step % PSTAGES) * (PM + PN) * 128;
#pragma unroll
        for (int ks = 0; ks < PK / 16; ++ks) {
            uint32_t a[2][4], b[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i)
                ldmatrix_x4(a[i], stage + swizzled(wm * 32 + i * 16 + (lane & 15), ks * 2 + (lane >> 4)));
#pragma unroll
            for (int j = 0; j < 2; ++j)                // two n-tiles of eight features a load
                ldmatrix_x4(b[j], stage + PM * 128 +
                                      swizzled(wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], &b[j >> 1][(j & 1) * 2]);
        }
    }
    cp_async_wait<0>();
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int a = rows_of[wm * 32 + i * 16 + g + half * 8];
            if (a < 0) continue;
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = n0 + wn * 32 + j * 8 + 2 * t + e;
                    if (n >= N) continue;
                    float v = acc[i][j][half * 2 + e];
                    if (EPI == EXP_SQUARED_RELU) {
                        v = fmaxf(v, 0.0f);
                        v *= v;
                    }
                    Elem<O>::store(out + (int64_t)a * out_stride + n, v);
                }
        }
}

// ----------------------------------------------------------------------------- the weighted sum

__global__ void expert_combine_kernel(const float* __restrict__ y, const float* __restrict__ weights,
                                      const float* __restrict__ base, float* __restrict__ out, int width, int top) {
    pdl_trigger();
    pdl_wait();
    const int64_t row = blockIdx.x;
    const float* w = weights + row * top;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < width; j += gridDim.y * blockDim.x) {
        float sum = 0.0f;
        for (int s = 0; s < top; ++s) sum = fmaf(w[s], y[(row * top + s) * width + j], sum);
        if (base != nullptr) sum += base[row * width + j];
        out[row * width + j] = sum;
    }
}

template <typename T, typename O>
int launch_linear(const void* in, int64_t in_stride, const void* W, void* out, int64_t out_stride, const int* offsets,
                  const int* order, int assignments, int experts, int top_div, int N, int K, int epilogue,
                  cudaStream_t stream) {
    const dim3 grid((N + BN - 1) / BN, (assignments + BM - 1) / BM + experts);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (epilogue == EXP_SQUARED_RELU)
        launched = tb_launch_pdl(expert_linear_kernel<T, O, EXP_SQUARED_RELU>, grid, dim3(256), 0, stream, (const T*)in,
                                 in_stride, (const T*)W, (O*)out, out_stride, offsets, order, experts, top_div, N, K);
    else
        launched = tb_launch_pdl(expert_linear_kernel<T, O, EXP_PLAIN>, grid, dim3(256), 0, stream, (const T*)in,
                                 in_stride, (const T*)W, (O*)out, out_stride, offsets, order, experts, top_div, N, K);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename O, int EPI>
int launch_linear_pipe(const void* in, int64_t in_stride, const void* W, void* out, int64_t out_stride,
                       const int* offsets, const int* order, int assignments, int experts, int top_div, int N, int K,
                       cudaStream_t stream) {
    const dim3 grid((N + PN - 1) / PN, (assignments + PM - 1) / PM + experts);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    auto kernel = expert_linear_pipe_kernel<O, EPI>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPipeSmem);
    if (err != cudaSuccess) return (int)err;
    cudaError_t launched = tb_launch_pdl(kernel, grid, dim3(256), (size_t)kPipeSmem, stream, (const __nv_bfloat16*)in,
                                         in_stride, (const __nv_bfloat16*)W, (O*)out, out_stride, offsets, order,
                                         experts, top_div, N, K);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename O>
int launch_linear_mma(const void* in, int64_t in_stride, const void* W, void* out, int64_t out_stride,
                      const int* offsets, const int* order, int assignments, int experts, int top_div, int N, int K,
                      int epilogue, cudaStream_t stream) {
    if (K % PK == 0)
        return epilogue == EXP_SQUARED_RELU
                   ? launch_linear_pipe<O, EXP_SQUARED_RELU>(in, in_stride, W, out, out_stride, offsets, order, assignments,
                                                             experts, top_div, N, K, stream)
                   : launch_linear_pipe<O, EXP_PLAIN>(in, in_stride, W, out, out_stride, offsets, order, assignments,
                                                      experts, top_div, N, K, stream);
    const dim3 grid((N + BN - 1) / BN, (assignments + BM - 1) / BM + experts);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (epilogue == EXP_SQUARED_RELU)
        launched = tb_launch_pdl(expert_linear_mma_kernel<O, EXP_SQUARED_RELU>, grid, dim3(128), 0, stream,
                                 (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)W, (O*)out, out_stride,
                                 offsets, order, experts, top_div, N, K);
    else
        launched = tb_launch_pdl(expert_linear_mma_kernel<O, EXP_PLAIN>, grid, dim3(128), 0, stream,
                                 (const __nv_bfloat16*)in, in_stride, (const __nv_bfloat16*)W, (O*)out, out_stride,
                                 offsets, order, experts, top_div, N, K);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

}  // namespace

// logits: 32-bit [rows, experts], contiguous.
TB_EXPORT int tb_choose_topk(const float* logits, int* ids, float* weights, int rows, int experts, int top,
                             cudaStream_t stream) {
    if (rows == 0) return 0;
    if (experts < 1 || top < 1 || top > experts) return TB_ERR_BAD_SIZE;
    const size_t smem = (size_t)kRouteWarps * experts * sizeof(float);
    if (smem > 40 * 1024) return TB_ERR_BAD_SIZE;
    cudaError_t launched = tb_launch_pdl(choose_topk_kernel, dim3((rows + kRouteWarps - 1) / kRouteWarps),
                                         dim3(kRouteWarps * 32), smem, stream, logits, ids, weights, rows, experts, top);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// logits: 32-bit [rows, experts], contiguous; `groups` divides `experts`, keep <= groups, top <= keep * experts / groups.
TB_EXPORT int tb_choose_grouped(const float* logits, int* ids, float* weights, int rows, int experts, int top, int groups,
                                int keep, float weight_scale, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (experts < 1 || top < 1 || groups < 1 || experts % groups != 0 || keep < 1 || keep > groups) return TB_ERR_BAD_SIZE;
    if (top > keep * (experts / groups)) return TB_ERR_BAD_SIZE;
    const size_t smem = (size_t)kRouteWarps * (experts + groups) * sizeof(float);
    if (smem > 40 * 1024) return TB_ERR_BAD_SIZE;
    cudaError_t launched = tb_launch_pdl(choose_grouped_kernel, dim3((rows + kRouteWarps - 1) / kRouteWarps),
                                         dim3(kRouteWarps * 32), smem, stream, logits, ids, weights, rows, experts, top,
                                         groups, keep, weight_scale);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// ids: int32 [assignments]; offsets: int32 [experts + 1]; order: int32 [assignments].
TB_EXPORT int tb_expert_plan(const int* ids, int assignments, int experts, int* offsets, int* order,
                             cudaStream_t stream) {
    if (experts < 1 || experts > 8192 || assignments < 0) return TB_ERR_BAD_SIZE;
    cudaError_t launched = tb_launch_pdl(expert_plan_kernel, dim3(1), dim3(1024), (size_t)2 * experts * sizeof(int),
                                         stream, ids, assignments, experts, offsets, order);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// in: [*, K] of dtype (row stride in_stride); W: [experts, N, K] of dtype; out: [assignments, N] of out_dtype (row
// stride out_stride); top_div: the source row of assignment a is a / top_div.  epilogue: 0 plain, 1 squared ReLU.
// tensor_cores != 0 asks for the mma.sync kernels (bfloat16, K a multiple of 32, 16-byte aligned rows; the pipelined
// one where K is a multiple of 64); the entry point refuses it where it cannot run.
TB_EXPORT int tb_expert_linear(const void* in, int64_t in_stride, const void* W, void* out, int64_t out_stride,
                               const int* offsets, const int* order, int assignments, int experts, int top_div, int N,
                               int K, int epilogue, int dtype, int out_dtype, int tensor_cores, cudaStream_t stream) {
    if (assignments == 0 || N == 0) return 0;
    if (K < 1 || top_div < 1 || experts < 1) return TB_ERR_BAD_SIZE;
    if (epilogue != EXP_PLAIN && epilogue != EXP_SQUARED_RELU) return TB_ERR_BAD_SIZE;
    if (tensor_cores) {
        if (dtype != TB_BF16) return TB_ERR_BAD_DTYPE;
        if (K % MK != 0 || in_stride % 8 != 0 || ((uintptr_t)in | (uintptr_t)W) % 16 != 0) return TB_ERR_BAD_ALIGN;
        if (out_dtype == TB_F32)
            return launch_linear_mma<float>(in, in_stride, W, out, out_stride, offsets, order, assignments, experts,
                                            top_div, N, K, epilogue, stream);
        if (out_dtype == TB_BF16)
            return launch_linear_mma<__nv_bfloat16>(in, in_stride, W, out, out_stride, offsets, order, assignments,
                                                    experts, top_div, N, K, epilogue, stream);
        return TB_ERR_BAD_DTYPE;
    }
    if (dtype == TB_F32 && out_dtype == TB_F32)
        return launch_linear<float, float>(in, in_stride, W, out, out_stride, offsets, order, assignments, experts,
                                           top_div, N, K, epilogue, stream);
    if (dtype == TB_BF16 && out_dtype == TB_F32)
        return launch_linear<__nv_bfloat16, float>(in, in_stride, W, out, out_stride, offsets, order, assignments,
                                                   experts, top_div, N, K, epilogue, stream);
    if (dtype == TB_BF16 && out_dtype == TB_BF16)
        return launch_linear<__nv_bfloat16, __nv_bfloat16>(in, in_stride, W, out, out_stride, offsets, order,
                                                           assignments, experts, top_div, N, K, epilogue, stream);
    return TB_ERR_BAD_DTYPE;
}

// y: 32-bit [rows * top, width]; weights: 32-bit [rows, top]; base: null or 32-bit [rows, width]; out: 32-bit
// [rows, width] (may alias base).
TB_EXPORT int tb_expert_combine(const float* y, const float* weights, const float* base, float* out, int rows,
                                int width, int top, cudaStream_t stream) {
    if (rows == 0 || width == 0) return 0;
    if (top < 1) return TB_ERR_BAD_SIZE;
    int by = (width + 255) / 256;
    if (by > 32) by = 32;
    cudaError_t launched = tb_launch_pdl(expert_combine_kernel, dim3(rows, by), dim3(256), 0, stream, y, weights, base,
                                         out, width, top);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
