// Linear attention with a fixed decay per head:  S_t = a S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  (S: [dim, vdim], 32-bit,
// kept per request in its state slot), with q = silu(.), k = silu(.), v = silu(.) of the projected rows, or, for a
// mixer that rotates its queries and keys (retention), of rows that tb_retention_prepare left in 32-bit:
//
//   tb_retention_prepare   q and k heads turned in the rotate-half layout by position * inv_freq[i] (32-bit angle,
//                          sincosf), k times k_scale, v copied; everything widened to 32-bit
//   tb_head_norm_gate      o / sqrt(mean(o^2) + eps) per head (no weight), times silu or sigmoid of a gate row
//
// A block takes one (sequence, head, slice of 32 value columns) and walks the sequence's rows of this step in chunks of
// up to C rows.  With S the state at the chunk's start and rows 0 .. c-1 of the chunk,
//
//   A[t][s] = (q_t . k_s) a^(t-s)                       s <= t          (scores, 32-bit)
//   o_t     = a^(t+1) (S^T q_t) + sum_(s<=t) A[t][s] v_s
//   S'      = a^c S + sum_s a^(c-1-s) k_s v_s^T
//
// so that only non-negative powers of the decay appear (taken in 64-bit, once a block).  A step of single rows is
// the chunk c = 1.  The order of the sums depends on where a step's rows start, so cutting a prompt differently moves
// the result by rounding only.  q, k, v, the scores and the state are 32-bit inside the kernel whatever the run dtype.
// A step of single rows has a kernel of its own that keeps no copy of the state in shared memory.
//
// A step with long prompt portions takes three launches instead, so that the chunks of a sequence run side by side:
// a tile is one chunk of one sequence (which block takes which follows from row_start alone);
//   1. every tile's own sum  U = sum_s a^(c-1-s) k_s v_s^T                       (a block a tile, head and slice)
//   2. per sequence, head and slice, the tiles in order:  S_0 = state,  S_(i+1) = a^(c_i) S_i + U_i ; every S_i is kept
//      where U_i was, the last one goes back to the state slot
//   3. every tile's outputs from its S_i and its own rows, as above.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kSlice = 32;          // value columns a block owns
constexpr int kRows = 8;            // rows (or key dimensions) a warp carries in registers at a time
static_assert(kRows == 8, "the vector forms below are written for eight");

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

// What q, k and v go through before the recurrence: ACT_SILU, or ACT_NONE for rows that a kernel in front prepared.
enum RowActivation : int { ACT_NONE = 0, ACT_SILU = 1 };
__device__ __forceinline__ float activate(float z, int act) { return act == ACT_SILU ? silu(z) : z; }

// Floats of a query or key row in shared memory.  Where dim is a multiple of four, rows start on 16 bytes and are read
// four numbers at a time (the padding of four keeps a quarter-warp's rows on different banks); otherwise a number at a time.
__host__ __device__ __forceinline__ int row_floats(int dim) { return dim % 4 == 0 ? dim + 4 : dim + 1; }

// sum += a[0 .. n) . b[0 .. n), the products added in order
__device__ __forceinline__ float dot_in_order(const float* a, const float* b, int n, bool vec, float sum) {
    if (vec) {
        for (int i = 0; i < n; i += 4) {
            const float4 x = *reinterpret_cast<const float4*>(a + i), y = *reinterpret_cast<const float4*>(b + i);
            sum = fmaf(x.x, y.x, sum); sum = fmaf(x.y, y.y, sum); sum = fmaf(x.z, y.z, sum); sum = fmaf(x.w, y.w, sum);
        }
    } else {
        for (int i = 0; i < n; ++i) sum = fmaf(a[i], b[i], sum);
    }
    return sum;
}

// dst[t][0 .. n) = act(src[t][0 .. valid)) and zeros behind, for c rows (src rows `stride` elements apart, dst rows
// `dst_stride` floats): with PACKETS 16 bytes of the source at a time where its rows allow it, else an element at a time.
template <typename T, bool PACKETS>
__device__ __forceinline__ void load_silu_rows(float* dst, int dst_stride, const T* src, int64_t stride, int c, int n,
                                               int valid, int act) {
    constexpr int N = Packet<T>::N;
    if (PACKETS && n % N == 0 && valid % N == 0 && stride % N == 0 && (uintptr_t)src % 16 == 0) {
        const int packets = n / N;
        for (int e = threadIdx.x; e < c * packets; e += kThreads) {
            const int t = e / packets, i = (e % packets) * N;
            float v[N];
            if (i < valid) {
                Packet<T>::load(src + (int64_t)t * stride + i, v);
#pragma unroll
                for (int u = 0; u < N; ++u) v[u] = activate(v[u], act);
            } else {
#pragma unroll
                for (int u = 0; u < N; ++u) v[u] = 0.0f;
            }
#pragma unroll
            for (int u = 0; u < N; ++u) dst[t * dst_stride + i + u] = v[u];
        }
    } else {
        for (int e = threadIdx.x; e < c * n; e += kThreads) {
            const int t = e / n, i = e % n;
            dst[t * dst_stride + i] = i < valid ? activate(Elem<T>::load(src + (int64_t)t * stride + i), act) : 0.0f;
        }
    }
}

// The tile-th chunk of the step, counting every sequence's chunks in order: its sequence, first row and row count.
__device__ __forceinline__ bool find_tile(const int* row_start, int num_seqs, int chunk, int tile, int& seq, int& r0, int& n) {
    for (int s = 0; s < num_seqs; ++s) {
        const int begin = row_start[s], rows = row_start[s + 1] - begin;
        const int tiles = (rows + chunk - 1) / chunk;
        if (tile < tiles) {
            seq = s; r0 = begin + tile * chunk; n = min(chunk, rows - tile * chunk);
            return true;
        }
        tile -= tiles;
    }
    return false;
}

// tile_state == nullptr: a block walks all rows of its sequence (blockIdx.x) from the state slot and renews the slot.
// Otherwise blockIdx.x is a tile: its rows alone, from the state kept for it in tile_state; nothing is written back.
// WIDE: chunks of kRows rows or more (prompt portions), a warp carrying kRows rows or key dimensions in registers;
// otherwise (steps of few rows a sequence, decoded ones) a warp a row, which needs half the registers: twice the blocks
// stream their states side by side.
template <typename T, bool WIDE>
__global__ void __launch_bounds__(kThreads)
lightning_kernel(const T* __restrict__ proj, int64_t proj_stride, int q_off, int k_off, int v_off,
                 const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                 const int* __restrict__ row_start, const int* __restrict__ state_slots, int heads, int dim, int vdim,
                 int chunk, const float* __restrict__ tile_state, int num_seqs, int act) {
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    const int head = blockIdx.y, col0 = blockIdx.z * kSlice;
    const int cols = min(kSlice, vdim - col0);
    const int dpad = row_floats(dim);
    const bool vec = dim % 4 == 0;
    float* qs = smem;                              // [chunk][row_floats(dim)]
    float* ks = qs + chunk * dpad;                 // [chunk][row_floats(dim)]
    float* vs = ks + chunk * dpad;                 // [chunk][kSlice]
    float* A = vs + chunk * kSlice;                // [chunk][chunk]
    float* S = A + chunk * chunk;                  // [dim][kSlice]
    float* pw = S + dim * kSlice;                  // [chunk + 1]
    const float a = decay[head];
    for (int i = threadIdx.x; i <= chunk; i += kThreads) pw[i] = (float)pow((double)a, (double)i);
    pdl_wait();                                    // rows, state and the step's metadata come from kernels in front
    int seq = blockIdx.x, first, last;
    if (tile_state != nullptr) {
        int n;
        if (!find_tile(row_start, num_seqs, chunk, blockIdx.x, seq, first, n)) return;
        last = first + n;
    } else {
        first = row_start[seq];
        last = row_start[seq + 1];
    }
    if (first >= last) return;
    float* slot = tile_state != nullptr ? const_cast<float*>(tile_state) + ((int64_t)blockIdx.x * heads + head) * dim * vdim
                                        : state + ((int64_t)state_slots[seq] * heads + head) * dim * vdim;
    for (int e = threadIdx.x; e < dim * kSlice; e += kThreads) {
        const int i = e / kSlice, j = e % kSlice;
        S[e] = j < cols ? slot[(int64_t)i * vdim + col0 + j] : 0.0f;
    }
    const int lane = threadIdx.x & 31, group = threadIdx.x >> 5;          // kSlice == 32: a lane a value column
    for (int row0 = first; row0 < last; row0 += chunk) {
        const int c = min(chunk, last - row0);
        __syncthreads();                           // the chunk before is done with qs, ks, vs, A (and S is written)
        const T* rows_at = proj + (int64_t)row0 * proj_stride;
        load_silu_rows<T, WIDE>(qs, dpad, rows_at + q_off + (int64_t)head * dim, proj_stride, c, dim, dim, act);
        load_silu_rows<T, WIDE>(ks, dpad, rows_at + k_off + (int64_t)head * dim, proj_stride, c, dim, dim, act);
        load_silu_rows<T, WIDE>(vs, kSlice, rows_at + v_off + (int64_t)head * vdim + col0, proj_stride, c, kSlice, cols, act);
        __syncthreads();
        // scores of the chunk: thread e takes (t, s) with s fastest, so neighbouring lanes read neighbouring key rows
        for (int e = threadIdx.x; e < c * c; e += kThreads) {
            const int t = e / c, s = e % c;
            float dot = 0.0f;
            if (s <= t) {
                dot = dot_in_order(qs + t * dpad, ks + s * dpad, dim, vec, 0.0f) * pw[t - s];
            }
            A[t * chunk + s] = dot;
        }
        __syncthreads();
        // outputs: a warp takes kRows neighbouring rows at a time, a lane a value column, so that a number of the state or
        // of the values is read once for all of them
        for (int t = group; (!WIDE || c < kRows) && t < c; t += kThreads / 32) {       // few rows: a warp a row
            const float* qr = qs + t * dpad;
            float from_state = 0.0f;
            for (int i = 0; i < dim; ++i) from_state = fmaf(qr[i], S[i * kSlice + lane], from_state);
            float inside = 0.0f;
            for (int s = 0; s <= t; ++s) inside = fmaf(A[t * chunk + s], vs[s * kSlice + lane], inside);
            if (lane < cols)
                out[(int64_t)(row0 + t) * heads * vdim + (int64_t)head * vdim + col0 + lane] = fmaf(pw[t + 1], from_state, inside);
        }
        for (int t0 = group * kRows; WIDE && c >= kRows && t0 < c; t0 += (kThreads / 32) * kRows) {
            const float* qr[kRows];
            const float* ar[kRows];
            float from_state[kRows], inside[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int t = min(t0 + r, c - 1);
                qr[r] = qs + t * dpad;
                ar[r] = A + t * chunk;
                from_state[r] = 0.0f;
                inside[r] = 0.0f;
            }
            if (vec) {
                for (int i = 0; i < dim; i += 4) {
                    const float s0 = S[i * kSlice + lane], s1 = S[(i + 1) * kSlice + lane];
                    const float s2 = S[(i + 2) * kSlice + lane], s3 = S[(i + 3) * kSlice + lane];
#pragma unroll
                    for (int r = 0; r < kRows; ++r) {
                        const float4 qv = *reinterpret_cast<const float4*>(qr[r] + i);
                        from_state[r] = fmaf(qv.x, s0, from_state[r]); from_state[r] = fmaf(qv.y, s1, from_state[r]);
                        from_state[r] = fmaf(qv.z, s2, from_state[r]); from_state[r] = fmaf(qv.w, s3, from_state[r]);
                    }
                }
            } else {
                for (int i = 0; i < dim; ++i) {
                    const float sv = S[i * kSlice + lane];
#pragma unroll
                    for (int r = 0; r < kRows; ++r) from_state[r] = fmaf(qr[r][i], sv, from_state[r]);
                }
            }
            const int reach = min(t0 + kRows, c);                 // (a row's scores behind itself are zeros)
            int s = 0;
            for (; s + 4 <= reach; s += 4) {                      // (chunk is a multiple of four here: rows of A start on 16 bytes)
                const float v0 = vs[s * kSlice + lane], v1 = vs[(s + 1) * kSlice + lane];
                const float v2 = vs[(s + 2) * kSlice + lane], v3 = vs[(s + 3) * kSlice + lane];
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const float4 av = *reinterpret_cast<const float4*>(ar[r] + s);
                    inside[r] = fmaf(av.x, v0, inside[r]); inside[r] = fmaf(av.y, v1, inside[r]);
                    inside[r] = fmaf(av.z, v2, inside[r]); inside[r] = fmaf(av.w, v3, inside[r]);
                }
            }
            for (; s < reach; ++s) {
                const float vv = vs[s * kSlice + lane];
#pragma unroll
                for (int r = 0; r < kRows; ++r) inside[r] = fmaf(ar[r][s], vv, inside[r]);
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                if (t0 + r < c && lane < cols)
                    out[(int64_t)(row0 + t0 + r) * heads * vdim + (int64_t)head * vdim + col0 + lane] =
                        fmaf(pw[t0 + r + 1], from_state[r], inside[r]);
        }
        if (tile_state != nullptr) return;         // (a tile is one chunk; its state was made by the scan)
        __syncthreads();                           // every output of the chunk has read S
        // the state behind the chunk: warp `group` takes key dimensions group, group + 8, ... (WIDE: kRows at a time)
        for (int i = group; !WIDE && i < dim; i += kThreads / 32) {
            float add = 0.0f;
            for (int s = 0; s < c; ++s) add = fmaf(ks[s * dpad + i] * pw[c - 1 - s], vs[s * kSlice + lane], add);
            S[i * kSlice + lane] = fmaf(pw[c], S[i * kSlice + lane], add);
        }
        for (int i0 = group * kRows; WIDE && i0 < dim; i0 += (kThreads / 32) * kRows) {
            float add[kRows];
            int at[kRows];
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                add[r] = 0.0f;
                at[r] = min(i0 + r, dim - 1);
            }
            if (vec && i0 + kRows <= dim) {
                for (int s = 0; s < c; ++s) {
                    const float vv = vs[s * kSlice + lane], power = pw[c - 1 - s];
                    const float4 k0 = *reinterpret_cast<const float4*>(ks + s * dpad + i0);
                    const float4 k1 = *reinterpret_cast<const float4*>(ks + s * dpad + i0 + 4);
                    add[0] = fmaf(k0.x * power, vv, add[0]); add[1] = fmaf(k0.y * power, vv, add[1]);
                    add[2] = fmaf(k0.z * power, vv, add[2]); add[3] = fmaf(k0.w * power, vv, add[3]);
                    add[4] = fmaf(k1.x * power, vv, add[4]); add[5] = fmaf(k1.y * power, vv, add[5]);
                    add[6] = fmaf(k1.z * power, vv, add[6]); add[7] = fmaf(k1.w * power, vv, add[7]);
                }
            } else {
                for (int s = 0; s < c; ++s) {
                    const float vv = vs[s * kSlice + lane], power = pw[c - 1 - s];
#pragma unroll
                    for (int r = 0; r < kRows; ++r) add[r] = fmaf(ks[s * dpad + at[r]] * power, vv, add[r]);
                }
            }
#pragma unroll
            for (int r = 0; r < kRows; ++r)
                if (i0 + r < dim) S[(i0 + r) * kSlice + lane] = fmaf(pw[c], S[(i0 + r) * kSlice + lane], add[r]);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < dim * kSlice; e += kThreads) {
        const int i = e / kSlice, j = e % kSlice;
        if (j < cols) slot[(int64_t)i * vdim + col0 + j] = S[e];
    }
}

// A step of single rows (decoded ones): every number of the state is read once, renewed and written once, straight
// from and to the slot; a lane a value column, a warp every eighth key dimension, the warps' parts of S^T q summed in
// warp order.  o = a (S^T q) + (q . k) v,  S' = a S + k v^T.
template <typename T>
__global__ void __launch_bounds__(kThreads)
lightning_step_kernel(const T* __restrict__ proj, int64_t proj_stride, int q_off, int k_off, int v_off,
                      const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                      const int* __restrict__ row_start, const int* __restrict__ state_slots, int heads, int dim, int vdim,
                      int act) {
    extern __shared__ __align__(16) float smem[];
    float* qs = smem;                              // [dim]
    float* ks = qs + dim;                          // [dim]
    float* parts = ks + dim;                       // [warps][kSlice], then the dot product q . k
    pdl_trigger();
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * kSlice;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int kWarps = kThreads / 32;
    const float a = decay[head];
    pdl_wait();
    const int row = row_start[seq];
    if (row >= row_start[seq + 1]) return;
    const T* p = proj + (int64_t)row * proj_stride + (int64_t)head * dim;
    for (int i = threadIdx.x; i < dim; i += kThreads) {
        qs[i] = activate(Elem<T>::load(p + q_off + i), act);
        ks[i] = activate(Elem<T>::load(p + k_off + i), act);
    }
    const bool there = col0 + lane < vdim;
    const float v = there ? activate(Elem<T>::load(proj + (int64_t)row * proj_stride + v_off + (int64_t)head * vdim + col0 + lane), act) : 0.0f;
    __syncthreads();
    float* slot = state + ((int64_t)state_slots[seq] * heads + head) * dim * vdim + col0 + lane;
    float from_state = 0.0f;
    if (there)
        for (int i = warp; i < dim; i += kWarps) {
            const float old = slot[(int64_t)i * vdim];
            from_state = fmaf(qs[i], old, from_state);
            slot[(int64_t)i * vdim] = fmaf(a, old, ks[i] * v);
        }
    parts[warp * kSlice + lane] = from_state;
    if (warp == 0) {
        float dot = 0.0f;
        for (int i = lane; i < dim; i += 32) dot = fmaf(qs[i], ks[i], dot);
        dot = warp_sum(dot);
        if (lane == 0) parts[kWarps * kSlice] = dot;
    }
    __syncthreads();
    if (warp == 0 && there) {
        float total = 0.0f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) total += parts[w * kSlice + lane];
        out[(int64_t)row * heads * vdim + (int64_t)head * vdim + col0 + lane] = fmaf(a, total, parts[kWarps * kSlice] * v);
    }
}

// Launch 1 of the tiled form: U = sum_s a^(c-1-s) k_s v_s^T of one tile, head and slice of value columns, into
// tile_state[tile][head] ([dim][vdim]).
template <typename T>
__global__ void __launch_bounds__(kThreads)
lightning_tile_sum_kernel(const T* __restrict__ proj, int64_t proj_stride, int k_off, int v_off,
                          const float* __restrict__ decay, float* __restrict__ tile_state,
                          const int* __restrict__ row_start, int num_seqs, int heads, int dim, int vdim, int chunk,
                          int act) {
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    const int head = blockIdx.y, col0 = blockIdx.z * kSlice;
    const int cols = min(kSlice, vdim - col0);
    const int dpad = row_floats(dim);
    const bool vec = dim % 4 == 0;
    float* ks = smem;                              // [chunk][row_floats(dim)]
    float* vs = ks + chunk * dpad;                 // [chunk][kSlice]
    float* pw = vs + chunk * kSlice;               // [chunk + 1]
    const float a = decay[head];
    for (int i = threadIdx.x; i <= chunk; i += kThreads) pw[i] = (float)pow((double)a, (double)i);
    pdl_wait();
    int seq, r0, c;
    if (!find_tile(row_start, num_seqs, chunk, blockIdx.x, seq, r0, c)) return;
    const T* rows_at = proj + (int64_t)r0 * proj_stride;
    load_silu_rows<T, true>(ks, dpad, rows_at + k_off + (int64_t)head * dim, proj_stride, c, dim, dim, act);
    load_silu_rows<T, true>(vs, kSlice, rows_at + v_off + (int64_t)head * vdim + col0, proj_stride, c, kSlice, cols, act);
    __syncthreads();
    const int lane = threadIdx.x & 31, group = threadIdx.x >> 5;
    float* mine = tile_state + ((int64_t)blockIdx.x * heads + head) * dim * vdim;
    for (int i0 = group * kRows; i0 < dim; i0 += (kThreads / 32) * kRows) {
        float add[kRows];
        int at[kRows];
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            add[r] = 0.0f;
            at[r] = min(i0 + r, dim - 1);
        }
        if (vec && i0 + kRows <= dim) {
            for (int s = 0; s < c; ++s) {
                const float vv = vs[s * kSlice + lane], power = pw[c - 1 - s];
                const float4 k0 = *reinterpret_cast<const float4*>(ks + s * dpad + i0);
                const float4 k1 = *reinterpret_cast<const float4*>(ks + s * dpad + i0 + 4);
                add[0] = fmaf(k0.x * power, vv, add[0]); add[1] = fmaf(k0.y * power, vv, add[1]);
                add[2] = fmaf(k0.z * power, vv, add[2]); add[3] = fmaf(k0.w * power, vv, add[3]);
                add[4] = fmaf(k1.x * power, vv, add[4]); add[5] = fmaf(k1.y * power, vv, add[5]);
                add[6] = fmaf(k1.z * power, vv, add[6]); add[7] = fmaf(k1.w * power, vv, add[7]);
            }
        } else {
            for (int s = 0; s < c; ++s) {
                const float vv = vs[s * kSlice + lane], power = pw[c - 1 - s];
#pragma unroll
                for (int r = 0; r < kRows; ++r) add[r] = fmaf(ks[s * dpad + at[r]] * power, vv, add[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r)
            if (i0 + r < dim && lane < cols) mine[(int64_t)(i0 + r) * vdim + col0 + lane] = add[r];
    }
}

// Launch 2: per sequence and head, the tiles in order.  Every number of the state is a chain of its own.
__global__ void __launch_bounds__(kThreads)
lightning_scan_kernel(const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ tile_state,
                      const int* __restrict__ row_start, const int* __restrict__ state_slots, int heads, int dim, int vdim,
                      int chunk) {
    pdl_trigger();
    pdl_wait();
    const int seq = blockIdx.x, head = blockIdx.y;
    const int rows = row_start[seq + 1] - row_start[seq];
    if (rows <= 0) return;
    int first_tile = 0;
    for (int s = 0; s < seq; ++s) first_tile += (row_start[s + 1] - row_start[s] + chunk - 1) / chunk;
    const int tiles = (rows + chunk - 1) / chunk;
    const float a = decay[head];
    const float whole = (float)pow((double)a, (double)chunk);
    const float rest = (float)pow((double)a, (double)(rows - (tiles - 1) * chunk));
    float* slot = state + ((int64_t)state_slots[seq] * heads + head) * dim * vdim;
    const int64_t stride = (int64_t)heads * dim * vdim;
    float* kept = tile_state + ((int64_t)first_tile * heads + head) * dim * vdim;
    for (int e = blockIdx.z * kThreads + threadIdx.x; e < dim * vdim; e += gridDim.z * kThreads) {
        float current = slot[e];
        for (int i = 0; i < tiles; ++i) {
            const float own = kept[i * stride + e];
            kept[i * stride + e] = current;
            current = fmaf(i + 1 < tiles ? whole : rest, current, own);
        }
        slot[e] = current;
    }
}


// ----------------------------------------------------------------------------- around the recurrence

// One warp per (row, head of q, k or v); out row: [H * dim q | H * dim k | H * vdim v], 32-bit.
template <typename T>
__global__ void __launch_bounds__(128)
retention_prepare_kernel(const T* __restrict__ proj, int64_t proj_stride, int q_off, int k_off, int v_off,
                         float* __restrict__ out, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                         int heads, int dim, int vdim, int rot_dims, float amplitude, float k_scale) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, slot = blockIdx.y * 4 + warp;
    if (slot >= 3 * heads) return;
    const int64_t out_stride = (int64_t)heads * (2 * dim + vdim);
    const T* prow = proj + (int64_t)row * proj_stride;
    float* orow = out + (int64_t)row * out_stride;
    if (slot >= 2 * heads) {
        const int head = slot - 2 * heads;
        const T* src = prow + v_off + (int64_t)head * vdim;
        float* dst = orow + (int64_t)2 * heads * dim + (int64_t)head * vdim;
        for (int i = lane; i < vdim; i += 32) dst[i] = Elem<T>::load(src + i);
        return;
    }
    const bool is_key = slot >= heads;
    const int head = is_key ? slot - heads : slot;
    const T* src = prow + (is_key ? k_off : q_off) + (int64_t)head * dim;
    float* dst = orow + (int64_t)slot * dim;
    const float factor = is_key ? k_scale : 1.0f;
    const float pos = (float)positions[row];
    const int half = rot_dims >> 1;
    for (int i = lane; i < half; i += 32) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        sn *= amplitude;
        cs *= amplitude;
        const float u = Elem<T>::load(src + i), v = Elem<T>::load(src + i + half);
        dst[i] = (u * cs - v * sn) * factor;
        dst[i + half] = (v * cs + u * sn) * factor;
    }
    for (int i = rot_dims + lane; i < dim; i += 32) dst[i] = Elem<T>::load(src + i) * factor;
}

enum GateKind : int { GATE_SIGMOID = 0, GATE_SILU = 1 };

// One warp per (row, head): the head's 32-bit numbers over their root mean square, times the activated gate.
template <typename T>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ gate, int64_t gate_stride, T* __restrict__ out,
                      int64_t out_stride, int heads, int vdim, float eps, int gate_kind) {
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x, head = blockIdx.y * 4 + warp;
    if (head >= heads) return;
    const float* orow = o + ((int64_t)row * heads + head) * vdim;
    float ss = 0.0f;
    for (int i = lane; i < vdim; i += 32) ss = fmaf(orow[i], orow[i], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + eps);
    const T* grow = gate + (int64_t)row * gate_stride + (int64_t)head * vdim;
    T* dst = out + (int64_t)row * out_stride + (int64_t)head * vdim;
    for (int i = lane; i < vdim; i += 32) {
        const float g = Elem<T>::load(grow + i);
        const float s = 1.0f / (1.0f + expf(-g));
        Elem<T>::store(dst + i, orow[i] * inv * (gate_kind == GATE_SILU ? g * s : s));
    }
}

size_t smem_for(int chunk, int dim) {
    return sizeof(float) * ((size_t)2 * chunk * row_floats(dim) + (size_t)chunk * kSlice + (size_t)chunk * chunk +
                            (size_t)dim * kSlice + chunk + 1);
}

int chunk_for(int dim, int max_new) {
    int chunk = 64;
    while (chunk > 1 && (chunk / 2 >= max_new || smem_for(chunk, dim) > 200 * 1024)) chunk /= 2;
    return chunk;
}

// Tiles of the three-launch form for a step of `rows` rows in `num_seqs` sequences (an upper bound that follows from
// the counts alone), or 0 where a block walks its sequence: steps whose longest portion is shorter than four chunks.
int tiles_for(int rows, int num_seqs, int dim, int max_new) {
    const int chunk = chunk_for(dim, max_new);
    if (max_new < 4 * chunk) return 0;
    return (rows + chunk - 1) / chunk + num_seqs;
}

template <typename T>
int launch(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, const float* decay, float* state,
           float* out, const int* row_start, const int* state_slots, int rows, int num_seqs, int heads, int dim, int vdim,
           int max_new, float* tile_state, int act, cudaStream_t stream) {
    const int chunk = chunk_for(dim, max_new);
    const size_t smem = smem_for(chunk, dim);
    if (smem > 220 * 1024) return TB_ERR_BAD_SIZE;
    auto kernel = chunk >= kRows ? lightning_kernel<T, true> : lightning_kernel<T, false>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    const int slices = (vdim + kSlice - 1) / kSlice;
    if (max_new == 1) {                                           // single rows: the state straight from and to its slot
        const size_t step_smem = sizeof(float) * ((size_t)2 * dim + (kThreads / 32) * kSlice + 1);
        if (step_smem > 40 * 1024) return TB_ERR_BAD_SIZE;
        cudaError_t launched = tb_launch_pdl(lightning_step_kernel<T>, dim3(num_seqs, heads, slices), dim3(kThreads),
                                             step_smem, stream, (const T*)proj, proj_stride, q_off, k_off, v_off, decay,
                                             state, out, row_start, state_slots, heads, dim, vdim, act);
        return launched == cudaSuccess ? tb_launch_status() : (int)launched;
    }
    const int tiles = tiles_for(rows, num_seqs, dim, max_new);
    if (tiles == 0) {
        cudaError_t launched = tb_launch_pdl(kernel, dim3(num_seqs, heads, slices), dim3(kThreads), smem, stream,
                                             (const T*)proj, proj_stride, q_off, k_off, v_off, decay, state, out, row_start,
                                             state_slots, heads, dim, vdim, chunk, (const float*)nullptr, num_seqs, act);
        return launched == cudaSuccess ? tb_launch_status() : (int)launched;
    }
    if (tile_state == nullptr) return TB_ERR_BAD_SIZE;
    auto sums = lightning_tile_sum_kernel<T>;
    const size_t sums_smem = sizeof(float) * ((size_t)chunk * row_floats(dim) + (size_t)chunk * kSlice + chunk + 1);
    if (sums_smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(sums, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sums_smem);
        if (err != cudaSuccess) return (int)err;
    }
    cudaError_t launched = tb_launch_pdl(sums, dim3(tiles, heads, slices), dim3(kThreads), sums_smem, stream, (const T*)proj,
                                         proj_stride, k_off, v_off, decay, tile_state, row_start, num_seqs, heads, dim,
                                         vdim, chunk, act);
    if (launched != cudaSuccess) return (int)launched;
    const int parts = max(1, min(64, (dim * vdim + kThreads - 1) / kThreads));
    launched = tb_launch_pdl(lightning_scan_kernel, dim3(num_seqs, heads, parts), dim3(kThreads), (size_t)0, stream, decay,
                             state, tile_state, row_start, state_slots, heads, dim, vdim, chunk);
    if (launched != cudaSuccess) return (int)launched;
    launched = tb_launch_pdl(kernel, dim3(tiles, heads, slices), dim3(kThreads), smem, stream, (const T*)proj, proj_stride,
                             q_off, k_off, v_off, decay, state, out, row_start, state_slots, heads, dim, vdim, chunk,
                             (const float*)tile_state, num_seqs, act);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

}  // namespace

// proj: [rows, ...] in `dtype`, row stride proj_stride (elements); q at column q_off ([heads, dim]), k at k_off ([heads, dim]),
// v at v_off ([heads, vdim]), all before their activation.  decay: float32 [heads].  state: float32 [slots, heads, dim, vdim].
// out: float32 [rows, heads * vdim].  max_new: the most rows any sequence brings (it sizes the chunk).  tile_state: float32
// [tb_lightning_tiles(...), heads, dim, vdim] of scratch where that count is not 0.  act: 1 applies SiLU to q, k and v as
// they are read, 0 takes them as they are.
TB_EXPORT int tb_lightning_tiles(int rows, int num_seqs, int dim, int max_new) {
    return (rows < 1 || num_seqs < 1 || dim < 1 || max_new < 1) ? 0 : tiles_for(rows, num_seqs, dim, max_new);
}

TB_EXPORT int tb_lightning(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, const float* decay,
                           float* state, float* out, const int* row_start, const int* state_slots, int rows, int num_seqs,
                           int heads, int dim, int vdim, int max_new, float* tile_state, int act, int dtype,
                           cudaStream_t stream) {
    if (num_seqs == 0 || rows == 0) return 0;
    if (act != ACT_NONE && act != ACT_SILU) return TB_ERR_BAD_SIZE;
    if (heads < 1 || heads > 65535 || dim < 1 || vdim < 1 || (vdim + kSlice - 1) / kSlice > 65535 || max_new < 1)
        return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32)
        return launch<float>(proj, proj_stride, q_off, k_off, v_off, decay, state, out, row_start, state_slots, rows,
                             num_seqs, heads, dim, vdim, max_new, tile_state, act, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(proj, proj_stride, q_off, k_off, v_off, decay, state, out, row_start, state_slots,
                                     rows, num_seqs, heads, dim, vdim, max_new, tile_state, act, stream);
    return TB_ERR_BAD_DTYPE;
}

// proj as for tb_lightning; out: float32 [rows, heads * (2 * dim + vdim)] (q heads, k heads, v heads); inv_freq: float32
// [rot_dims / 2] (may be null when rot_dims is 0).
TB_EXPORT int tb_retention_prepare(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, float* out,
                                   const int* positions, const float* inv_freq, int rows, int heads, int dim, int vdim,
                                   int rot_dims, float amplitude, float k_scale, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (heads < 1 || dim < 1 || vdim < 1 || rot_dims < 0 || rot_dims % 2 || rot_dims > dim) return TB_ERR_BAD_SIZE;
    if (rot_dims > 0 && inv_freq == nullptr) return TB_ERR_BAD_SIZE;
    const dim3 grid(rows, (3 * heads + 3) / 4);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(retention_prepare_kernel<float>, grid, dim3(128), (size_t)0, stream, (const float*)proj,
                                 proj_stride, q_off, k_off, v_off, out, positions, inv_freq, heads, dim, vdim, rot_dims,
                                 amplitude, k_scale);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(retention_prepare_kernel<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream,
                                 (const __nv_bfloat16*)proj, proj_stride, q_off, k_off, v_off, out, positions, inv_freq,
                                 heads, dim, vdim, rot_dims, amplitude, k_scale);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// o: float32 [rows, heads * vdim], contiguous; gate and out: [rows, >= heads * vdim] in `dtype` with row strides of their own.
TB_EXPORT int tb_head_norm_gate(const float* o, const void* gate, int64_t gate_stride, void* out, int64_t out_stride,
                                int rows, int heads, int vdim, float eps, int gate_kind, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (heads < 1 || vdim < 1 || (gate_kind != GATE_SIGMOID && gate_kind != GATE_SILU)) return TB_ERR_BAD_SIZE;
    const dim3 grid(rows, (heads + 3) / 4);
    if (grid.y > 65535) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(head_norm_gate_kernel<float>, grid, dim3(128), (size_t)0, stream, o, (const float*)gate,
                                 gate_stride, (float*)out, out_stride, heads, vdim, eps, gate_kind);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(head_norm_gate_kernel<__nv_bfloat16>, grid, dim3(128), (size_t)0, stream, o,
                                 (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, out_stride, heads, vdim, eps,
                                 gate_kind);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
