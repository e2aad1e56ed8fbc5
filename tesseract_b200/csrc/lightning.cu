// Linear attention with a fixed decay per head:  S_t = a S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t  (S: [dim, vdim], 32-bit,
// kept per request in its state slot), with q = silu(.), k = silu(.), v = silu(.) of the projected rows.
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
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kSlice = 32;          // value columns a block owns

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(kThreads)
lightning_kernel(const T* __restrict__ proj, int64_t proj_stride, int q_off, int k_off, int v_off,
                 const float* __restrict__ decay, float* __restrict__ state, float* __restrict__ out,
                 const int* __restrict__ row_start, const int* __restrict__ state_slots, int heads, int dim, int vdim,
                 int chunk) {
    extern __shared__ __align__(16) float smem[];
    pdl_trigger();
    const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * kSlice;
    const int cols = min(kSlice, vdim - col0);
    const int dpad = dim + 1;
    float* qs = smem;                              // [chunk][dim + 1]
    float* ks = qs + chunk * dpad;                 // [chunk][dim + 1]
    float* vs = ks + chunk * dpad;                 // [chunk][kSlice]
    float* A = vs + chunk * kSlice;                // [chunk][chunk]
    float* S = A + chunk * chunk;                  // [dim][kSlice]
    float* pw = S + dim * kSlice;                  // [chunk + 1]
    const float a = decay[head];
    for (int i = threadIdx.x; i <= chunk; i += kThreads) pw[i] = (float)pow((double)a, (double)i);
    pdl_wait();                                    // rows, state and the step's metadata come from kernels in front
    const int first = row_start[seq], last = row_start[seq + 1];
    if (first >= last) return;
    float* slot = state + ((int64_t)state_slots[seq] * heads + head) * dim * vdim;
    for (int e = threadIdx.x; e < dim * kSlice; e += kThreads) {
        const int i = e / kSlice, j = e % kSlice;
        S[e] = j < cols ? slot[(int64_t)i * vdim + col0 + j] : 0.0f;
    }
    const int lane = threadIdx.x & 31, group = threadIdx.x >> 5;          // kSlice == 32: a lane a value column
    for (int row0 = first; row0 < last; row0 += chunk) {
        const int c = min(chunk, last - row0);
        __syncthreads();                           // the chunk before is done with qs, ks, vs, A (and S is written)
        for (int e = threadIdx.x; e < c * dim; e += kThreads) {
            const int t = e / dim, i = e % dim;
            const T* p = proj + (int64_t)(row0 + t) * proj_stride + (int64_t)head * dim + i;
            qs[t * dpad + i] = silu(Elem<T>::load(p + q_off));
            ks[t * dpad + i] = silu(Elem<T>::load(p + k_off));
        }
        for (int e = threadIdx.x; e < c * kSlice; e += kThreads) {
            const int t = e / kSlice, j = e % kSlice;
            vs[e] = j < cols ? silu(Elem<T>::load(proj + (int64_t)(row0 + t) * proj_stride + v_off + (int64_t)head * vdim + col0 + j))
                             : 0.0f;
        }
        __syncthreads();
        // scores of the chunk: thread e takes (t, s) with s fastest, so neighbouring lanes read neighbouring key rows
        for (int e = threadIdx.x; e < c * c; e += kThreads) {
            const int t = e / c, s = e % c;
            float dot = 0.0f;
            if (s <= t) {
                const float* qr = qs + t * dpad;
                const float* kr = ks + s * dpad;
                for (int i = 0; i < dim; ++i) dot = fmaf(qr[i], kr[i], dot);
                dot *= pw[t - s];
            }
            A[t * chunk + s] = dot;
        }
        __syncthreads();
        // outputs: warp `group` takes rows group, group + 8, ...; a lane a value column
        for (int t = group; t < c; t += kThreads / 32) {
            const float* qr = qs + t * dpad;
            float from_state = 0.0f;
            for (int i = 0; i < dim; ++i) from_state = fmaf(qr[i], S[i * kSlice + lane], from_state);
            float inside = 0.0f;
            for (int s = 0; s <= t; ++s) inside = fmaf(A[t * chunk + s], vs[s * kSlice + lane], inside);
            if (lane < cols)
                out[(int64_t)(row0 + t) * heads * vdim + (int64_t)head * vdim + col0 + lane] = fmaf(pw[t + 1], from_state, inside);
        }
        __syncthreads();                           // every output of the chunk has read S
        // the state behind the chunk: warp `group` takes key dimensions group, group + 8, ...
        for (int i = group; i < dim; i += kThreads / 32) {
            float add = 0.0f;
            for (int s = 0; s < c; ++s) add = fmaf(ks[s * dpad + i] * pw[c - 1 - s], vs[s * kSlice + lane], add);
            S[i * kSlice + lane] = fmaf(pw[c], S[i * kSlice + lane], add);
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < dim * kSlice; e += kThreads) {
        const int i = e / kSlice, j = e % kSlice;
        if (j < cols) slot[(int64_t)i * vdim + col0 + j] = S[e];
    }
}

size_t smem_for(int chunk, int dim) {
    return sizeof(float) * ((size_t)2 * chunk * (dim + 1) + (size_t)chunk * kSlice + (size_t)chunk * chunk +
                            (size_t)dim * kSlice + chunk + 1);
}

template <typename T>
int launch(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, const float* decay, float* state,
           float* out, const int* row_start, const int* state_slots, int num_seqs, int heads, int dim, int vdim,
           int max_new, cudaStream_t stream) {
    int chunk = 64;
    while (chunk > 1 && (chunk / 2 >= max_new || smem_for(chunk, dim) > 200 * 1024)) chunk /= 2;
    const size_t smem = smem_for(chunk, dim);
    if (smem > 220 * 1024) return TB_ERR_BAD_SIZE;
    auto kernel = lightning_kernel<T>;
    if (smem > 40 * 1024) {
        cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (err != cudaSuccess) return (int)err;
    }
    const dim3 grid(num_seqs, heads, (vdim + kSlice - 1) / kSlice);
    cudaError_t launched = tb_launch_pdl(kernel, grid, dim3(kThreads), smem, stream, (const T*)proj, proj_stride, q_off,
                                         k_off, v_off, decay, state, out, row_start, state_slots, heads, dim, vdim, chunk);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

}  // namespace

// proj: [rows, ...] in `dtype`, row stride proj_stride (elements); q at column q_off ([heads, dim]), k at k_off ([heads, dim]),
// v at v_off ([heads, vdim]), all before their activation.  decay: float32 [heads].  state: float32 [slots, heads, dim, vdim].
// out: float32 [rows, heads * vdim].  max_new: the most rows any sequence brings (it sizes the chunk).
TB_EXPORT int tb_lightning(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, const float* decay,
                           float* state, float* out, const int* row_start, const int* state_slots, int num_seqs,
                           int heads, int dim, int vdim, int max_new, int dtype, cudaStream_t stream) {
    if (num_seqs == 0) return 0;
    if (heads < 1 || heads > 65535 || dim < 1 || vdim < 1 || (vdim + kSlice - 1) / kSlice > 65535 || max_new < 1)
        return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32)
        return launch<float>(proj, proj_stride, q_off, k_off, v_off, decay, state, out, row_start, state_slots, num_seqs,
                             heads, dim, vdim, max_new, stream);
    if (dtype == TB_BF16)
        return launch<__nv_bfloat16>(proj, proj_stride, q_off, k_off, v_off, decay, state, out, row_start, state_slots,
                                     num_seqs, heads, dim, vdim, max_new, stream);
    return TB_ERR_BAD_DTYPE;
}
