// Norms around a sublayer whose result is normed before it joins the residual stream, for a stream kept in 32-bit.
//
//   tb_norm_add_norm   u  = post(upd)                       post: nothing, a layer norm (weight, bias) or an RMS norm (weight)
//                      x  = res + u                         (32-bit, stored back to res; without upd x = res)
//                      y  = round(next(x))                  next: nothing, a layer norm or an RMS norm; y in the run dtype
//                      c  = round(x)                        (when a rounded copy of the stream is asked for)
//                      layer norm: (v - mean) / sqrt(mean((v - mean)^2) + eps) * w + b, the mean first, then the
//                      deviations' squares, both from the row held in shared memory; RMS norm: v / sqrt(mean(v^2) + eps) * w.
//   tb_gated_rms_norm  y = round(v / sqrt(mean(v^2) + eps) * w * sigmoid(g)) over rows of 32-bit v and a gate in the run dtype.
//
// One block per row; block size and reduction tree follow from the width alone, so a row's result does not depend on the
// batch around it.  Everything is 32-bit up to the single rounding of an output.
#include "common.cuh"

namespace {

enum NormKind : int { NORM_NONE = 0, NORM_LAYER = 1, NORM_RMS = 2 };

// mean and 1 / sqrt(variance + eps) (layer norm) or 0 and 1 / sqrt(mean square + eps) (RMS) of row[0 .. width)
__device__ __forceinline__ void row_statistics(const float* row, int width, int kind, float eps, float* scratch,
                                               float& mean, float& inv) {
    mean = 0.0f;
    if (kind == NORM_LAYER) {
        float s = 0.0f;
        for (int j = threadIdx.x; j < width; j += blockDim.x) s += row[j];
        mean = block_sum(s, scratch) / (float)width;
    }
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float d = row[j] - mean;
        ss = fmaf(d, d, ss);
    }
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / (float)width + eps);
}

template <typename T>
__global__ void __launch_bounds__(1024)
norm_add_norm_kernel(float* __restrict__ res, const float* __restrict__ upd, int post_kind,
                     const float* __restrict__ post_w, const float* __restrict__ post_b, int next_kind,
                     const float* __restrict__ next_w, const float* __restrict__ next_b, T* __restrict__ out,
                     T* __restrict__ copy, int width, float eps) {
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();                                   // the stream and the update come from kernels in front
    const int64_t base = (int64_t)blockIdx.x * width;
    if (upd != nullptr) {
        for (int j = threadIdx.x; j < width; j += blockDim.x) row[j] = upd[base + j];
        __syncthreads();
        float mean = 0.0f, inv = 1.0f;
        if (post_kind != NORM_NONE) row_statistics(row, width, post_kind, eps, scratch, mean, inv);
        for (int j = threadIdx.x; j < width; j += blockDim.x) {      // each thread rewrites what it wrote
            float u = row[j];
            if (post_kind != NORM_NONE) {
                u = (u - mean) * inv * post_w[j];
                if (post_kind == NORM_LAYER) u += post_b[j];
            }
            const float x = res[base + j] + u;
            res[base + j] = x;
            row[j] = x;
        }
    } else {
        for (int j = threadIdx.x; j < width; j += blockDim.x) row[j] = res[base + j];
    }
    __syncthreads();
    if (copy != nullptr)
        for (int j = threadIdx.x; j < width; j += blockDim.x) Elem<T>::store(copy + base + j, row[j]);
    if (next_kind == NORM_NONE || out == nullptr) return;
    float mean, inv;
    row_statistics(row, width, next_kind, eps, scratch, mean, inv);
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float y = (row[j] - mean) * inv * next_w[j];
        if (next_kind == NORM_LAYER) y += next_b[j];
        Elem<T>::store(out + base + j, y);
    }
}

template <typename T>
__global__ void __launch_bounds__(1024)
gated_rms_norm_kernel(const float* __restrict__ v, const float* __restrict__ w, const T* __restrict__ gate,
                      int64_t gate_stride, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* row = v + (int64_t)blockIdx.x * width;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) ss = fmaf(row[j], row[j], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    const T* g = gate + (int64_t)blockIdx.x * gate_stride;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float s = 1.0f / (1.0f + expf(-Elem<T>::load(g + j)));
        Elem<T>::store(out + (int64_t)blockIdx.x * width + j, row[j] * inv * w[j] * s);
    }
}

int threads_for(int width) {
    int threads = 32;
    while (threads < 1024 && threads * 4 < width) threads <<= 1;
    return threads;
}

}  // namespace

// res: float32 [rows, width], updated in place when upd (float32 [rows, width]) is given.  post_kind / next_kind:
// 0 none, 1 layer norm (w, b), 2 RMS norm (w).  out, copy: null or [rows, width] in `dtype`.
TB_EXPORT int tb_norm_add_norm(float* res, const float* upd, int post_kind, const float* post_w, const float* post_b,
                               int next_kind, const float* next_w, const float* next_b, void* out, void* copy,
                               int rows, int width, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1 || (size_t)width * sizeof(float) > 200 * 1024) return TB_ERR_BAD_SIZE;
    if (post_kind < NORM_NONE || post_kind > NORM_RMS || next_kind < NORM_NONE || next_kind > NORM_RMS) return TB_ERR_BAD_SIZE;
    if ((post_kind != NORM_NONE && (upd == nullptr || post_w == nullptr)) || (post_kind == NORM_LAYER && post_b == nullptr))
        return TB_ERR_BAD_SIZE;
    if ((next_kind != NORM_NONE && (out == nullptr || next_w == nullptr)) || (next_kind == NORM_LAYER && next_b == nullptr))
        return TB_ERR_BAD_SIZE;
    const size_t smem = (size_t)width * sizeof(float);
    const int threads = threads_for(width);
#define TB_RUN(T)                                                                                                    \
    do {                                                                                                             \
        auto kernel = norm_add_norm_kernel<T>;                                                                       \
        if (smem > 40 * 1024) {                                                                                      \
            cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);  \
            if (err != cudaSuccess) return (int)err;                                                                 \
        }                                                                                                            \
        cudaError_t launched = tb_launch_pdl(kernel, dim3(rows), dim3(threads), smem, stream, res, upd, post_kind,   \
                                             post_w, post_b, next_kind, next_w, next_b, (T*)out, (T*)copy, width,    \
                                             eps);                                                                   \
        return launched == cudaSuccess ? tb_launch_status() : (int)launched;                                         \
    } while (0)
    if (dtype == TB_F32) TB_RUN(float);
    if (dtype == TB_BF16) TB_RUN(__nv_bfloat16);
#undef TB_RUN
    return TB_ERR_BAD_DTYPE;
}

// v: float32 [rows, width]; w: float32 [width]; gate: [rows, width] in `dtype` with row stride gate_stride; out: [rows, width].
TB_EXPORT int tb_gated_rms_norm(const float* v, const float* w, const void* gate, int64_t gate_stride, void* out,
                                int rows, int width, float eps, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1) return TB_ERR_BAD_SIZE;
    const int threads = threads_for(width);
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(gated_rms_norm_kernel<float>, dim3(rows), dim3(threads), 0, stream, v, w,
                                 (const float*)gate, gate_stride, (float*)out, width, eps);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(gated_rms_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), 0, stream, v, w,
                                 (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, width, eps);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
