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

// Four neighbouring numbers at a time where the width is a multiple of four (VEC): 16-byte loads of 32-bit rows, 8- or
// 16-byte stores of the outputs; a number at a time otherwise.
template <bool VEC>
__device__ __forceinline__ void load4(const float* p, int j, float* v) {
    if (VEC) {
        const float4 t = *reinterpret_cast<const float4*>(p + j);
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    } else {
        v[0] = p[j];
    }
}
template <bool VEC>
__device__ __forceinline__ void store4(float* p, int j, const float* v) {
    if (VEC) *reinterpret_cast<float4*>(p + j) = make_float4(v[0], v[1], v[2], v[3]);
    else p[j] = v[0];
}
template <bool VEC>
__device__ __forceinline__ void store4(__nv_bfloat16* p, int j, const float* v) {
    if (VEC) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p + j) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    } else {
        p[j] = __float2bfloat16_rn(v[0]);
    }
}
template <bool VEC>
__device__ __forceinline__ void load4(const __nv_bfloat16* p, int j, float* v) {
    if (VEC) {
        const uint2 t = *reinterpret_cast<const uint2*>(p + j);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&t.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
        v[0] = __low2float(lo); v[1] = __high2float(lo); v[2] = __low2float(hi); v[3] = __high2float(hi);
    } else {
        v[0] = __bfloat162float(p[j]);
    }
}

// mean and 1 / sqrt(variance + eps) (layer norm) or 0 and 1 / sqrt(mean square + eps) (RMS) of row[0 .. width)
template <bool VEC>
__device__ __forceinline__ void row_statistics(const float* row, int width, int kind, float eps, float* scratch,
                                               float& mean, float& inv) {
    constexpr int N = VEC ? 4 : 1;
    mean = 0.0f;
    if (kind == NORM_LAYER) {
        float s = 0.0f;
        for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {
            float v[4];
            load4<VEC>(row, j, v);
#pragma unroll
            for (int e = 0; e < N; ++e) s += v[e];
        }
        mean = block_sum(s, scratch) / (float)width;
    }
    float ss = 0.0f;
    for (int j = threadIdx.x * N; j < width; j += blockDim.x * N) {
        float v[4];
        load4<VEC>(row, j, v);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            const float d = v[e] - mean;
            ss = fmaf(d, d, ss);
        }
    }
    ss = block_sum(ss, scratch);
    inv = 1.0f / sqrtf(ss / (float)width + eps);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(1024)
norm_add_norm_kernel(float* __restrict__ res, const float* __restrict__ upd, int post_kind,
                     const float* __restrict__ post_w, const float* __restrict__ post_b, int next_kind,
                     const float* __restrict__ next_w, const float* __restrict__ next_b, T* __restrict__ out,
                     T* __restrict__ copy, int width, float eps) {
    constexpr int N = VEC ? 4 : 1;
    extern __shared__ __align__(16) float row[];
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();                                   // the stream and the update come from kernels in front
    const int64_t base = (int64_t)blockIdx.x * width;
    const int first = threadIdx.x * N, step = blockDim.x * N;
    float v[4], w[4], b[4], x[4];
    if (upd != nullptr) {
        for (int j = first; j < width; j += step) {
            load4<VEC>(upd + base, j, v);
            store4<VEC>(row, j, v);
        }
        __syncthreads();
        float mean = 0.0f, inv = 1.0f;
        if (post_kind != NORM_NONE) row_statistics<VEC>(row, width, post_kind, eps, scratch, mean, inv);
        for (int j = first; j < width; j += step) {                  // each thread rewrites what it wrote
            load4<VEC>(row, j, v);
            if (post_kind != NORM_NONE) {
                load4<VEC>(post_w, j, w);
#pragma unroll
                for (int e = 0; e < N; ++e) v[e] = (v[e] - mean) * inv * w[e];
                if (post_kind == NORM_LAYER) {
                    load4<VEC>(post_b, j, b);
#pragma unroll
                    for (int e = 0; e < N; ++e) v[e] += b[e];
                }
            }
            load4<VEC>(res + base, j, x);
#pragma unroll
            for (int e = 0; e < N; ++e) x[e] += v[e];
            store4<VEC>(res + base, j, x);
            store4<VEC>(row, j, x);
        }
    } else {
        for (int j = first; j < width; j += step) {
            load4<VEC>(res + base, j, v);
            store4<VEC>(row, j, v);
        }
    }
    __syncthreads();
    if (copy != nullptr)
        for (int j = first; j < width; j += step) {
            load4<VEC>(row, j, v);
            store4<VEC>(copy + base, j, v);
        }
    if (next_kind == NORM_NONE || out == nullptr) return;
    float mean, inv;
    row_statistics<VEC>(row, width, next_kind, eps, scratch, mean, inv);
    for (int j = first; j < width; j += step) {
        load4<VEC>(row, j, v);
        load4<VEC>(next_w, j, w);
#pragma unroll
        for (int e = 0; e < N; ++e) v[e] = (v[e] - mean) * inv * w[e];
        if (next_kind == NORM_LAYER) {
            load4<VEC>(next_b, j, b);
#pragma unroll
            for (int e = 0; e < N; ++e) v[e] += b[e];
        }
        store4<VEC>(out + base, j, v);
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(1024)
gated_rms_norm_kernel(const float* __restrict__ v, const float* __restrict__ w, const T* __restrict__ gate,
                      int64_t gate_stride, T* __restrict__ out, int width, float eps) {
    constexpr int N = VEC ? 4 : 1;
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const float* row = v + (int64_t)blockIdx.x * width;
    const int first = threadIdx.x * N, step = blockDim.x * N;
    float x[4], wv[4], gv[4];
    float ss = 0.0f;
    for (int j = first; j < width; j += step) {
        load4<VEC>(row, j, x);
#pragma unroll
        for (int e = 0; e < N; ++e) ss = fmaf(x[e], x[e], ss);
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    const T* g = gate + (int64_t)blockIdx.x * gate_stride;
    for (int j = first; j < width; j += step) {
        load4<VEC>(row, j, x);
        load4<VEC>(w, j, wv);
        load4<VEC>(g, j, gv);
#pragma unroll
        for (int e = 0; e < N; ++e) x[e] = x[e] * inv * wv[e] * (1.0f / (1.0f + expf(-gv[e])));
        store4<VEC>(out + (int64_t)blockIdx.x * width, j, x);
    }
}

// (eight numbers a thread: a row of 2,048 is a block of 256, whose reductions cost less than those of 512 threads
// with four numbers each, and more rows are in flight on a multiprocessor)
int threads_for(int width) {
    int threads = 32;
    while (threads < 1024 && threads * 8 < width) threads <<= 1;
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
    const bool vec = width % 4 == 0 && ((uintptr_t)res | (uintptr_t)upd | (uintptr_t)post_w | (uintptr_t)post_b |
                                        (uintptr_t)next_w | (uintptr_t)next_b | (uintptr_t)out | (uintptr_t)copy) % 16 == 0;
#define TB_RUN(T)                                                                                                    \
    do {                                                                                                             \
        auto kernel = vec ? norm_add_norm_kernel<T, true> : norm_add_norm_kernel<T, false>;                          \
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
    const bool vec = width % 4 == 0 && gate_stride % 4 == 0 &&
                     ((uintptr_t)v | (uintptr_t)w | (uintptr_t)gate | (uintptr_t)out) % 16 == 0;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(vec ? gated_rms_norm_kernel<float, true> : gated_rms_norm_kernel<float, false>, dim3(rows),
                                 dim3(threads), 0, stream, v, w, (const float*)gate, gate_stride, (float*)out, width, eps);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(vec ? gated_rms_norm_kernel<__nv_bfloat16, true> : gated_rms_norm_kernel<__nv_bfloat16, false>,
                                 dim3(rows), dim3(threads), 0, stream, v, w, (const __nv_bfloat16*)gate, gate_stride,
                                 (__nv_bfloat16*)out, width, eps);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
