// A sublayer's result joins a 32-bit residual stream through a scale per feature and a gate per row and feature, and
// the norm in front of the next sublayer is taken in the same pass:
//
//   residual[r, :] += update[r, :] * scale[:] * sigmoid(gate[r, :] + gate_bias[:])         (all 32-bit)
//   out[r, :]       = residual[r, :] / sqrt(mean(residual[r, :]^2) + eps) * weight[:]       (rounded once; optional)
//
// `gate` holds the logits of the gate's product (32-bit, no bias yet).  One block a row; a thread keeps its share of the
// new row in registers between the statistic and the output where the row is short enough, and reads it back otherwise.
// The order of a row's sum of squares depends on the width alone.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kKeep = 4;            // packets of four a thread keeps: rows of up to 4096 numbers stay in registers

template <typename T>
__global__ void __launch_bounds__(kThreads)
gated_add_norm_kernel(float* __restrict__ residual, const float* __restrict__ update, const float* __restrict__ gate,
                      const float* __restrict__ gate_bias, const float* __restrict__ scale,
                      const float* __restrict__ weight, T* __restrict__ out, int width, float eps) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int64_t at = (int64_t)blockIdx.x * width;
    float* res = residual + at;
    const float* upd = update + at;
    const float* gat = gate + at;
    float ss = 0.0f;
    if (width % 4 == 0) {
        float4 kept[kKeep];
        const int packets = width / 4;
        int n = 0;
        for (int p = threadIdx.x; p < packets; p += kThreads, ++n) {
            const int i = p * 4;
            float4 r = *reinterpret_cast<const float4*>(res + i);
            const float4 u = *reinterpret_cast<const float4*>(upd + i), g = *reinterpret_cast<const float4*>(gat + i);
            const float4 b = *reinterpret_cast<const float4*>(gate_bias + i), s = *reinterpret_cast<const float4*>(scale + i);
            r.x += u.x * s.x * (1.0f / (1.0f + expf(-(g.x + b.x))));
            r.y += u.y * s.y * (1.0f / (1.0f + expf(-(g.y + b.y))));
            r.z += u.z * s.z * (1.0f / (1.0f + expf(-(g.z + b.z))));
            r.w += u.w * s.w * (1.0f / (1.0f + expf(-(g.w + b.w))));
            *reinterpret_cast<float4*>(res + i) = r;
            if (n < kKeep) kept[n] = r;
            ss = fmaf(r.x, r.x, ss); ss = fmaf(r.y, r.y, ss); ss = fmaf(r.z, r.z, ss); ss = fmaf(r.w, r.w, ss);
        }
        if (out == nullptr) return;
        const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
        n = 0;
        for (int p = threadIdx.x; p < packets; p += kThreads, ++n) {
            const int i = p * 4;
            const float4 r = n < kKeep ? kept[n] : *reinterpret_cast<const float4*>(res + i);   // (its own store)
            const float4 w = *reinterpret_cast<const float4*>(weight + i);
            T* to = out + at + i;
            Elem<T>::store(to, r.x * inv * w.x);
            Elem<T>::store(to + 1, r.y * inv * w.y);
            Elem<T>::store(to + 2, r.z * inv * w.z);
            Elem<T>::store(to + 3, r.w * inv * w.w);
        }
        return;
    }
    for (int i = threadIdx.x; i < width; i += kThreads) {
        const float r = res[i] + upd[i] * scale[i] * (1.0f / (1.0f + expf(-(gat[i] + gate_bias[i]))));
        res[i] = r;
        ss = fmaf(r, r, ss);
    }
    if (out == nullptr) return;
    const float inv = 1.0f / sqrtf(block_sum(ss, scratch) / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += kThreads) Elem<T>::store(out + at + i, res[i] * inv * weight[i]);
}

}  // namespace

// residual, update, gate: float32 [rows, width], contiguous; gate_bias, scale, weight: float32 [width]; out: [rows, width]
// in `dtype`, or null together with weight where no norm follows.
TB_EXPORT int tb_gated_add_norm(float* residual, const float* update, const float* gate, const float* gate_bias,
                                const float* scale, const float* weight, void* out, int rows, int width, float eps,
                                int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1 || (out != nullptr && weight == nullptr)) return TB_ERR_BAD_SIZE;
    const uintptr_t bits = (uintptr_t)residual | (uintptr_t)update | (uintptr_t)gate | (uintptr_t)gate_bias |
                           (uintptr_t)scale | (uintptr_t)weight;
    if (width % 4 == 0 && bits % 16 != 0) return TB_ERR_BAD_ALIGN;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(gated_add_norm_kernel<float>, dim3(rows), dim3(kThreads), (size_t)0, stream, residual,
                                 update, gate, gate_bias, scale, weight, (float*)out, width, eps);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(gated_add_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(kThreads), (size_t)0, stream,
                                 residual, update, gate, gate_bias, scale, weight, (__nv_bfloat16*)out, width, eps);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
