// Element-by-element kernels of feed-forwards with biases or other activations than SwiGLU, of scaled embeddings
// and of scaled logits.  All arithmetic is 32-bit; each stored value is rounded once.
//
//   tb_gated_activation   out[t, j] = act(gate[t, j] + bg[j]) * (up[t, j] + bu[j]); gate and up are the two halves
//                         of a row of `gu`; the biases (32-bit, [2 * inter], gate then up) may be null.
//                         act: 0 = SiLU, 1 = GELU in its tanh form
//                         0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))).
//   tb_squared_relu       out[t, j] = max(z[t, j], 0)^2
//   tb_add_bias           y[t, j] += b[j]                      (y 32-bit or bfloat16, b 32-bit)
//   tb_scale_rows         y[t, j] *= s                         (32-bit y)
//   tb_add_rows           a[t, j] += b[t, j]                   (32-bit)
//   tb_blend_rows         a[t, j] = x * a[t, j] + y * b[t, j]  (32-bit: two mixers side by side, each with a weight)
//   tb_sigmoid_mul        out[t, j] = a[t, j] * sigmoid(g[t, j])      (an output gate; 32-bit arithmetic)
//   tb_embedding_scaled   out[t, :] = float(table[token[t], :]) * s   (32-bit out; the table 32-bit or bfloat16)
//   tb_token_gate         out[t, j] = act(z[t, j]) * table[token[t], offset + j]     (32-bit z; a slice of a second
//                         embedding table gated by a projection of the stream)
#include "common.cuh"

namespace {

enum Activation : int { ACT_SILU = 0, ACT_GELU_TANH = 1 };

template <int ACT>
__device__ __forceinline__ float activate(float z) {
    if (ACT == ACT_SILU) return z * (1.0f / (1.0f + expf(-z)));
    const float inner = 0.7978845608028654f * (z + 0.044715f * z * z * z);
    return 0.5f * z * (1.0f + tanhf(inner));
}

template <typename T, int ACT>
__global__ void gated_activation_kernel(const T* __restrict__ gu, int64_t gu_stride, const float* __restrict__ bias,
                                        T* __restrict__ out, int64_t out_stride, int inter) {
    pdl_trigger();
    pdl_wait();
    const T* g = gu + (int64_t)blockIdx.x * gu_stride;
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < inter; j += gridDim.y * blockDim.x) {
        float gv = Elem<T>::load(g + j), uv = Elem<T>::load(g + inter + j);
        if (bias != nullptr) {
            gv += bias[j];
            uv += bias[inter + j];
        }
        Elem<T>::store(o + j, activate<ACT>(gv) * uv);
    }
}

// 16-byte packets of gate and up (inter a multiple of the packet, rows aligned).
template <typename T, int ACT>
__global__ void gated_activation_packets_kernel(const T* __restrict__ gu, int64_t gu_stride,
                                                const float* __restrict__ bias, T* __restrict__ out,
                                                int64_t out_stride, int inter) {
    constexpr int N = Packet<T>::N;
    pdl_trigger();
    pdl_wait();
    const T* g = gu + (int64_t)blockIdx.x * gu_stride;
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * N; j < inter; j += gridDim.y * blockDim.x * N) {
        float gv[N], uv[N], ov[N];
        Packet<T>::load(g + j, gv);
        Packet<T>::load(g + inter + j, uv);
#pragma unroll
        for (int e = 0; e < N; ++e) {
            if (bias != nullptr) {
                gv[e] += bias[j + e];
                uv[e] += bias[inter + j + e];
            }
            ov[e] = activate<ACT>(gv[e]) * uv[e];
        }
        Packet<T>::store(o + j, ov);
    }
}

template <typename T>
__global__ void squared_relu_kernel(const T* __restrict__ z, int64_t z_stride, T* __restrict__ out, int64_t out_stride,
                                    int width) {
    pdl_trigger();
    pdl_wait();
    const T* zr = z + (int64_t)blockIdx.x * z_stride;
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < width; j += gridDim.y * blockDim.x) {
        const float v = fmaxf(Elem<T>::load(zr + j), 0.0f);
        Elem<T>::store(o + j, v * v);
    }
}

template <typename T>
__global__ void add_bias_kernel(T* __restrict__ y, int64_t y_stride, const float* __restrict__ bias, int width) {
    pdl_trigger();
    pdl_wait();
    T* yr = y + (int64_t)blockIdx.x * y_stride;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < width; j += gridDim.y * blockDim.x)
        Elem<T>::store(yr + j, Elem<T>::load(yr + j) + bias[j]);
}

__global__ void scale_rows_kernel(float* __restrict__ y, int64_t total, float s) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        y[i] *= s;
}

__global__ void add_rows_kernel(float* __restrict__ a, const float* __restrict__ b, int64_t total) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        a[i] += b[i];
}

__global__ void blend_rows_kernel(float* __restrict__ a, const float* __restrict__ b, int64_t total, float x, float y) {
    pdl_trigger();
    pdl_wait();
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
        a[i] = x * a[i] + y * b[i];
}

template <typename T>
__global__ void sigmoid_mul_kernel(const T* __restrict__ a, int64_t a_stride, const T* __restrict__ g, int64_t g_stride,
                                   T* __restrict__ out, int64_t out_stride, int width) {
    pdl_trigger();
    pdl_wait();
    const T* ar = a + (int64_t)blockIdx.x * a_stride;
    const T* gr = g + (int64_t)blockIdx.x * g_stride;
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < width; j += gridDim.y * blockDim.x)
        Elem<T>::store(o + j, Elem<T>::load(ar + j) * (1.0f / (1.0f + expf(-Elem<T>::load(gr + j)))));
}

// 16-byte packets of a, g and out (width a multiple of the packet, rows aligned).
template <typename T>
__global__ void sigmoid_mul_packets_kernel(const T* __restrict__ a, int64_t a_stride, const T* __restrict__ g, int64_t g_stride,
                                           T* __restrict__ out, int64_t out_stride, int width) {
    constexpr int N = Packet<T>::N;
    pdl_trigger();
    pdl_wait();
    const T* ar = a + (int64_t)blockIdx.x * a_stride;
    const T* gr = g + (int64_t)blockIdx.x * g_stride;
    T* o = out + (int64_t)blockIdx.x * out_stride;
    for (int j = (blockIdx.y * blockDim.x + threadIdx.x) * N; j < width; j += gridDim.y * blockDim.x * N) {
        float av[N], gv[N];
        Packet<T>::load(ar + j, av);
        Packet<T>::load(gr + j, gv);
#pragma unroll
        for (int e = 0; e < N; ++e) av[e] *= 1.0f / (1.0f + expf(-gv[e]));
        Packet<T>::store(o + j, av);
    }
}

template <typename T>
__global__ void embedding_scaled_kernel(const int* __restrict__ tokens, const T* __restrict__ table,
                                        float* __restrict__ out, int hidden, int vocab, float s) {
    pdl_trigger();
    pdl_wait();                                   // the token ids may come from the kernel in front
    int from = tokens[blockIdx.x];
    if (from < 0 || from >= vocab) from = 0;      // the host validates; never read out of bounds
    const T* src = table + (int64_t)from * hidden;
    float* dst = out + (int64_t)blockIdx.x * hidden;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = Elem<T>::load(src + i) * s;
}

template <typename T, int ACT>
__global__ void token_gate_kernel(const float* __restrict__ z, const int* __restrict__ tokens,
                                  const T* __restrict__ table, int64_t table_stride, int offset, T* __restrict__ out,
                                  int width, int vocab) {
    pdl_trigger();
    pdl_wait();
    int from = tokens[blockIdx.x];
    if (from < 0 || from >= vocab) from = 0;      // the host validates; never read out of bounds
    const T* e = table + (int64_t)from * table_stride + offset;
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        Elem<T>::store(out + (int64_t)blockIdx.x * width + j,
                       activate<ACT>(z[(int64_t)blockIdx.x * width + j]) * Elem<T>::load(e + j));
}

inline dim3 row_grid(int rows, int width, int threads, int per_thread = 1) {
    int by = (width + threads * per_thread - 1) / (threads * per_thread);
    if (by > 64) by = 64;
    if (by < 1) by = 1;
    return dim3(rows, by);
}

inline int grid_for(int64_t total, int threads) {
    int64_t blocks = (total + threads - 1) / threads;
    return (int)(blocks > 148 * 16 ? 148 * 16 : (blocks < 1 ? 1 : blocks));
}

template <typename T, int ACT>
int launch_gated(const void* gu, int64_t gu_stride, const float* bias, void* out, int64_t out_stride, int rows, int inter,
                 cudaStream_t stream) {
    constexpr int N = Packet<T>::N;
    const int threads = 256;
    const bool packets = inter % N == 0 && gu_stride % N == 0 && out_stride % N == 0 &&
                         ((uintptr_t)gu | (uintptr_t)out) % 16 == 0;
    cudaError_t launched;
    if (packets)
        launched = tb_launch_pdl(gated_activation_packets_kernel<T, ACT>, row_grid(rows, inter, threads, N), dim3(threads),
                                 0, stream, (const T*)gu, gu_stride, bias, (T*)out, out_stride, inter);
    else
        launched = tb_launch_pdl(gated_activation_kernel<T, ACT>, row_grid(rows, inter, threads), dim3(threads), 0,
                                 stream, (const T*)gu, gu_stride, bias, (T*)out, out_stride, inter);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

}  // namespace

TB_EXPORT int tb_gated_activation(const void* gu, int64_t gu_stride, const float* bias, void* out, int64_t out_stride,
                                  int rows, int inter, int activation, int dtype, cudaStream_t stream) {
    if (rows == 0 || inter == 0) return 0;
    if (activation != ACT_SILU && activation != ACT_GELU_TANH) return TB_ERR_BAD_SIZE;
    if (dtype == TB_F32)
        return activation == ACT_SILU
                   ? launch_gated<float, ACT_SILU>(gu, gu_stride, bias, out, out_stride, rows, inter, stream)
                   : launch_gated<float, ACT_GELU_TANH>(gu, gu_stride, bias, out, out_stride, rows, inter, stream);
    if (dtype == TB_BF16)
        return activation == ACT_SILU
                   ? launch_gated<__nv_bfloat16, ACT_SILU>(gu, gu_stride, bias, out, out_stride, rows, inter, stream)
                   : launch_gated<__nv_bfloat16, ACT_GELU_TANH>(gu, gu_stride, bias, out, out_stride, rows, inter, stream);
    return TB_ERR_BAD_DTYPE;
}

TB_EXPORT int tb_squared_relu(const void* z, int64_t z_stride, void* out, int64_t out_stride, int rows, int width,
                              int dtype, cudaStream_t stream) {
    if (rows == 0 || width == 0) return 0;
    const int threads = 256;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(squared_relu_kernel<float>, row_grid(rows, width, threads), dim3(threads), 0, stream,
                                 (const float*)z, z_stride, (float*)out, out_stride, width);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(squared_relu_kernel<__nv_bfloat16>, row_grid(rows, width, threads), dim3(threads), 0,
                                 stream, (const __nv_bfloat16*)z, z_stride, (__nv_bfloat16*)out, out_stride, width);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

TB_EXPORT int tb_add_bias(void* y, int64_t y_stride, const float* bias, int rows, int width, int dtype,
                          cudaStream_t stream) {
    if (rows == 0 || width == 0) return 0;
    const int threads = 256;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(add_bias_kernel<float>, row_grid(rows, width, threads), dim3(threads), 0, stream,
                                 (float*)y, y_stride, bias, width);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(add_bias_kernel<__nv_bfloat16>, row_grid(rows, width, threads), dim3(threads), 0, stream,
                                 (__nv_bfloat16*)y, y_stride, bias, width);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

TB_EXPORT int tb_scale_rows(float* y, int64_t total, float s, cudaStream_t stream) {
    if (total == 0) return 0;
    cudaError_t launched = tb_launch_pdl(scale_rows_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, y, total, s);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

TB_EXPORT int tb_add_rows(float* a, const float* b, int64_t total, cudaStream_t stream) {
    if (total == 0) return 0;
    cudaError_t launched = tb_launch_pdl(add_rows_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, a, b, total);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

template <typename T>
static cudaError_t launch_sigmoid_mul(const void* a, int64_t a_stride, const void* g, int64_t g_stride, void* out, int64_t out_stride,
                               int rows, int width, cudaStream_t stream) {
    constexpr int N = Packet<T>::N;
    const int threads = 256;
    const bool packets = width % N == 0 && a_stride % N == 0 && g_stride % N == 0 && out_stride % N == 0 &&
                         ((uintptr_t)a | (uintptr_t)g | (uintptr_t)out) % 16 == 0;
    if (packets)
        return tb_launch_pdl(sigmoid_mul_packets_kernel<T>, row_grid(rows, width, threads, N), dim3(threads), 0, stream,
                             (const T*)a, a_stride, (const T*)g, g_stride, (T*)out, out_stride, width);
    return tb_launch_pdl(sigmoid_mul_kernel<T>, row_grid(rows, width, threads), dim3(threads), 0, stream, (const T*)a,
                         a_stride, (const T*)g, g_stride, (T*)out, out_stride, width);
}

TB_EXPORT int tb_blend_rows(float* a, const float* b, int64_t total, float x, float y, cudaStream_t stream) {
    if (total == 0) return 0;
    cudaError_t launched = tb_launch_pdl(blend_rows_kernel, dim3(grid_for(total, 256)), dim3(256), 0, stream, a, b, total, x, y);
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

TB_EXPORT int tb_sigmoid_mul(const void* a, int64_t a_stride, const void* g, int64_t g_stride, void* out, int64_t out_stride,
                             int rows, int width, int dtype, cudaStream_t stream) {
    if (rows == 0 || width == 0) return 0;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = launch_sigmoid_mul<float>(a, a_stride, g, g_stride, out, out_stride, rows, width, stream);
    else if (dtype == TB_BF16)
        launched = launch_sigmoid_mul<__nv_bfloat16>(a, a_stride, g, g_stride, out, out_stride, rows, width, stream);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

TB_EXPORT int tb_embedding_scaled(const int* tokens, const void* table, int table_dtype, float* out, int rows, int hidden,
                                  int vocab, float s, cudaStream_t stream) {
    if (rows == 0) return 0;
    cudaError_t launched;
    if (table_dtype == TB_F32)
        launched = tb_launch_pdl(embedding_scaled_kernel<float>, dim3(rows), dim3(256), 0, stream, tokens,
                                 (const float*)table, out, hidden, vocab, s);
    else if (table_dtype == TB_BF16)
        launched = tb_launch_pdl(embedding_scaled_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, tokens,
                                 (const __nv_bfloat16*)table, out, hidden, vocab, s);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// z: float32 [rows, width]; table: [vocab, table_stride] in `dtype`, the row's slice starts at column `offset`;
// out: [rows, width] in `dtype`.
TB_EXPORT int tb_token_gate(const float* z, const int* tokens, const void* table, int64_t table_stride, int offset,
                            void* out, int rows, int width, int vocab, int activation, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (width < 1 || offset < 0 || offset + width > table_stride) return TB_ERR_BAD_SIZE;
    if (activation != ACT_SILU && activation != ACT_GELU_TANH) return TB_ERR_BAD_SIZE;
    const int threads = width >= 256 ? 256 : ((width + 31) / 32) * 32;
    cudaError_t launched;
#define TB_RUN(T, ACT)                                                                                                \
    launched = tb_launch_pdl(token_gate_kernel<T, ACT>, dim3(rows), dim3(threads), 0, stream, z, tokens, (const T*)table, \
                             table_stride, offset, (T*)out, width, vocab)
    if (dtype == TB_F32) { if (activation == ACT_SILU) TB_RUN(float, ACT_SILU); else TB_RUN(float, ACT_GELU_TANH); }
    else if (dtype == TB_BF16) { if (activation == ACT_SILU) TB_RUN(__nv_bfloat16, ACT_SILU); else TB_RUN(__nv_bfloat16, ACT_GELU_TANH); }
    else return TB_ERR_BAD_DTYPE;
#undef TB_RUN
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
