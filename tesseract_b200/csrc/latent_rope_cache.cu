// Attention over a latent vector per token: what stands between the projections and the attention kernel.
//
// Per row the down projection gives `rank` numbers, which are divided by their root mean square and weighted (the
// latent c), and `rot_width` numbers that are one rotated key part shared by all heads.  The page keeps, per token,
// [c | rotated part]: one "key" of rank + rot_width numbers whose first `rank` numbers are also the "value" (scores and
// outputs are taken in the latent space: the per-head key and value matrices are applied to the query in front of the
// attention kernel and to its output behind it).  A query row is [heads][rank + rot_width]: the first `rank` numbers
// of a head are written by the product in front, this kernel fills in the head's rotated part.
//
// Rotation: neighbouring pairs (2i, 2i + 1) of the first rot_dims numbers of the rotated part turn by
// position * inv_freq[i], cosine and sine both multiplied by `amplitude`; angle, sine, cosine and the norm are 32-bit;
// every stored number is rounded once.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
latent_rope_cache_kernel(const float* __restrict__ down, int64_t down_stride, const T* __restrict__ q,
                         int64_t q_stride, T* __restrict__ q_full, int64_t full_stride, T* __restrict__ cache,
                         const float* __restrict__ weight, const int* __restrict__ positions,
                         const int* __restrict__ seq_of_row, const int* __restrict__ block_table, int bt_stride,
                         const float* __restrict__ inv_freq, int heads, int dim, int rank, int rot_width, int rot_dims,
                         int page_size, float eps, float amplitude) {
    __shared__ float scratch[32];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    const int64_t page = block_table[(int64_t)seq * bt_stride + pos / page_size];
    const int width = rank + rot_width;
    T* entry = cache + (page * page_size + pos % page_size) * width;
    const float* drow = down + (int64_t)row * down_stride;
    float ss = 0.0f;
    for (int j = threadIdx.x; j < rank; j += blockDim.x) ss = fmaf(drow[j], drow[j], ss);
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)rank + eps);
    for (int j = threadIdx.x; j < rank; j += blockDim.x) Elem<T>::store(entry + j, drow[j] * inv * weight[j]);
    // slot 0 .. half-1 of "head" -1 is the shared key part, then the heads' query parts
    const int half = (rot_width + 1) / 2;
    for (int e = threadIdx.x; e < (heads + 1) * half; e += blockDim.x) {
        const int head = e / half - 1, i = e % half;
        const int c = 2 * i;
        float u, v = 0.0f;
        T* to;
        if (head < 0) {
            u = drow[rank + c];
            if (c + 1 < rot_width) v = drow[rank + c + 1];
            to = entry + rank + c;
        } else {
            const T* from = q + (int64_t)row * q_stride + (int64_t)head * (dim + rot_width) + dim + c;
            u = Elem<T>::load(from);
            if (c + 1 < rot_width) v = Elem<T>::load(from + 1);
            to = q_full + (int64_t)row * full_stride + (int64_t)head * width + rank + c;
        }
        if (c + 1 >= rot_width) {
            Elem<T>::store(to, u);
            continue;
        }
        if (c + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            sn *= amplitude;
            cs *= amplitude;
            Elem<T>::store(to, u * cs - v * sn);
            Elem<T>::store(to + 1, v * cs + u * sn);
        } else {
            Elem<T>::store(to, u);
            Elem<T>::store(to + 1, v);
        }
    }
}

}  // namespace

// down: float32 [rows, rank + rot_width]; q: [rows, heads * (dim + rot_width)]; q_full: [rows, heads * (rank + rot_width)]
// (only the rotated parts are written); cache: pages of [page_size][rank + rot_width]; weight: float32 [rank].
TB_EXPORT int tb_latent_rope_cache(const float* down, int64_t down_stride, const void* q, int64_t q_stride, void* q_full,
                                   int64_t full_stride, void* cache, const float* weight, const int* positions,
                                   const int* seq_of_row, const int* block_table, int bt_stride, const float* inv_freq,
                                   int rows, int heads, int dim, int rank, int rot_width, int rot_dims, int page_size,
                                   float eps, float amplitude, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (heads < 1 || dim < 0 || rank < 1 || rot_width < 0 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > rot_width || (rot_dims > 0 && inv_freq == nullptr)) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(latent_rope_cache_kernel<float>, dim3(rows), dim3(256), 0, stream, down, down_stride,
                                 (const float*)q, q_stride, (float*)q_full, full_stride, (float*)cache, weight, positions,
                                 seq_of_row, block_table, bt_stride, inv_freq, heads, dim, rank, rot_width, rot_dims,
                                 page_size, eps, amplitude);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(latent_rope_cache_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, down,
                                 down_stride, (const __nv_bfloat16*)q, q_stride, (__nv_bfloat16*)q_full, full_stride,
                                 (__nv_bfloat16*)cache, weight, positions, seq_of_row, block_table, bt_stride, inv_freq,
                                 heads, dim, rank, rot_width, rot_dims, page_size, eps, amplitude);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
