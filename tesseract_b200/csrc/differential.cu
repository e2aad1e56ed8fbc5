// Attention with two score maps per head over the same values: rotation and cache write in front of the attention
// kernel, and the combination of the two maps' outputs behind it.
//
//   tb_pair_rope_cache       neighbouring pairs (2i, 2i + 1) of the first rot_dims numbers of every query and key head
//                            turn by position * inv_freq[i] (angle, sine and cosine 32-bit); queries go to q_out, keys
//                            and values into the row's page.  Key heads and value heads are counted apart: a page is
//                            [key_heads][page][dim] keys followed by [value_heads][page][vdim] values.
//   tb_differential_combine  o = a1 - lambda a2 per head, o / sqrt(mean(o^2) + eps) * post, times sigmoid(gate):
//                            32-bit from the 32-bit outputs of the two maps, rounded once.  The attention kernel saw
//                            the maps as query heads laid out [kv head][map][head within the group]; the result is laid
//                            out by head.
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
pair_rope_cache_kernel(const T* __restrict__ proj, int64_t proj_stride, T* __restrict__ q_out, int64_t q_stride,
                       T* __restrict__ cache, const int* __restrict__ positions, const int* __restrict__ seq_of_row,
                       const int* __restrict__ block_table, int bt_stride, const float* __restrict__ inv_freq,
                       int q_heads, int key_heads, int value_heads, int dim, int vdim, int rot_dims, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const int pos = positions[row];
    const int seq = seq_of_row[row];
    const int64_t page = block_table[(int64_t)seq * bt_stride + pos / page_size];
    const int in_page = pos % page_size;
    const int64_t page_elems = (int64_t)page_size * ((int64_t)key_heads * dim + (int64_t)value_heads * vdim);
    T* keys = cache + page * page_elems;
    T* values = keys + (int64_t)key_heads * page_size * dim;
    const T* src = proj + (int64_t)row * proj_stride;
    const int half = (dim + 1) / 2;                  // slots of a head: pairs, and a last single number if dim is odd
    const int qk_slots = (q_heads + key_heads) * half;
    for (int e = threadIdx.x; e < qk_slots; e += blockDim.x) {
        const int head = e / half, i = e % half;
        const int c = 2 * i;
        const T* from = src + (int64_t)head * dim + c;            // queries then keys lie side by side in proj
        T* to = head < q_heads ? q_out + (int64_t)row * q_stride + (int64_t)head * dim + c
                               : keys + ((int64_t)(head - q_heads) * page_size + in_page) * dim + c;
        const float u = Elem<T>::load(from);
        if (c + 1 >= dim) {                          // the odd last number of a head passes
            Elem<T>::store(to, u);
            continue;
        }
        const float v = Elem<T>::load(from + 1);
        if (c + 1 < rot_dims) {
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            Elem<T>::store(to, u * cs - v * sn);
            Elem<T>::store(to + 1, v * cs + u * sn);
        } else {
            Elem<T>::store(to, u);
            Elem<T>::store(to + 1, v);
        }
    }
    const T* vsrc = src + (int64_t)(q_heads + key_heads) * dim;
    for (int e = threadIdx.x; e < value_heads * vdim; e += blockDim.x) {
        const int head = e / vdim, c = e % vdim;
        values[((int64_t)head * page_size + in_page) * vdim + c] = vsrc[e];
    }
}

// one warp per (row, head)
template <typename T>
__global__ void __launch_bounds__(128)
differential_combine_kernel(const float* __restrict__ maps, const T* __restrict__ gate, int64_t gate_stride,
                            T* __restrict__ out, int rows, int heads, int kv_heads, int vdim, float lambda, float post,
                            float eps) {
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)rows * heads) return;
    const int row = (int)(item / heads), head = (int)(item % heads);
    const int per = heads / kv_heads;
    const int g = head / per, within = head % per;
    const float* first = maps + ((int64_t)row * 2 * heads + (int64_t)(g * 2) * per + within) * vdim;
    const float* second = first + (int64_t)per * vdim;
    float ss = 0.0f;
    for (int c = lane; c < vdim; c += 32) {
        const float o = first[c] - lambda * second[c];
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = post / sqrtf(ss / (float)vdim + eps);
    const T* grow = gate == nullptr ? nullptr : gate + (int64_t)row * gate_stride + (int64_t)head * vdim;
    T* orow = out + ((int64_t)row * heads + head) * vdim;
    for (int c = lane; c < vdim; c += 32) {
        float o = (first[c] - lambda * second[c]) * inv;
        if (grow != nullptr) o *= 1.0f / (1.0f + expf(-Elem<T>::load(grow + c)));
        Elem<T>::store(orow + c, o);
    }
}

}  // namespace

// proj: [rows, q_heads * dim | key_heads * dim | value_heads * vdim | ...] (row stride proj_stride, elements).
TB_EXPORT int tb_pair_rope_cache(const void* proj, int64_t proj_stride, void* q_out, int64_t q_stride, void* cache,
                                 const int* positions, const int* seq_of_row, const int* block_table, int bt_stride,
                                 const float* inv_freq, int rows, int q_heads, int key_heads, int value_heads, int dim,
                                 int vdim, int rot_dims, int page_size, int dtype, cudaStream_t stream) {
    if (rows == 0) return 0;
    if (q_heads < 1 || key_heads < 1 || value_heads < 1 || dim < 1 || vdim < 1 || page_size < 1) return TB_ERR_BAD_SIZE;
    if (rot_dims < 0 || rot_dims % 2 || rot_dims > dim || (rot_dims > 0 && inv_freq == nullptr)) return TB_ERR_BAD_SIZE;
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(pair_rope_cache_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)proj,
                                 proj_stride, (float*)q_out, q_stride, (float*)cache, positions, seq_of_row, block_table,
                                 bt_stride, inv_freq, q_heads, key_heads, value_heads, dim, vdim, rot_dims, page_size);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(pair_rope_cache_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream,
                                 (const __nv_bfloat16*)proj, proj_stride, (__nv_bfloat16*)q_out, q_stride,
                                 (__nv_bfloat16*)cache, positions, seq_of_row, block_table, bt_stride, inv_freq, q_heads,
                                 key_heads, value_heads, dim, vdim, rot_dims, page_size);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}

// maps: float32 [rows, 2 * heads * vdim], query heads laid out [kv head][map][head within the group]; gate: null or
// [rows, heads * vdim] in `dtype` (row stride gate_stride); out: [rows, heads * vdim] in `dtype`, laid out by head.
TB_EXPORT int tb_differential_combine(const float* maps, const void* gate, int64_t gate_stride, void* out, int rows,
                                      int heads, int kv_heads, int vdim, float lambda, float post, float eps, int dtype,
                                      cudaStream_t stream) {
    if (rows == 0) return 0;
    if (heads < 1 || kv_heads < 1 || heads % kv_heads || vdim < 1) return TB_ERR_BAD_SIZE;
    const int64_t items = (int64_t)rows * heads;
    const dim3 grid((unsigned)((items + 3) / 4));
    cudaError_t launched;
    if (dtype == TB_F32)
        launched = tb_launch_pdl(differential_combine_kernel<float>, grid, dim3(128), 0, stream, maps, (const float*)gate,
                                 gate_stride, (float*)out, rows, heads, kv_heads, vdim, lambda, post, eps);
    else if (dtype == TB_BF16)
        launched = tb_launch_pdl(differential_combine_kernel<__nv_bfloat16>, grid, dim3(128), 0, stream, maps,
                                 (const __nv_bfloat16*)gate, gate_stride, (__nv_bfloat16*)out, rows, heads, kv_heads, vdim,
                                 lambda, post, eps);
    else
        return TB_ERR_BAD_DTYPE;
    return launched == cudaSuccess ? tb_launch_status() : (int)launched;
}
