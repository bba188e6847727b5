// Causal grouped-query attention over the paged cache for any head size (multiples of 8
// up to 256) and either storage type, written with plain loads and float32 arithmetic.
// It serves the float32 path of the whole model and every shape the tensor-core kernels
// refuse.  One warp owns one (query row, query head); keys are taken 32 at a time, one per
// lane, with the online softmax of the reference's split kernel
// (engine/kernels/attention.py:40-137: m' = max(m, rowmax), c = exp(m - m'),
// l = l*c + sum p, acc = acc*c + p.V) and its mask `key <= position of the query`.
#include "common.cuh"

namespace dfi {

constexpr int kGenericWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void attention_generic_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out,
                                         int out_row_stride, const T* __restrict__ k_cache,
                                         const T* __restrict__ v_cache, const int* __restrict__ block_table,
                                         int table_width, const int* __restrict__ row_seq,
                                         const int* __restrict__ row_pos, int n_q, int n_kv, int D, int page_size,
                                         int ring_tokens, int window, float scale) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float q_s[kGenericWarps][kMaxHeadDim];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * kGenericWarps + warp;
    const int row = blockIdx.x;
    if (head >= n_q) return;
    const int kv_head = head / (n_q / n_kv);
    const int pos = row_pos[row];
    const int* table = block_table + (size_t)row_seq[row] * table_width;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;

    const T* q_row = q + (size_t)row * q_row_stride + (size_t)head * D;
    for (int d = lane; d < D; d += 32) q_s[warp][d] = to_float(q_row[d]) * scale;
    __syncwarp();

    constexpr int n = Vec16<T>::n;
    float acc[kMaxHeadDim / 32];
#pragma unroll
    for (int j = 0; j < kMaxHeadDim / 32; ++j) acc[j] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int base = first; base <= pos; base += 32) {
        const int key = base + lane;
        const bool live = key <= pos;
        unsigned long long offset = 0;
        float s = -INFINITY;
        if (live) {
            const int place = place_of(key, ring_tokens);
            const int page = table[place / page_size];
            offset = (((unsigned long long)page * n_kv + kv_head) * page_size + place % page_size) * D;
            const T* kp = k_cache + offset;
            float dot = 0.f;
            for (int d = 0; d < D; d += n) {
                float kv[n];
                load16(kp + d, kv);
#pragma unroll
                for (int e = 0; e < n; ++e) dot += q_s[warp][d + e] * kv[e];
            }
            s = dot;
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);  // m = -inf on the first tile gives 0
        const float p = live ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int j = 0; j < kMaxHeadDim / 32; ++j) acc[j] *= corr;
        m = m_new;
        const int count = min(32, pos - base + 1);
        for (int kk = 0; kk < count; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            const unsigned long long off = __shfl_sync(0xffffffffu, offset, kk);
            const T* vp = v_cache + off;
#pragma unroll
            for (int j = 0; j < kMaxHeadDim / 32; ++j) {
                const int d = lane + 32 * j;
                if (d < D) acc[j] += pk * to_float(vp[d]);
            }
        }
    }
    T* o = out + (size_t)row * out_row_stride + (size_t)head * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int j = 0; j < kMaxHeadDim / 32; ++j) {
        const int d = lane + 32 * j;
        if (d < D) o[d] = from_float<T>(acc[j] * inv);
    }
}

}  // namespace dfi

using namespace dfi;

// q [rows, q_row_stride] holds n_q heads of head_dim per row (already normalised and
// rotated); out [rows, out_row_stride].  row_seq gives each row's line of block_table and
// row_pos its absolute position; the cache already holds the keys up to that position.
DFI_EXPORT int dfi_attention_generic(const void* q, int q_row_stride, void* out, int out_row_stride,
                                     const void* k_cache, const void* v_cache, const int* block_table,
                                     int table_width, const int* row_seq, const int* row_pos, int rows, int n_q,
                                     int n_kv, int head_dim, int page_size, int ring_tokens, int window,
                                     float scale, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (head_dim <= 0 || head_dim > kMaxHeadDim || n_q <= 0 || n_kv <= 0 || n_q % n_kv) return DFI_ERR_SHAPE;
    if (page_size <= 0 || table_width <= 0 || window < 0 || ring_tokens < 0) return DFI_ERR_SHAPE;
    const int vec = dtype == DFI_DTYPE_F32 ? 4 : 8;
    if (head_dim % vec) return DFI_ERR_SHAPE;
    if (!aligned16(k_cache) || !aligned16(v_cache)) return DFI_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid(rows, (n_q + kGenericWarps - 1) / kGenericWarps);
    if (grid.y > 65535) return DFI_ERR_LIMIT;
    if (dtype == DFI_DTYPE_F32)
        launch(attention_generic_kernel<float>, grid, kGenericWarps * 32, 0, st, 
            (const float*)q, q_row_stride, (float*)out, out_row_stride, (const float*)k_cache,
            (const float*)v_cache, block_table, table_width, row_seq, row_pos, n_q, n_kv, head_dim, page_size,
            ring_tokens, window, scale);
    else if (dtype == DFI_DTYPE_BF16)
        launch(attention_generic_kernel<bf16>, grid, kGenericWarps * 32, 0, st, 
            (const bf16*)q, q_row_stride, (bf16*)out, out_row_stride, (const bf16*)k_cache,
            (const bf16*)v_cache, block_table, table_width, row_seq, row_pos, n_q, n_kv, head_dim, page_size,
            ring_tokens, window, scale);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
