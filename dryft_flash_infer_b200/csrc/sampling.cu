// Token selection from float32 logits on the device: argmax (lowest index on ties, as
// engine/engine.py:1026 and :1046 take it) and sampling at a temperature by inverse CDF
// over softmax(logits / temperature).  One block per row; the order of every sum is fixed
// by the thread layout alone, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

namespace dfi {

constexpr int kSampleThreads = 1024;

constexpr int kArgmaxParts = 64;       // CTAs that share one row
constexpr int kArgmaxMaxRows = 4096;   // rows the arrival counters cover

// Arrival counters of the rows (zero between calls) and the parts' candidates.
__device__ int g_argmax_counters[kArgmaxMaxRows];
__device__ float g_argmax_value[kArgmaxMaxRows * kArgmaxParts];
__device__ int g_argmax_index[kArgmaxMaxRows * kArgmaxParts];

__device__ __forceinline__ void keep_better(float& v, int& idx, float ov, int oi) {
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
}

// grid (parts, rows).  Each CTA finds the best of its share of the row; the CTA that arrives last
// (a ticket per row, no waiting) reduces the parts' candidates in index order and writes the row's
// result, so the choice does not depend on which CTA finished when.
__global__ void argmax_kernel(const float* __restrict__ logits, int row_stride, int vocab, int* __restrict__ out) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    __shared__ int ticket_s;
    const int row = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
    const float* x = logits + (size_t)row * row_stride;
    const int per = (vocab + parts - 1) / parts;
    const int begin = min(vocab, part * per), end = min(vocab, begin + per);
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) keep_better(v, idx, x[i], i);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        v = lane < n_warps ? best_v[lane] : -INFINITY;
        idx = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
            keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
        if (lane == 0) {
            g_argmax_value[row * kArgmaxParts + part] = v;
            g_argmax_index[row * kArgmaxParts + part] = idx;
            __threadfence();
            ticket_s = atomicAdd(&g_argmax_counters[row], 1);
        }
    }
    __syncthreads();
    if (ticket_s != parts - 1 || warp != 0) return;
    __threadfence();
    v = -INFINITY;
    idx = 0x7fffffff;
    for (int p = lane; p < parts; p += 32)
        keep_better(v, idx, __ldcg(&g_argmax_value[row * kArgmaxParts + p]), __ldcg(&g_argmax_index[row * kArgmaxParts + p]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        keep_better(v, idx, __shfl_xor_sync(0xffffffffu, v, o), __shfl_xor_sync(0xffffffffu, idx, o));
    if (lane == 0) {
        out[row] = idx == 0x7fffffff ? 0 : idx;
        g_argmax_counters[row] = 0;
    }
}

// Each thread owns a contiguous chunk of the vocabulary.  Pass 1: row maximum.  Pass 2:
// the chunk's sum of exp((x - max) / T).  A scan over the chunk sums finds the chunk in
// which the running sum passes u * total; its owner walks the chunk to the element.
__global__ void sample_temperature_kernel(const float* __restrict__ logits, int row_stride, int vocab,
                                          const float* __restrict__ uniforms, float inv_temperature,
                                          int* __restrict__ out) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float scratch[32];
    __shared__ float sums[kSampleThreads];
    __shared__ float warp_tot[32];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    const int chunk = (vocab + kSampleThreads - 1) / kSampleThreads;
    const int begin = min(vocab, (int)threadIdx.x * chunk), end = min(vocab, begin + chunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    float mx = -INFINITY;
    for (int i = begin; i < end; ++i) mx = fmaxf(mx, x[i]);
    mx = warp_max(mx);
    if (lane == 0) scratch[warp] = mx;
    __syncthreads();
    mx = warp_max(scratch[lane]);
    __syncthreads();

    float mine = 0.f;
    for (int i = begin; i < end; ++i) mine += expf((x[i] - mx) * inv_temperature);
    sums[threadIdx.x] = mine;
    // inclusive scan inside each warp, then over the warps' totals
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    float before_warp = 0.f, total = 0.f;
    for (int w = 0; w < 32; ++w) {
        if (w < warp) before_warp += warp_tot[w];
        total += warp_tot[w];
    }
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = 0.f;
    // before + mine of one thread is bit for bit the `before` of the next: no gaps, no overlaps
    const float before = before_warp + excl;
    const float upto = before_warp + incl;
    const float target = uniforms[blockIdx.x] * total;
    __shared__ int chosen;
    if (threadIdx.x == 0) chosen = -1;
    __syncthreads();
    if (mine > 0.f && target >= before && target < upto) {
        float run = before;
        int pick = end - 1;
        for (int i = begin; i < end; ++i) {
            run += expf((x[i] - mx) * inv_temperature);
            if (target < run) { pick = i; break; }
        }
        atomicMax(&chosen, pick);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int pick = chosen;
        if (pick < 0) {
            // rounding left the target at or past the total: take the last element with weight
            pick = 0;
            for (int t = kSampleThreads - 1; t >= 0; --t)
                if (sums[t] > 0.f) {
                    const int b = min(vocab, t * chunk), e = min(vocab, b + chunk);
                    pick = e - 1;
                    for (int i = e - 1; i >= b; --i)
                        if (expf((x[i] - mx) * inv_temperature) > 0.f) { pick = i; break; }
                    break;
                }
        }
        out[blockIdx.x] = pick;
    }
}

}  // namespace dfi

using namespace dfi;

DFI_EXPORT int dfi_argmax(const float* logits, int rows, int row_stride, int vocab, int* out, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (vocab <= 0) return DFI_ERR_SHAPE;
    for (int first = 0; first < rows; first += kArgmaxMaxRows) {
        const int n = rows - first < kArgmaxMaxRows ? rows - first : kArgmaxMaxRows;
        const int parts = vocab >= 8192 ? kArgmaxParts : 1;
        launch(argmax_kernel, dim3(parts, n), 256, 0, (cudaStream_t)stream, logits + (size_t)first * row_stride, row_stride,
               vocab, out + first);
    }
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// uniforms [rows] in [0, 1); temperature > 0.
DFI_EXPORT int dfi_sample_temperature(const float* logits, int rows, int row_stride, int vocab,
                                      const float* uniforms, float temperature, int* out, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (vocab <= 0 || !(temperature > 0.f)) return DFI_ERR_SHAPE;
    launch(sample_temperature_kernel, rows, kSampleThreads, 0, (cudaStream_t)stream, 
        logits, row_stride, vocab, uniforms, 1.0f / temperature, out);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
