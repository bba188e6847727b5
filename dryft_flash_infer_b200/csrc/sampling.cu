// Token selection from float32 logits on the device: argmax (lowest index on ties, as
// engine/engine.py:1026 and :1046 take it) and sampling at a temperature by inverse CDF
// over softmax(logits / temperature).  One block per row; the order of every sum is fixed
// by the thread layout alone, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

namespace dfi {

constexpr int kSampleThreads = 1024;

__global__ void argmax_kernel(const float* __restrict__ logits, int row_stride, int vocab, int* __restrict__ out) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* x = logits + (size_t)blockIdx.x * row_stride;
    float v = -INFINITY;
    int idx = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float c = x[i];
        if (c > v || (c == v && i < idx)) { v = c; idx = i; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (lane == 0) { best_v[warp] = v; best_i[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        const int n_warps = blockDim.x >> 5;
        v = lane < n_warps ? best_v[lane] : -INFINITY;
        idx = lane < n_warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
        }
        if (lane == 0) out[blockIdx.x] = idx == 0x7fffffff ? 0 : idx;
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
    launch(argmax_kernel, rows, 1024, 0, (cudaStream_t)stream, logits, row_stride, vocab, out);
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
