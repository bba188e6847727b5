// Token selection from float32 logits on the device: argmax (lowest index on ties, as
// engine/engine.py:1026 and :1046 take it) and sampling at a temperature by inverse CDF
// over softmax(logits / temperature).  Several CTAs share a row; the order of every sum is fixed
// by the layout alone, so a row's result does not depend on what else is in the batch.
#include "common.cuh"

namespace dfi {

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

// Sampling at a temperature: a row's vocabulary is cut into segments of at most kSegment logits, one CTA
// each (grid: segments x rows).  A CTA brings its segment into shared memory with coalesced loads and
// works out the segment's maximum m and the sum s of exp((x - m) / T), every thread over a short contiguous
// run of the segment and the runs' sums scanned in the order of the indices.  The CTA that arrives last at
// the row's ticket puts the segments' sums on the scale of the row's maximum, adds them in index order,
// finds the segment in which the running sum passes u * total, brings that segment in again, repeats its
// scan (the same instructions on the same numbers: the same sums) and walks the one run that holds the
// target.  Nothing depends on which CTA arrived when, nor on the other rows of the batch.
constexpr int kSegment = 4096;             // logits per segment: 16 KB of shared memory
constexpr int kSegThreads = 256;
constexpr int kMaxSegments = 1024;         // per row: a vocabulary of up to four million
constexpr int kSampleMaxRows = 256;        // rows per launch (more rows: more launches)
__device__ int g_sample_counters[kSampleMaxRows];
__device__ float g_sample_max[kSampleMaxRows * kMaxSegments];
__device__ float g_sample_sum[kSampleMaxRows * kMaxSegments];

// The segment [begin, end) of row x in shared memory, its maximum, and the scan of its runs' sums:
// thread t's run is elements t * run .. t * run + run - 1 of the segment; `before` is the sum of the runs
// before it and `mine` its own.  Returns the segment's sum.  All threads of the CTA call it.
__device__ __forceinline__ float segment_scan(const float* __restrict__ x, int begin, int end, float inv_temperature,
                                              float* seg, float* warp_part, float& seg_max, float& before, float& mine) {
    const int n = end - begin;
    for (int i = threadIdx.x; i < n; i += kSegThreads) seg[i] = x[begin + i];
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int run = (n + kSegThreads - 1) / kSegThreads;
    const int a = min(n, (int)threadIdx.x * run), b = min(n, a + run);
    float mx = -INFINITY;
    for (int i = a; i < b; ++i) mx = fmaxf(mx, seg[i]);
    mx = warp_max(mx);
    if (lane == 0) warp_part[warp] = mx;
    __syncthreads();
    mx = warp_max(lane < kSegThreads / 32 ? warp_part[lane] : -INFINITY);
    __syncthreads();
    seg_max = mx;
    mine = 0.f;
    if (mx > -INFINITY)
        for (int i = a; i < b; ++i) mine += expf((seg[i] - mx) * inv_temperature);
    float incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) warp_part[warp] = incl;
    __syncthreads();
    float before_warp = 0.f, total = 0.f;
#pragma unroll
    for (int w = 0; w < kSegThreads / 32; ++w) {
        if (w < warp) before_warp += warp_part[w];
        total += warp_part[w];
    }
    float excl = __shfl_up_sync(0xffffffffu, incl, 1);
    if (lane == 0) excl = 0.f;
    before = before_warp + excl;       // before + mine of one thread is bit for bit the `before` of the next
    __syncthreads();
    return total;
}

__global__ void __launch_bounds__(kSegThreads)
sample_temperature_kernel(const float* __restrict__ logits, int row_stride, int vocab, int first_row,
                          const float* __restrict__ uniforms, float inv_temperature, int* __restrict__ out) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float seg[kSegment];
    __shared__ float warp_part[32];
    __shared__ int ticket_s, chosen_seg_s, chosen_s;
    __shared__ float local_target_s;
    const int row = blockIdx.y, part = blockIdx.x, parts = gridDim.x;
    const float* x = logits + (size_t)(first_row + row) * row_stride;
    const int per = (vocab + parts - 1) / parts;
    const int begin = min(vocab, part * per), end = min(vocab, begin + per);
    float seg_max, before, mine;
    const float total = segment_scan(x, begin, end, inv_temperature, seg, warp_part, seg_max, before, mine);
    if (threadIdx.x == 0) {
        g_sample_max[row * kMaxSegments + part] = seg_max;
        g_sample_sum[row * kMaxSegments + part] = total;
        __threadfence();
        ticket_s = atomicAdd(&g_sample_counters[row], 1);
    }
    __syncthreads();
    if (ticket_s != parts - 1) return;
    // ---- the last CTA of the row to arrive: which segment, then which element
    if (threadIdx.x == 0) {
        __threadfence();
        float row_max = -INFINITY;
        for (int p = 0; p < parts; ++p) row_max = fmaxf(row_max, __ldcg(&g_sample_max[row * kMaxSegments + p]));
        float all = 0.f;
        for (int p = 0; p < parts; ++p) {
            const float m = __ldcg(&g_sample_max[row * kMaxSegments + p]);
            if (m > -INFINITY) all += __ldcg(&g_sample_sum[row * kMaxSegments + p]) * expf((m - row_max) * inv_temperature);
        }
        const float target = uniforms[first_row + row] * all;
        float run = 0.f, local = 0.f;
        int pick = -1, last_with_weight = -1;
        for (int p = 0; p < parts; ++p) {
            const float m = __ldcg(&g_sample_max[row * kMaxSegments + p]);
            if (!(m > -INFINITY)) continue;
            const float scale = expf((m - row_max) * inv_temperature);
            const float weight = __ldcg(&g_sample_sum[row * kMaxSegments + p]) * scale;
            if (!(weight > 0.f)) continue;
            last_with_weight = p;
            if (target < run + weight) {
                pick = p;
                local = (target - run) / scale;        // the target on the segment's own scale
                break;
            }
            run += weight;
        }
        if (pick < 0) {                                // rounding left the target at or past the total
            pick = max(last_with_weight, 0);
            local = INFINITY;
        }
        chosen_seg_s = pick;
        local_target_s = local;
        chosen_s = -1;
        g_sample_counters[row] = 0;                    // ready for the next call
    }
    __syncthreads();
    const int p = chosen_seg_s;
    const float target = local_target_s;
    const int b2 = min(vocab, p * per), e2 = min(vocab, b2 + per);
    segment_scan(x, b2, e2, inv_temperature, seg, warp_part, seg_max, before, mine);
    const int n = e2 - b2;
    const int run_len = (n + kSegThreads - 1) / kSegThreads;
    const int a = min(n, (int)threadIdx.x * run_len), b = min(n, a + run_len);
    if (mine > 0.f && target >= before && target < before + mine) {
        float run = before;
        int pick = b - 1;
        for (int i = a; i < b; ++i) {
            run += expf((seg[i] - seg_max) * inv_temperature);
            if (target < run) { pick = i; break; }
        }
        atomicMax(&chosen_s, b2 + pick);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int pick = chosen_s;
        if (pick < 0) {
            // the target lies at or past the segment's sum: the segment's last element with weight
            pick = b2;
            for (int i = n - 1; i >= 0; --i)
                if (expf((seg[i] - seg_max) * inv_temperature) > 0.f) { pick = b2 + i; break; }
        }
        out[first_row + row] = pick;
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
    const int parts = (vocab + kSegment - 1) / kSegment;
    if (parts > kMaxSegments) return DFI_ERR_LIMIT;
    for (int first = 0; first < rows; first += kSampleMaxRows) {
        const int n = rows - first < kSampleMaxRows ? rows - first : kSampleMaxRows;
        launch(sample_temperature_kernel, dim3(parts, n), kSegThreads, 0, (cudaStream_t)stream, logits, row_stride, vocab,
               first, uniforms, 1.0f / temperature, out);
    }
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
