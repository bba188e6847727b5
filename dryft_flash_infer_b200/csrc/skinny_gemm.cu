// out[M, N] = x[M, K] . W[N, K]^T for a few rows of activations (M <= 64, the decode step),
// bfloat16 operands, float32 accumulation.  The work is reading W once at memory speed.
//
// W's rows are the 16-row operand of mma.sync m16n8k16 and the activations the 8-column
// one, so the batch pads to a multiple of 8 instead of 16 or more.  Fragments load
// straight from global memory as 16-byte vectors: within a chunk of 32 k, lane (g, t)
// reads k = 8t..8t+7 of W rows g and g+8 and of activation row g.  This permutes k inside
// the chunk the same way for both operands, which a dot product does not see.
//
// A CTA of four warps owns 64 rows of W (16 per warp) and one slice of K; the slices of
// one row block run in parallel CTAs (split-K) so that a matrix with few rows still fills
// the GPU.  Each CTA leaves its float32 partial sums in scratch memory, takes a ticket
// from the row block's counter, and the CTA that draws the last ticket adds the slices in
// slice order (so the result does not depend on who finished when), applies the epilogue
// and resets the counter.  No CTA ever waits for another.
//
// SWIGLU variant: W is [2*I, K] with the gate rows first; a warp's 16 rows are 8 gate
// rows and the 8 up rows that belong to them, and the epilogue writes
// silu(gate) * up to out[M, I] (engine/kernels/reference.py:74-79; the fusion follows
// the idea of engine/kernels/cuda_mlp.py:39-125).
#include "common.cuh"

namespace dfi {

constexpr int kGemmThreads = 128;
constexpr int kSub = 256;            // k per staging pass of the activations
constexpr int kSubStride = kSub + 8; // padded: conflict-free 16-byte reads down a column of rows

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 load_stream(const bf16* p) {
    uint4 v;
    asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

// NT: 8-row tiles of the batch (M <= 8*NT).  out_dtype: 0 float32, 1 bfloat16.
template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(kGemmThreads)
skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, void* __restrict__ out, int M, int N, int K,
                   int k_per_split, int n_splits, float* __restrict__ partials, int* __restrict__ counters,
                   int out_dtype) {
    __shared__ __align__(16) bf16 x_s[NT * 8 * kSubStride];
    __shared__ int ticket_s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int row_block = blockIdx.x, split = blockIdx.y;
    // N_rows: rows of W; for SWIGLU, N is the width of the output (I) and W has 2*N rows
    const int rows_per_block = SWIGLU ? 32 : 64;
    const int block_row0 = row_block * rows_per_block;
    int row_lo, row_hi;          // the two rows of W this lane reads (fragment rows g and g+8)
    bool live_lo, live_hi;
    if (SWIGLU) {
        const int r = block_row0 + warp * 8 + g;
        live_lo = live_hi = r < N;
        row_lo = r;
        row_hi = N + r;
    } else {
        row_lo = block_row0 + warp * 16 + g;
        row_hi = row_lo + 8;
        live_lo = row_lo < N;
        live_hi = row_hi < N;
    }
    const bf16* w_lo = w + (size_t)(live_lo ? row_lo : 0) * K;
    const bf16* w_hi = w + (size_t)(live_hi ? row_hi : 0) * K;

    const int k_begin = split * k_per_split, k_end = min(K, k_begin + k_per_split);
    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    for (int k0 = k_begin; k0 < k_end; k0 += kSub) {
        // this warp's weights for the pass: 8 chunks of 32 k, two rows, 16 bytes each
        uint4 a_lo[8], a_hi[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int k = k0 + c * 32 + t4 * 8;
            const bool in = k < k_end;
            a_lo[c] = (in && live_lo) ? load_stream(w_lo + k) : make_uint4(0, 0, 0, 0);
            a_hi[c] = (in && live_hi) ? load_stream(w_hi + k) : make_uint4(0, 0, 0, 0);
        }
        __syncthreads();   // the previous pass no longer reads x_s
        for (int i = threadIdx.x; i < NT * 8 * (kSub / 8); i += kGemmThreads) {
            const int m = i / (kSub / 8), c = i % (kSub / 8);
            const int k = k0 + c * 8;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (m < M && k < k_end) v = *reinterpret_cast<const uint4*>(x + (size_t)m * K + k);
            *reinterpret_cast<uint4*>(x_s + m * kSubStride + c * 8) = v;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint4 b = *reinterpret_cast<const uint4*>(x_s + (j * 8 + g) * kSubStride + c * 32 + t4 * 8);
                mma16816(acc[j], a_lo[c].x, a_hi[c].x, a_lo[c].y, a_hi[c].y, b.x, b.y);
                mma16816(acc[j], a_lo[c].z, a_hi[c].z, a_lo[c].w, a_hi[c].w, b.z, b.w);
            }
        }
    }

    // acc[j][e]: row of W = (e < 2 ? lo : hi), batch row m = j*8 + 2*t4 + (e & 1)
    const int w_rows = SWIGLU ? 2 * N : N;
    if (n_splits == 1) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int m = j * 8 + 2 * t4 + e;
                if (m >= M) continue;
                if (SWIGLU) {
                    if (live_lo) {
                        const float v = silu_mul(acc[j][e], acc[j][e + 2]);
                        if (out_dtype == DFI_DTYPE_F32) ((float*)out)[(size_t)m * N + row_lo] = v;
                        else ((bf16*)out)[(size_t)m * N + row_lo] = __float2bfloat16_rn(v);
                    }
                } else {
                    if (live_lo) {
                        if (out_dtype == DFI_DTYPE_F32) ((float*)out)[(size_t)m * N + row_lo] = acc[j][e];
                        else ((bf16*)out)[(size_t)m * N + row_lo] = __float2bfloat16_rn(acc[j][e]);
                    }
                    if (live_hi) {
                        if (out_dtype == DFI_DTYPE_F32) ((float*)out)[(size_t)m * N + row_hi] = acc[j][e + 2];
                        else ((bf16*)out)[(size_t)m * N + row_hi] = __float2bfloat16_rn(acc[j][e + 2]);
                    }
                }
            }
        }
        return;
    }

    float* mine = partials + (size_t)split * M * w_rows;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = j * 8 + 2 * t4 + e;
            if (m >= M) continue;
            if (live_lo) mine[(size_t)m * w_rows + row_lo] = acc[j][e];
            if (live_hi) mine[(size_t)m * w_rows + row_hi] = acc[j][e + 2];
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_s = atomicAdd(&counters[row_block], 1);
    __syncthreads();
    if (ticket_s != n_splits - 1) return;
    __threadfence();   // the other slices' partial sums are visible now
    const int out_cols = min(rows_per_block, N - block_row0);
    for (int i = threadIdx.x; i < M * out_cols; i += kGemmThreads) {
        const int m = i / out_cols, n = block_row0 + i % out_cols;
        float v;
        if (SWIGLU) {
            float gate = 0.f, up = 0.f;
            for (int s = 0; s < n_splits; ++s) {
                const float* p = partials + ((size_t)s * M + m) * w_rows;
                gate += __ldcg(p + n);
                up += __ldcg(p + N + n);
            }
            v = silu_mul(gate, up);
        } else {
            v = 0.f;
            for (int s = 0; s < n_splits; ++s) v += __ldcg(partials + ((size_t)s * M + m) * w_rows + n);
        }
        if (out_dtype == DFI_DTYPE_F32) ((float*)out)[(size_t)m * N + n] = v;
        else ((bf16*)out)[(size_t)m * N + n] = __float2bfloat16_rn(v);
    }
    if (threadIdx.x == 0) counters[row_block] = 0;   // ready for the next call
}

template <int NT, bool SWIGLU>
static void launch_skinny(const bf16* x, const bf16* w, void* out, int M, int N, int K, int k_per_split, int n_splits,
                          float* partials, int* counters, int out_dtype, cudaStream_t st) {
    const int rows_per_block = SWIGLU ? 32 : 64;
    dim3 grid((N + rows_per_block - 1) / rows_per_block, n_splits);
    skinny_gemm_kernel<NT, SWIGLU><<<grid, kGemmThreads, 0, st>>>(x, w, out, M, N, K, k_per_split, n_splits, partials,
                                                                   counters, out_dtype);
}

}  // namespace dfi

using namespace dfi;

// How the caller sizes the scratch: floats for the partial sums of `n_splits` slices
// (0 when n_splits == 1) and ints for the row blocks' counters (always; they must be
// zero before the first call and are left zero by every call).
DFI_EXPORT long long dfi_skinny_gemm_partial_floats(int M, int N, int swiglu, int n_splits) {
    return n_splits <= 1 ? 0 : (long long)n_splits * M * (swiglu ? 2 * N : N);
}
DFI_EXPORT int dfi_skinny_gemm_counters(int N, int swiglu) { return (N + (swiglu ? 31 : 63)) / (swiglu ? 32 : 64); }

// x [M, K] bfloat16 (rows contiguous), w [N, K] (or [2N, K] with swiglu) bfloat16,
// out [M, N] of out_dtype.  K must be a multiple of 8; M at most 64.  n_splits slices of
// K run in parallel (each a multiple of 32 long).
DFI_EXPORT int dfi_skinny_gemm(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int n_splits,
                               float* partials, int* counters, int out_dtype, void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (M > 64 || K <= 0 || K % 8) return DFI_ERR_SHAPE;
    if (out_dtype != DFI_DTYPE_F32 && out_dtype != DFI_DTYPE_BF16) return DFI_ERR_DTYPE;
    if (!aligned16(x) || !aligned16(w)) return DFI_ERR_ALIGN;
    if (n_splits < 1 || n_splits > 65535 || counters == nullptr || (n_splits > 1 && partials == nullptr))
        return DFI_ERR_SHAPE;
    int k_per_split = (K + n_splits - 1) / n_splits;
    k_per_split = (k_per_split + 31) / 32 * 32;
    if ((long long)k_per_split * (n_splits - 1) >= K && n_splits > 1) return DFI_ERR_SHAPE;   // an empty slice
    cudaStream_t st = (cudaStream_t)stream;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    const int nt = (M + 7) / 8;
#define DFI_LAUNCH(NTV)                                                                                             \
    do {                                                                                                            \
        if (swiglu) launch_skinny<NTV, true>(xp, wp, out, M, N, K, k_per_split, n_splits, partials, counters, out_dtype, st); \
        else launch_skinny<NTV, false>(xp, wp, out, M, N, K, k_per_split, n_splits, partials, counters, out_dtype, st);      \
    } while (0)
    if (nt <= 1) DFI_LAUNCH(1);
    else if (nt <= 2) DFI_LAUNCH(2);
    else if (nt <= 4) DFI_LAUNCH(4);
    else DFI_LAUNCH(8);
#undef DFI_LAUNCH
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
