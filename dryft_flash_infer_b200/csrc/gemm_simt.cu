// The plain matrix product: out[M, N] = x[M, K] . w[N, K]^T on the ordinary float32 pipes, for float32
// and bfloat16 operands of any size.
//
// It is the product of the true 32-bit path (every multiply and add in float32, summed in the order
// of k: no tensor core, no reduced-precision mode) and the product for bfloat16 matrices whose width is
// no multiple of 8, which the TMA-fed tensor-core kernels do not take.  A CTA of 256 threads computes a
// 64 x 64 tile of the result from 64 x 16 tiles of both operands staged in shared memory (converted to
// float32 on the way in), each thread a 4 x 4 patch.  Edges are handled by bounds checks on the loads
// (zeros beyond the matrix) and on the stores.
#include "common.cuh"

namespace dfi {

constexpr int kSimtTile = 64;
constexpr int kSimtK = 16;
constexpr int kSimtThreads = 256;

// Loads the 64 x 16 tile of `m` [rows, K] that starts at (row0, k0) into tile[k][row]; a thread takes
// four consecutive k of one row (one 16-byte or 8-byte load when `vec`, i.e. K % 4 == 0 and the base aligned).
template <typename T, bool vec>
__device__ __forceinline__ void load_tile(const T* __restrict__ m, int rows, int K, int row0, int k0,
                                          float (&tile)[kSimtK][kSimtTile + 4]) {
    const int r = threadIdx.x >> 2, kq = (threadIdx.x & 3) * 4;
    const int row = row0 + r, k = k0 + kq;
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < rows) {
        const T* p = m + (size_t)row * K + k;
        if (vec && k + 4 <= K) {
            if constexpr (sizeof(T) == 4) {
                const float4 f = *reinterpret_cast<const float4*>(p);
                v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
            } else {
                const uint2 raw = *reinterpret_cast<const uint2*>(p);
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
                const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
                v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (k + i < K) v[i] = to_float(p[i]);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) tile[kq + i][r] = v[i];
}

template <typename T, typename TO, bool vec>
__global__ void __launch_bounds__(kSimtThreads) gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                                 TO* __restrict__ out, int M, int N, int K) {
    __shared__ float xs[kSimtK][kSimtTile + 4];
    __shared__ float ws[kSimtK][kSimtTile + 4];
    pdl_launch_next();
    pdl_wait();
    const int row0 = blockIdx.y * kSimtTile, col0 = blockIdx.x * kSimtTile;
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;          // rows ty*4.., columns tx*4..
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += kSimtK) {
        load_tile<T, vec>(x, M, K, row0, k0, xs);
        load_tile<T, vec>(w, N, K, col0, k0, ws);
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kSimtK; ++k) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[k][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[k][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row0 + ty * 4 + i;
        if (row >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int col = col0 + tx * 4 + j;
            if (col < N) out[(size_t)row * N + col] = from_float<TO>(acc[i][j]);
        }
    }
}

template <typename T, typename TO>
static int run(const void* x, const void* w, void* out, int M, int N, int K, cudaStream_t stream) {
    const dim3 grid((N + kSimtTile - 1) / kSimtTile, (M + kSimtTile - 1) / kSimtTile);
    const bool vec = K % 4 == 0 && (reinterpret_cast<uintptr_t>(x) % 16 == 0) && (reinterpret_cast<uintptr_t>(w) % 16 == 0);
    if (vec)
        launch(gemm_simt_kernel<T, TO, true>, grid, dim3(kSimtThreads), 0, stream, (const T*)x, (const T*)w, (TO*)out, M, N, K);
    else
        launch(gemm_simt_kernel<T, TO, false>, grid, dim3(kSimtThreads), 0, stream, (const T*)x, (const T*)w, (TO*)out, M, N, K);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

}  // namespace dfi

using namespace dfi;

// out[M, N] = x[M, K] . w[N, K]^T; x, w and out contiguous.  `dtype` is that of x and w; `out_dtype` may
// be float32 for bfloat16 operands (unrounded results, as logits want them).
DFI_EXPORT int dfi_gemm_simt(const void* x, const void* w, void* out, int M, int N, int K, int dtype, int out_dtype,
                             void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (K <= 0) return DFI_ERR_SHAPE;
    if ((long long)((M + kSimtTile - 1) / kSimtTile) > 65535) return DFI_ERR_LIMIT;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32 && out_dtype == DFI_DTYPE_F32) return run<float, float>(x, w, out, M, N, K, s);
    if (dtype == DFI_DTYPE_BF16 && out_dtype == DFI_DTYPE_BF16) return run<bf16, bf16>(x, w, out, M, N, K, s);
    if (dtype == DFI_DTYPE_BF16 && out_dtype == DFI_DTYPE_F32) return run<bf16, float>(x, w, out, M, N, K, s);
    return DFI_ERR_DTYPE;
}
