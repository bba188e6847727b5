// bfloat16 GEMM on the fifth-generation tensor cores: D[m, n] = sum_k A[m, k] * B[n, k], both
// operands K-major (rows contiguous in k), float32 accumulation in tensor memory.
//
//   TMA (cp.async.bulk.tensor, 128-byte swizzle) brings 128 x 64 tiles of A and BN x 64 tiles
//   of B into a ring of shared-memory stages; one thread issues tcgen05.mma (M = 128, N = BN,
//   K = 16 per instruction) straight from shared memory into a TMEM accumulator; stages are
//   handed back by tcgen05.commit on an mbarrier; four warps read the accumulator back with
//   tcgen05.ld and write the output.  Warp 0 produces, warp 1 issues, warps 2-5 drain.
//
// Modes
//   NORMAL  out[m, n]   A = activations [M, K], B = weights [N, K]            (prefill projections)
//   SWIGLU  out[m, j] = silu(D[m, j]) * D[m, N + j], B = [gate; up] of 2N rows: a tile's B rows
//           are BN/2 gate rows and the BN/2 up rows that belong to them, so the activation is
//           applied on the accumulator (engine/kernels/reference.py:74-79; the reference fuses it
//           into its prefill kernel the same way, engine/kernels/prefill_mlp.py:19-44)
//   SWAP    out[n, m]   A = weights [M, K], B = activations [N <= BN, K]: the weights take the
//           128-row side of the instruction so that a small batch wastes nothing (decode)
//
// Every wait on an mbarrier is bounded: a wait that runs out records a code in an error word that
// the host can read (dfi_gemm_tcgen05_error) and the CTA winds down, frees its tensor memory and returns.
#include "tcgen05.cuh"

namespace dfi {

template <int BN> struct TcConfig {
    static constexpr int kBBytes = BN * kTileK * 2;
    static constexpr int kABytes = kTileM * kTileK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStagesRaw = (kSmemBudget - 1024) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr int kTmemCols = BN <= 32 ? 32 : (BN <= 64 ? 64 : (BN <= 128 ? 128 : 256));
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024;   // + slack to align the ring to 1024 bytes
};

// out_dtype 0: float32, 1: bfloat16.  ldo: row stride of out in elements.
template <int BN, int MODE>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                    void* __restrict__ out, int rows_a, int rows_b, int K, int ldo, int out_dtype) {
    using Cfg = TcConfig<BN>;
    pdl_launch_next();
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[Cfg::kStages];
    __shared__ __align__(8) uint64_t empty_bar[Cfg::kStages];
    __shared__ __align__(8) uint64_t accum_bar;
    __shared__ uint32_t tmem_base_s;

    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * kTileM;
    // SWIGLU: a tile covers BN/2 output columns; rows_b is the width of the output (rows of gate)
    const int n0 = blockIdx.y * (MODE == MODE_SWIGLU ? BN / 2 : BN);
    const int k_chunks = (K + kTileK - 1) / kTileK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < Cfg::kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&accum_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();    // set-up is done; everything below reads what earlier kernels wrote

    if (warp == 0) {
        if (lane == 0) {
            for (int kc = 0; kc < k_chunks; ++kc) {
                const int s = kc % Cfg::kStages;
                const uint32_t round = kc / Cfg::kStages;
                if (round > 0 && !mbar_wait(&empty_bar[s], (round - 1) & 1, 1)) break;
                unsigned char* a_tile = ring + (size_t)s * Cfg::kStageBytes;
                unsigned char* b_tile = a_tile + Cfg::kABytes;
                mbar_expect_tx(&full_bar[s], Cfg::kStageBytes);
                tma_load_2d(a_tile, &map_a, kc * kTileK, m0, &full_bar[s]);
                if (MODE == MODE_SWIGLU) {
                    tma_load_2d(b_tile, &map_b, kc * kTileK, n0, &full_bar[s]);
                    tma_load_2d(b_tile + Cfg::kBBytes / 2, &map_b, kc * kTileK, rows_b + n0, &full_bar[s]);
                } else if (MODE == MODE_NN) {
                    // B is [K, N] with N contiguous: 64 x 64 boxes, one per 64 columns of the tile
#pragma unroll
                    for (int h = 0; h < BN / 64; ++h)
                        tma_load_2d(b_tile + h * 8192, &map_b, n0 + h * 64, kc * kTileK, &full_bar[s]);
                } else {
                    tma_load_2d(b_tile, &map_b, kc * kTileK, n0, &full_bar[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: float32 accumulator, bfloat16 A and B, both K-major, N = BN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(kTileM >> 4) << 24) | (MODE == MODE_NN ? (1u << 16) : 0u);
            bool ok = true;
            for (int kc = 0; kc < k_chunks && ok; ++kc) {
                const int s = kc % Cfg::kStages;
                ok = mbar_wait(&full_bar[s], (kc / Cfg::kStages) & 1, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* a_tile = ring + (size_t)s * Cfg::kStageBytes;
                const uint64_t a_desc = umma_desc(a_tile), b_desc = umma_desc(a_tile + Cfg::kABytes);
#pragma unroll
                for (int k = 0; k < kTileK / kUmmaK; ++k) {
                    // 16 elements further along k = 32 bytes = 2 units of the descriptor's address field;
                    // in an MN-major tile 16 steps of k are 16 rows of 128 bytes
                    const uint64_t b_k = MODE == MODE_NN ? umma_desc_mn(a_tile + Cfg::kABytes + k * 2048, 8192) : b_desc + 2 * k;
                    umma_bf16(tmem_base, a_desc + 2 * k, b_k, idesc, (kc > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty_bar[s]);        // the stage is free once these MMAs have read it
            }
            umma_commit(&accum_bar);               // the accumulator is complete once all MMAs are done
        }
    } else {
        // warps 2..5 drain the accumulator: a warp reads the 32 lanes of its quarter (warp % 4)
        const int quarter = warp & 3;
        const bool ok = mbar_wait(&accum_bar, 0, 3);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const int row = m0 + quarter * 32 + lane;      // row of A this thread holds
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        if (ok) {
            if (MODE == MODE_SWIGLU) {
                constexpr int kHalf = BN / 2;
#pragma unroll
                for (int c = 0; c < kHalf; c += 16) {
                    uint32_t g[16], u[16];
                    tmem_load16(lane_addr + c, g);
                    tmem_load16(lane_addr + kHalf + c, u);
                    if (row < rows_a) {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            const int col = n0 + c + j;
                            if (col + 8 <= rows_b) {
                                float v[8];
#pragma unroll
                                for (int e = 0; e < 8; ++e) v[e] = silu_times(__uint_as_float(g[j + e]), __uint_as_float(u[j + e]));
                                if (out_dtype == DFI_DTYPE_BF16) {
                                    store16((bf16*)out + (size_t)row * ldo + col, v);
                                } else {
                                    store16((float*)out + (size_t)row * ldo + col, v);
                                    store16((float*)out + (size_t)row * ldo + col + 4, v + 4);
                                }
                            } else {
                                for (int e = 0; e < 8 && col + e < rows_b; ++e) {
                                    const float v = silu_times(__uint_as_float(g[j + e]), __uint_as_float(u[j + e]));
                                    if (out_dtype == DFI_DTYPE_BF16) ((bf16*)out)[(size_t)row * ldo + col + e] = __float2bfloat16_rn(v);
                                    else ((float*)out)[(size_t)row * ldo + col + e] = v;
                                }
                            }
                        }
                    }
                }
            } else {
#pragma unroll
                for (int c = 0; c < BN; c += 16) {
                    uint32_t d[16];
                    tmem_load16(lane_addr + c, d);
                    if (row >= rows_a) continue;
                    if (MODE == MODE_SWAP) {
                        // out[b, row]: this thread's 16 values go to 16 rows of out
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int b = n0 + c + e;
                            if (b < rows_b) {
                                if (out_dtype == DFI_DTYPE_BF16) ((bf16*)out)[(size_t)b * ldo + row] = __float2bfloat16_rn(__uint_as_float(d[e]));
                                else ((float*)out)[(size_t)b * ldo + row] = __uint_as_float(d[e]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            const int col = n0 + c + j;
                            float v[8];
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(d[j + e]);
                            if (col + 8 <= rows_b) {
                                if (out_dtype == DFI_DTYPE_BF16) {
                                    store16((bf16*)out + (size_t)row * ldo + col, v);
                                } else {
                                    store16((float*)out + (size_t)row * ldo + col, v);
                                    store16((float*)out + (size_t)row * ldo + col + 4, v + 4);
                                }
                            } else {
                                for (int e = 0; e < 8 && col + e < rows_b; ++e) {
                                    if (out_dtype == DFI_DTYPE_BF16) ((bf16*)out)[(size_t)row * ldo + col + e] = __float2bfloat16_rn(v[e]);
                                    else ((float*)out)[(size_t)row * ldo + col + e] = v[e];
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
    }
}

template <int BN, int MODE>
static int launch_tc(const void* a, const void* b, void* out, int rows_a, int rows_b, int K, int ldo, int out_dtype,
                     cudaStream_t st) {
    using Cfg = TcConfig<BN>;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    CUtensorMap map_a, map_b;
    const int b_rows_total = MODE == MODE_SWIGLU ? 2 * rows_b : rows_b;
    if (!make_tile_map(&map_a, a, rows_a, K, kTileM)) return DFI_ERR_LAUNCH;
    if (MODE == MODE_NN) {
        if (!make_tile_map(&map_b, b, K, rows_b, 64)) return DFI_ERR_LAUNCH;      // [K, N]: rows are k
    } else if (!make_tile_map(&map_b, b, b_rows_total, K, MODE == MODE_SWIGLU ? BN / 2 : BN)) {
        return DFI_ERR_LAUNCH;
    }
    const int cols_per_tile = MODE == MODE_SWIGLU ? BN / 2 : BN;
    dim3 grid((rows_a + kTileM - 1) / kTileM, (rows_b + cols_per_tile - 1) / cols_per_tile);
    launch(gemm_tcgen05_kernel<BN, MODE>, grid, kTcThreads, Cfg::kSmemBytes, st, map_a, map_b, out, rows_a, rows_b, K, ldo, out_dtype);
    return DFI_OK;
}

}  // namespace dfi

using namespace dfi;

// The error word of the kernels above: 0, or which wait ran out first (1 producer, 2 issuer, 3 drain).
// Reading it synchronises the device.  `reset` != 0 clears it afterwards.
DFI_EXPORT int dfi_gemm_tcgen05_error(int reset) {
    int value = 0;
    if (cudaMemcpyFromSymbol(&value, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    if (reset && value != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_tc_error, &zero, sizeof(int));
    }
    return value;
}

// mode 0: out[M, N] = x[M, K] . w[N, K]^T            (x rows on the 128-row side)
// mode 1: out[M, N] = silu(x . gate^T) * (x . up^T), w = [gate; up] of 2N rows
// mode 2: the same product as mode 0 computed with w on the 128-row side (M <= 256: small batches)
// mode 3: out[M, N] = x[M, K] . w[K, N] with w stored [K, N] (N contiguous)
// K a multiple of 8, x and w 16-byte aligned and contiguous; out row stride = N.
DFI_EXPORT int dfi_gemm_tcgen05(const void* x, const void* w, void* out, int M, int N, int K, int mode, int out_dtype,
                                void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (K <= 0 || K % 8) return DFI_ERR_SHAPE;
    if (out_dtype != DFI_DTYPE_F32 && out_dtype != DFI_DTYPE_BF16) return DFI_ERR_DTYPE;
    if (!aligned16(x) || !aligned16(w) || !aligned16(out)) return DFI_ERR_ALIGN;
    cudaStream_t st = (cudaStream_t)stream;
    int rc = DFI_ERR_SHAPE;
    if (mode == MODE_NORMAL) {
        if (N % 8) return DFI_ERR_SHAPE;
        rc = launch_tc<128, MODE_NORMAL>(x, w, out, M, N, K, N, out_dtype, st);
    } else if (mode == MODE_SWIGLU) {
        if (N % 8) return DFI_ERR_SHAPE;
        rc = launch_tc<256, MODE_SWIGLU>(x, w, out, M, N, K, N, out_dtype, st);
    } else if (mode == MODE_NN) {
        if (N % 8) return DFI_ERR_SHAPE;
        rc = launch_tc<128, MODE_NN>(x, w, out, M, N, K, N, out_dtype, st);
    } else if (mode == MODE_SWAP) {
        if (M <= 16) rc = launch_tc<16, MODE_SWAP>(w, x, out, N, M, K, N, out_dtype, st);
        else if (M <= 32) rc = launch_tc<32, MODE_SWAP>(w, x, out, N, M, K, N, out_dtype, st);
        else if (M <= 64) rc = launch_tc<64, MODE_SWAP>(w, x, out, N, M, K, N, out_dtype, st);
        else if (M <= 128) rc = launch_tc<128, MODE_SWAP>(w, x, out, N, M, K, N, out_dtype, st);
        else if (M <= 256) rc = launch_tc<256, MODE_SWAP>(w, x, out, N, M, K, N, out_dtype, st);
        else return DFI_ERR_LIMIT;
    }
    if (rc != DFI_OK) return rc;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
