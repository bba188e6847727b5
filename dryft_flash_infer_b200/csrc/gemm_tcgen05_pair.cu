// bfloat16 GEMM for many rows (prompts) on pairs of SMs: out[m, n] = sum_k x[m, k] * w[n, k].
//
// Two CTAs on the two SMs of a pair form a cluster and share one tcgen05.mma.cta_group::2 of
// M = 256, N = 256, K = 16: each CTA holds 128 rows of x and one half (128 rows) of the w tile in its
// own shared memory, the instruction reads both halves from both CTAs, and each CTA's tensor memory
// receives its own 128 rows of the 256 x 256 result.  Per CTA that is 8 KB of operands for 128 clocks
// of arithmetic where a single-CTA instruction of the same shape needs 12 KB.
//
// The kernel is persistent: a cluster walks over output tiles (tile t, t + clusters, ...).  In each
// CTA warp 0 feeds a ring of shared-memory stages by TMA (the transaction bytes of both CTAs count
// on the leader's barrier), warp 1 of the leader CTA issues the MMAs and hands stages back to both
// CTAs with a multicast commit, and warps 2-5 of each CTA drain one of two accumulators in tensor
// memory while the other is being filled.
//
// SWIGLU variant: w = [gate; up] of 2N rows.  The leader CTA loads 128 gate rows and the other CTA
// the 128 up rows that belong to them, so an accumulator holds gate in columns 0-127 and up in
// 128-255, and the epilogue writes silu(gate) * up (engine/kernels/reference.py:74-79): the
// [rows, 2N] intermediate is never written.
//
// Every wait is bounded; a wait that runs out records a code (dfi_gemm_pair_error), and every
// thread of both CTAs still reaches the cluster barrier at the end before tensor memory is freed.
#include "tcgen05.cuh"

namespace dfi {

constexpr int kPairThreads = 192;
constexpr int kPairN = 256;                                   // columns of an accumulator
constexpr int kPairStages = 6;
constexpr int kPairHalfBytes = kTileM * kTileK * 2;           // 128 rows x 64 k of x, and the same of w
constexpr int kPairStageBytes = 2 * kPairHalfBytes;
constexpr int kPairSmem = kPairStages * kPairStageBytes + 1024;
constexpr int kPairTmemCols = 512;                            // two accumulators of 256 columns

__device__ __forceinline__ uint32_t pair_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// The address of this CTA's shared-memory location in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t pair_map(const void* own, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(s32(own)), "r"(rank));
    return out;
}
// TMA tile load whose bytes count on a barrier that may live in the other CTA of the pair.
__device__ __forceinline__ void pair_tma_load(void* dst, const CUtensorMap* map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void pair_mma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both CTAs once every MMA issued so far is complete.
__device__ __forceinline__ void pair_commit_both(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;\n"
        ::"r"(s32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void pair_arrive_remote(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void pair_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
}

struct PairShape {
    int M, N, K;              // N: columns of the output
    int tiles_m, tiles_n;     // tiles of 256 rows; tiles of 256 (SWIGLU: 128) output columns
    int ldo;                  // row stride of out in elements
};

// Tiles are numbered so that the clusters, which take consecutive numbers, work on a compact block of
// the output at any time: bands of kBandTiles row tiles, inside a band column by column.  The rows of
// x of a band (8 x 256 rows) and the rows of w of the columns in flight then stay in L2, whatever the
// number of rows; numbering row tiles first over the whole matrix streams x from memory once per
// column tile as soon as x outgrows L2.
constexpr int kBandTiles = 8;
__device__ __forceinline__ void tile_place(const PairShape& s, int t, int& tile_m, int& tile_n) {
    const int per_band = kBandTiles * s.tiles_n;
    const int band = t / per_band, in_band = t % per_band;
    const int rows_here = min(kBandTiles, s.tiles_m - band * kBandTiles);
    tile_m = band * kBandTiles + in_band % rows_here;
    tile_n = in_band / rows_here;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kPairThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 bf16* __restrict__ out, PairShape s) {
    pdl_launch_next();
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[kPairStages];     // the leader's are used
    __shared__ __align__(8) uint64_t empty_bar[kPairStages];    // each CTA's own
    __shared__ __align__(8) uint64_t acc_full[2];               // each CTA's own
    __shared__ __align__(8) uint64_t acc_empty[2];              // the leader's are used: one arrival per CTA
    __shared__ uint32_t tmem_base_s;

    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = pair_rank();
    const int cluster = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    const int n_tiles = s.tiles_m * s.tiles_n;
    const int k_chunks = (s.K + kTileK - 1) / kTileK;
    constexpr int kOutCols = SWIGLU ? kPairN / 2 : kPairN;      // output columns of a tile

    if (threadIdx.x == 0) {
        for (int i = 0; i < kPairStages; ++i) {
            mbar_init(&full_bar[i], 1);
            mbar_init(&empty_bar[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], 2);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(kPairTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    pair_sync_all();         // both CTAs' barriers are initialised before either is used from the other side
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t i = 0;          // stages filled so far, over all tiles
            bool ok = true;
            for (int t = cluster; t < n_tiles && ok; t += n_clusters) {
                int tile_m, tile_n;
                tile_place(s, t, tile_m, tile_n);
                const int m0 = tile_m * 2 * kTileM + (int)rank * kTileM;
                // rows of w for this CTA's half of the tile
                const int w_row = SWIGLU ? (rank == 0 ? 0 : s.N) + tile_n * kOutCols : tile_n * kPairN + (int)rank * kTileM;
                for (int kc = 0; kc < k_chunks; ++kc, ++i) {
                    const int st = i % kPairStages;
                    const uint32_t round = i / kPairStages;
                    if (round > 0) {
                        ok = mbar_wait(&empty_bar[st], (round - 1) & 1, 1);
                        if (!ok) break;
                    }
                    if (rank == 0) mbar_expect_tx(&full_bar[st], 2 * kPairStageBytes);
                    const uint32_t bar = pair_map(&full_bar[st], 0);
                    unsigned char* tile = ring + (size_t)st * kPairStageBytes;
                    pair_tma_load(tile, &map_x, kc * kTileK, m0, bar);
                    pair_tma_load(tile + kPairHalfBytes, &map_w, kc * kTileK, w_row, bar);
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && lane == 0) {
            // float32 accumulator, bfloat16 operands, both K-major, N = 256, M = 256 over the pair
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kPairN >> 3) << 17) |
                                       ((uint32_t)((2 * kTileM) >> 4) << 24);
            uint32_t i = 0;
            int j = 0;               // tiles done by this cluster
            bool ok = true;
            for (int t = cluster; t < n_tiles && ok; t += n_clusters, ++j) {
                const int buf = j & 1;
                if (j >= 2) {
                    ok = mbar_wait(&acc_empty[buf], ((j >> 1) - 1) & 1, 4);      // both CTAs have drained this accumulator
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                }
                for (int kc = 0; kc < k_chunks; ++kc, ++i) {
                    const int st = i % kPairStages;
                    ok = mbar_wait(&full_bar[st], (i / kPairStages) & 1, 2);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const unsigned char* tile = ring + (size_t)st * kPairStageBytes;
                    const uint64_t a_desc = umma_desc(tile), b_desc = umma_desc(tile + kPairHalfBytes);
#pragma unroll
                    for (int k = 0; k < kTileK / kUmmaK; ++k)
                        pair_mma(tmem_base + buf * kPairN, a_desc + 2 * k, b_desc + 2 * k, idesc, (kc > 0 || k > 0) ? 1u : 0u);
                    pair_commit_both(&empty_bar[st]);
                }
                if (ok) pair_commit_both(&acc_full[buf]);
            }
        }
    } else {
        // warps 2-5: thread t of the 128 holds row t of this CTA's 128 rows (TMEM lane t)
        const int quarter = warp & 3;
        const int row_in_cta = quarter * 32 + lane;
        const uint32_t empty_at_leader[2] = {pair_map(&acc_empty[0], 0), pair_map(&acc_empty[1], 0)};
        int j = 0;
        bool ok = true;
        for (int t = cluster; t < n_tiles && ok; t += n_clusters, ++j) {
            const int buf = j & 1;
            ok = mbar_wait(&acc_full[buf], (j >> 1) & 1, 3);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            int tile_m, tile_n;
            tile_place(s, t, tile_m, tile_n);
            const int row = tile_m * 2 * kTileM + (int)rank * kTileM + row_in_cta;
            const int col0 = tile_n * kOutCols;
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kPairN;
            bf16* dst = out + (size_t)row * s.ldo + col0;
            const bool vector = (s.ldo % 8 == 0) && (reinterpret_cast<uintptr_t>(out) & 15) == 0 && col0 % 8 == 0;
#pragma unroll 1
            for (int c = 0; c < kOutCols; c += 32) {
                uint32_t v[32];
                tmem_load32(taddr + c, v);
                float f[32];
                if (SWIGLU) {
                    uint32_t u[32];
                    tmem_load32(taddr + kPairN / 2 + c, u);
#pragma unroll
                    for (int e = 0; e < 32; ++e) f[e] = silu_times(__uint_as_float(v[e]), __uint_as_float(u[e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 32; ++e) f[e] = __uint_as_float(v[e]);
                }
                if (row < s.M) {
                    if (vector && col0 + c + 32 <= s.N) {
#pragma unroll
                        for (int e = 0; e < 32; e += 8) store16(dst + c + e, f + e);
                    } else {
                        for (int e = 0; e < 32; ++e)
                            if (col0 + c + e < s.N) dst[c + e] = __float2bfloat16_rn(f[e]);
                    }
                }
            }
            // this CTA is done with the accumulator: one arrival per CTA on the leader's barrier
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (row_in_cta == 0) pair_arrive_remote(empty_at_leader[buf]);
        }
    }
    // no CTA leaves (or frees tensor memory) while the other may still read its shared memory or
    // arrive on its barriers
    __syncwarp();
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    pair_sync_all();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kPairTmemCols) : "memory");
    }
}

static int g_pair_clusters = 0;

template <bool SWIGLU>
static int pair_clusters() {
    if (g_pair_clusters > 0) return g_pair_clusters;
    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(sms & ~1);
    config.blockDim = dim3(kPairThreads);
    config.dynamicSmemBytes = kPairSmem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_pair_kernel<SWIGLU>, &config) != cudaSuccess || clusters <= 0) {
        cudaGetLastError();
        clusters = sms / 2;
    }
    if (clusters > sms / 2) clusters = sms / 2;
    g_pair_clusters = clusters;
    return clusters;
}

template <bool SWIGLU>
static int launch_pair(const void* x, const void* w, void* out, PairShape s, cudaStream_t st) {
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_pair_kernel<SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmem) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    CUtensorMap map_x, map_w;
    if (!make_tile_map(&map_x, x, s.M, s.K, kTileM)) return DFI_ERR_LAUNCH;
    if (!make_tile_map(&map_w, w, SWIGLU ? 2 * s.N : s.N, s.K, kTileM)) return DFI_ERR_LAUNCH;
    int clusters = pair_clusters<SWIGLU>();
    if (clusters <= 0) return DFI_ERR_LAUNCH;
    const int n_tiles = s.tiles_m * s.tiles_n;
    if (clusters > n_tiles) clusters = n_tiles;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * clusters);
    config.blockDim = dim3(kPairThreads);
    config.dynamicSmemBytes = kPairSmem;
    config.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl_enabled() ? 2 : 1;
    if (cudaLaunchKernelEx(&config, gemm_pair_kernel<SWIGLU>, map_x, map_w, (bf16*)out, s) != cudaSuccess) {
        cudaGetLastError();
        return DFI_ERR_LAUNCH;
    }
    return DFI_OK;
}

}  // namespace dfi

using namespace dfi;

DFI_TCGEN05_STATUS_ENTRIES(gemm_pair)

// out[M, N] bfloat16 (row stride ldo) = x[M, K] . w[N, K]^T, or with swiglu: silu(x . gate^T) * (x . up^T)
// for w = [gate; up] of 2N rows.  K a multiple of 8; x and w 16-byte aligned.
DFI_EXPORT int dfi_gemm_pair(const void* x, const void* w, void* out, int M, int N, int K, int ldo, int swiglu,
                             void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (K <= 0 || K % 8 || ldo < N) return DFI_ERR_SHAPE;
    if (!aligned16(x) || !aligned16(w)) return DFI_ERR_ALIGN;
    PairShape s;
    s.M = M; s.N = N; s.K = K; s.ldo = ldo;
    s.tiles_m = (M + 2 * kTileM - 1) / (2 * kTileM);
    s.tiles_n = (N + (swiglu ? kPairN / 2 : kPairN) - 1) / (swiglu ? kPairN / 2 : kPairN);
    if ((long long)s.tiles_m * s.tiles_n > (1 << 24)) return DFI_ERR_LIMIT;
    const int rc = swiglu ? launch_pair<true>(x, w, out, s, (cudaStream_t)stream)
                          : launch_pair<false>(x, w, out, s, (cudaStream_t)stream);
    if (rc != DFI_OK) return rc;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
