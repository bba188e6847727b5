// Building blocks of the tcgen05 kernels: mbarriers with bounded waits, TMA tile loads, shared-memory
// and instruction descriptors, MMA issue and commit, tensor-memory loads.
#pragma once

#include <cuda.h>
#include <string.h>

#include "common.cuh"

namespace dfi {

constexpr int kTileM = 128;
constexpr int kTileK = 64;                    // 64 bfloat16 = 128 bytes: one swizzle row
constexpr int kUmmaK = 16;
constexpr int kTcThreads = 192;
constexpr int kSmemBudget = 200 * 1024;
// Tries of mbarrier.try_wait before a wait gives up.  A try that does not succeed returns after a few
// microseconds (the hardware's own time limit), so this bound is about a second: no wait of these kernels
// lasts longer than microseconds unless something is broken, and a broken kernel then ends in a second
// (measured: a deadlock built by mistake ended after 16 s with a bound of 2^22) with its code recorded.
constexpr uint32_t kSpinLimit = 1u << 18;

enum { MODE_NORMAL = 0, MODE_SWIGLU = 1, MODE_SWAP = 2, MODE_NN = 3 };

// One error word per translation unit (each .cu that includes this header reads its own), and, if the
// host has named one, a word in the host's own status buffer that receives the same code: the host
// reads that buffer together with a step's results, so a wait that ran out is noticed without a
// synchronisation of its own.
static __device__ int g_tc_error = 0;
static __device__ int* g_status_word = nullptr;

__device__ __forceinline__ void record_error(int code) {
    atomicCAS(&g_tc_error, 0, code);
    int* word = g_status_word;
    if (word != nullptr) atomicCAS(word, 0, code);
}

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(s32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(s32(bar)), "r"(bytes) : "memory");
}
// Waits for the phase with the given parity to complete; false if the bound ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int code, uint32_t limit = kSpinLimit) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}\n"
            : "=r"(done) : "r"(s32(bar)), "r"(parity) : "memory");
        if (done) return true;
    }
    record_error(code);
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(s32(dst)), "l"(map), "r"(x), "r"(y), "r"(s32(bar)) : "memory");
}
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    // K-major, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
    return (uint64_t)((s32(tile) >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (rows of the tile run along k, each row holds 64 contiguous elements of the M or
// N side, 128-byte swizzle): 8-row groups 1024 bytes apart, 64-element column blocks `block_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn(const void* tile, uint32_t block_bytes) {
    return (uint64_t)((s32(tile) >> 4) & 0x3FFF) | ((uint64_t)((block_bytes >> 4) & 0x3FFF) << 16) | (64ull << 32) |
           (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
// silu(gate) * up for an epilogue whose result is rounded to bfloat16: the fast exponential and division
// (a few units in the last place of float32) cost a quarter of the instructions of the exact ones, and the
// epilogue of a step of many rows is a chain of such instructions.
__device__ __forceinline__ float silu_times(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }


// A [rows, K] bfloat16 matrix (row stride K) as a TMA map with boxes of box_rows x 64, 128-byte swizzle.
static inline bool make_tile_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows,
                                 long long row_stride_elems = 0) {
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)(row_stride_elems > 0 ? row_stride_elems : K) * 2};
    cuuint32_t box[2] = {(cuuint32_t)kTileK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return cuTensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}


// ---- a word about the matrix product that the step runs next
// How a decode product deals its units of 128 rows x 64 k to its CTAs: equal contiguous runs over the whole
// matrix (parts == 0), or every row block cut into the same number of parts, one CTA each.
struct UnitDeal {
    int units, k_chunks, n_ctas, parts;
};
__host__ __device__ __forceinline__ int deal_begin(const UnitDeal& d, int cta) {
    if (d.parts > 0) {
        if (cta >= d.n_ctas) return d.units;
        return (cta / d.parts) * d.k_chunks + d.k_chunks * (cta % d.parts) / d.parts;
    }
    return (int)((unsigned)d.units * (unsigned)cta / (unsigned)d.n_ctas);
}
// A decode kernel may be told which weights the step streams after it.  Between the moment a CTA has asked
// for the last of its own stream and the moment the next product can use its first tiles, the memory has
// nothing to do (the epilogue, the end of the grid and the next product's activations take about 4 us); the
// next product already holds its first ring (it loads it before it waits for this kernel), so the CTA asks
// the `count` tiles that follow that ring, for the next product's CTA of the same number, into L2.  A hint
// only: nothing waits for these tiles, and a wrong hint costs a little bandwidth.  More than a few tiles
// were measured slower than none: the epilogue's own dependent loads then queue behind them.  The products
// take the hint; decode attention does not (given one for the output projection it ran slower, hint or no hint).
struct alignas(64) NextStream {
    CUtensorMap map;        // the next product's weights with the boxes that product loads
    UnitDeal deal;
    int up_row0;            // >= 0: [gate; up] weights in boxes of 64 rows, the up rows starting at this row
    int skip;               // tiles of a CTA's run that its first ring holds
    int count;              // tiles to ask for after those; 0: no hint
    int reserved;
};
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];\n" ::"l"(map), "r"(x), "r"(y) : "memory");
}
// Called by one thread of CTA `cta` of `n_here`.
__device__ __forceinline__ void prefetch_next_stream(const NextStream& next, int cta, int n_here) {
    if (next.count <= 0) return;
    for (int c = cta; c < next.deal.n_ctas; c += n_here) {
        const int first = deal_begin(next.deal, c) + next.skip;
        const int last = min(deal_begin(next.deal, c + 1), first + next.count);
        for (int u = first; u < last; ++u) {
            const int rb = u / next.deal.k_chunks, kc = u % next.deal.k_chunks;
            if (next.up_row0 >= 0) {
                tma_prefetch_2d(&next.map, kc * kTileK, rb * (kTileM / 2));
                tma_prefetch_2d(&next.map, kc * kTileK, next.up_row0 + rb * (kTileM / 2));
            } else {
                tma_prefetch_2d(&next.map, kc * kTileK, rb * kTileM);
            }
        }
    }
}
// The kernel argument from the host's copy of a hint (any alignment), or no hint.
static inline NextStream next_stream_arg(const void* host_hint) {
    NextStream next;
    memset(&next, 0, sizeof(next));
    if (host_hint != nullptr) memcpy(&next, host_hint, sizeof(next));
    return next;
}

// What a kernel of this header does when a wait runs out, alone: one warp takes 32 columns of tensor
// memory, waits `limit` tries on a barrier that nothing ever arrives on, records `code`, gives the
// tensor memory back and returns.  It exists so that the path from the error word to the host's
// exception can be tested without any other kernel failing.
static __global__ void wait_selftest_kernel(uint32_t limit, int code) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_base_s;
    if (threadIdx.x == 0) mbar_init(&bar, 1);
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(32) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    if (threadIdx.x == 0) mbar_wait(&bar, 0, code, limit);
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(32) : "memory");
}

}  // namespace dfi

// The three host entry points every translation unit of this header exports under its own name:
//   dfi_<name>_error(reset)            the unit's error word (synchronises), optionally reset to 0
//   dfi_<name>_set_status_word(ptr)    a device word of the host's that receives the codes too (or null)
//   dfi_<name>_wait_selftest(limit, code, stream)   the self-test kernel above
#define DFI_TCGEN05_STATUS_ENTRIES(name)                                                              \
    DFI_EXPORT int dfi_##name##_error(int reset) {                                                    \
        int value = 0;                                                                                \
        if (cudaMemcpyFromSymbol(&value, dfi::g_tc_error, sizeof(int)) != cudaSuccess) return -1;     \
        if (reset && value != 0) {                                                                    \
            const int zero = 0;                                                                       \
            cudaMemcpyToSymbol(dfi::g_tc_error, &zero, sizeof(int));                                  \
        }                                                                                             \
        return value;                                                                                 \
    }                                                                                                 \
    DFI_EXPORT int dfi_##name##_set_status_word(int* word) {                                          \
        return cudaMemcpyToSymbol(dfi::g_status_word, &word, sizeof(int*)) == cudaSuccess ? DFI_OK    \
                                                                                           : DFI_ERR_LAUNCH; \
    }                                                                                                 \
    DFI_EXPORT int dfi_##name##_wait_selftest(unsigned limit, int code, void* stream) {               \
        dfi::wait_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(limit, code);                   \
        DFI_CHECK_LAUNCH();                                                                           \
        return DFI_OK;                                                                                \
    }
