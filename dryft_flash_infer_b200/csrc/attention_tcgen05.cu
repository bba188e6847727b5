// Causal grouped-query flash attention for prompts on the fifth-generation tensor cores
// (head sizes 64 and 128, bfloat16), reading keys and values from the paged cache.
//
// One CTA owns 128 query rows of one head of one sequence and walks the sequence's pages of 64
// keys up to the diagonal (or through the window).  Per page:
//     S = Q K^T      tcgen05.mma, M = 128, N = 64, operands in shared memory (TMA, 128-byte swizzle),
//                    accumulator in tensor memory (two buffers, so the next S is computed while
//                    this one is being turned into probabilities)
//     P = exp2(S * scale - max)   by 128 threads, one query row each: a row's maximum and sum need
//                    no exchange between threads; the online softmax is the reference's
//                    (engine/kernels/attention.py:40-137) with float32 maximum, sum and output
//     O_page = P V   tcgen05.mma with P (bfloat16, written to shared memory in the swizzled layout)
//                    as the 128-row operand and V, as it lies in the cache ([key][d]), as an
//                    MN-major second operand; the page's product is added into the thread's
//                    float32 output row, which is rescaled when the maximum moves
// Warp 0 feeds a ring of K/V pages with TMA, warp 1 issues the MMAs, warps 2-5 do the softmax and
// the output.  Every wait on an mbarrier is bounded (see tcgen05.cuh).
//
// Rows of the last page that no token was written to may hold anything: their scores are
// replaced (not added to) by -inf, and their value rows are zeroed in shared memory before use.
#include "tcgen05.cuh"

#ifndef DFI_HEAD_DIM
#define DFI_HEAD_DIM 128
#endif

namespace dfi {

#if DFI_HEAD_DIM == 64 || DFI_HEAD_DIM == 128
#define DFI_FA_ENABLED 1
constexpr int kFaD = DFI_HEAD_DIM;
#else
#define DFI_FA_ENABLED 0
constexpr int kFaD = 128;
#endif

constexpr int kFaRows = 128;                          // query rows per CTA
constexpr int kFaKeys = 64;                           // keys per page
constexpr int kFaThreads = 192;
constexpr int kFaBlocks = kFaD / 64;                  // 64-wide column blocks of a head
constexpr int kFaQBytes = kFaRows * kFaD * 2;
constexpr int kFaKBytes = kFaKeys * kFaD * 2;
constexpr int kFaPBytes = kFaRows * kFaKeys * 2;
constexpr int kFaStages = 3;
constexpr int kFaSmem = kFaQBytes + kFaStages * 2 * kFaKBytes + 2 * kFaPBytes + 1024;
constexpr int kFaTmemCols = 256;                      // S0 at 0, S1 at 64, O_page at 128
constexpr float kFaLog2e = 1.4426950408889634f;

__device__ __forceinline__ void fa_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ float fa_exp2(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

// The product with the first operand in tensor memory (rows = lanes, 16 k = 8 columns of bfloat16 pairs).
__device__ __forceinline__ void umma_bf16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}

#if DFI_FA_ENABLED
__global__ void __launch_bounds__(kFaThreads, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int out_stride,
                            const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_rows,
                            const int* __restrict__ seq_start, int n_q, int n_kv, int ring_tokens, int window,
                            float scale_log2) {
    pdl_launch_next();
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, kv_full[kFaStages], kv_empty[kFaStages];
    __shared__ __align__(8) uint64_t s_full[2], s_empty[2], p_full[2], pv_done[2], o_empty;
    __shared__ uint32_t tmem_base_s;

    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = base;                                   // [blocks][128 rows][128 bytes]
    unsigned char* kv_s = q_s + kFaQBytes;                       // [stages][K: blocks x 64 x 128 B | V: blocks x 64 x 128 B]
    unsigned char* p_s = kv_s + kFaStages * 2 * kFaKBytes;       // [2][128 rows][128 bytes]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int row0 = cu_rows[seq], q_len = cu_rows[seq + 1] - row0;
    // the heaviest tiles (the last rows of a prompt) are started first
    const int n_row_tiles = (q_len + kFaRows - 1) / kFaRows;
    if ((int)blockIdx.x >= n_row_tiles) return;
    const int r0 = (n_row_tiles - 1 - blockIdx.x) * kFaRows;
    const int rows_here = min(kFaRows, q_len - r0);
    const int start = seq_start[seq];
    const int kv_len = start + q_len;
    const int kv_head = head / (n_q / n_kv);
    const int* table = block_table + (size_t)seq * table_width;
    const int last_key = start + r0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, start + r0 - window + 1) : 0;
    const int t_begin = first_key / kFaKeys, t_end = last_key / kFaKeys;
    const int n_tiles = t_end - t_begin + 1;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < kFaStages; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&s_empty[i], 128);
            mbar_init(&p_full[i], 128);
            mbar_init(&pv_done[i], 1);
        }
        mbar_init(&o_empty, 128);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(kFaTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();        // the queries and this step's keys and values come from the kernel before

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, kFaQBytes);
#pragma unroll
            for (int b = 0; b < kFaBlocks; ++b)
                tma_load_2d(q_s + b * (kFaRows * 128), &map_q, head * kFaD + b * 64, row0 + r0, &q_full);
            for (int j = 0; j < n_tiles; ++j) {
                const int st = j % kFaStages;
                const uint32_t round = j / kFaStages;
                if (round > 0 && !mbar_wait(&kv_empty[st], (round - 1) & 1, 11)) break;
                const int tile = t_begin + j;
                const int place = place_of(tile * kFaKeys, ring_tokens);
                const int page = table[place / kFaKeys];
                const int cache_row = (page * n_kv + kv_head) * kFaKeys;
                unsigned char* k_tile = kv_s + (size_t)st * 2 * kFaKBytes;
                unsigned char* v_tile = k_tile + kFaKBytes;
                mbar_expect_tx(&kv_full[st], 2 * kFaKBytes);
#pragma unroll
                for (int b = 0; b < kFaBlocks; ++b) {
                    tma_load_2d(k_tile + b * (kFaKeys * 128), &map_k, b * 64, cache_row, &kv_full[st]);
                    tma_load_2d(v_tile + b * (kFaKeys * 128), &map_v, b * 64, cache_row, &kv_full[st]);
                }
            }
        }
    } else if (warp == 1) {
        // S = Q K^T: N = 64 keys.  O_page = P V: N = head size, second operand MN-major.
        constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kFaKeys >> 3) << 17) | ((uint32_t)(kFaRows >> 4) << 24);
        constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kFaD >> 3) << 17) | ((uint32_t)(kFaRows >> 4) << 24);
        bool ok = mbar_wait(&q_full, 0, 12);
        auto issue_pv = [&](int j) {
            // the page's P is in shared memory, and the output of the page before has been taken
            if (!mbar_wait(&p_full[j & 1], (j >> 1) & 1, 13)) return false;
            if (j >= 1 && !mbar_wait(&o_empty, (j - 1) & 1, 14)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int st = j % kFaStages;
            unsigned char* v_tile = kv_s + (size_t)st * 2 * kFaKBytes + kFaKBytes;
            // value rows of keys that were never written (only in a sequence's last page) are zeroed
            const int dead_from = kv_len - (t_begin + j) * kFaKeys;
            if (dead_from < kFaKeys) {
                for (int i = lane; i < (kFaKeys - max(dead_from, 0)) * 8 * kFaBlocks; i += 32) {
                    const int b = i / ((kFaKeys - max(dead_from, 0)) * 8), rest = i % ((kFaKeys - max(dead_from, 0)) * 8);
                    const int row = max(dead_from, 0) + rest / 8, chunk = rest % 8;
                    *reinterpret_cast<uint4*>(v_tile + b * (kFaKeys * 128) + row * 128 + chunk * 16) = make_uint4(0, 0, 0, 0);
                }
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncwarp();
            }
            if (lane == 0) {
                const uint64_t p_desc = umma_desc(p_s + (j & 1) * kFaPBytes);
#pragma unroll
                for (int k = 0; k < kFaKeys / kUmmaK; ++k)
                    umma_bf16(tmem_base + 128, p_desc + 2 * k, umma_desc_mn(v_tile + k * 2048, kFaKeys * 128), idesc_pv, k > 0 ? 1u : 0u);
                umma_commit(&pv_done[j & 1]);
                umma_commit(&kv_empty[st]);
            }
            __syncwarp();
            return true;
        };
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int st = j % kFaStages;
            ok = mbar_wait(&kv_full[st], (j / kFaStages) & 1, 15);
            if (ok && j >= 2) ok = mbar_wait(&s_empty[j & 1], ((j >> 1) - 1) & 1, 16);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                const unsigned char* k_tile = kv_s + (size_t)st * 2 * kFaKBytes;
#pragma unroll
                for (int kk = 0; kk < kFaD / kUmmaK; ++kk) {
                    const uint64_t a = umma_desc(q_s + (kk / 4) * (kFaRows * 128)) + 2 * (kk % 4);
                    const uint64_t b = umma_desc(k_tile + (kk / 4) * (kFaKeys * 128)) + 2 * (kk % 4);
                    umma_bf16(tmem_base + (j & 1) * 64, a, b, idesc_qk, kk > 0 ? 1u : 0u);
                }
                umma_commit(&s_full[j & 1]);
            }
            __syncwarp();
            if (j >= 1) ok = issue_pv(j - 1);
        }
        if (ok) issue_pv(n_tiles - 1);
    } else {
        // ---- softmax and output: thread `t` owns query row r0 + t (tensor-memory lane t)
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;
        const int pos = start + r0 + t;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        float o[kFaD];
#pragma unroll
        for (int d = 0; d < kFaD; ++d) o[d] = 0.f;
        float m = -INFINITY, l = 0.f;
        bool ok = true;
        auto take_page_output = [&](int j) {
            if (!mbar_wait(&pv_done[j & 1], (j >> 1) & 1, 17)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll
            for (int c = 0; c < kFaD; c += 32) {
                uint32_t v[32];
                tmem_load32(lane_addr + 128 + c, v);
#pragma unroll
                for (int e = 0; e < 32; ++e) o[c + e] += __uint_as_float(v[e]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            fa_arrive(&o_empty);
            return true;
        };
        for (int j = 0; j < n_tiles && ok; ++j) {
            ok = mbar_wait(&s_full[j & 1], (j >> 1) & 1, 18);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            uint32_t sv[64];
            {
                uint32_t half[32];
                tmem_load32(lane_addr + (j & 1) * 64, half);
#pragma unroll
                for (int e = 0; e < 32; ++e) sv[e] = half[e];
                tmem_load32(lane_addr + (j & 1) * 64 + 32, half);
#pragma unroll
                for (int e = 0; e < 32; ++e) sv[32 + e] = half[e];
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            fa_arrive(&s_empty[j & 1]);

            const int key0 = (t_begin + j) * kFaKeys;
            const bool partial = key0 + kFaKeys - 1 > pos || (window > 0 && key0 < pos - window + 1);
            // the maximum is kept in the scores' own units; the scale enters in the exponent's multiply-add
            float mx = -INFINITY;
            if (partial) {
#pragma unroll
                for (int e = 0; e < 64; ++e) {
                    const int key = key0 + e;
                    const bool seen = key <= pos && (window <= 0 || key > pos - window);
                    const float x = seen ? __uint_as_float(sv[e]) : -INFINITY;
                    sv[e] = __float_as_uint(x);
                    mx = fmaxf(mx, x);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 64; ++e) mx = fmaxf(mx, __uint_as_float(sv[e]));
            }
            const float m_new = fmaxf(m, mx);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = fa_exp2((m - m_use) * scale_log2);
            const float shift = -m_use * scale_log2;
            float sum = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const float p0 = fa_exp2(fmaf(__uint_as_float(sv[e]), scale_log2, shift));
                const float p1 = fa_exp2(fmaf(__uint_as_float(sv[e + 1]), scale_log2, shift));
                sum += p0 + p1;
                __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                packed[e >> 1] = *reinterpret_cast<uint32_t*>(&pair);
            }
            // row t of P: 128 bytes, its 16-byte pieces placed as the 128-byte swizzle places them
            unsigned char* p_row = p_s + (j & 1) * kFaPBytes + t * 128;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4*>(p_row + ((c ^ (t & 7)) << 4)) =
                    make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            fa_arrive(&p_full[j & 1]);
            // while the tensor core multiplies this page's P by V: add the page before into the row,
            // then rescale the row for this page's maximum (skipped when no row of the warp moved)
            if (j >= 1) ok = take_page_output(j - 1);
            if (!ok) break;
            l = l * corr + sum;
            m = m_new;
            if (__any_sync(0xffffffffu, corr != 1.0f)) {
#pragma unroll
                for (int d = 0; d < kFaD; ++d) o[d] *= corr;
            }
        }
        if (ok) ok = take_page_output(n_tiles - 1);
        if (ok && t < rows_here) {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + (size_t)(row0 + r0 + t) * out_stride + (size_t)head * kFaD;
#pragma unroll
            for (int d = 0; d < kFaD; d += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = o[d + e] * inv;
                store16(dst + d, v);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFaTmemCols) : "memory");
    }
}

#ifdef DFI_TRACE
// Timing of the two-tile kernel's phases, summed per CTA: [wait scores, load, arithmetic, store and
// arrive, total, pages, issuer's wait for P, issuer's issue] in nanoseconds (first softmax thread of
// tile 0 and the issuing thread).
__device__ unsigned long long g_fa_trace[1024 * 8];
__device__ __forceinline__ unsigned long long fa_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}
#define FA_T(var) const unsigned long long var = fa_now()
#define FA_ADD(slot, value) do { if (trace_cta < 1024) g_fa_trace[trace_cta * 8 + (slot)] += (value); } while (0)
#else
#define FA_T(var)
#define FA_ADD(slot, value)
#endif

// ------------------------------------------------------------------ two query tiles per CTA
// For prompts longer than one tile: a CTA owns 256 query rows as two tiles of 128, each with a
// softmax warp group of its own, and the tensor core alternates between them, so that the scores of
// one tile are turned into probabilities while the other tile's products run.  The output rows stay
// in tensor memory and are accumulated there by the MMA itself; a row is rescaled (by its softmax
// thread, between two pages) only when its maximum has grown by more than 2^8 since the scale was
// last fixed, which after the first pages of a row happens rarely.  The probabilities never touch
// shared memory: a thread writes its row's bfloat16 pairs into tensor memory (tcgen05.st), and the
// product with V takes them from there as its first operand.  A tcgen05.commit arrives only
// when every MMA issued before it is complete, so "the next scores are ready" also tells the
// softmax threads that the products issued before them have finished reading P and writing the output.
//
// Pages are taken two at a time: the keys of a pair of pages lie in shared memory as one tile of 128 keys,
// and the scores of a query tile against both come from one group of MMAs with N = 128 (the query operand,
// 4 KB of shared memory per MMA, is fetched once for 128 keys instead of once for 64: an MMA of 128 x 64 x 16
// took 84 clocks for 32 clocks of arithmetic).  The softmax still goes page by page (64 scores a row at a
// time), and the second page's scores are there while the first page's product with V runs.  The
// probabilities of a page overwrite the first half of that page's scores.
constexpr int kFa2Threads = 320;                                   // producer, issuer, 2 x 4 softmax warps
constexpr int kFa2Stages = 2;                                      // pairs of pages of keys and values in flight
constexpr int kFa2PairBytes = 4 * kFaKBytes;                       // keys of two pages as one tile, values page by page
constexpr int kFa2Smem = 2 * kFaQBytes + kFa2Stages * kFa2PairBytes + 1024;
constexpr int kFa2TmemCols = 512;      // S of tile X at 128 X (page p of the pair at + 64 p, its P over its first 32), output at 256 + 128 X
constexpr float kFaRescaleStep = 8.0f;                             // in log2 units

__global__ void __launch_bounds__(kFa2Threads, 1)
attention_prefill_tc2_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, int out_stride,
                             const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_rows,
                             const int* __restrict__ seq_start, int n_q, int n_kv, int ring_tokens, int window,
                             float scale_log2) {
    pdl_launch_next();
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t q_full, kv_full[kFa2Stages], kv_empty[kFa2Stages];
    __shared__ __align__(8) uint64_t s_full[2], p_full[2][2], pv_first[2], all_done;
    __shared__ uint32_t tmem_base_s;

    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* q_s = base;                                   // [tile][blocks][128 rows][128 bytes]
    unsigned char* kv_s = q_s + 2 * kFaQBytes;                   // [stage][K: blocks x 128 keys x 128 B | V: 2 pages x blocks x 64 x 128 B]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // CTAs start in the order of blockIdx.x, then y: the head is x and the rows are y, latest rows
    // first, so that the CTAs with the most keys to walk all start in the first wave
    const int seq = blockIdx.z, head = blockIdx.x;
#ifdef DFI_TRACE
    const int trace_cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
#endif
    const int row0 = cu_rows[seq], q_len = cu_rows[seq + 1] - row0;
    const int n_row_tiles = (q_len + 2 * kFaRows - 1) / (2 * kFaRows);
    const int behind = (int)gridDim.y - 1 - (int)blockIdx.y;              // row tiles after this one
    if (behind >= n_row_tiles) return;
    const int r0 = behind * 2 * kFaRows;
    const int rows_here = min(2 * kFaRows, q_len - r0);
    const bool has_b = rows_here > kFaRows;
    const int start = seq_start[seq];
    const int kv_len = start + q_len;
    const int kv_head = head / (n_q / n_kv);
    const int* table = block_table + (size_t)seq * table_width;
    const int first_key = window > 0 ? max(0, start + r0 - window + 1) : 0;
    const int t_begin = first_key / kFaKeys;
    // pages each tile walks (both start at t_begin; a tile stops at its own diagonal)
    const int n_a = (start + r0 + min(rows_here, kFaRows) - 1) / kFaKeys - t_begin + 1;
    const int n_b = has_b ? (start + r0 + rows_here - 1) / kFaKeys - t_begin + 1 : 0;
    const int n_tiles = max(n_a, n_b);

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int i = 0; i < kFa2Stages; ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1);
            mbar_init(&p_full[i][0], 128);     // one barrier for each page of a pair: the softmax threads go from a pair's
            mbar_init(&p_full[i][1], 128);     // first page to its second without waiting, and a barrier must not be two phases ahead of its waiter
            mbar_init(&pv_first[i], 1);
        }
        mbar_init(&all_done, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(kFa2TmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(&q_full, (has_b ? 2 : 1) * kFaQBytes);
            for (int x = 0; x < (has_b ? 2 : 1); ++x)
#pragma unroll
                for (int b = 0; b < kFaBlocks; ++b)
                    tma_load_2d(q_s + x * kFaQBytes + b * (kFaRows * 128), &map_q, head * kFaD + b * 64,
                                row0 + r0 + x * kFaRows, &q_full);
            const int n_pairs = (n_tiles + 1) / 2;
            for (int pr = 0; pr < n_pairs; ++pr) {
                const int st = pr % kFa2Stages;
                const uint32_t round = pr / kFa2Stages;
                if (round > 0 && !mbar_wait(&kv_empty[st], (round - 1) & 1, 21)) break;
                const int pages = min(2, n_tiles - 2 * pr);
                unsigned char* k_pair = kv_s + (size_t)st * kFa2PairBytes;
                unsigned char* v_pair = k_pair + 2 * kFaKBytes;
                mbar_expect_tx(&kv_full[st], pages * 2 * kFaKBytes);
                for (int p = 0; p < pages; ++p) {
                    const int place = place_of((t_begin + 2 * pr + p) * kFaKeys, ring_tokens);
                    const int page = table[place / kFaKeys];
                    const int cache_row = (page * n_kv + kv_head) * kFaKeys;
#pragma unroll
                    for (int b = 0; b < kFaBlocks; ++b) {
                        // keys: rows 64 p .. 64 p + 63 of the pair's tile of 128 keys; values: the page's own tile
                        tma_load_2d(k_pair + b * (2 * kFaKeys * 128) + p * (kFaKeys * 128), &map_k, b * 64, cache_row, &kv_full[st]);
                        tma_load_2d(v_pair + p * kFaKBytes + b * (kFaKeys * 128), &map_v, b * 64, cache_row, &kv_full[st]);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // S = Q K^T for a pair of pages: N = 128 keys.  O += P V page by page: N = head size, V MN-major.
        constexpr uint32_t idesc_qk = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)((2 * kFaKeys) >> 3) << 17) | ((uint32_t)(kFaRows >> 4) << 24);
        constexpr uint32_t idesc_pv = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(kFaD >> 3) << 17) | ((uint32_t)(kFaRows >> 4) << 24);
        bool ok = mbar_wait(&q_full, 0, 22);
        auto n_of = [&](int x) { return x == 0 ? n_a : n_b; };
        const int n_pairs = (n_tiles + 1) / 2;
        auto issue_qk = [&](int x, int pr) {        // lane 0 only: the scores of tile x against the pair's 128 keys
            const unsigned char* k_pair = kv_s + (size_t)(pr % kFa2Stages) * kFa2PairBytes;
#pragma unroll
            for (int kk = 0; kk < kFaD / kUmmaK; ++kk) {
                const uint64_t a = umma_desc(q_s + x * kFaQBytes + (kk / 4) * (kFaRows * 128)) + 2 * (kk % 4);
                const uint64_t b = umma_desc(k_pair + (kk / 4) * (2 * kFaKeys * 128)) + 2 * (kk % 4);
                umma_bf16(tmem_base + x * 128, a, b, idesc_qk, kk > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[x]);
        };
        // pair 0: scores of both tiles
        if (ok) ok = mbar_wait(&kv_full[0], 0, 23);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                issue_qk(0, 0);
                if (has_b) issue_qk(1, 0);
            }
            __syncwarp();
        }
        for (int pr = 0; pr < n_pairs && ok; ++pr) {
            const int st = pr % kFa2Stages;
            unsigned char* v_pair = kv_s + (size_t)st * kFa2PairBytes + 2 * kFaKBytes;
            // value rows of keys that were never written (only in the sequence's last page) are zeroed
            for (int p = 0; p < 2; ++p) {
                const int dead_from = max(kv_len - (t_begin + 2 * pr + p) * kFaKeys, 0);
                if (2 * pr + p < n_tiles && dead_from < kFaKeys) {
                    const int n_dead = kFaKeys - dead_from;
                    for (int i = lane; i < n_dead * 8 * kFaBlocks; i += 32) {
                        const int b = i / (n_dead * 8), rest = i % (n_dead * 8);
                        *reinterpret_cast<uint4*>(v_pair + p * kFaKBytes + b * (kFaKeys * 128) + (dead_from + rest / 8) * 128 + (rest % 8) * 16) = make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    __syncwarp();
                }
            }
            bool next_landed = false;                          // the next pair's keys, needed by the first scores against them
            for (int p = 0; p < 2 && ok; ++p) {
                const int j = 2 * pr + p;
                for (int x = 0; x < 2 && ok; ++x) {
                    if (j >= n_of(x)) continue;
                    const bool last_of_pair = !(p == 0 && j + 1 < n_of(x));
                    if (last_of_pair && 2 * (pr + 1) < n_of(x) && !next_landed) {
                        ok = mbar_wait(&kv_full[(pr + 1) % kFa2Stages], ((pr + 1) / kFa2Stages) & 1, 24);
                        if (!ok) break;
                        next_landed = true;
                    }
                    FA_T(ti0);
                    ok = mbar_wait(&p_full[x][p], pr & 1, 25);    // P of page j is in tensor memory, its scores have been read
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    FA_T(ti1);
                    if (lane == 0) FA_ADD(6, ti1 - ti0);
                    if (lane == 0) {
                        // P lies over the first 32 columns of the page's scores: 16 keys of a row are 8 columns of pairs
#pragma unroll
                        for (int k = 0; k < kFaKeys / kUmmaK; ++k)
                            umma_bf16_ts(tmem_base + 256 + x * 128, tmem_base + x * 128 + p * 64 + 8 * k,
                                         umma_desc_mn(v_pair + p * kFaKBytes + k * 2048, kFaKeys * 128), idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
                        if (p == 0 && j + 1 < n_of(x)) {
                            umma_commit(&pv_first[x]);             // the softmax of the pair's second page may rescale the output after this
                        } else if (2 * (pr + 1) < n_of(x)) {
                            issue_qk(x, pr + 1);                   // the tile is through with this pair; its commit also covers the product just issued
                        }
                        FA_T(ti2);
                        FA_ADD(7, ti2 - ti1);
                    }
                    __syncwarp();
                }
            }
            if (lane == 0) umma_commit(&kv_empty[st]);         // the pair's last user has been issued
            __syncwarp();
        }
        if (lane == 0) umma_commit(&all_done);
        __syncwarp();
    } else {
        // ---- softmax warp groups: warps 2-5 own tile 0, warps 6-9 tile 1; thread t of a group owns row t
        const int x = (warp - 2) >> 2;
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;
        const int n_mine = x == 0 ? n_a : n_b;
        const int pos = start + r0 + x * kFaRows + t;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t s_pair = lane_addr + x * 128, o_addr = lane_addr + 256 + x * 128;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
#ifdef DFI_TRACE
        const bool tracer = x == 0 && t == 0;
        const unsigned long long t_begin_all = fa_now();
#endif
        for (int j = 0; j < n_mine && ok; ++j) {
            FA_T(ts0);
            const int pr = j >> 1, p = j & 1;                  // page p of pair pr: its scores at + 64 p
            const uint32_t s_addr = s_pair + p * 64;
            if (p == 0) {
                ok = mbar_wait(&s_full[x], pr & 1, 26);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            }
            FA_T(ts1);
            uint32_t sv[64];
            {
                uint32_t half[32];
                tmem_load32(s_addr, half);
#pragma unroll
                for (int e = 0; e < 32; ++e) sv[e] = half[e];
                tmem_load32(s_addr + 32, half);
#pragma unroll
                for (int e = 0; e < 32; ++e) sv[32 + e] = half[e];
            }
            FA_T(ts2);
            const int key0 = (t_begin + j) * kFaKeys;
            const bool partial = key0 + kFaKeys - 1 > pos || (window > 0 && key0 < pos - window + 1);
            float mx = -INFINITY;
            if (partial) {
#pragma unroll
                for (int e = 0; e < 64; ++e) {
                    const int key = key0 + e;
                    const bool seen = key <= pos && (window <= 0 || key > pos - window);
                    const float v = seen ? __uint_as_float(sv[e]) : -INFINITY;
                    sv[e] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
            } else {
#pragma unroll
                for (int e = 0; e < 64; ++e) mx = fmaxf(mx, __uint_as_float(sv[e]));
            }
            // the scale of the row is moved only when its maximum has outgrown it by 2^8
            float corr = 1.0f;
            if (mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * scale_log2 > kFaRescaleStep)) {
                corr = m_ref == -INFINITY ? 0.f : fa_exp2((m_ref - mx) * scale_log2);
                m_ref = mx;
            }
            if (j > 0 && __any_sync(0xffffffffu, corr != 1.0f)) {
                // The product of the page before must be complete before the output is touched.  For a pair's first
                // page it is: the pair's scores were issued after it.  For the second page the issuing thread
                // commits the first page's product to a barrier of its own.
                if (p == 1) {
                    ok = mbar_wait(&pv_first[x], pr & 1, 30);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                }
#pragma unroll
                for (int c = 0; c < kFaD; c += 32) {
                    uint32_t v[32];
                    tmem_load32(o_addr + c, v);
#pragma unroll
                    for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * corr);
                    asm volatile(
                        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                        ::"r"(o_addr + c), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
                          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
                          "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                          "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                        : "memory");
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            }
            const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
            const float shift = -m_use * scale_log2;
            float sum = 0.f;
            uint32_t packed[32];
#pragma unroll
            for (int e = 0; e < 64; e += 2) {
                const float p0 = fa_exp2(fmaf(__uint_as_float(sv[e]), scale_log2, shift));
                const float p1 = fa_exp2(fmaf(__uint_as_float(sv[e + 1]), scale_log2, shift));
                sum += p0 + p1;
                __nv_bfloat162 pair = __floats2bfloat162_rn(p0, p1);
                packed[e >> 1] = *reinterpret_cast<uint32_t*>(&pair);
            }
            l = l * corr + sum;
            // the probabilities go over the first half of the page's scores (all 64 are in registers by now), where the
            // product with V takes them as its first operand
            asm volatile(
                "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
                "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n"
                ::"r"(s_addr), "r"(packed[0]), "r"(packed[1]), "r"(packed[2]), "r"(packed[3]), "r"(packed[4]),
                  "r"(packed[5]), "r"(packed[6]), "r"(packed[7]), "r"(packed[8]), "r"(packed[9]), "r"(packed[10]), "r"(packed[11]),
                  "r"(packed[12]), "r"(packed[13]), "r"(packed[14]), "r"(packed[15]), "r"(packed[16]), "r"(packed[17]),
                  "r"(packed[18]), "r"(packed[19]), "r"(packed[20]), "r"(packed[21]), "r"(packed[22]), "r"(packed[23]),
                  "r"(packed[24]), "r"(packed[25]), "r"(packed[26]), "r"(packed[27]), "r"(packed[28]), "r"(packed[29]),
                  "r"(packed[30]), "r"(packed[31])
                : "memory");
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            FA_T(ts3);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            fa_arrive(&p_full[x][p]);
#ifdef DFI_TRACE
            if (tracer) {
                const unsigned long long ts4 = fa_now();
                FA_ADD(0, ts1 - ts0); FA_ADD(1, ts2 - ts1); FA_ADD(2, ts3 - ts2); FA_ADD(3, ts4 - ts3); FA_ADD(5, 1);
            }
#endif
        }
#ifdef DFI_TRACE
        if (tracer) FA_ADD(4, fa_now() - t_begin_all);
#endif
        if (ok && n_mine > 0) ok = mbar_wait(&all_done, 0, 27);
        if (ok && n_mine > 0) {
            // every thread of the warp takes part in the loads; rows past the prompt's end store nothing
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const bool mine = x * kFaRows + t < rows_here;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = out + (size_t)(row0 + r0 + x * kFaRows + (mine ? t : 0)) * out_stride + (size_t)head * kFaD;
#pragma unroll
            for (int c = 0; c < kFaD; c += 32) {
                uint32_t v[32];
                tmem_load32(o_addr + c, v);
                if (mine) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        float f[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(v[d + e]) * inv;
                        store16(dst + c + d, f);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(kFa2TmemCols) : "memory");
    }
}
#endif  // DFI_FA_ENABLED

}  // namespace dfi

using namespace dfi;

DFI_TCGEN05_STATUS_ENTRIES(attention_prefill_tc)

#ifdef DFI_TRACE
DFI_EXPORT int dfi_attention_prefill_trace(unsigned long long* host) {
    if (cudaMemcpyFromSymbol(host, g_fa_trace, sizeof(unsigned long long) * 1024 * 8) != cudaSuccess) return -1;
    cudaMemset(nullptr, 0, 0);
    return 0;
}
DFI_EXPORT int dfi_attention_prefill_trace_reset() {
    static unsigned long long zeros[1024 * 8];
    return cudaMemcpyToSymbol(g_fa_trace, zeros, sizeof(zeros)) == cudaSuccess ? 0 : -1;
}
#endif

// 1 if this build (head size) has the tcgen05 prefill kernel.
DFI_EXPORT int dfi_attention_prefill_tc_available() { return DFI_FA_ENABLED; }

// q [rows, q_stride] (the head's columns start at head * head_dim), out [rows, out_stride];
// k_cache, v_cache [pages, n_kv, 64, head_dim]; cache_pages = number of pages in them.
// tiles_per_cta: 1 or 2 query tiles of 128 rows per CTA, or 0 to let the launch choose.
DFI_EXPORT int dfi_attention_prefill_tc(const void* q, int q_rows, int q_stride, void* out, int out_stride,
                                        const void* k_cache, const void* v_cache, long long cache_pages,
                                        const int* block_table, int table_width, const int* cu_rows,
                                        const int* seq_start, int n_seqs, int max_q_len, int n_q, int n_kv,
                                        int page_size, int ring_tokens, int window, float scale, int tiles_per_cta,
                                        void* stream) {
#if DFI_FA_ENABLED
    if (n_seqs <= 0 || max_q_len <= 0) return DFI_OK;
    if (page_size != kFaKeys || n_q <= 0 || n_kv <= 0 || n_q % n_kv || ring_tokens % kFaKeys) return DFI_ERR_SHAPE;
    if (q_stride % 8 || out_stride % 8 || !aligned16(q) || !aligned16(out) || !aligned16(k_cache) || !aligned16(v_cache))
        return DFI_ERR_ALIGN;
    if (n_q > 65535 || n_seqs > 65535 || max_q_len / (2 * kFaRows) >= 65535) return DFI_ERR_LIMIT;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFaSmem) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    CUtensorMap map_q, map_k, map_v;
    const long long cache_rows = cache_pages * n_kv * kFaKeys;
    if (cache_rows > 0x7fffffffLL) return DFI_ERR_LIMIT;
    if (!make_tile_map(&map_q, q, q_rows, n_q * kFaD, kFaRows, q_stride)) return DFI_ERR_LAUNCH;
    if (!make_tile_map(&map_k, k_cache, (int)cache_rows, kFaD, kFaKeys)) return DFI_ERR_LAUNCH;
    if (!make_tile_map(&map_v, v_cache, (int)cache_rows, kFaD, kFaKeys)) return DFI_ERR_LAUNCH;
    static int sms = 0;
    if (sms == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
            sms = 1;
    }
    // CTAs of two tiles each; if they would leave half the SMs idle (one prompt of up to 512 tokens with 32 heads),
    // CTAs of one tile do better although a tile alone runs its pages more slowly (measured at 512 tokens:
    // 16.4 against 19.3 us; at 768 tokens 29.4 against 25.2)
    // (counted from the rows there are: a step laid out at a larger shape has sequences without rows)
    const long long ctas2 = (long long)n_q * ((q_rows + 2 * kFaRows - 1) / (2 * kFaRows));
    if (tiles_per_cta < 0 || tiles_per_cta > 2) return DFI_ERR_SHAPE;
    if (max_q_len > kFaRows && (tiles_per_cta == 2 || (tiles_per_cta == 0 && ctas2 * 2 > sms))) {
        // long shares: two query tiles per CTA, each with softmax warps of its own
        static bool configured2 = false;
        if (!configured2) {
            if (cudaFuncSetAttribute(attention_prefill_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFa2Smem) != cudaSuccess)
                return DFI_ERR_LAUNCH;
            configured2 = true;
        }
        dim3 grid2(n_q, (max_q_len + 2 * kFaRows - 1) / (2 * kFaRows), n_seqs);
        launch(attention_prefill_tc2_kernel, grid2, kFa2Threads, kFa2Smem, (cudaStream_t)stream, map_q, map_k, map_v,
               (bf16*)out, out_stride, block_table, table_width, cu_rows, seq_start, n_q, n_kv, ring_tokens, window,
               scale * kFaLog2e);
        DFI_CHECK_LAUNCH();
        return DFI_OK;
    }
    dim3 grid((max_q_len + kFaRows - 1) / kFaRows, n_q, n_seqs);
    launch(attention_prefill_tc_kernel, grid, kFaThreads, kFaSmem, (cudaStream_t)stream, map_q, map_k, map_v, (bf16*)out,
           out_stride, block_table, table_width, cu_rows, seq_start, n_q, n_kv, ring_tokens, window, scale * kFaLog2e);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
#else
    return DFI_ERR_SHAPE;
#endif
}
