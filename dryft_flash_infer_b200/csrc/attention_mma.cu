// bfloat16 attention over the paged cache on the tensor cores, for one head size per
// build (-DDFI_HEAD_DIM=..., a multiple of 16 up to 128).
//
//   dfi_attention_prefill   any number of query rows per sequence (a whole prompt, a chunk
//                           of one): flash attention with causal mask, grouped-query heads,
//                           optional window.  One CTA per (64 query rows, query head).
//   dfi_attention_decode    one query row per sequence: the G query heads of a key/value
//                           head are the rows of one MMA tile.  One kernel: the pages of all
//                           (sequence, head) groups are dealt to the CTAs (equal parts per
//                           group when all sequences are as long, else equal contiguous runs),
//                           and the parts of a group are merged by the last CTA to arrive
//                           or, four parts in a thread-block cluster, through distributed
//                           shared memory.  No CTA waits for another outside a cluster barrier.
//   dfi_attention_decode_prepared   the same, and the kernel also does the per-head RMS norm and
//                           rotation of the step's q and k and writes the new key and value
//                           into the cache (what a kernel before attention would do).
//
// Both follow the online softmax of the reference's split kernel
// (engine/kernels/attention.py:40-137; merge :140-177): float32 scores, maximum, sum and
// accumulator; probabilities rounded to bfloat16 for the product with V.  Keys and values
// come one page (64 tokens) at a time; the tensor-core instruction is mma.sync m16n8k16 (operands
// in registers via ldmatrix).  The decode kernel, for head sizes 64 and 128, fetches a page as TMA
// boxes of 64 tokens x 64 elements with the 128-byte swizzle (one thread asks, an mbarrier says when
// the page has landed; ldmatrix applies the same swizzle, which keeps it free of bank conflicts
// without padding); the other head sizes and the prompt kernel use cp.async into padded rows.
//
// Places of the cache that no token was written to may hold anything (NaN included):
// scores of masked keys are replaced, not added to, and value rows past the sequence's
// end are zero-filled on load, so such places never reach a result.
#include <stdlib.h>

#include "decode_plan.h"
#include "tcgen05.cuh"

#ifndef DFI_HEAD_DIM
#define DFI_HEAD_DIM 128
#endif

namespace dfi {

constexpr int D = DFI_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 128, "head size must be a multiple of 16 up to 128");
constexpr int kStride = D + 8;      // padded row: 16-byte chunks at an odd stride are conflict-free for ldmatrix
constexpr int kRedStride = D + 8;   // floats per row of the merge buffers: eight rows stored at once fall into different banks
constexpr int kChunks = D / 8;      // 16-byte chunks per row
constexpr int kThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;
constexpr bool kTmaPages = D % 64 == 0;                               // the decode kernel's pages come by TMA
constexpr int kDecTile = kTmaPages ? kPage * D : kPage * kStride;     // elements of one tile of its ring

// Address of the 16-byte chunk at (row, col), col a multiple of 8, of a tile of 64 rows: padded rows, or
// (SW) column blocks of 64 elements, each [64 rows][128 bytes] with the chunk index XORed by row mod 8.
template <bool SW>
__device__ __forceinline__ const bf16* tile_chunk(const bf16* tile, int row, int col) {
    if (SW) return tile + (col >> 6) * (kPage * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3);
    return tile + row * kStride + col;
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Copies one page of one key/value head ([64][D], contiguous) into padded shared memory.
// Rows whose key index is not below `live_keys` are zero-filled when `zero_dead` is set.
__device__ __forceinline__ void load_page(bf16* dst, const bf16* src, int first_key, int live_keys, bool zero_dead) {
    for (int i = threadIdx.x; i < kPage * kChunks; i += kThreads) {
        const int row = i / kChunks, c = i % kChunks;
        const bool valid = !zero_dead || first_key + row < live_keys;
        cp_async16(dst + row * kStride + c * 8, src + (size_t)row * D + c * 8, valid);
    }
}

__device__ __forceinline__ const bf16* page_ptr(const bf16* cache, const int* table, int tile, int ring_tokens,
                                                int n_kv, int kv_head) {
    const int place = place_of(tile * kPage, ring_tokens);
    const int page = table[place / kPage];
    return cache + ((size_t)page * n_kv + kv_head) * kPage * D;
}

// S[16 x 8*NT] += Q[16 x D] . K[keys x D]^T for the NT key tiles starting at row `key0` of k_s.
template <int NT, bool SW = false>
__device__ __forceinline__ void scores(float (&s)[NT][4], const uint32_t (&qf)[D / 16][4], const bf16* k_s, int key0,
                                       int lane) {
    static_assert(NT % 2 == 0, "key tiles come in pairs");
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int j = 0; j < NT; j += 2) {
            uint32_t b[4];
            ldmatrix_x4(b, tile_chunk<SW>(k_s, key0 + j * 8 + r + (mi >> 1) * 8, kk * 16 + (mi & 1) * 8));
            mma_bf16(s[j], qf[kk], b[0], b[1]);
            mma_bf16(s[j + 1], qf[kk], b[2], b[3]);
        }
    }
}

// O[16 x D] += P[16 x 8*NT] . V[keys x D] for the keys starting at row `key0` of v_s.
template <int NT, bool SW = false>
__device__ __forceinline__ void weighted_values(float (&o)[D / 8][4], const float (&p)[NT][4], const bf16* v_s, int key0,
                                                int lane) {
    const int mi = lane >> 3, r = lane & 7;
#pragma unroll
    for (int c = 0; c < NT / 2; ++c) {
        uint32_t a[4];
        a[0] = pack_bf16(p[2 * c][0], p[2 * c][1]);
        a[1] = pack_bf16(p[2 * c][2], p[2 * c][3]);
        a[2] = pack_bf16(p[2 * c + 1][0], p[2 * c + 1][1]);
        a[3] = pack_bf16(p[2 * c + 1][2], p[2 * c + 1][3]);
#pragma unroll
        for (int n = 0; n < D / 8; n += 2) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, tile_chunk<SW>(v_s, key0 + c * 16 + r + (mi & 1) * 8, n * 8 + (mi >> 1) * 8));
            mma_bf16(o[n], a, b[0], b[1]);
            mma_bf16(o[n + 1], a, b[2], b[3]);
        }
    }
}

// One online-softmax update of the two rows (g, g+8) a thread holds, over NT key tiles.
// `s` holds scores in the log2 domain (already scaled); masked entries are -inf.
template <int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&o)[D / 8][4]) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < NT; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * h], s[j][2 * h + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[h], mx);
        const float m_use = m_new == -INFINITY ? 0.f : m_new;   // a row with nothing to see yet
        const float corr = exp2f(m[h] - m_use);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            s[j][2 * h] = exp2f(s[j][2 * h] - m_use);
            s[j][2 * h + 1] = exp2f(s[j][2 * h + 1] - m_use);
            sum += s[j][2 * h] + s[j][2 * h + 1];
        }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        l[h] = l[h] * corr + sum;
        m[h] = m_new;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][2 * h] *= corr;
            o[n][2 * h + 1] *= corr;
        }
    }
}

// ------------------------------------------------------------------ prefill
__global__ void __launch_bounds__(kThreads)
attention_prefill_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                         const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                         const int* __restrict__ block_table, int table_width, const int* __restrict__ cu_rows,
                         const int* __restrict__ seq_start, int n_q, int n_kv, int ring_tokens, int window,
                         float scale_log2) {
    pdl_launch_next();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    bf16* q_s = reinterpret_cast<bf16*>(smem_raw);   // [64][kStride]
    bf16* k_s = q_s + kPage * kStride;               // [2][64][kStride]
    bf16* v_s = k_s + 2 * kPage * kStride;           // [2][64][kStride]

    const int seq = blockIdx.z, head = blockIdx.y;
    const int row0 = cu_rows[seq], q_len = cu_rows[seq + 1] - row0;
    const int r0 = blockIdx.x * 64;
    if (r0 >= q_len) return;
    const int rows_here = min(64, q_len - r0);
    const int start = seq_start[seq];
    const int kv_len = start + q_len;
    const int kv_head = head / (n_q / n_kv);
    const int* table = block_table + (size_t)seq * table_width;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;

    // the query tile; rows past the sequence's share are zeros
    for (int i = threadIdx.x; i < 64 * kChunks; i += kThreads) {
        const int row = i / kChunks, c = i % kChunks;
        const bool valid = row < rows_here;
        const bf16* src = q + (size_t)(row0 + r0 + (valid ? row : 0)) * q_stride + (size_t)head * D + c * 8;
        cp_async16(q_s + row * kStride + c * 8, src, valid);
    }
    const int last_key = start + r0 + rows_here - 1;
    const int first_key = window > 0 ? max(0, start + r0 - window + 1) : 0;
    const int t_begin = first_key / kPage, t_end = last_key / kPage;
    load_page(k_s, page_ptr(k_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, false);
    load_page(v_s, page_ptr(v_cache, table, t_begin, ring_tokens, n_kv, kv_head), t_begin * kPage, kv_len, true);
    cp_async_commit();

    uint32_t qf[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    // positions of the two query rows this thread holds
    const int pos_lo = start + r0 + warp * 16 + g, pos_hi = pos_lo + 8;

    for (int t = t_begin; t <= t_end; ++t) {
        const int stage = (t - t_begin) & 1;
        if (t < t_end) {
            bf16* k_next = k_s + (stage ^ 1) * kPage * kStride;
            bf16* v_next = v_s + (stage ^ 1) * kPage * kStride;
            load_page(k_next, page_ptr(k_cache, table, t + 1, ring_tokens, n_kv, kv_head), (t + 1) * kPage, kv_len, false);
            load_page(v_next, page_ptr(v_cache, table, t + 1, ring_tokens, n_kv, kv_head), (t + 1) * kPage, kv_len, true);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (t == t_begin) {
            const int mi = lane >> 3, r = lane & 7;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk)
                ldmatrix_x4(qf[kk], q_s + (warp * 16 + r + (mi & 1) * 8) * kStride + kk * 16 + (mi >> 1) * 8);
        }
        const bf16* k_t = k_s + stage * kPage * kStride;
        const bf16* v_t = v_s + stage * kPage * kStride;
        float s[8][4];
        scores<8>(s, qf, k_t, 0, lane);
        const int key_base = t * kPage;
        // the tile needs masking if any of its keys is hidden from any row of this warp
        const bool partial = key_base + kPage - 1 > start + r0 + warp * 16 ||
                             (window > 0 && key_base < start + r0 + warp * 16 + 15 - window + 1);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float v = s[j][e] * scale_log2;
                if (partial) {
                    const int key = key_base + j * 8 + t4 * 2 + (e & 1);
                    const int pos = (e & 2) ? pos_hi : pos_lo;
                    const bool seen = key <= pos && (window <= 0 || key > pos - window);
                    v = seen ? v : -INFINITY;
                }
                s[j][e] = v;
            }
        }
        softmax_update<8>(s, m, l, o);
        weighted_values<8>(o, s, v_t, 0, lane);
        __syncthreads();   // everyone is done with this stage before the next load overwrites it
    }

#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int row = warp * 16 + g + h * 8;
        if (row < rows_here) {
            const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
            bf16* dst = out + (size_t)(row0 + r0 + row) * out_stride + (size_t)head * D;
#pragma unroll
            for (int n = 0; n < D / 8; ++n)
                *reinterpret_cast<uint32_t*>(dst + n * 8 + t4 * 2) = pack_bf16(o[n][2 * h] * inv, o[n][2 * h + 1] * inv);
        }
    }
}

// ------------------------------------------------------------------ decode
// One query row per sequence.  The work is the list of (sequence, key/value head, page of keys)
// triples, sequence after sequence; it is dealt to the CTAs in equal contiguous runs, so that a
// batch of unequal contexts, or one that does not fill a whole number of waves, still keeps every
// SM busy for the same time.  A run visits one (sequence, head) group after another.  A CTA that
// sees all the pages of a group writes the group's output itself.  Otherwise it leaves its
// unnormalised accumulator with (maximum, sum) in scratch memory and takes a ticket from the
// group's counter; the CTA that draws the last ticket merges the parts by their log-sum-exp in
// the order of their key ranges (engine/kernels/attention.py:140-177), writes the output and
// resets the counter.  No CTA waits for another.
//
//   part_o  [cta][2][16][D] float32, part_ml [cta][2][16][2]: a CTA's first and last group
//   counters [sequences * kv heads] int32, zero between calls
// Thread-block cluster helpers for the decode kernel's merge.
__device__ __forceinline__ uint32_t dec_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t dec_cluster_map(const void* own, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"((uint32_t)__cvta_generic_to_shared(own)), "r"(rank));
    return out;
}
constexpr bool kFullClusterFits = (D / kDecodeClusterFull) % 4 == 0;
constexpr bool kWideClusterFits = (D / kDecodeClusterWide) % 4 == 0;     // a CTA's share of the columns in fours
__device__ __forceinline__ void dec_cluster_arrive() { asm volatile("barrier.cluster.arrive.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void dec_cluster_wait() { asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory"); }
// The merge of a group's parts inside a cluster of CL CTAs (2, 4, 8 or 16).  Every CTA owns D / CL columns of the
// head and receives, in the space of its query tile, [sender][row][its columns] of the others' sums and then
// [sender][row][maximum, sum]; the space holds dec_cluster_rows(CL) rows of a group (8 query heads, 4 with
// eight CTAs or more), kRows * D * 4 + CL * kRows * 8 bytes, which the query tile's 16 rows always cover.
template <int CL>
__device__ __forceinline__ void dec_cluster_send(const bf16* q_s, int row, int d, float4 acc, float mx, float sum) {
    constexpr int kRows = dec_cluster_rows(CL);
    constexpr int share = D / CL;
    const uint32_t owner = (uint32_t)(d / share);
    const uint32_t base = dec_cluster_map(q_s, owner);
    const int me = (int)dec_cluster_rank();
    const uint32_t o_at = base + (uint32_t)(((me * kRows + row) * share + d % share) * 4);
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(o_at), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
    if (d % share == 0) {
        const uint32_t ml_at = base + (uint32_t)((CL * kRows * share + (me * kRows + row) * 2) * 4);
        asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};\n" ::"r"(ml_at), "f"(mx), "f"(sum) : "memory");
    }
}
// All parts have arrived (the caller has passed the cluster barrier): this CTA adds them, in the order of the
// parts' pages, for its share of the columns and writes the group's rows; `dst` is the group's first row.
template <int CL>
__device__ __forceinline__ void dec_cluster_finish(const bf16* q_s, bf16* dst_group, int group) {
    constexpr int kRows = dec_cluster_rows(CL);
    constexpr int share = D / CL;
    const float* recv_o = reinterpret_cast<const float*>(q_s);
    const float* recv_ml = recv_o + CL * kRows * share;
    const int me = (int)dec_cluster_rank();
    for (int i = threadIdx.x; i < group * (share / 4); i += kThreads) {
        const int row = i / (share / 4), dl = (i % (share / 4)) * 4;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < CL; ++j) mx = fmaxf(mx, recv_ml[(j * kRows + row) * 2]);
        const float m_use = mx == -INFINITY ? 0.f : mx;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < CL; ++j) {
            const float w = exp2f(recv_ml[(j * kRows + row) * 2] - m_use);
            const float4 part = *reinterpret_cast<const float4*>(recv_o + (j * kRows + row) * share + dl);
            acc.x += w * part.x; acc.y += w * part.y; acc.z += w * part.z; acc.w += w * part.w;
            sum += w * recv_ml[(j * kRows + row) * 2 + 1];
        }
        const float inv = sum > 0.f ? 1.0f / sum : 0.f;
        bf16* dst = dst_group + (size_t)row * D + me * share + dl;
        *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    }
}

#ifdef DFI_TRACE
__device__ unsigned long long g_attn_trace[4096 * 8];
__device__ __forceinline__ void atrace(int slot) {
    if (threadIdx.x == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        g_attn_trace[blockIdx.x * 8 + slot] = now;
    }
}
#else
__device__ __forceinline__ void atrace(int) {}
#endif

// The step's own token, prepared inside the decode kernel instead of by a kernel before it: the
// per-head RMS norm and the rotation of q and k (engine/kernels/reference.py:31-46) and the write of
// the new key and value into the cache.  qkv == null: q is ready and the cache holds the token.
struct DecodePrep {
    const bf16* qkv;          // [sequences, qkv_stride]: q heads, then k heads, then v heads of the step's tokens
    int qkv_stride;
    const float* q_weight;    // [D] or null (no per-head norm)
    const float* k_weight;
    float eps;
    const float* cos_table;   // [positions, D/2] or null (no rotation)
    const float* sin_table;
    bf16* k_cache;            // where the new key and value go when write_cache is set
    bf16* v_cache;
    int write_cache;
};
constexpr bool kPrepHeadDim = (D & (D - 1)) == 0;    // the rotation's partner is a lane away by a power of two

// One head vector of D elements, four per lane.  head_load issues every load that the preparation
// needs (so that they travel together); head_finish does the norm (if weight), the rotation (if
// tables) and stores the result as bfloat16 to `dst` (shared or global memory) and, if dst2 is not
// null, there as well.  src == null: zeros.
struct HeadInput {
    uint2 raw;
    float4 weight, cosine, sine;
};
// What the preparation of a head at position `pos` needs besides the head itself: the same for every head of a
// kind at that position, and known before the step's projection has run.
struct HeadTables {
    float4 weight, cosine, sine;
};
__device__ __forceinline__ HeadTables head_tables(const float* weight, const float* cos_t, const float* sin_t, int pos, int lane) {
    constexpr int kLanes = D / 4;
    HeadTables tb;
    tb.weight = tb.cosine = tb.sine = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lane < kLanes) {
        if (weight != nullptr) tb.weight = *reinterpret_cast<const float4*>(weight + 4 * lane);
        if (cos_t != nullptr) {
            const int at = (4 * lane) % (D / 2);
            tb.cosine = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * (D / 2) + at);
            tb.sine = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * (D / 2) + at);
        }
    }
    return tb;
}
__device__ __forceinline__ HeadInput head_load(const bf16* src, const HeadTables& tb, int lane) {
    HeadInput in;
    in.raw = make_uint2(0u, 0u);
    in.weight = tb.weight;
    in.cosine = tb.cosine;
    in.sine = tb.sine;
    if (lane < D / 4 && src != nullptr) in.raw = *reinterpret_cast<const uint2*>(src + 4 * lane);
    return in;
}
__device__ __forceinline__ HeadInput head_load(const bf16* src, const float* weight, const float* cos_t,
                                               const float* sin_t, int pos, int lane) {
    return head_load(src, head_tables(weight, cos_t, sin_t, pos, lane), lane);
}
// `sw_row` >= 0: dst is a swizzled tile (see tile_chunk) and the vector is its row sw_row.
__device__ __forceinline__ void head_finish(const HeadInput& in, bool norm, float eps, bool rotate, bf16* dst, bf16* dst2,
                                            int lane, int sw_row = -1) {
    constexpr int kLanes = D / 4;
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.raw.y));
    float v[4] = {a.x, a.y, b.x, b.y};
    if (norm) {
        float ssq = v[0] * v[0] + v[1] * v[1] + v[2] * v[2] + v[3] * v[3];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        const float scale = 1.0f / sqrtf(ssq / (float)D + eps);
        v[0] *= scale * in.weight.x; v[1] *= scale * in.weight.y; v[2] *= scale * in.weight.z; v[3] *= scale * in.weight.w;
    }
    if (rotate) {
        float partner[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) partner[e] = __shfl_xor_sync(0xffffffffu, v[e], (kLanes / 2) & 31);
        const bool low = lane < kLanes / 2;
        const float cs[4] = {in.cosine.x, in.cosine.y, in.cosine.z, in.cosine.w};
        const float ss[4] = {in.sine.x, in.sine.y, in.sine.z, in.sine.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) v[e] = low ? v[e] * cs[e] - partner[e] * ss[e] : v[e] * cs[e] + partner[e] * ss[e];
    }
    if (lane < kLanes) {
        uint2 packed;
        *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(v[2], v[3]);
        bf16* at = sw_row < 0 ? dst + 4 * lane
                              : const_cast<bf16*>(tile_chunk<true>(dst, sw_row, (4 * lane) & ~7)) + ((4 * lane) & 7);
        *reinterpret_cast<uint2*>(at) = packed;
        if (dst2 != nullptr) *reinterpret_cast<uint2*>(dst2 + 4 * lane) = packed;
    }
}

constexpr int kKvStages = 3;            // pages of keys and values in the decode kernel's ring
constexpr int kMaxParts = 16;           // parts of a group that the merge holds at once (it takes more in rounds)
constexpr int kMaxDecodeSeqs = 1024;    // sequences per launch (their page counts sit in shared memory)

// The plans of every CTA of a launch, worked out once: by one CTA, for the launches of all layers of a step that
// deal the same pages (same sequences, heads, window and launch shape).  Working the plan out costs a CTA that
// starts on an SM where another kernel ran until then one to two microseconds (its divisions, and above all its
// instructions, none of which the SM holds yet), every layer, on the way to its first page; reading it costs
// one load.  This kernel lets no later kernel start before it has ended (it never says launch_dependents), so
// that every reader finds the plans complete, and it waits for everything before it, so that no reader of the
// step before is still looking at them.
template <int CL>
__global__ void __launch_bounds__(kThreads)
attention_decode_plan_kernel(DecodePlan* __restrict__ plans, const int* __restrict__ seq_start, int n_seqs, int n_kv,
                             int group, int window, int launched) {
    __shared__ int cum_s[kMaxDecodeSeqs + 1];
    __shared__ int longest_s, shortest_s;
    for (int i = threadIdx.x; i < n_seqs; i += kThreads) {
        const int pos = seq_start[i];
        const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
        cum_s[i + 1] = pos / kPage - first_key / kPage + 1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // (a thousand sequences at most, once a step: one thread sums)
        int total = 0, longest = 0, shortest = 0x7fffffff;
        cum_s[0] = 0;
        for (int i = 1; i <= n_seqs; ++i) {
            const int tiles = cum_s[i];
            total += tiles;
            cum_s[i] = total;
            longest = max(longest, tiles);
            shortest = min(shortest, tiles);
        }
        longest_s = longest;
        shortest_s = shortest;
    }
    __syncthreads();
    pdl_wait();
    for (int cta = threadIdx.x; cta < launched; cta += kThreads) {
        DecodePlan plan;
        dec_plan<CL, D>(&plan, cum_s, longest_s, shortest_s, n_seqs, n_kv, group, launched, cta);
        plan.reserved[0] = plan.reserved[1] = 0;
        plans[cta] = plan;
    }
    // The launch behind this kernel starts when this CTA has ended and reads the plans before its own
    // griddepcontrol.wait: they are in L2 before the CTA ends (and are read from there, not through an SM's L1,
    // which may still hold the plans of the step before).
    __threadfence();
}

// CL: CTAs per thread-block cluster of the launch (1: no clusters).  A kernel of its own for each, so that the
// merge inside a cluster is compiled once, for one size, with its shares of the columns divided by constants.
template <int CL>
__global__ void __launch_bounds__(kThreads)
attention_decode_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                        const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                        const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                        const int* __restrict__ block_table, int table_width, const int* __restrict__ seq_start,
                        int n_seqs, int n_q, int n_kv, int ring_tokens, int window, float scale_log2,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int* __restrict__ counters,
                        DecodePrep prep, const DecodePlan* __restrict__ plans) {
    constexpr int cluster_size = CL;
    // the merge in the cluster needs a CTA's share of the head's columns in fours
    constexpr bool kClusterMerge = CL > 1 && (D / (CL > 1 ? CL : 1)) % 4 == 0;
    atrace(0);
    pdl_launch_next();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    // the tiles first, on a 1024-byte boundary (the swizzle's period); the query tile behind them
    bf16* k_s = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_raw) + (kTmaPages ? 1023 : 0)) &
                                        ~uintptr_t(kTmaPages ? 1023 : 0));   // [kKvStages][tile]
    bf16* v_s = k_s + kKvStages * kDecTile;          // [kKvStages][tile]
    bf16* q_s = v_s + kKvStages * kDecTile;          // [16][kStride]
    __shared__ __align__(8) uint64_t page_bar[kKvStages];     // a page's keys and values have landed (TMA)
    uint32_t page_parity = 0;                        // bit s: the parity of the next wait on stage s
    if (kTmaPages && threadIdx.x == 0) {
        for (int i = 0; i < kKvStages; ++i) mbar_init(&page_bar[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // One page into a stage of the ring: by TMA one thread asks for the boxes (two column blocks of keys, two
    // of values), else every thread copies its chunks.  `zero_from` is the first key index that holds nothing.
    auto fetch_page = [&](int stage, const int* table, int t, int kv_head, int live_keys) {
        if (kTmaPages) {
            if (threadIdx.x == 0) {
                const int place = place_of(t * kPage, ring_tokens);
                const int row = (table[place / kPage] * n_kv + kv_head) * kPage;
                mbar_expect_tx(&page_bar[stage], 2 * kPage * D * (int)sizeof(bf16));
#pragma unroll
                for (int h = 0; h < D / 64; ++h) {
                    tma_load_2d(k_s + stage * kDecTile + h * kPage * 64, &map_k, h * 64, row, &page_bar[stage]);
                    tma_load_2d(v_s + stage * kDecTile + h * kPage * 64, &map_v, h * 64, row, &page_bar[stage]);
                }
            }
        } else {
            load_page(k_s + stage * kDecTile, page_ptr(k_cache, table, t, ring_tokens, n_kv, kv_head), t * kPage, live_keys, false);
            load_page(v_s + stage * kDecTile, page_ptr(v_cache, table, t, ring_tokens, n_kv, kv_head), t * kPage, live_keys, true);
        }
    };
    __shared__ int cum_s[kMaxDecodeSeqs + 1];        // pages of the sequences before each one
    __shared__ int warp_tot_s[4];
    __shared__ int warp_max_s[4];
    __shared__ int warp_min_s[4];
    __shared__ int ticket_s;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int group = n_q / n_kv;

    // ---- how many pages each sequence brings: known before this step's kernels ran, so this part
    // overlaps the kernel before (the positions were uploaded ahead of the step)
    __shared__ DecodePlan plan_s;
    const int cta = blockIdx.x;
    if (n_seqs <= 32) {
        // Up to 32 sequences: one warp counts, scans and plans, and the CTA meets once.  (For the CTAs that get their
        // place on an SM only when the kernel before leaves it, all of this is on the way to their first page.)
        if (warp == 0) {
            int tiles = 0;
            if (lane < n_seqs) {
                const int pos = seq_start[lane];
                const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
                tiles = pos / kPage - first_key / kPage + 1;
            }
            int incl = tiles;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += up;
            }
            const int longest = __reduce_max_sync(0xffffffffu, tiles);
            const int shortest = __reduce_min_sync(0xffffffffu, lane < n_seqs ? tiles : 0x7fffffff);
            if (lane < n_seqs) cum_s[lane] = incl - tiles;
            if (lane == n_seqs - 1) cum_s[n_seqs] = incl;
            __syncwarp();
            if (lane == 0 && plans == nullptr)
                dec_plan<CL, D>(&plan_s, cum_s, longest, shortest, n_seqs, n_kv, group, (int)gridDim.x, cta);
        } else if (warp == 1 && lane < 3 && plans != nullptr) {
            // worked out before this launch (attention_decode_plan_kernel): three 16-byte words
            reinterpret_cast<int4*>(&plan_s)[lane] = __ldcg(reinterpret_cast<const int4*>(plans + cta) + lane);
        }
    } else {
        const int per = (n_seqs + kThreads - 1) / kThreads;
        const int lo = min(n_seqs, (int)threadIdx.x * per), hi = min(n_seqs, lo + per);
        int mine = 0, longest = 0, shortest = 0x7fffffff;
        for (int i = lo; i < hi; ++i) {
            const int pos = seq_start[i];
            const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
            const int tiles = pos / kPage - first_key / kPage + 1;
            mine += tiles;
            longest = max(longest, tiles);
            shortest = min(shortest, tiles);
        }
        longest = __reduce_max_sync(0xffffffffu, longest);
        shortest = __reduce_min_sync(0xffffffffu, shortest);
        if (lane == 0) { warp_max_s[warp] = longest; warp_min_s[warp] = shortest; }
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_tot_s[warp] = incl;
        __syncthreads();
        int before = incl - mine;
        for (int w = 0; w < warp; ++w) before += warp_tot_s[w];
        for (int i = lo; i < hi; ++i) {
            cum_s[i] = before;
            const int pos = seq_start[i];
            const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
            before += pos / kPage - first_key / kPage + 1;
        }
        if (threadIdx.x == kThreads - 1) cum_s[n_seqs] = before;
        __syncthreads();
        if (threadIdx.x == 0 && plans == nullptr) {
            const int longest = max(max(warp_max_s[0], warp_max_s[1]), max(warp_max_s[2], warp_max_s[3]));
            const int shortest = min(min(warp_min_s[0], warp_min_s[1]), min(warp_min_s[2], warp_min_s[3]));
            dec_plan<CL, D>(&plan_s, cum_s, longest, shortest, n_seqs, n_kv, group, (int)gridDim.x, cta);
        } else if (threadIdx.x >= 32 && threadIdx.x < 35 && plans != nullptr) {
            reinterpret_cast<int4*>(&plan_s)[threadIdx.x - 32] = __ldcg(reinterpret_cast<const int4*>(plans + cta) + (threadIdx.x - 32));
        }
    }
    __syncthreads();
    const DecodeRun run = plan_s.run;
    // When the launch groups CTAs into clusters and every group of this step is cut into exactly that
    // many parts, the CTAs of a cluster hold the parts of one group and merge them through distributed
    // shared memory: each owns a share of the head's columns and receives the others' sums for them in
    // the space of its query tile (free once the queries are in registers; a first cluster barrier
    // says so), and a second barrier tells it that all parts have arrived.  All CTAs of a cluster
    // take the same decision, since they compute it from the same numbers.
    // (the cluster's size is a constant of this file, so that the shares of the columns below are divided by a constant)
    const bool clustered = kClusterMerge && run.parts == cluster_size && group <= dec_cluster_rows(cluster_size);
    const bool idle = cta >= run.n_ctas;
    const int u_begin = plan_s.first_unit, u_end = plan_s.end_unit;
    int seq = plan_s.first_seq;
    // Pages that lie wholly before this step's token were written by earlier steps: the first of them
    // are asked for now, while the kernel before (which writes the new token's keys and values and
    // the queries) may still be running.
    unsigned preloaded = 0;
    HeadTables tables_q = {};
    float4 tables_kw = make_float4(0.f, 0.f, 0.f, 0.f);
    int tables_pos = -1;          // the position that tables_q and tables_kw were loaded for
    if (!idle) {
        // (in equal runs a group's first `gc` units stand for its fixed cost and hold no pages)
        const int gc = run.group_cost;
        const int seq_tiles = cum_s[seq + 1] - cum_s[seq];
        const int in_seq = u_begin - (cum_s[seq] + seq * gc) * n_kv;
        const int kv_head = in_seq / (seq_tiles + gc), off = in_seq % (seq_tiles + gc);
        const int t_a = max(0, off - gc);
        const int t_b = max(0, min(seq_tiles + gc, off + (u_end - u_begin)) - gc);
        const int pos = seq_start[seq];
        const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
        const int t_begin = first_key / kPage + t_a, t_end = first_key / kPage + t_b - 1;
        const int* table = block_table + (size_t)seq * table_width;
#pragma unroll
        for (int i = 0; i < kKvStages - 1; ++i) {
            const int t = t_begin + i;
            if (t <= t_end && t < pos / kPage) {
                fetch_page(i, table, t, kv_head, pos + 1);
                preloaded |= 1u << i;
            }
        }
        // The norm's weights and the rotation's row of the token's position do not wait for the projection either.
        // (After the wait every CTA of the launch asks for the same few lines at once; these are off that queue.)
        if (kPrepHeadDim && prep.qkv != nullptr) {
            tables_q = head_tables(prep.q_weight, prep.cos_table, prep.sin_table, pos, lane);
            if (warp == 0 && prep.k_weight != nullptr && lane < D / 4)
                tables_kw = *reinterpret_cast<const float4*>(prep.k_weight + 4 * lane);
            tables_pos = pos;
        }
    }
    atrace(1);
    pdl_wait();        // from here on the queries and the new keys and values are read
    if (idle) return;
    atrace(2);
    if constexpr (kClusterMerge) {
        if (run.uneven && run.parts > 0 && u_begin == u_end) {
            // A part without pages (its group has fewer pages than the cluster has CTAs) still takes its place in
            // the cluster's merge: it has nothing to send but "no keys seen", and finishes its share of the columns.
            const int gi = cta / run.parts;
            dec_cluster_arrive();
            dec_cluster_wait();
            for (int i = threadIdx.x; i < group * (D / 4); i += kThreads)
                dec_cluster_send<CL>(q_s, i / (D / 4), (i % (D / 4)) * 4, make_float4(0.f, 0.f, 0.f, 0.f), -INFINITY, 0.f);
            dec_cluster_arrive();
            dec_cluster_wait();
            dec_cluster_finish<CL>(q_s, out + (size_t)(gi / n_kv) * out_stride + (size_t)((gi % n_kv) * group) * D, group);
            return;
        }
    }
    int u = u_begin;
    bool first_segment = true;
    const int gc = run.group_cost;       // equal runs: a group's first `gc` units stand for its fixed cost, no pages
    while (u < u_end) {
        while ((cum_s[seq + 1] + (seq + 1) * gc) * n_kv <= u) ++seq;
        const int seq_tiles = cum_s[seq + 1] - cum_s[seq];
        const int in_seq = u - (cum_s[seq] + seq * gc) * n_kv;
        const int kv_head = in_seq / (seq_tiles + gc), off = in_seq % (seq_tiles + gc);
        const int end_off = min(seq_tiles + gc, off + (u_end - u));
        const int t_a = max(0, off - gc), t_b = max(0, end_off - gc);  // tiles [t_a, t_b) of this group
        const int units_here = end_off - off;
        if (t_b == t_a) {
            u += units_here;             // the run ends inside the group's cost units: its pages are the next CTA's
            continue;
        }
        const bool whole = t_a == 0 && t_b == seq_tiles;
        const int group_first_unit = (cum_s[seq] + seq * gc) * n_kv + kv_head * (seq_tiles + gc);

        const int pos = seq_start[seq];
        const int kv_len = pos + 1;
        const int first_key = window > 0 ? max(0, pos - window + 1) : 0;
        const int t_first = first_key / kPage;
        const int* table = block_table + (size_t)seq * table_width;
        const int t_begin = t_first + t_a, t_end = t_first + t_b - 1;

        float o[D / 8][4];
#pragma unroll
        for (int n = 0; n < D / 8; ++n)
#pragma unroll
            for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
        float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
        HeadInput token_in = {};
        bool freed = false;          // in a cluster: this CTA has told the others that its query tile's space is free

        if (kPrepHeadDim && prep.qkv != nullptr) {
            // the group's query heads come raw from the projection: a warp prepares rows warp, warp + 4, ...
            HeadInput rows_in[4];
            if (pos != tables_pos) {
                tables_q = head_tables(prep.q_weight, prep.cos_table, prep.sin_table, pos, lane);
                if (warp == 0 && prep.k_weight != nullptr && lane < D / 4)
                    tables_kw = *reinterpret_cast<const float4*>(prep.k_weight + 4 * lane);
                tables_pos = pos;
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = warp + 4 * i;
                rows_in[i] = head_load(row < group ? prep.qkv + (size_t)seq * prep.qkv_stride + (size_t)(kv_head * group + row) * D : nullptr,
                                       tables_q, lane);
            }
            // the step's own key and value, if this share of the group holds their page
            if (prep.write_cache && warp < 2 && t_end == pos / kPage) {
                const bf16* raw = prep.qkv + (size_t)seq * prep.qkv_stride + (size_t)(warp == 0 ? n_q + kv_head : n_q + n_kv + kv_head) * D;
                HeadTables tables_k = tables_q;
                tables_k.weight = tables_kw;
                token_in = head_load(raw, tables_k, lane);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // rows past the group are the padding of the 16-row MMA tile: zeros, without the norm's and the
                // rotation's chains of shuffles (with four query heads a group, three of a warp's four rows)
                if (warp + 4 * i < group)
                    head_finish(rows_in[i], prep.q_weight != nullptr, prep.eps, prep.cos_table != nullptr,
                                q_s + (warp + 4 * i) * kStride, nullptr, lane);
                else if (lane < D / 4)
                    *reinterpret_cast<uint2*>(q_s + (warp + 4 * i) * kStride + 4 * lane) = make_uint2(0u, 0u);
            }
        } else {
            for (int i = threadIdx.x; i < 16 * kChunks; i += kThreads) {
                const int row = i / kChunks, c = i % kChunks;
                const bool valid = row < group;
                const bf16* src = q + (size_t)seq * q_stride + (size_t)(kv_head * group + (valid ? row : 0)) * D + c * 8;
                cp_async16(q_s + row * kStride + c * 8, src, valid);
            }
        }
        // a ring of kKvStages pages of keys and values: kKvStages - 1 of them are on their way while one is used
        auto load_tile = [&](int t) { fetch_page((t - t_begin) % kKvStages, table, t, kv_head, kv_len); };
#pragma unroll
        for (int i = 0; i < kKvStages - 1; ++i) {
            if (t_begin + i <= t_end && !(first_segment && ((preloaded >> i) & 1u))) load_tile(t_begin + i);
            cp_async_commit();
        }
        // which CTAs hold the group's parts, and whether the first of them holds it in its second place:
        // divisions whose latency is better spent here, while the queries and the first pages are on
        // their way, than after the last page
        int c_first = cta, c_last = cta, first_slot = 0;
        if (!whole && !clustered) {
            if (run.parts > 0) {
                // every group is cut into the same number of parts and no run crosses into another group
                c_first = (seq * n_kv + kv_head) * run.parts;
                c_last = c_first + run.parts - 1;
            } else {
                c_first = dec_cta_of_unit(run, group_first_unit + gc);                  // who holds the first page
                c_last = dec_cta_of_unit(run, group_first_unit + gc + seq_tiles - 1);
                first_slot = dec_run_begin(run, c_first) >= group_first_unit ? 0 : 1;
            }
        }
        uint32_t qf[D / 16][4];
        for (int t = t_begin; t <= t_end; ++t) {
            const int stage = (t - t_begin) % kKvStages;
            cp_async_wait<kKvStages - 2>();
            if (kTmaPages) {
                mbar_wait(&page_bar[stage], (page_parity >> stage) & 1u, 31);      // bounded; a wait that runs out is recorded
                page_parity ^= 1u << stage;
            }
            __syncthreads();     // page t has landed for everyone, and everyone is done with the stage refilled next
            if (clustered && t == t_begin + 1) {
                dec_cluster_arrive();      // every warp has its queries in registers: the query tile's space is free
                freed = true;
            }
            if (t + kKvStages - 1 <= t_end) load_tile(t + kKvStages - 1);
            cp_async_commit();
            const bool own_token_here = kPrepHeadDim && prep.qkv != nullptr && prep.write_cache && t == pos / kPage;
            if (own_token_here || (kTmaPages && t == pos / kPage)) {
                if (kTmaPages) {
                    // a page that came by TMA came whole: the value rows of keys past the sequence's end may hold
                    // anything and are zeroed here (their probabilities are zero, but zero times NaN is not)
                    const int first_dead = pos % kPage + 1;
                    bf16* v_tile = v_s + stage * kDecTile;
                    for (int i = threadIdx.x; i < (kPage - first_dead) * (D / 8); i += kThreads) {
                        const int row = first_dead + i / (D / 8), c = i % (D / 8);
                        *reinterpret_cast<uint4*>(v_tile + (c >> 3) * (kPage * 64) + row * 64 + (c & 7) * 8) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                // this page holds the step's own token: its key (normalised, rotated) and value go into
                // the page in shared memory and into the cache
                if (own_token_here && warp < 2) {
                    const int row = pos % kPage;
                    bf16* tile = (warp == 0 ? k_s : v_s) + stage * kDecTile + (kTmaPages ? 0 : row * kStride);
                    bf16* cached = const_cast<bf16*>(page_ptr(warp == 0 ? prep.k_cache : prep.v_cache, table, t, ring_tokens, n_kv, kv_head)) + (size_t)row * D;
                    if (warp == 0) head_finish(token_in, prep.k_weight != nullptr, prep.eps, prep.cos_table != nullptr, tile, cached, lane, kTmaPages ? row : -1);
                    else head_finish(token_in, false, 0.f, false, tile, cached, lane, kTmaPages ? row : -1);
                }
                // (the stage's next page comes through the async proxy: these writes are ordered before it)
                if (kTmaPages) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                __syncthreads();
            }
            if (t == t_begin) {
                atrace(3);
                const int mi = lane >> 3, r = lane & 7;
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    ldmatrix_x4(qf[kk], q_s + (r + (mi & 1) * 8) * kStride + kk * 16 + (mi >> 1) * 8);
            }
            const bf16* k_t = k_s + stage * kDecTile;
            const bf16* v_t = v_s + stage * kDecTile;
            // each warp takes 16 of the tile's 64 keys
            float sc[2][4];
            scores<2, kTmaPages>(sc, qf, k_t, warp * 16, lane);
            const int key_base = t * kPage + warp * 16;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int key = key_base + j * 8 + t4 * 2 + (e & 1);
                    const bool seen = key <= pos && key >= first_key;
                    sc[j][e] = seen ? sc[j][e] * scale_log2 : -INFINITY;
                }
            softmax_update<2>(sc, m, l, o);
            weighted_values<2, kTmaPages>(o, sc, v_t, warp * 16, lane);
        }
        atrace(4);
        cp_async_wait<0>();
        __syncthreads();         // everyone is done with the pages: their memory is reused below
        if (clustered && !freed) dec_cluster_arrive();

        // merge the four warps' results: the tile buffers are free now.  Rows are kRedStride floats apart, so
        // that the eight rows a warp stores at once fall into different banks; rows past the group are the
        // padding of the 16-row MMA tile and are left out.
        float* red_o = reinterpret_cast<float*>(k_s);        // [4][16][kRedStride]
        float* red_ml = red_o + 4 * 16 * kRedStride;         // [4][16][2]
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = g + h * 8;
            if (row < group) {
#pragma unroll
                for (int n = 0; n < D / 8; ++n)
                    *reinterpret_cast<float2*>(red_o + (warp * 16 + row) * kRedStride + n * 8 + t4 * 2) =
                        make_float2(o[n][2 * h], o[n][2 * h + 1]);
                if (t4 == 0) *reinterpret_cast<float2*>(red_ml + (warp * 16 + row) * 2) = make_float2(m[h], l[h]);
            }
        }
        __syncthreads();
        if (clustered) dec_cluster_wait();       // every CTA of the cluster has freed its query tile's space
        const int slot = cta * 2 + (first_segment ? 0 : 1);
        // a thread takes four neighbouring output elements of a row at a time
        for (int i = threadIdx.x; i < group * (D / 4); i += kThreads) {
            const int row = i / (D / 4), d = (i % (D / 4)) * 4;
            float mx = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mx = fmaxf(mx, red_ml[(w * 16 + row) * 2]);
            const float m_use = mx == -INFINITY ? 0.f : mx;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float c = exp2f(red_ml[(w * 16 + row) * 2] - m_use);
                const float4 part = *reinterpret_cast<const float4*>(red_o + (w * 16 + row) * kRedStride + d);
                acc.x += c * part.x; acc.y += c * part.y; acc.z += c * part.z; acc.w += c * part.w;
                sum += c * red_ml[(w * 16 + row) * 2 + 1];
            }
            if (clustered) {
                if constexpr (kClusterMerge) dec_cluster_send<CL>(q_s, row, d, acc, mx, sum);
            } else if (whole) {
                const float inv = sum > 0.f ? 1.0f / sum : 0.f;
                bf16* dst = out + (size_t)seq * out_stride + (size_t)(kv_head * group + row) * D + d;
                *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
            } else {
                *reinterpret_cast<float4*>(part_o + ((size_t)slot * 16 + row) * D + d) = acc;
                if (d == 0) *reinterpret_cast<float2*>(part_ml + ((size_t)slot * 16 + row) * 2) = make_float2(mx, sum);
            }
        }
        if (clustered) {
            // all parts have arrived; this CTA finishes its share of the columns
            dec_cluster_arrive();
            dec_cluster_wait();
            bf16* dst = out + (size_t)seq * out_stride + (size_t)(kv_head * group) * D;
            if constexpr (kClusterMerge) dec_cluster_finish<CL>(q_s, dst, group);
        } else if (!whole) {
            __syncthreads();
            atrace(5);
            if (threadIdx.x == 0) {
                // one acquire-release add at GPU scope: this CTA's part (ordered before it by the barrier
                // above) is visible to whoever reads a later ticket, and the earlier parts are visible here
                const int ticket = ticket_add(&counters[seq * n_kv + kv_head]);
                ticket_s = ticket;
            }
            __syncthreads();
            if (ticket_s == c_last - c_first) {
                // a part lies in its CTA's first place if the group is the first of its run: true for
                // every part after the first, whose runs begin inside the group
                const int n_parts = c_last - c_first + 1;       // at most kMaxGroupParts by the choice of run length
                // four neighbouring elements of a row per thread; the parts come in rounds of kMaxParts, the loads
                // of a round issued before any is used, and are added in the order of their pages
                for (int i = threadIdx.x; i < group * (D / 4); i += kThreads) {
                    const int row = i / (D / 4), d = (i % (D / 4)) * 4;
                    float run_m = -INFINITY, sum = 0.f;
                    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int base = 0; base < n_parts; base += kMaxParts) {
                        float2 pml[kMaxParts];
                        float4 po[kMaxParts];
#pragma unroll
                        for (int j = 0; j < kMaxParts; ++j) {
                            const bool live = base + j < n_parts;
                            const size_t sl = (size_t)(c_first + (live ? base + j : 0)) * 2 + (base + j == 0 ? first_slot : 0);
                            pml[j] = live ? __ldcg(reinterpret_cast<const float2*>(part_ml + (sl * 16 + row) * 2))
                                          : make_float2(-INFINITY, 0.f);
                            po[j] = live ? __ldcg(reinterpret_cast<const float4*>(part_o + (sl * 16 + row) * D + d))
                                         : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
                        float mx = run_m;
#pragma unroll
                        for (int j = 0; j < kMaxParts; ++j) mx = fmaxf(mx, pml[j].x);
                        const float m_use = mx == -INFINITY ? 0.f : mx;
                        if (base > 0) {
                            const float keep = exp2f(run_m - m_use);       // what was added so far, on the new scale
                            acc.x *= keep; acc.y *= keep; acc.z *= keep; acc.w *= keep;
                            sum *= keep;
                        }
#pragma unroll
                        for (int j = 0; j < kMaxParts; ++j) {
                            const float w = exp2f(pml[j].x - m_use);
                            acc.x += w * po[j].x; acc.y += w * po[j].y; acc.z += w * po[j].z; acc.w += w * po[j].w;
                            sum += w * pml[j].y;
                        }
                        run_m = mx;
                    }
                    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
                    bf16* dst = out + (size_t)seq * out_stride + (size_t)(kv_head * group + row) * D + d;
                    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
                    *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
                }
                if (threadIdx.x == 0) counters[seq * n_kv + kv_head] = 0;   // ready for the next call
            }
        }
        atrace(6);
        // (the next group's pages come through the async proxy into memory this group's merge wrote)
        if (kTmaPages) asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncthreads();     // the reduction buffers alias the tile buffers of the next group
        u += units_here;
        first_segment = false;
    }
}

constexpr int kPrefillSmem = (64 + 4 * kPage) * kStride * (int)sizeof(bf16);
constexpr int kDecodeTiles = (16 * kStride + 2 * kKvStages * kDecTile) * (int)sizeof(bf16) + (kTmaPages ? 1024 : 0);
constexpr int kDecodeReduce = 16 * kStride * (int)sizeof(bf16) + (4 * 16 * kRedStride + 4 * 16 * 2) * (int)sizeof(float) + (kTmaPages ? 1024 : 0);
constexpr int kDecodeSmem = kDecodeTiles > kDecodeReduce ? kDecodeTiles : kDecodeReduce;

}  // namespace dfi

using namespace dfi;

// 1: kernels of this library are launched so that they may overlap the tail of the kernel before
// them (programmatic dependent launch); 0: plain launches.  Returns the previous setting.
DFI_EXPORT int dfi_attention_set_pdl(int enabled) {
    const int before = pdl_enabled();
    pdl_enabled() = enabled ? 1 : 0;
    return before;
}

#ifdef DFI_TRACE
DFI_EXPORT int dfi_attention_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(unsigned long long) * 4096 * 8) == cudaSuccess ? 0 : 1;
}
#endif

DFI_EXPORT int dfi_attention_head_dim() { return D; }

// the decode kernel's waits for its pages are bounded like those of the tcgen05 kernels
DFI_TCGEN05_STATUS_ENTRIES(attention_decode)

// Scratch of the decode kernel for a launch of `n_ctas` CTAs: floats for part_o, then for part_ml.
DFI_EXPORT long long dfi_attention_decode_scratch_floats(int n_ctas) { return (long long)n_ctas * 2 * 16 * (D + 2); }

// CTAs of the decode kernel that one SM holds at a time, times the SMs: what one wave can run.
static int decode_clusters_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* text = getenv("DRYFT_ATTENTION_CLUSTER");      // "off": parts always meet through scratch memory
        enabled = (text != nullptr && (text[0] == 'o' || text[0] == 'O') && (text[1] == 'f' || text[1] == 'F')) ? 0 : 1;
    }
    return enabled;
}

static int wide_clusters_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* text = getenv("DRYFT_ATTENTION_CLUSTER");      // "4": clusters of four only
        enabled = (text != nullptr && text[0] == '4') ? 0 : 1;
    }
    return enabled;
}

DFI_EXPORT int dfi_attention_decode_wave() {
    static int wave = -1;
    if (wave >= 0) return wave;
    int device = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    cudaFuncSetAttribute(attention_decode_kernel<kDecodeCluster>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_decode_kernel<kDecodeCluster>, kThreads, kDecodeSmem) != cudaSuccess)
        return 0;
    int ctas = sms * per_sm;
    if (decode_clusters_enabled()) {
        // launched as clusters, only whole clusters that fit their part of the device run at once
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3((ctas / kDecodeCluster) * kDecodeCluster);
        config.blockDim = dim3(kThreads);
        config.dynamicSmemBytes = kDecodeSmem;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = kDecodeCluster;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        config.attrs = attr;
        config.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, attention_decode_kernel<kDecodeCluster>, &config) == cudaSuccess && clusters > 0)
            ctas = min(ctas / kDecodeCluster, clusters) * kDecodeCluster;
        else
            cudaGetLastError();
    }
    wave = ctas;
    return wave;
}

DFI_EXPORT int dfi_attention_prefill(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                     const void* v_cache, const int* block_table, int table_width,
                                     const int* cu_rows, const int* seq_start, int n_seqs, int max_q_len, int n_q,
                                     int n_kv, int page_size, int ring_tokens, int window, float scale,
                                     void* stream) {
    if (n_seqs <= 0 || max_q_len <= 0) return DFI_OK;
    if (page_size != kPage || n_q <= 0 || n_kv <= 0 || n_q % n_kv || ring_tokens % kPage) return DFI_ERR_SHAPE;
    if (q_stride % 8 || !aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return DFI_ERR_ALIGN;
    if (n_q > 65535 || n_seqs > 65535) return DFI_ERR_LIMIT;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPrefillSmem) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    dim3 grid((max_q_len + 63) / 64, n_q, n_seqs);
    launch(attention_prefill_kernel, grid, kThreads, kPrefillSmem, (cudaStream_t)stream, 
        (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_cache, (const bf16*)v_cache, block_table,
        table_width, cu_rows, seq_start, n_q, n_kv, ring_tokens, window, scale * kLog2e);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// How many clusters of sixteen CTAs of the decode kernel the device runs at once (0: none, or switched off).  A
// cluster of more than eight CTAs is one the kernel has to ask for by an attribute of its own.
static int full_clusters_at_once() {
    static int clusters = -1;
    if (clusters >= 0) return clusters;
    clusters = 0;
    if (!kFullClusterFits || !decode_clusters_enabled() || !wide_clusters_enabled()) return clusters;
    auto kernel = attention_decode_kernel<kDecodeClusterFull>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess ||
        cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) {
        cudaGetLastError();
        return clusters;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(kDecodeClusterFull * 16);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kDecodeSmem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kDecodeClusterFull;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    config.attrs = attr;
    config.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &config) == cudaSuccess && n > 0) clusters = n;
    else cudaGetLastError();
    return clusters;
}

// One query row per sequence (row i belongs to sequence i).  `scratch` holds
// dfi_attention_decode_scratch_floats(n_ctas) floats; `counters` holds n_seqs * n_kv ints, zero
// before the first call and left zero by every call.  n_ctas <= 0: as many as run at once.
static int attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                            const void* v_cache, long long cache_pages, const int* block_table, int table_width,
                            const int* seq_start, int n_seqs, int n_q, int n_kv, int page_size,
                            int ring_tokens, int window, float scale, int n_ctas, float* scratch,
                            int* counters, const DecodePrep& prep, int max_kv_len, void* plans, int plans_fresh,
                            void* stream) {
    if (n_seqs <= 0) return DFI_OK;
    if (plans != nullptr && !aligned16(plans)) return DFI_ERR_ALIGN;
    if (page_size != kPage || n_q <= 0 || n_kv <= 0 || n_q % n_kv || n_q / n_kv > 16 || ring_tokens % kPage)
        return DFI_ERR_SHAPE;
    if (n_seqs > kMaxDecodeSeqs) return DFI_ERR_LIMIT;
    if (scratch == nullptr || counters == nullptr) return DFI_ERR_SHAPE;
    if (prep.qkv == nullptr && (q_stride % 8 || !aligned16(q))) return DFI_ERR_ALIGN;
    if (!aligned16(k_cache) || !aligned16(v_cache)) return DFI_ERR_ALIGN;
    if (out_stride % 2 || (reinterpret_cast<uintptr_t>(out) & 3)) return DFI_ERR_ALIGN;      // outputs are stored in pairs
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_decode_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess ||
            cudaFuncSetAttribute(attention_decode_kernel<kDecodeClusterPair>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess ||
            cudaFuncSetAttribute(attention_decode_kernel<kDecodeCluster>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess ||
            cudaFuncSetAttribute(attention_decode_kernel<kDecodeClusterWide>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDecodeSmem) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    if (n_ctas <= 0) n_ctas = dfi_attention_decode_wave();
    if (n_ctas <= 0) return DFI_ERR_LAUNCH;
    if (n_ctas > 4096) n_ctas = 4096;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)n_ctas * 2 * 16 * D;
    // the caches as TMA maps of boxes of 64 rows x 64 elements (rows: page, head, token)
    CUtensorMap map_k = {}, map_v = {};
    if (kTmaPages) {
        const long long rows = cache_pages * n_kv * kPage;
        if (cache_pages <= 0 || rows > 0x7fffffffLL) return DFI_ERR_LIMIT;
        if (!make_tile_map(&map_k, k_cache, (int)rows, D, kPage) || !make_tile_map(&map_v, v_cache, (int)rows, D, kPage))
            return DFI_ERR_LAUNCH;
    }
    // clusters only where the kernel can use them: every group cut into kDecodeCluster parts needs that many CTAs
    int cluster = (decode_clusters_enabled() && n_ctas % kDecodeCluster == 0 &&
                   (long long)n_seqs * n_kv * kDecodeCluster <= n_ctas) ? kDecodeCluster : 1;
    // too many groups for four CTAs each, but not for two
    if (cluster == 1 && decode_clusters_enabled() && wide_clusters_enabled() && n_ctas % kDecodeClusterPair == 0 &&
        (long long)n_seqs * n_kv * kDecodeClusterPair <= n_ctas)
        cluster = kDecodeClusterPair;
    // eight CTAs a cluster where that still covers every group and a group's rows fit the receive space
    // (the grid is then a whole number of them: up to seven CTAs fewer, none of which would have had pages)
    int grid = n_ctas;
    const int wide_grid = n_ctas / kDecodeClusterWide * kDecodeClusterWide;
    // Measured at 32/8 heads of 128: a launch in clusters of eight gains 1.4 to 4.9 % of the step for one or two
    // sequences of up to 4,096 keys, and loses 1 to 4 % for four sequences or for longer ones, whose parts do
    // not meet in the cluster and whose CTAs the wider clusters place less evenly.  Hence: at most 16 groups,
    // and only if the caller says that no sequence of this launch can be longer than the kernel's limit.
    if (cluster == kDecodeCluster && kWideClusterFits && wide_clusters_enabled() && n_q / n_kv <= dec_cluster_rows(kDecodeClusterWide) &&
        n_seqs * n_kv <= 16 && max_kv_len > 0 && max_kv_len <= kWideMostPages * kPage &&
        (long long)n_seqs * n_kv * kDecodeClusterWide <= wide_grid) {
        cluster = kDecodeClusterWide;
        grid = wide_grid;
    }
    // Sixteen CTAs a cluster for the groups of one sequence (fewer groups than sixteen) that may grow past
    // kFullLeastKeys keys but not past ten pages a part: a CTA alone on its SM takes about a microsecond a page (three
    // pages in flight), so half the pages a CTA are worth more than the wider meeting costs.
    if (cluster >= kDecodeCluster && kFullClusterFits && wide_clusters_enabled() && n_q / n_kv <= dec_cluster_rows(kDecodeClusterFull) &&
        n_seqs * n_kv < 16 && max_kv_len > kFullLeastKeys &&
        max_kv_len <= kPartMostPages * kDecodeClusterFull * kPage && n_seqs * n_kv <= full_clusters_at_once()) {
        const int full_grid = n_ctas / kDecodeClusterFull * kDecodeClusterFull;
        // (what the plan keeps of a cluster launch: see dec_plan)
        if ((long long)n_seqs * n_kv * kDecodeClusterFull <= (full_grid - full_grid / 16) / kDecodeClusterFull * kDecodeClusterFull) {
            cluster = kDecodeClusterFull;
            grid = full_grid;
        }
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kDecodeSmem;
    config.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (cluster > 1) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = cluster;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    config.attrs = attr;
    config.numAttrs = n_attr;
    if (plans != nullptr && plans_fresh) {
        // the plans of this launch shape, for this launch and those that say they deal the same pages
        auto planner = cluster == kDecodeClusterFull ? attention_decode_plan_kernel<kDecodeClusterFull>
                       : cluster == kDecodeClusterWide ? attention_decode_plan_kernel<kDecodeClusterWide>
                       : cluster == kDecodeCluster   ? attention_decode_plan_kernel<kDecodeCluster>
                       : cluster == kDecodeClusterPair ? attention_decode_plan_kernel<kDecodeClusterPair>
                                                       : attention_decode_plan_kernel<1>;
        if (launch(planner, 1, kThreads, 0, (cudaStream_t)stream, (DecodePlan*)plans, seq_start, n_seqs, n_kv, n_q / n_kv,
                   window, grid) != cudaSuccess) {
            cudaGetLastError();
            return DFI_ERR_LAUNCH;
        }
    }
    auto kernel = cluster == kDecodeClusterFull ? attention_decode_kernel<kDecodeClusterFull>
                  : cluster == kDecodeClusterWide ? attention_decode_kernel<kDecodeClusterWide>
                  : cluster == kDecodeCluster   ? attention_decode_kernel<kDecodeCluster>
                  : cluster == kDecodeClusterPair ? attention_decode_kernel<kDecodeClusterPair>
                                                  : attention_decode_kernel<1>;
    if (cudaLaunchKernelEx(&config, kernel, map_k, map_v, (const bf16*)q, q_stride, (bf16*)out, out_stride,
                           (const bf16*)k_cache, (const bf16*)v_cache, block_table, table_width, seq_start, n_seqs, n_q,
                           n_kv, ring_tokens, window, scale * kLog2e, part_o, part_ml, counters, prep,
                           (const DecodePlan*)plans) != cudaSuccess) {
        cudaGetLastError();
        return DFI_ERR_LAUNCH;
    }
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// Bytes of the plans of a launch of up to n_ctas CTAs (n_ctas <= 0: as many as run at once).
DFI_EXPORT long long dfi_attention_decode_plan_bytes(int n_ctas) {
    if (n_ctas <= 0) n_ctas = dfi_attention_decode_wave();
    return (long long)sizeof(DecodePlan) * (n_ctas > 4096 ? 4096 : n_ctas < 1 ? 1 : n_ctas);
}

// max_kv_len: no sequence of this launch, or of any later replay of it in a CUDA graph, holds more keys than this
// (0: not known).  It only chooses between launch shapes.
// plans: null, or dfi_attention_decode_plan_bytes(n_ctas) bytes on the device that hold how the launch deals its
// pages.  With plans_fresh they are worked out now, by a kernel before the launch; without, the launch reads what
// an earlier call with the same seq_start, n_seqs, n_q, n_kv, window, n_ctas and max_kv_len left there (the layers
// of one step).  Null: every CTA works its plan out itself.
DFI_EXPORT int dfi_attention_decode(const void* q, int q_stride, void* out, int out_stride, const void* k_cache,
                                    const void* v_cache, long long cache_pages, const int* block_table, int table_width,
                                    const int* seq_start, int n_seqs, int n_q, int n_kv, int page_size,
                                    int ring_tokens, int window, float scale, int n_ctas, float* scratch,
                                    int* counters, int max_kv_len, void* plans, int plans_fresh, void* stream) {
    DecodePrep none = {};
    return attention_decode(q, q_stride, out, out_stride, k_cache, v_cache, cache_pages, block_table, table_width,
                            seq_start, n_seqs, n_q, n_kv, page_size, ring_tokens, window, scale, n_ctas, scratch, counters,
                            none, max_kv_len, plans, plans_fresh, stream);
}

// The lengths (in keys) at which the launch shape chosen by `max_kv_len` changes, in rising order; 0 past the
// last.  A caller that knows how long its sequences are picks the smallest of them that covers the longest.
DFI_EXPORT int dfi_attention_decode_kv_step(int i) {
    const int steps[3] = {kFullLeastKeys, kWideMostPages * kPage, kPartMostPages * kDecodeClusterFull * kPage};
    return i >= 0 && i < 3 ? steps[i] : 0;
}

// 1 if this build (head size) has the variant that prepares the step's token itself.
DFI_EXPORT int dfi_attention_decode_prepares() { return kPrepHeadDim ? 1 : 0; }

// The same with the step's token prepared inside the kernel: qkv [n_seqs, qkv_stride] holds the raw
// projection (q heads, k heads, v heads) of each sequence's new token at position seq_start[i].  q and k
// heads are RMS-normalised with q_weight / k_weight (null: not) and rotated by the tables (null: not);
// with write_cache the new key and value are stored into the cache, else the cache holds them already.
DFI_EXPORT int dfi_attention_decode_prepared(const void* qkv, int qkv_stride, const float* q_weight,
                                             const float* k_weight, float eps, const float* cos_table,
                                             const float* sin_table, int write_cache, void* out, int out_stride,
                                             void* k_cache, void* v_cache, long long cache_pages,
                                             const int* block_table, int table_width,
                                             const int* seq_start, int n_seqs, int n_q, int n_kv, int page_size,
                                             int ring_tokens, int window, float scale, int n_ctas, float* scratch,
                                             int* counters, int max_kv_len, void* plans, int plans_fresh, void* stream) {
    if (!kPrepHeadDim) return DFI_ERR_SHAPE;
    if (qkv == nullptr || qkv_stride % 4 || (reinterpret_cast<uintptr_t>(qkv) & 7)) return DFI_ERR_ALIGN;
    if (!aligned16(q_weight) || !aligned16(k_weight) || !aligned16(cos_table) || !aligned16(sin_table)) return DFI_ERR_ALIGN;
    if ((cos_table == nullptr) != (sin_table == nullptr)) return DFI_ERR_SHAPE;
    DecodePrep prep;
    prep.qkv = (const bf16*)qkv;
    prep.qkv_stride = qkv_stride;
    prep.q_weight = q_weight;
    prep.k_weight = k_weight;
    prep.eps = eps;
    prep.cos_table = cos_table;
    prep.sin_table = sin_table;
    prep.k_cache = (bf16*)k_cache;
    prep.v_cache = (bf16*)v_cache;
    prep.write_cache = write_cache;
    return attention_decode(nullptr, 0, out, out_stride, k_cache, v_cache, cache_pages, block_table, table_width,
                            seq_start, n_seqs, n_q, n_kv, page_size, ring_tokens, window, scale, n_ctas, scratch, counters,
                            prep, max_kv_len, plans, plans_fresh, stream);
}
