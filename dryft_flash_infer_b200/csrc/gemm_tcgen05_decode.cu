// The decode step's matrix product on tcgen05: out[M, N] = x[M, K] . W[N, K]^T for a small batch
// (M <= 64), bound by reading W once.  W's rows take the 128-row side of tcgen05.mma and the
// batch the narrow side (N = 16, 32 or 64 of the instruction), so a batch of 8 pads to 16 columns
// of tensor memory and nothing else.
//
// One persistent CTA per SM.  W is cut into units of 128 rows x 64 k; units are numbered row block
// by row block and dealt to the CTAs in equal contiguous runs (stream-K), so that every SM reads
// the same number of bytes even when W has few rows.  Inside a CTA: warp 0 feeds a ring of
// shared-memory stages with TMA, warp 1 issues the MMAs into one of two TMEM accumulators, warps
// 2-9 drain the other (two warps for each quarter of the lanes, which share its columns) and run the
// epilogue: its chains of dependent instructions are what a step of many rows waits for, so they are
// spread over eight warps, two to a scheduler.  A CTA whose run covers a whole row block stores the result itself;
// otherwise it leaves float32 partial sums in scratch memory and takes a ticket from the row
// block's counter, and the CTA that draws the last ticket adds the parts in the order of their k
// ranges (the result does not depend on who finished when), applies the epilogue and resets the
// counter.  No CTA waits for another CTA; waits inside a CTA (on its own mbarriers) are bounded.
//
// CLUSTER variant, for a matrix with few row blocks cut into 2 to 8 parts each: the CTAs of a row
// block form a thread-block cluster and meet once at the cluster barrier instead of taking tickets.
// Every CTA owns the columns c of the row block with (c / 4) mod parts equal to its rank.  With a
// batch of at most 16 rows each CTA stores its sums for a column straight into the owner's shared
// memory; with more rows it writes its part to scratch memory and the owners read their columns
// from there after the barrier (the barrier's release and acquire order both).  Every owner adds
// the parts in the order of their k ranges and applies the epilogue to its columns.
//
// Two optional fusions with the RMS norm around the product, both in the adding CTA's epilogue:
// * scaled input: x holds rows w (.) r that still lack their 1/rms factor; the sums of squares of r
//   come as partial sums per row, and since the factor is one number per row it is applied to the
//   float32 result instead (before SwiGLU, to gate and up alike);
// * add-norm output: the product y is a residual delta; the epilogue forms r = residual + y in
//   place (y rounded to bfloat16 first, as an unfused step would store it), writes w (.) r as the
//   next product's scaled input and this row block's sum of r^2 per row.
// With both, the add + norm kernel between two products disappears.
//
// A word about the next product (NextStream, tcgen05.cuh): when the producer has asked for the last tile of
// its CTA's run it asks a few tiles of the product that the step runs next into L2, for the time in which
// this kernel's epilogue and the next kernel's wait leave the memory idle.
//
// SWIGLU variant: W = [gate; up] of 2N rows; a row block is 64 gate rows and the 64 up rows that
// belong to them, and the epilogue writes silu(gate) * up (engine/kernels/reference.py:74-79;
// the fusion follows the idea of engine/kernels/cuda_mlp.py:39-125).
#include <stdlib.h>

#include "tcgen05.cuh"

namespace dfi {

constexpr int kEpThreads = 256;              // the epilogue's threads: eight warps, two for each quarter of the TMEM lanes
constexpr int kDecThreads = 64 + kEpThreads; // producer warp, issuing warp, epilogue warps
constexpr int kDecSmemBudget = 110 * 1024;   // two CTAs fit an SM: the next kernel sets up and loads weights beside this one

struct StreamShape {
    int M, N, K;          // N: columns of the output
    int k_chunks;         // units per row block
    int row_blocks;
    int units;
    int n_ctas;
    int parts;            // > 0: every row block is cut into this many parts, one CTA each (n_ctas = row_blocks * parts)
    int wide_out;         // plain outputs may be stored four at a time (N a multiple of 4, out on a 16-byte boundary)
};

constexpr int kSsqStride = 64;   // floats per part in a sum-of-squares array: one per row of the batch

struct RowFusion {
    const float* in_ssq;      // scaled input: [in_parts][kSsqStride] partial sums of squares, or null
    int in_parts;
    float in_inv_dim, in_eps;
    bf16* residual;           // add-norm output: [M, N] updated in place, or null
    const float* norm_weight; // [N]
    float* out_ssq;           // [row_blocks][kSsqStride]
};

// First unit of a CTA's run.  Two ways of dealing the units out: equal contiguous runs over the
// whole matrix (stream-K), or, for a matrix with few row blocks, each row block cut into the same
// number of parts, so that no CTA's run crosses from one row block into the next.
__device__ __forceinline__ int sk_run_begin(const StreamShape& s, int cta) {
    return deal_begin(UnitDeal{s.units, s.k_chunks, s.n_ctas, s.parts}, cta);
}
__device__ __forceinline__ int sk_cta_of_unit(const StreamShape& s, int u) {
    int c;
    if (s.parts > 0) {
        const int rb = u / s.k_chunks, kc = u % s.k_chunks;
        c = rb * s.parts + min(s.parts - 1, kc * s.parts / s.k_chunks);
    } else {
        c = (int)((unsigned)u * (unsigned)s.n_ctas / (unsigned)s.units);
    }
    while (c + 1 < s.n_ctas && sk_run_begin(s, c + 1) <= u) ++c;
    while (c > 0 && sk_run_begin(s, c) > u) --c;
    return c;
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, %0;\n" ::"n"(kEpThreads) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(s32(bar)) : "memory");
}

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// Address of this CTA's shared-memory location `addr` in the CTA of rank `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_map(uint32_t addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void cluster_store(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_store4(uint32_t addr, float4 v) {
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1, %2, %3, %4};\n" ::"r"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w)
                 : "memory");
}
// Every thread of every CTA of the cluster arrives (release) and waits (acquire).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.aligned;\n" ::: "memory");
}
// Columns of a row block come in groups of four; group g belongs to rank g mod parts.
__device__ __forceinline__ int owned_groups(int rank, int parts, int groups) { return (groups - rank + parts - 1) / parts; }

// -DDFI_TRACE: every CTA records the global timer at a few points of its life (a debugging build).
#ifdef DFI_TRACE
__device__ unsigned long long g_trace[512 * 8];
__device__ __forceinline__ void trace(int slot) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    g_trace[blockIdx.x * 8 + slot] = now;
}
#else
__device__ __forceinline__ void trace(int) {}
#endif

template <int BN, bool CLUSTER> struct DecConfig {
    static constexpr int kABytes = kTileM * kTileK * 2;
    static constexpr int kBBytes = BN * kTileK * 2;
    static constexpr int kStageBytes = kABytes + kBBytes;
    // float [BN][128] for the epilogue; in a cluster [parts][BN][owned columns], at most 144 BN floats; none in a
    // cluster with more than 16 rows, whose parts meet through scratch memory
    static constexpr int kStagingBytes = (CLUSTER && BN > 16) ? 0 : BN * 144 * 4;
    static constexpr int kStagesRaw = (kDecSmemBudget - 1024 - kStagingBytes) / kStageBytes;
    static constexpr int kStages = kStagesRaw > 10 ? 10 : kStagesRaw;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;      // two accumulators
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingBytes + 1024;
    static constexpr int kSlotFloats = BN * kTileM;                  // one part of one row block
};

// What the epilogue of one group of four columns needs from memory besides the sums: asked for
// early, so that it travels together with the parts.
struct FinishInput {
    uint2 residual;
    float4 norm_weight;
    bool inside;
};
template <bool SWIGLU>
__device__ __forceinline__ FinishInput finish_begin(const RowFusion& fusion, const StreamShape& s, int col, int b) {
    FinishInput in;
    in.residual = make_uint2(0u, 0u);
    in.norm_weight = make_float4(0.f, 0.f, 0.f, 0.f);
    in.inside = col < s.N;       // N is a multiple of 4 with an add-norm output: a group is inside the matrix or outside it
    if (!SWIGLU && fusion.residual != nullptr && in.inside) {
        in.residual = __ldcg(reinterpret_cast<const uint2*>(fusion.residual + (size_t)b * s.N + col));
        in.norm_weight = __ldg(reinterpret_cast<const float4*>(fusion.norm_weight + col));
    }
    return in;
}
// Sums v (and u, the "up" half with SwiGLU) of row b, columns col..col+3, become outputs: the input
// rows' 1/rms factor, SwiGLU, then either the add-norm output or a plain store.  With an add-norm
// output every lane of the warp must call this (inactive lanes contribute nothing); `seg` lanes
// hold the columns of one row and share its sum of squares, written as part `ssq_part`.
template <bool SWIGLU>
__device__ __forceinline__ void finish_group(const RowFusion& fusion, const StreamShape& s, void* out, int out_dtype,
                                             const float* row_scale, const FinishInput& in, int col, int b, float4 v,
                                             float4 u, bool active, int seg, int ssq_part, int lane) {
    if (fusion.in_ssq != nullptr && active) {
        const float rs = row_scale[b];
        v.x *= rs; v.y *= rs; v.z *= rs; v.w *= rs;
        if (SWIGLU) { u.x *= rs; u.y *= rs; u.z *= rs; u.w *= rs; }
    }
    if (SWIGLU) {
        v.x = silu_times(v.x, u.x); v.y = silu_times(v.y, u.y);
        v.z = silu_times(v.z, u.z); v.w = silu_times(v.w, u.w);
    }
    const float vals[4] = {v.x, v.y, v.z, v.w};
    if (!SWIGLU && fusion.residual != nullptr) {
        float ssq = 0.f;
        if (active && in.inside) {
            const float2 r01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.residual.x));
            const float2 r23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in.residual.y));
            const float old_r[4] = {r01.x, r01.y, r23.x, r23.y};
            const float w4[4] = {in.norm_weight.x, in.norm_weight.y, in.norm_weight.z, in.norm_weight.w};
            float r[4], xs[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float delta = __bfloat162float(__float2bfloat16_rn(vals[e]));
                r[e] = __bfloat162float(__float2bfloat16_rn(old_r[e] + delta));
                xs[e] = r[e] * w4[e];
                ssq += r[e] * r[e];
            }
            uint2 r_out, x_out;
            *reinterpret_cast<__nv_bfloat162*>(&r_out.x) = __floats2bfloat162_rn(r[0], r[1]);
            *reinterpret_cast<__nv_bfloat162*>(&r_out.y) = __floats2bfloat162_rn(r[2], r[3]);
            *reinterpret_cast<__nv_bfloat162*>(&x_out.x) = __floats2bfloat162_rn(xs[0], xs[1]);
            *reinterpret_cast<__nv_bfloat162*>(&x_out.y) = __floats2bfloat162_rn(xs[2], xs[3]);
            const size_t at = (size_t)b * s.N + col;
            *reinterpret_cast<uint2*>(fusion.residual + at) = r_out;
            *reinterpret_cast<uint2*>((bf16*)out + at) = x_out;
        }
        for (int o = seg >> 1; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
        if (active && (lane & (seg - 1)) == 0) fusion.out_ssq[ssq_part * kSsqStride + b] = ssq;
        return;
    }
    if (!active) return;
    if (s.wide_out && col + 3 < s.N) {
        // four outputs as one store: N is a multiple of four and the output starts on a 16-byte boundary
        if (out_dtype == DFI_DTYPE_F32) {
            *reinterpret_cast<float4*>((float*)out + (size_t)b * s.N + col) = make_float4(vals[0], vals[1], vals[2], vals[3]);
        } else {
            uint2 packed;
            *reinterpret_cast<__nv_bfloat162*>(&packed.x) = __floats2bfloat162_rn(vals[0], vals[1]);
            *reinterpret_cast<__nv_bfloat162*>(&packed.y) = __floats2bfloat162_rn(vals[2], vals[3]);
            *reinterpret_cast<uint2*>((bf16*)out + (size_t)b * s.N + col) = packed;
        }
        return;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (col + e < s.N) {
            if (out_dtype == DFI_DTYPE_F32) ((float*)out)[(size_t)b * s.N + col + e] = vals[e];
            else ((bf16*)out)[(size_t)b * s.N + col + e] = __float2bfloat16_rn(vals[e]);
        }
    }
}

template <int BN, bool SWIGLU, bool CLUSTER>
__global__ void __launch_bounds__(kDecThreads, 2)
gemm_decode_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* __restrict__ out, StreamShape s, float* __restrict__ partials, int* __restrict__ counters,
                   int out_dtype, RowFusion fusion, const __grid_constant__ NextStream next) {
    using Cfg = DecConfig<BN, CLUSTER>;
    if (threadIdx.x == 0) trace(0);
    pdl_launch_next();
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[Cfg::kStages];
    __shared__ __align__(8) uint64_t empty_bar[Cfg::kStages];
    __shared__ __align__(8) uint64_t acc_full[2];
    __shared__ __align__(8) uint64_t acc_empty[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int ticket_s;
    __shared__ float row_scale[BN];

    unsigned char* ring = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* staging = reinterpret_cast<float*>(ring + (size_t)Cfg::kStages * Cfg::kStageBytes);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int cl_stride = 0, cl_owned = 0, cl_pad_log2 = 2;      // CLUSTER: set by the epilogue threads before they wait
    const int cta = blockIdx.x;
    const int u_begin = sk_run_begin(s, cta), u_end = sk_run_begin(s, cta + 1);
    const int n_units = u_end - u_begin;
    const int first_rb = u_begin / s.k_chunks, first_kc = u_begin % s.k_chunks;
    constexpr int kCols = SWIGLU ? kTileM / 2 : kTileM;      // output columns per row block

    auto load_w = [&](int st, int rb, int kc) {
        unsigned char* a_tile = ring + (size_t)st * Cfg::kStageBytes;
        mbar_expect_tx(&full_bar[st], Cfg::kStageBytes);
        if (SWIGLU) {
            tma_load_2d(a_tile, &map_w, kc * kTileK, rb * 64, &full_bar[st]);
            tma_load_2d(a_tile + Cfg::kABytes / 2, &map_w, kc * kTileK, s.N + rb * 64, &full_bar[st]);
        } else {
            tma_load_2d(a_tile, &map_w, kc * kTileK, rb * kTileM, &full_bar[st]);
        }
    };
    auto load_x = [&](int st, int kc) {
        tma_load_2d(ring + (size_t)st * Cfg::kStageBytes + Cfg::kABytes, &map_x, kc * kTileK, 0, &full_bar[st]);
    };
    const int first_round = min(n_units, Cfg::kStages);
    int prod_rb = first_rb, prod_kc = first_kc;      // the producer's place (thread 0 only)

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kStages; ++i) {
            mbar_init(&full_bar[i], 1);
            mbar_init(&empty_bar[i], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&acc_full[i], 1);
            mbar_init(&acc_empty[i], kEpThreads);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        // The weights depend on no earlier kernel and on no other thread of this CTA: the first
        // round of the ring is on its way before the CTA has finished setting up.
        for (int i = 0; i < first_round; ++i) {
            load_w(i, prod_rb, prod_kc);
            if (++prod_kc == s.k_chunks) { prod_kc = 0; ++prod_rb; }
        }
        trace(1);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(s32(&tmem_base_s)), "r"(Cfg::kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem_base = tmem_base_s;

    if (warp == 0) {
        if (lane == 0) {
            pdl_wait();          // from here on the activations are read
            trace(2);
            int kc_x = first_kc;
            for (int i = 0; i < first_round; ++i) {
                load_x(i, kc_x);
                if (++kc_x == s.k_chunks) kc_x = 0;
            }
            for (int i = first_round; i < n_units; ++i) {
                const int st = i % Cfg::kStages;
                const uint32_t round = i / Cfg::kStages;
                if (!mbar_wait(&empty_bar[st], (round - 1) & 1, 1)) break;
                load_w(st, prod_rb, prod_kc);
                load_x(st, prod_kc);
                if (++prod_kc == s.k_chunks) { prod_kc = 0; ++prod_rb; }
            }
            prefetch_next_stream(next, cta, (int)gridDim.x);      // this CTA's own stream has been asked for
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) |
                                       ((uint32_t)(kTileM >> 4) << 24);
            int kc = first_kc, segment = 0;
            bool fresh = true;       // the next MMA starts a row block's sum
            bool ok = true;
            for (int i = 0; i < n_units && ok; ++i) {
                const int buf = segment & 1;
                if (fresh && segment >= 2) {
                    // the drain of the accumulator's previous use must be over
                    ok = mbar_wait(&acc_empty[buf], ((segment >> 1) - 1) & 1, 4);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                }
                const int st = i % Cfg::kStages;
                ok = mbar_wait(&full_bar[st], (i / Cfg::kStages) & 1, 2);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const unsigned char* a_tile = ring + (size_t)st * Cfg::kStageBytes;
                const uint64_t a_desc = umma_desc(a_tile), b_desc = umma_desc(a_tile + Cfg::kABytes);
#pragma unroll
                for (int k = 0; k < kTileK / kUmmaK; ++k)
                    umma_bf16(tmem_base + buf * BN, a_desc + 2 * k, b_desc + 2 * k, idesc, (!fresh || k > 0) ? 1u : 0u);
                umma_commit(&empty_bar[st]);
                fresh = false;
                if (++kc == s.k_chunks || i == n_units - 1) {
                    umma_commit(&acc_full[buf]);     // this row block's share of the CTA is summed
                    kc = 0;
                    ++segment;
                    fresh = true;
                }
            }
        }
    } else {
        // warps 2..9: thread t of a set of four warps holds row `t` of the row block (TMEM lane t); the two sets
        // share the batch's columns when there are 32 or more, and the work of the epilogue always
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;
        const int half = (warp - 2) >> 2;
        const int t2 = half * 128 + t;                         // 0..255: this thread's place in the epilogue's work
        constexpr bool kSplitCols = BN >= 32;
        const int c_begin = kSplitCols ? half * (BN / 2) : 0;
        const int c_end = kSplitCols ? c_begin + BN / 2 : (half == 0 ? BN : 0);
        int rb = first_rb, seg_first_kc = first_kc, done = 0, segment = 0;
        bool ok = true;
        uint32_t cl_dest = 0;
        if (CLUSTER) {
            // Where this thread's sums go in the cluster, and what the CTA owns: divisions by the number of
            // parts, done now, while the weights stream, and not between the last MMA and the stores.
            constexpr bool kTurn = BN > 16;
            const int parts = s.parts, rank = (int)cluster_rank();
            cl_stride = ((kTileM / 4 + parts - 1) / parts) * 4;
            cl_owned = owned_groups(rank, parts, kTileM / 4);
            while ((parts << cl_pad_log2) < kTileM / 4) ++cl_pad_log2;
            // a group is four neighbouring rows of the block: a thread sends its own row's sums, or (turned) a whole group's
            const int group = kTurn ? (t & 31) : (t >> 2);
            cl_dest = cluster_map(s32(staging), (uint32_t)(group % parts)) +
                      (uint32_t)((rank * BN * cl_stride + (group / parts) * 4 + (kTurn ? 0 : (t & 3))) * 4);
            asm volatile("" : "+r"(cl_stride), "+r"(cl_owned), "+r"(cl_pad_log2), "+r"(cl_dest));      // computed here, not later
        }
        if (fusion.in_ssq != nullptr || fusion.residual != nullptr) {
            pdl_wait();          // these threads read what the kernel before wrote
            if (fusion.in_ssq != nullptr) {
                if (t2 < BN) {
                    float ssq = 0.f;
                    if (t2 < s.M)
                        for (int p = 0; p < fusion.in_parts; ++p) ssq += fusion.in_ssq[p * kSsqStride + t2];
                    row_scale[t2] = 1.0f / sqrtf(ssq * fusion.in_inv_dim + fusion.in_eps);
                }
                epilogue_barrier();
            }
        }
        if (CLUSTER) {
            // The run is one part of row block first_rb: every sum goes to the CTA that owns its column.
            // A thread holds one row of the block, a group is four neighbouring rows.  With at most 16 rows
            // in the batch every sum travels on its own into the owner's shared memory.  With more, the
            // remote stores (32 KB a CTA at 64 rows) took longer to land than the whole stream of a small
            // matrix takes: the CTA writes its part to scratch memory instead, rows of the batch along the
            // row block (512 contiguous bytes a warp), and the owners read their columns from L2.
            constexpr bool kTurn = BN > 16;
            float* turn = partials + (size_t)cta * 2 * Cfg::kSlotFloats;      // this CTA's part, [row of the batch][row of the block]
            ok = mbar_wait(&acc_full[0], 0, 3);
            if (t2 == 0) trace(3);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
                for (int c = c_begin; c < c_end; c += 16) {
                    if (c >= s.M) break;                 // the same for a whole warp: columns past the batch hold nothing
                    uint32_t d[16];
                    tmem_load16(taddr + c, d);
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        if (c + e < s.M) {
                            if (kTurn) turn[(c + e) * kTileM + t] = __uint_as_float(d[e]);
                            else cluster_store(cl_dest + (uint32_t)((c + e) * cl_stride * 4), __uint_as_float(d[e]));
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            }
            // (kTurn: the sums lie in scratch memory now; the cluster barrier below, with its release and acquire at
            // cluster scope, makes them visible to the CTAs that own their columns)
        }
        while (!CLUSTER && done < n_units && ok) {
            const int seg_units = min(s.k_chunks - seg_first_kc, n_units - done);
            const bool complete = seg_units == s.k_chunks;
            const int buf = segment & 1;
            ok = mbar_wait(&acc_full[buf], (segment >> 1) & 1, 3);
            if (!ok) break;
            if (t2 == 0 && done + seg_units >= n_units) trace(3);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
            // D[t][b] goes, transposed, either to the staging buffer (this CTA summed the whole row
            // block) or straight to this CTA's part in scratch memory: [b][t], so that what follows
            // reads along the row block
            float* dest = complete ? staging
                                   : partials + ((size_t)cta * 2 + (rb == first_rb ? 0 : 1)) * Cfg::kSlotFloats;
            for (int c = c_begin; c < c_end; c += 16) {
                if (c >= s.M) break;                     // the same for a whole warp
                uint32_t d[16];
                tmem_load16(taddr + c, d);
#pragma unroll
                for (int e = 0; e < 16; ++e)
                    if (c + e < s.M) dest[(c + e) * kTileM + t] = __uint_as_float(d[e]);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(&acc_empty[buf]);            // the issuer may reuse this accumulator
            epilogue_barrier();                      // the 128 threads' writes are ordered before what thread 0 does next

            bool reduce = complete;
            int c_first = cta, c_last = cta, first_slot = 0;
            if (!complete) {
                const int rb_first_unit = rb * s.k_chunks;
                c_first = sk_cta_of_unit(s, rb_first_unit);
                c_last = sk_cta_of_unit(s, rb_first_unit + s.k_chunks - 1);
                first_slot = sk_run_begin(s, c_first) >= rb_first_unit ? 0 : 1;
                if (t2 == 0) {
                    if (done + seg_units >= n_units) trace(4);
                    // one acquire-release add at GPU scope: this CTA's part (ordered before it by the barrier
                    // above) is visible to whoever reads a later ticket, and the earlier parts are visible here
                    const int ticket = ticket_add(&counters[rb]);
                    ticket_s = ticket;
                    if (done + seg_units >= n_units) trace(5);
                }
                epilogue_barrier();
                reduce = ticket_s == c_last - c_first;      // the last of the row block's parts to arrive
            }
            if (reduce) {
                // 128 threads share the block's M x kCols outputs in groups of four columns; the parts'
                // loads of a group do not depend on each other, so they travel together
                constexpr int kGroups = kCols / 4;
                const float* first_part = complete ? staging
                                                   : partials + ((size_t)c_first * 2 + first_slot) * Cfg::kSlotFloats;
                const float* next_part = partials + ((size_t)c_first * 2 + 2) * Cfg::kSlotFloats;
                const int n_more = complete ? 0 : c_last - c_first;
                for (int item = t2; item < s.M * kGroups; item += kEpThreads) {
                    const int b = item / kGroups, c4 = (item % kGroups) * 4;
                    const int offset = b * kTileM + c4;
                    const FinishInput in = finish_begin<SWIGLU>(fusion, s, rb * kCols + c4, b);
                    float4 v = complete ? *reinterpret_cast<const float4*>(first_part + offset)
                                        : __ldcg(reinterpret_cast<const float4*>(first_part + offset));
                    float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (SWIGLU) u = complete ? *reinterpret_cast<const float4*>(first_part + offset + 64)
                                             : __ldcg(reinterpret_cast<const float4*>(first_part + offset + 64));
                    const float* p = next_part + offset;
                    // the parts' loads are issued eight at a time and added in the order of their k ranges
                    for (int part0 = 0; part0 < n_more; part0 += 8, p += 16 * Cfg::kSlotFloats) {
                        float4 w4[8], u4[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const bool live = part0 + j < n_more;
                            const float* q = p + (size_t)j * 2 * Cfg::kSlotFloats;
                            w4[j] = live ? __ldcg(reinterpret_cast<const float4*>(q)) : make_float4(0.f, 0.f, 0.f, 0.f);
                            if (SWIGLU) u4[j] = live ? __ldcg(reinterpret_cast<const float4*>(q + 64)) : make_float4(0.f, 0.f, 0.f, 0.f);
                        }
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            v.x += w4[j].x; v.y += w4[j].y; v.z += w4[j].z; v.w += w4[j].w;
                            if (SWIGLU) { u.x += u4[j].x; u.y += u4[j].y; u.z += u4[j].z; u.w += u4[j].w; }
                        }
                    }
                    // a warp holds one row's columns of this row block: 32 lanes share a sum of squares
                    finish_group<SWIGLU>(fusion, s, out, out_dtype, row_scale, in, rb * kCols + c4, b, v, u, true, 32, rb, lane);
                }
                if (!complete && t2 == 0) counters[rb] = 0;   // ready for the next call
            }
            if (t2 == 0 && done + seg_units >= n_units) trace(6);
            epilogue_barrier();          // staging is free for the next row block
            done += seg_units;
            seg_first_kc = 0;
            ++rb;
            ++segment;
        }
    }
    if (CLUSTER) {
        // every thread of every CTA of the cluster comes here, whatever happened to it before
        __syncwarp();
        const int ep_t = warp >= 2 ? ((warp - 2) >> 2) * 128 + (warp & 3) * 32 + lane : 0;
        const int ep_parts = s.parts, ep_rank = (int)cluster_rank();
        const int ep_pad = 1 << cl_pad_log2;                    // lanes per row: a power of two that holds the owned groups
        const int ep_total = s.M << cl_pad_log2;
        const int ep_rounded = (ep_total + 31) & ~31;      // whole warps: the lanes of a row share its sum of squares
        // What the first pass of the epilogue needs from memory besides the sums (the old residual, the norm's
        // weight) depends on no other CTA of the cluster: it is asked for before the barrier and travels
        // while the CTAs meet.
        FinishInput ahead[2] = {};
        if (warp >= 2) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int item = ep_t + u * kEpThreads;
                const int j = item & (ep_pad - 1);
                if ((u == 0 || ep_t + kEpThreads < ep_rounded) && item < ep_total && j < cl_owned)
                    ahead[u] = finish_begin<false>(fusion, s, first_rb * kTileM + (ep_rank + ep_parts * j) * 4, item >> cl_pad_log2);
            }
        }
        if (threadIdx.x == 64) trace(4);
        cluster_sync_all();
        if (threadIdx.x == 64) trace(5);
        if (warp >= 2) {
            const int t = ep_t;
            const int parts = ep_parts, rank = ep_rank;
            const int stride = cl_stride, n_owned = cl_owned, pad_log2 = cl_pad_log2;
            const int pad = ep_pad;
            const int total = ep_total;
            const int rounded = ep_rounded;
            const int ssq_part = first_rb * parts + rank;
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            // two items per pass: the second one's loads from memory travel with the first one's
            for (int first = t; first < rounded; first += 2 * kEpThreads) {
                const bool two = first + kEpThreads < rounded;     // the same for a whole warp
                FinishInput in[2] = {};
                float4 v[2] = {zero4, zero4};
                int col[2], row[2];
                bool active[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int item = first + u * kEpThreads;
                    const int j = item & (pad - 1);
                    row[u] = item >> pad_log2;
                    active[u] = (u == 0 || two) && item < total && j < n_owned;
                    col[u] = first_rb * kTileM + (rank + parts * j) * 4;
                    if (active[u]) in[u] = first == t ? ahead[u] : finish_begin<false>(fusion, s, col[u], row[u]);
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    if (active[u]) {
                        if (BN > 16) {
                            // the parts lie in scratch memory, one slot per CTA of the cluster (neighbours in the grid)
                            const float* from = partials + (size_t)(cta - rank) * 2 * Cfg::kSlotFloats + row[u] * kTileM +
                                                (rank + parts * ((first + u * kEpThreads) & (pad - 1))) * 4;
                            float4 w4[8];
#pragma unroll
                            for (int p = 0; p < 8; ++p)
                                w4[p] = p < parts ? __ldcg(reinterpret_cast<const float4*>(from + (size_t)p * 2 * Cfg::kSlotFloats))
                                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                            for (int p = 0; p < 8; ++p) { v[u].x += w4[p].x; v[u].y += w4[p].y; v[u].z += w4[p].z; v[u].w += w4[p].w; }
                        } else {
                            const float* from = staging + row[u] * stride + ((first + u * kEpThreads) & (pad - 1)) * 4;
#pragma unroll
                            for (int p = 0; p < 8; ++p) {
                                if (p < parts) {
                                    const float4 w4 = *reinterpret_cast<const float4*>(from + p * BN * stride);
                                    v[u].x += w4.x; v[u].y += w4.y; v[u].z += w4.z; v[u].w += w4.w;
                                }
                            }
                        }
                    }
                }
                finish_group<false>(fusion, s, out, out_dtype, row_scale, in[0], col[0], row[0], v[0], zero4, active[0], pad,
                                    ssq_part, lane);
                if (two)
                    finish_group<false>(fusion, s, out, out_dtype, row_scale, in[1], col[1], row[1], v[1], zero4, active[1], pad,
                                        ssq_part, lane);
            }
        }
        if (threadIdx.x == 64) trace(6);
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(Cfg::kTmemCols) : "memory");
    }
}

static int cluster_enabled() {
    static int enabled = -1;
    if (enabled < 0) {
        const char* text = getenv("DRYFT_GEMM_CLUSTER");        // "off": parts meet through scratch memory and tickets
        enabled = (text != nullptr && (text[0] == 'o' || text[0] == 'O') && (text[1] == 'f' || text[1] == 'F')) ? 0 : 1;
    }
    return enabled;
}

static int g_dec_sm_count = 0;

static int dec_sm_count() {
    if (g_dec_sm_count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&g_dec_sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) g_dec_sm_count = 0;
    }
    return g_dec_sm_count;
}

template <int BN, bool SWIGLU, bool CLUSTER>
static int launch_decode(const void* x, const void* w, void* out, StreamShape s, float* partials, int* counters,
                         int out_dtype, const RowFusion& fusion, cudaStream_t st, const NextStream& next) {
    using Cfg = DecConfig<BN, CLUSTER>;
    static_assert(Cfg::kStages >= 2, "the ring needs at least two stages");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(gemm_decode_kernel<BN, SWIGLU, CLUSTER>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    CUtensorMap map_w, map_x;
    if (!make_tile_map(&map_w, w, SWIGLU ? 2 * s.N : s.N, s.K, SWIGLU ? 64 : kTileM)) return DFI_ERR_LAUNCH;
    if (!make_tile_map(&map_x, x, s.M, s.K, BN)) return DFI_ERR_LAUNCH;
    if (CLUSTER) {
        // the parts of a row block are neighbours in the grid: they form a cluster
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(s.n_ctas);
        config.blockDim = dim3(kDecThreads);
        config.dynamicSmemBytes = Cfg::kSmemBytes;
        config.stream = st;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = s.parts;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attr;
        config.numAttrs = pdl_enabled() ? 2 : 1;
        if (cudaLaunchKernelEx(&config, gemm_decode_kernel<BN, SWIGLU, CLUSTER>, map_w, map_x, out, s, partials, counters,
                               out_dtype, fusion, next) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        return DFI_OK;
    }
    launch(gemm_decode_kernel<BN, SWIGLU, CLUSTER>, s.n_ctas, kDecThreads, Cfg::kSmemBytes, st, map_w, map_x, out, s, partials, counters, out_dtype, fusion, next);
    return DFI_OK;
}

// The split of the work over CTAs: stream-K, or for few row blocks the same number of parts each.
static bool plan_decode(StreamShape& s, int M, int N, int K, int swiglu, int n_ctas) {
    s.M = M; s.N = N; s.K = K;
    s.k_chunks = (K + kTileK - 1) / kTileK;
    const int cols = swiglu ? kTileM / 2 : kTileM;
    s.row_blocks = (N + cols - 1) / cols;
    if ((long long)s.row_blocks * s.k_chunks > (1 << 22)) return false;
    s.units = s.row_blocks * s.k_chunks;
    s.parts = 0;
    s.n_ctas = s.units < n_ctas ? s.units : n_ctas;
    if (s.row_blocks * 2 <= n_ctas) {
        // few row blocks: the same number of parts for each, as many as fill the CTAs
        int parts = n_ctas / s.row_blocks;
        // one part more if fewer than 90 % of the SMs would be busy and that overshoots them by at most 16 %
        // (a few SMs then hold two CTAs): 40 row
        // blocks on 148 SMs run better as 4 x 40 than as 3 x 40 with 28 SMs idle (measured on the 8B and
        // 14B shapes; larger overshoots were measured slower)
        if (parts < 8 && parts * s.row_blocks * 100 < n_ctas * 90 && (parts + 1) * s.row_blocks * 100 <= n_ctas * 116) ++parts;
        if (parts > s.k_chunks) parts = s.k_chunks;
        s.parts = parts;
        s.n_ctas = s.row_blocks * parts;
    } else if (s.row_blocks > n_ctas && s.row_blocks <= 2 * n_ctas) {
        // up to two row blocks per SM: one CTA per row block (two CTAs fit an SM), and no sum is split
        s.parts = 1;
        s.n_ctas = s.row_blocks;
    } else if (s.row_blocks > 2 * n_ctas) {
        // a long stream (the vocabulary projection): two CTAs per SM keep more loads in flight
        // (measured 6.2 against 5.8 TB/s)
        s.n_ctas = s.units < 2 * n_ctas ? s.units : 2 * n_ctas;
    }
    return true;
}
// The parts of a row block meet in a cluster when there are 2 to 8 of them (and no SwiGLU epilogue).
static bool plan_uses_cluster(const StreamShape& s, int swiglu) {
    return !swiglu && s.parts >= 2 && s.parts <= 8 && cluster_enabled();
}

}  // namespace dfi

using namespace dfi;

#ifdef DFI_TRACE
DFI_EXPORT int dfi_gemm_decode_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, g_trace, sizeof(unsigned long long) * 512 * 8) == cudaSuccess ? 0 : 1;
}
#endif

DFI_TCGEN05_STATUS_ENTRIES(gemm_decode)

// Scratch: two parts of 128 x (padded batch) floats for each CTA, and the launch may use up to twice the
// CTAs it was asked for; one counter per row block (zero
// before the first call, left zero by every call).
DFI_EXPORT long long dfi_gemm_decode_partial_floats(int n_ctas) { return (long long)n_ctas * 2 * 2 * kTileM * 64; }
DFI_EXPORT int dfi_gemm_decode_counters(int N, int swiglu) {
    const int cols = swiglu ? kTileM / 2 : kTileM;
    return (N + cols - 1) / cols;
}

// out[M, N] (row stride N) = x[M, K] . w[N, K]^T, or with swiglu: silu(x . gate^T) * (x . up^T) for
// w = [gate; up] of 2N rows.  M <= 64; K a multiple of 8.  n_ctas <= 0: one per SM.
static int gemm_decode(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int n_ctas,
                       float* partials, int* counters, int out_dtype, const RowFusion& fusion, const void* next_hint,
                       void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (M > 64 || K <= 0 || K % 8) return DFI_ERR_SHAPE;
    if (out_dtype != DFI_DTYPE_F32 && out_dtype != DFI_DTYPE_BF16) return DFI_ERR_DTYPE;
    if (!aligned16(x) || !aligned16(w)) return DFI_ERR_ALIGN;
    if (counters == nullptr || partials == nullptr) return DFI_ERR_SHAPE;
    StreamShape s;
    if (n_ctas <= 0) n_ctas = dec_sm_count();
    if (n_ctas <= 0) return DFI_ERR_LAUNCH;
    if (n_ctas > 512) n_ctas = 512;
    if (!plan_decode(s, M, N, K, swiglu, n_ctas)) return DFI_ERR_LIMIT;
    if (s.n_ctas > 2 * n_ctas) return DFI_ERR_LIMIT;      // the scratch memory is sized for twice the CTAs asked for
    s.wide_out = (N % 4 == 0 && aligned16(out)) ? 1 : 0;
    const bool cluster = plan_uses_cluster(s, swiglu);
    cudaStream_t st = (cudaStream_t)stream;
    const NextStream next = next_stream_arg(next_hint);
    int rc;
#define DFI_DEC(BNV)                                                                                       \
    rc = swiglu ? launch_decode<BNV, true, false>(x, w, out, s, partials, counters, out_dtype, fusion, st, next)  \
         : cluster ? launch_decode<BNV, false, true>(x, w, out, s, partials, counters, out_dtype, fusion, st, next) \
                   : launch_decode<BNV, false, false>(x, w, out, s, partials, counters, out_dtype, fusion, st, next)
    if (M <= 16) DFI_DEC(16);
    else if (M <= 32) DFI_DEC(32);
    else DFI_DEC(64);
#undef DFI_DEC
    if (rc != DFI_OK) return rc;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// next_hint: null, or what dfi_gemm_decode_next_stream wrote about the product that the step runs after this one.
DFI_EXPORT int dfi_gemm_decode(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int n_ctas,
                               float* partials, int* counters, int out_dtype, const void* next_hint, void* stream) {
    RowFusion none = {};
    return gemm_decode(x, w, out, M, N, K, swiglu, n_ctas, partials, counters, out_dtype, none, next_hint, stream);
}

// The hint that a decode kernel takes about the product out = x[M, K] . w^T that follows it (same meaning of
// N, K, swiglu and n_ctas as in dfi_gemm_decode): written to `hint` (dfi_next_stream_bytes() bytes of host
// memory).  `tiles`: how many tiles per CTA to ask into L2.  The hint names w: it is good for as long as w
// stays where it is.
DFI_EXPORT int dfi_next_stream_bytes() { return (int)sizeof(NextStream); }
DFI_EXPORT int dfi_gemm_decode_next_stream(void* hint, const void* w, int M, int N, int K, int swiglu, int n_ctas, int tiles) {
    if (hint == nullptr || w == nullptr || M <= 0 || M > 64 || N <= 0 || K <= 0 || K % 8 || !aligned16(w)) return DFI_ERR_SHAPE;
    if (n_ctas <= 0) n_ctas = dec_sm_count();
    if (n_ctas <= 0) return DFI_ERR_LAUNCH;
    if (n_ctas > 512) n_ctas = 512;
    StreamShape s;
    if (!plan_decode(s, M, N, K, swiglu, n_ctas)) return DFI_ERR_LIMIT;
    NextStream next;
    memset(&next, 0, sizeof(next));
    if (!make_tile_map(&next.map, w, swiglu ? 2 * N : N, K, swiglu ? kTileM / 2 : kTileM)) return DFI_ERR_LAUNCH;
    next.deal = UnitDeal{s.units, s.k_chunks, s.n_ctas, s.parts};
    next.up_row0 = swiglu ? N : -1;
    const bool cluster = plan_uses_cluster(s, swiglu);
    next.skip = M <= 16 ? (cluster ? DecConfig<16, true>::kStages : DecConfig<16, false>::kStages)
              : M <= 32 ? (cluster ? DecConfig<32, true>::kStages : DecConfig<32, false>::kStages)
                        : (cluster ? DecConfig<64, true>::kStages : DecConfig<64, false>::kStages);
    next.count = tiles > 0 ? tiles : 0;
    memcpy(hint, &next, sizeof(next));
    return DFI_OK;
}

// Floats per part of a sum-of-squares array, and the number of parts a product with N output
// columns writes (one per row block).
DFI_EXPORT int dfi_gemm_decode_ssq_stride() { return kSsqStride; }
// Parts of the sum-of-squares array that a product with an add-norm output writes for this shape.
DFI_EXPORT int dfi_gemm_decode_ssq_parts(int M, int N, int K, int n_ctas) {
    StreamShape s;
    if (n_ctas <= 0) n_ctas = dec_sm_count();
    if (n_ctas > 512) n_ctas = 512;
    if (n_ctas <= 0 || !plan_decode(s, M, N, K, 0, n_ctas)) return 0;
    return plan_uses_cluster(s, 0) ? s.row_blocks * s.parts : s.row_blocks;
}

// The same product with the RMS norm around it fused in (see the top of this file).
// in_ssq != null: x's rows lack the factor 1/sqrt(sum(in_ssq parts) / in_dim + in_eps), applied to the result.
// residual != null (not with swiglu; out is bfloat16): residual[M, N] += bf16(product) in place,
// out = residual * norm_weight, out_ssq[row block][row] = this block's sum of squares of the new residual.
DFI_EXPORT int dfi_gemm_decode_fused(const void* x, const void* w, void* out, int M, int N, int K, int swiglu,
                                     int n_ctas, float* partials, int* counters, int out_dtype, const float* in_ssq,
                                     int in_parts, int in_dim, float in_eps, void* residual, const float* norm_weight,
                                     float* out_ssq, const void* next_hint, void* stream) {
    RowFusion fusion = {};
    if (in_ssq != nullptr) {
        if (in_parts <= 0 || in_dim <= 0) return DFI_ERR_SHAPE;
        fusion.in_ssq = in_ssq;
        fusion.in_parts = in_parts;
        fusion.in_inv_dim = 1.0f / (float)in_dim;
        fusion.in_eps = in_eps;
    }
    if (residual != nullptr) {
        if (swiglu || out_dtype != DFI_DTYPE_BF16 || norm_weight == nullptr || out_ssq == nullptr || N % 4) return DFI_ERR_SHAPE;
        if (!aligned16(residual) || !aligned16(norm_weight) || !aligned16(out)) return DFI_ERR_ALIGN;
        fusion.residual = (bf16*)residual;
        fusion.norm_weight = norm_weight;
        fusion.out_ssq = out_ssq;
    }
    return gemm_decode(x, w, out, M, N, K, swiglu, n_ctas, partials, counters, out_dtype, fusion, next_hint, stream);
}
