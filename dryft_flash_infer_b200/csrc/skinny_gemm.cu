// out[M, N] = x[M, K] . W[N, K]^T for a few rows of activations (M <= 64, the decode step),
// bfloat16 operands, float32 accumulation.  The work is reading W once at memory speed.
//
// One persistent CTA per SM streams its share of W through a ring of shared-memory
// stages filled by cp.async (16-byte copies that bypass L1), so that about a hundred
// kilobytes per SM are in flight whatever the registers hold.  W's rows are the 16-row
// operand of mma.sync m16n8k16 and the activations the 8-column one, so the batch pads
// to a multiple of 8 only.
//
// The matrix is cut into units of 128 rows x 64 k.  Units are numbered row block by row
// block and dealt to the CTAs in equal contiguous runs (stream-K), which keeps every SM
// busy for the same time even when W has few rows.  A CTA whose run covers a whole row
// block writes the result itself.  Otherwise it leaves its float32 partial sums in
// scratch memory and takes a ticket from the row block's counter; the CTA that draws the
// last ticket adds the parts in the order of their k ranges (so the result does not
// depend on who finished when), applies the epilogue and resets the counter.  No CTA ever
// waits for another.
//
// SWIGLU variant: W is [2*N, K] with the gate rows first; a row block holds 64 gate rows
// and the 64 up rows that belong to them, and the epilogue writes silu(gate) * up to
// out[M, N] (engine/kernels/reference.py:74-79; the fusion follows the idea of
// engine/kernels/cuda_mlp.py:39-125).
#include "common.cuh"

namespace dfi {

constexpr int kGemmThreads = 256;
constexpr int kBlockRows = 128;         // rows of W per unit (16 per warp)
constexpr int kBK = 64;                 // k per unit
constexpr int kRowStride = kBK + 8;     // padded shared-memory row: 9 16-byte chunks, conflict-free for ldmatrix
constexpr int kMaxSmem = 200 * 1024;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(dst)), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldsm2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float silu_mul(float gate, float up) { return gate / (1.0f + expf(-gate)) * up; }

struct GemmShape {
    int M, N, K;          // N: columns of the output
    int k_chunks;         // units per row block
    int row_blocks;
    int units;            // row_blocks * k_chunks (units * n_ctas stays below 2^31)
    int n_ctas;
};

__device__ __forceinline__ int run_begin(const GemmShape& s, int cta) { return (int)((unsigned)s.units * (unsigned)cta / (unsigned)s.n_ctas); }

// The row of W that shared-memory row `r` of row block `rb` holds, or -1 past the end.
template <bool SWIGLU>
__device__ __forceinline__ int weight_row(int rb, int r, int N) {
    if (SWIGLU) {
        const int warp = r >> 4, i = r & 15;
        const int col = rb * (kBlockRows / 2) + warp * 8 + (i & 7);
        if (col >= N) return -1;
        return i < 8 ? col : N + col;
    }
    const int row = rb * kBlockRows + r;
    return row < N ? row : -1;
}

template <int NT> struct Stages { static constexpr int n = NT <= 2 ? 8 : (NT == 4 ? 6 : 5); };

// The CTA whose run holds unit `u`.
__device__ __forceinline__ int cta_of_unit(const GemmShape& s, int u) {
    int c = (int)((unsigned)u * (unsigned)s.n_ctas / (unsigned)s.units);
    while (c + 1 < s.n_ctas && run_begin(s, c + 1) <= u) ++c;
    while (c > 0 && run_begin(s, c) > u) --c;
    return c;
}

__device__ __forceinline__ void store_out(void* out, int out_dtype, size_t index, float v) {
    if (out_dtype == DFI_DTYPE_F32) ((float*)out)[index] = v;
    else ((bf16*)out)[index] = __float2bfloat16_rn(v);
}

template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(kGemmThreads, 1)
skinny_gemm_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, void* __restrict__ out, GemmShape s,
                   float* __restrict__ partials, int* __restrict__ counters, int out_dtype) {
    pdl_launch_next();
    pdl_wait();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int kStages = Stages<NT>::n;
    constexpr int kXRows = NT * 8;
    constexpr int kStageElems = (kBlockRows + kXRows) * kRowStride;
    constexpr int kCols = SWIGLU ? kBlockRows / 2 : kBlockRows;   // output columns per row block
    bf16* ring = reinterpret_cast<bf16*>(smem_raw);
    __shared__ int ticket_s;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int cta = blockIdx.x;
    const int u_begin = run_begin(s, cta), u_end = run_begin(s, cta + 1);
    const int n_units = u_end - u_begin;
    if (n_units <= 0) return;
    const int first_rb = u_begin / s.k_chunks;

    // Each thread copies the same four 16-byte pieces of every unit: rows tid/8 + 32j, piece tid%8.
    const int piece = (threadIdx.x & 7) * 8, row_in_block = threadIdx.x >> 3;
    int load_rb = first_rb, load_kc = u_begin % s.k_chunks;
    auto load_unit = [&](int i) {
        const int k = load_kc * kBK + piece;
        const bool k_ok = k < s.K;
        bf16* stage = ring + (size_t)(i % kStages) * kStageElems;
#pragma unroll
        for (int j = 0; j < kBlockRows / 32; ++j) {
            const int r = row_in_block + 32 * j;
            const int row = weight_row<SWIGLU>(load_rb, r, s.N);
            const bool valid = row >= 0 && k_ok;
            cp16(stage + r * kRowStride + piece, w + (valid ? (size_t)row * s.K + k : 0), valid);
        }
        bf16* xs = stage + kBlockRows * kRowStride;
#pragma unroll
        for (int j = 0; j < (kXRows + 31) / 32; ++j) {
            const int m = row_in_block + 32 * j;
            if (m < kXRows) {
                const bool valid = m < s.M && k_ok;
                cp16(xs + m * kRowStride + piece, x + (valid ? (size_t)m * s.K + k : 0), valid);
            }
        }
        if (++load_kc == s.k_chunks) { load_kc = 0; ++load_rb; }
    };

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;

    for (int i = 0; i < kStages - 1; ++i) {
        if (i < n_units) load_unit(i);
        cp_commit();
    }
    int seg_first_kc = u_begin % s.k_chunks;
    int cur_rb = first_rb, cur_kc = seg_first_kc;
    const int mi = lane >> 3, r8 = lane & 7;
    for (int i = 0; i < n_units; ++i) {
        cp_wait<kStages - 2>();
        __syncthreads();   // unit i has landed for everyone, and everyone is done with the stage refilled next
        if (i + kStages - 1 < n_units) load_unit(i + kStages - 1);
        cp_commit();

        const bf16* stage = ring + (size_t)(i % kStages) * kStageElems;
        const bf16* ws = stage + (warp * 16) * kRowStride;
        const bf16* xs = stage + kBlockRows * kRowStride;
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
            uint32_t a[4];
            ldsm4(a, ws + (r8 + (mi & 1) * 8) * kRowStride + kk * 16 + (mi >> 1) * 8);
            if (NT == 1) {
                uint32_t b[2];
                ldsm2(b, xs + r8 * kRowStride + kk * 16 + (mi & 1) * 8);
                mma16816(acc[0], a, b[0], b[1]);
            } else {
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    uint32_t b[4];
                    ldsm4(b, xs + (j * 8 + r8 + (mi >> 1) * 8) * kRowStride + kk * 16 + (mi & 1) * 8);
                    mma16816(acc[j], a, b[0], b[1]);
                    mma16816(acc[j + 1 < NT ? j + 1 : j], a, b[2], b[3]);
                }
            }
        }

        const int rb = cur_rb, kc = cur_kc;
        if (++cur_kc == s.k_chunks) { cur_kc = 0; ++cur_rb; }
        if (kc != s.k_chunks - 1 && i != n_units - 1) continue;
        // ---- a row block's share of this CTA ends here
        const bool complete = seg_first_kc == 0 && kc == s.k_chunks - 1;
        if (complete) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int m = j * 8 + 2 * t4 + e;
                    if (m >= s.M) continue;
                    if (SWIGLU) {
                        const int col = rb * kCols + warp * 8 + g;
                        if (col < s.N) store_out(out, out_dtype, (size_t)m * s.N + col, silu_mul(acc[j][e], acc[j][e + 2]));
                    } else {
                        const int n0 = rb * kBlockRows + warp * 16 + g;
                        if (n0 < s.N) store_out(out, out_dtype, (size_t)m * s.N + n0, acc[j][e]);
                        if (n0 + 8 < s.N) store_out(out, out_dtype, (size_t)m * s.N + n0 + 8, acc[j][e + 2]);
                    }
                }
        } else {
            float* mine = partials + ((size_t)cta * 2 + (rb == first_rb ? 0 : 1)) * (kBlockRows * kXRows);
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int m = j * 8 + 2 * t4 + e;
                    mine[m * kBlockRows + warp * 16 + g] = acc[j][e];
                    mine[m * kBlockRows + warp * 16 + g + 8] = acc[j][e + 2];
                }
            __threadfence();
            __syncthreads();
            const int rb_first_unit = rb * s.k_chunks;
            const int c_first = cta_of_unit(s, rb_first_unit), c_last = cta_of_unit(s, rb_first_unit + s.k_chunks - 1);
            if (threadIdx.x == 0) ticket_s = atomicAdd(&counters[rb], 1);
            __syncthreads();
            if (ticket_s == c_last - c_first) {          // the last of the row block's parts to arrive
                __threadfence();
                // a part's sums lie in its slot 0 if the row block is the first of its run: true for every
                // part after the first, whose runs begin inside the row block
                const int first_slot = run_begin(s, c_first) >= rb_first_unit ? 0 : 1;
                constexpr int kSlot = kBlockRows * kXRows;
                for (int idx = threadIdx.x; idx < s.M * kCols; idx += kGemmThreads) {
                    const int m = idx / kCols, c = idx % kCols;
                    const int r = SWIGLU ? (c >> 3) * 16 + (c & 7) : c;
                    const float* p = partials + ((size_t)c_first * 2 + first_slot) * kSlot + m * kBlockRows + r;
                    float v = __ldcg(p), v_up = SWIGLU ? __ldcg(p + 8) : 0.f;
                    p = partials + ((size_t)c_first * 2 + 2) * kSlot + m * kBlockRows + r;
#pragma unroll 4
                    for (int part = c_first + 1; part <= c_last; ++part, p += 2 * kSlot) {
                        v += __ldcg(p);
                        if (SWIGLU) v_up += __ldcg(p + 8);
                    }
                    const int col = rb * kCols + c;
                    if (col < s.N) store_out(out, out_dtype, (size_t)m * s.N + col, SWIGLU ? silu_mul(v, v_up) : v);
                }
                if (threadIdx.x == 0) counters[rb] = 0;   // ready for the next call
            }
        }
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
        seg_first_kc = 0;
    }
    cp_wait<0>();
}

static int g_sm_count = 0;

template <int NT, bool SWIGLU>
static int launch_skinny(const bf16* x, const bf16* w, void* out, const GemmShape& s, float* partials, int* counters,
                         int out_dtype, cudaStream_t st) {
    constexpr int smem = Stages<NT>::n * (kBlockRows + NT * 8) * kRowStride * (int)sizeof(bf16);
    static_assert(smem <= kMaxSmem, "ring too large");
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(skinny_gemm_kernel<NT, SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return DFI_ERR_LAUNCH;
        configured = true;
    }
    launch(skinny_gemm_kernel<NT, SWIGLU>, s.n_ctas, kGemmThreads, smem, st, x, w, out, s, partials, counters, out_dtype);
    return DFI_OK;
}

}  // namespace dfi

using namespace dfi;

// How the caller sizes the scratch.  Partial sums: two parts of 128 x 64 floats for each CTA
// of the launch.  Counters: one int per row block, zero before the first call and left zero
// by every call.
DFI_EXPORT long long dfi_skinny_gemm_partial_floats(int n_ctas) { return (long long)n_ctas * 2 * kBlockRows * 64; }
DFI_EXPORT int dfi_skinny_gemm_counters(int N, int swiglu) {
    const int cols = swiglu ? kBlockRows / 2 : kBlockRows;
    return (N + cols - 1) / cols;
}
DFI_EXPORT int dfi_sm_count() {
    if (g_sm_count == 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess) return 0;
        if (cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) g_sm_count = 0;
    }
    return g_sm_count;
}

// x [M, K] bfloat16 (rows contiguous), w [N, K] (or [2N, K] with swiglu) bfloat16,
// out [M, N] of out_dtype.  K must be a multiple of 8; M at most 64.  n_ctas persistent
// CTAs share the work (0: one per SM); partials holds dfi_skinny_gemm_partial_floats(n_ctas).
DFI_EXPORT int dfi_skinny_gemm(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int n_ctas,
                               float* partials, int* counters, int out_dtype, void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (M > 64 || K <= 0 || K % 8) return DFI_ERR_SHAPE;
    if (out_dtype != DFI_DTYPE_F32 && out_dtype != DFI_DTYPE_BF16) return DFI_ERR_DTYPE;
    if (!aligned16(x) || !aligned16(w)) return DFI_ERR_ALIGN;
    if (counters == nullptr || partials == nullptr) return DFI_ERR_SHAPE;
    GemmShape s;
    s.M = M; s.N = N; s.K = K;
    s.k_chunks = (K + kBK - 1) / kBK;
    s.row_blocks = dfi_skinny_gemm_counters(N, swiglu);
    if ((long long)s.row_blocks * s.k_chunks > (1 << 22)) return DFI_ERR_LIMIT;
    s.units = s.row_blocks * s.k_chunks;
    if (n_ctas <= 0) n_ctas = dfi_sm_count();
    if (n_ctas <= 0) return DFI_ERR_LAUNCH;
    if (n_ctas > 512) n_ctas = 512;
    s.n_ctas = s.units < n_ctas ? s.units : n_ctas;
    cudaStream_t st = (cudaStream_t)stream;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    const int nt = (M + 7) / 8;
    int rc;
#define DFI_LAUNCH(NTV)                                                                                     \
    rc = swiglu ? launch_skinny<NTV, true>(xp, wp, out, s, partials, counters, out_dtype, st)                \
                : launch_skinny<NTV, false>(xp, wp, out, s, partials, counters, out_dtype, st)
    if (nt <= 1) DFI_LAUNCH(1);
    else if (nt <= 2) DFI_LAUNCH(2);
    else if (nt <= 4) DFI_LAUNCH(4);
    else DFI_LAUNCH(8);
#undef DFI_LAUNCH
    if (rc != DFI_OK) return rc;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// ------------------------------------------------------------------ the allocation-free entry point
// See skinny_gemm_static.h for who needs it and what it promises.
#include <mutex>

#include "skinny_gemm_static.h"

namespace dfi {

constexpr int kStaticCtas = 160;                                            // at least one per SM of a B200
constexpr int kStaticPartialFloats = kStaticCtas * 2 * kBlockRows * DFI_STATIC_MAX_ROWS;
constexpr int kStaticCounters = (DFI_STATIC_MAX_COLS + kBlockRows / 2 - 1) / (kBlockRows / 2);
constexpr int kMaxDevices = 64;

struct StaticScratch {
    float partials[kStaticPartialFloats];
    int counters[kStaticCounters];
};

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static __device__ __align__(256) StaticScratch g_static_scratch;

static StaticScratch* g_static_ptr[kMaxDevices] = {};
static std::mutex g_static_setup;          // first calls made by several host threads at once take turns

}  // namespace dfi

extern "C" __attribute__((visibility("default"))) const char* dfi_error_string(int code) {
    switch (code) {
        case DFI_OK: return "ok";
        case DFI_ERR_DTYPE: return "unsupported dtype code (0 float32, 1 bfloat16)";
        case DFI_ERR_SHAPE: return "a size the kernel does not take";
        case DFI_ERR_ALIGN: return "a pointer or stride is not aligned as required";
        case DFI_ERR_LAUNCH: return "a CUDA call failed";
        case DFI_ERR_LIMIT: return "a size beyond the stated maximum";
        default: return "unknown error code";
    }
}

extern "C" __attribute__((visibility("default")))
int dfi_skinny_gemm_static(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int out_dtype,
                           void* stream) {
    if (M <= 0 || N <= 0) return DFI_OK;
    if (M > DFI_STATIC_MAX_ROWS || N > DFI_STATIC_MAX_COLS) return DFI_ERR_LIMIT;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return DFI_ERR_LAUNCH;
    if (device < 0 || device >= kMaxDevices) return DFI_ERR_LIMIT;
    StaticScratch* scratch = nullptr;
    {
        // set-up, once per device, with that device current; threads that arrive together take turns
        std::lock_guard<std::mutex> lock(g_static_setup);
        if (g_static_ptr[device] == nullptr) {
            StaticScratch* ptr = nullptr;
            if (cudaGetSymbolAddress((void**)&ptr, g_static_scratch) != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return DFI_ERR_LAUNCH;
            }
            if (cudaMemsetAsync(ptr->counters, 0, sizeof(ptr->counters), (cudaStream_t)stream) != cudaSuccess) {
                cudaGetLastError();
                return DFI_ERR_LAUNCH;
            }
            g_static_ptr[device] = ptr;
        }
        scratch = g_static_ptr[device];
    }
    int n_ctas = dfi_sm_count();
    if (n_ctas <= 0) return DFI_ERR_LAUNCH;
    if (n_ctas > kStaticCtas) n_ctas = kStaticCtas;
    return dfi_skinny_gemm(x, w, out, M, N, K, swiglu, n_ctas, scratch->partials, scratch->counters, out_dtype, stream);
}
