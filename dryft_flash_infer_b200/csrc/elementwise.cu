// Row-wise kernels of the step: embedding gather, RMSNorm with and without the fused
// residual add, SwiGLU, row gather, and the fused per-head norm + rotary embedding +
// cache write.  Formulas follow the reference engine's plain-torch statement of its
// fused kernels (engine/kernels/reference.py:13-23, :31-71, :74-79) with one
// difference: values stay float32 inside a kernel and round once on store.
#include "common.cuh"

namespace dfi {

// ------------------------------------------------------------------ embedding
template <typename T, bool VEC>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids, T* __restrict__ out,
                                 int hidden, int vocab) {
    pdl_launch_next();
    pdl_wait();
    const int row = blockIdx.x;
    int id = ids[row];
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* src = table + (size_t)id * hidden;
    T* dst = out + (size_t)row * hidden;
    if (VEC) {
        constexpr int n = Vec16<T>::n;
        for (int i = threadIdx.x * n; i < hidden; i += blockDim.x * n)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = src[i];
    }
}

// ------------------------------------------------------------------ a * scale + b, and the cap on logits
// a[i] = a[i] * scale + (b ? b[i] : 0), in float32, in place: the factor some architectures put on the
// embedded rows, and the residual sum of a model without a final norm.
template <typename T>
__global__ void scale_add_kernel(T* __restrict__ a, const T* __restrict__ b, long long n, float scale) {
    pdl_launch_next();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = to_float(a[i]) * scale;
        if (b != nullptr) v += to_float(b[i]);
        a[i] = from_float<T>(v);
    }
}

// x = x * scale, then (cap > 0) x = cap * tanh(x / cap), in place on float32 logits.
__global__ void scale_cap_kernel(float* __restrict__ x, long long n, float scale, float cap) {
    pdl_launch_next();
    pdl_wait();
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        float v = x[i] * scale;
        if (cap > 0.f) v = cap * tanhf(v / cap);
        x[i] = v;
    }
}

// ------------------------------------------------------------------ gather rows
template <typename T, bool VEC>
__global__ void gather_rows_kernel(const T* __restrict__ x, const int* __restrict__ rows, T* __restrict__ out, int dim) {
    pdl_launch_next();
    pdl_wait();
    const T* src = x + (size_t)rows[blockIdx.x] * dim;
    T* dst = out + (size_t)blockIdx.x * dim;
    if (VEC) {
        constexpr int n = Vec16<T>::n;
        for (int i = threadIdx.x * n; i < dim; i += blockDim.x * n)
            *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = src[i];
    }
}

// ------------------------------------------------------------------ RMSNorm (+ residual add)
// ADD: residual[row] += delta[row] (float32 sum, rounded to T), then out = norm(residual) * w.
// else: out = norm(x) * w with x = residual (read only).
template <typename T, bool VEC, bool ADD>
__global__ void rmsnorm_kernel(T* __restrict__ residual, const T* __restrict__ delta,
                               const float* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float scratch[32];
    T* x = residual + (size_t)blockIdx.x * dim;
    const T* d = ADD ? delta + (size_t)blockIdx.x * dim : nullptr;
    T* y = out + (size_t)blockIdx.x * dim;
    float ssq = 0.f;
    if (VEC) {
        constexpr int n = Vec16<T>::n;
        for (int i = threadIdx.x * n; i < dim; i += blockDim.x * n) {
            float a[n];
            load16(x + i, a);
            if (ADD) {
                float b[n];
                load16(d + i, b);
#pragma unroll
                for (int j = 0; j < n; ++j) a[j] = to_float(from_float<T>(a[j] + b[j]));
                store16(x + i, a);
            }
#pragma unroll
            for (int j = 0; j < n; ++j) ssq += a[j] * a[j];
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            float a = to_float(x[i]);
            if (ADD) {
                T r = from_float<T>(a + to_float(d[i]));
                x[i] = r;
                a = to_float(r);
            }
            ssq += a * a;
        }
    }
    ssq = block_sum(ssq, scratch);
    const float scale = 1.0f / sqrtf(ssq / (float)dim + eps);
    // each thread re-reads exactly the elements it wrote above, so no barrier is needed
    if (VEC) {
        constexpr int n = Vec16<T>::n;
        for (int i = threadIdx.x * n; i < dim; i += blockDim.x * n) {
            float a[n];
            load16(x + i, a);
#pragma unroll
            for (int j = 0; j < n; ++j) a[j] = a[j] * scale * weight[i + j];
            store16(y + i, a);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x)
            y[i] = from_float<T>(to_float(x[i]) * scale * weight[i]);
    }
}

// The same for rows of up to kRowVectors 16-byte vectors per thread: the row stays in registers
// between the sum of squares and the scaling, so it is read once.
constexpr int kRowVectors = 4;

template <typename T, bool ADD>
__global__ void rmsnorm_registers_kernel(T* __restrict__ residual, const T* __restrict__ delta,
                                         const float* __restrict__ weight, T* __restrict__ out, int dim, float eps) {
    pdl_launch_next();
    pdl_wait();
    __shared__ float scratch[32];
    constexpr int n = Vec16<T>::n;
    T* x = residual + (size_t)blockIdx.x * dim;
    const T* d = ADD ? delta + (size_t)blockIdx.x * dim : nullptr;
    T* y = out + (size_t)blockIdx.x * dim;
    float a[kRowVectors][n];
    float ssq = 0.f;
#pragma unroll
    for (int v = 0; v < kRowVectors; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * n;
        if (i < dim) {
            load16(x + i, a[v]);
            if (ADD) {
                float b[n];
                load16(d + i, b);
#pragma unroll
                for (int j = 0; j < n; ++j) a[v][j] = to_float(from_float<T>(a[v][j] + b[j]));
                store16(x + i, a[v]);
            }
#pragma unroll
            for (int j = 0; j < n; ++j) ssq += a[v][j] * a[v][j];
        }
    }
    ssq = block_sum(ssq, scratch);
    const float scale = 1.0f / sqrtf(ssq / (float)dim + eps);
#pragma unroll
    for (int v = 0; v < kRowVectors; ++v) {
        const int i = (threadIdx.x + v * blockDim.x) * n;
        if (i < dim) {
            float w[n];
            load16(weight + i, w);
            if constexpr (n == 8) load16(weight + i + 4, w + 4);
#pragma unroll
            for (int j = 0; j < n; ++j) a[v][j] = a[v][j] * scale * w[j];
            store16(y + i, a[v]);
        }
    }
}

// ------------------------------------------------------------------ SwiGLU
// gate_up [rows, 2*inter] (gate first), out [rows, inter] = silu(gate) * up.
template <typename T, bool VEC>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int inter) {
    pdl_launch_next();
    pdl_wait();
    const T* g = gate_up + (size_t)blockIdx.y * 2 * inter;
    const T* u = g + inter;
    T* y = out + (size_t)blockIdx.y * inter;
    if (VEC) {
        constexpr int n = Vec16<T>::n;
        const int i = (blockIdx.x * blockDim.x + threadIdx.x) * n;
        if (i < inter) {
            float a[n], b[n];
            load16(g + i, a);
            load16(u + i, b);
#pragma unroll
            for (int j = 0; j < n; ++j) a[j] = a[j] / (1.0f + expf(-a[j])) * b[j];
            store16(y + i, a);
        }
    } else {
        const int i = blockIdx.x * blockDim.x + threadIdx.x;
        if (i < inter) {
            const float a = to_float(g[i]);
            y[i] = from_float<T>(a / (1.0f + expf(-a)) * to_float(u[i]));
        }
    }
}

// ------------------------------------------------------------------ per-head norm + rotary + cache write
// One warp per (row, head).  Heads 0..n_q-1 are queries (normalised and rotated in place
// in `qkv`), the next n_kv are keys (normalised, rotated, written to the key cache), the
// last n_kv are values (copied to the value cache).  A head vector pairs element i with
// i + D/2 (engine/kernels/reference.py:31-46).  q_w / k_w may be null (no per-head norm),
// cos may be null (no rotation).  cos/sin are [max_positions, D/2] float32.
constexpr int kMaxPairsPerLane = 4;  // D <= 256

__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void store2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store2(bf16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

template <typename T>
__global__ void qk_norm_rope_write_kernel(T* __restrict__ qkv, int row_stride, int n_q, int n_kv, int D,
                                          const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                          const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                          const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                                          T* __restrict__ k_cache, T* __restrict__ v_cache,
                                          const int* __restrict__ block_table, int table_width, int page_size,
                                          int ring_tokens, int write_cache) {
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int head = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int total_heads = n_q + 2 * n_kv;
    if (head >= total_heads) return;
    const int row = blockIdx.x;
    const bool is_q = head < n_q;
    const bool is_k = !is_q && head < n_q + n_kv;
    if (!is_q && !write_cache) return;
    const int half = D >> 1;
    T* src = qkv + (size_t)row * row_stride + (size_t)head * D;

    T* dst = src;
    if (!is_q) {
        const int pos = row_pos[row];
        const int place = place_of(pos, ring_tokens);
        const int page = block_table[(size_t)row_seq[row] * table_width + place / page_size];
        const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
        T* cache = is_k ? k_cache : v_cache;
        dst = cache + (((size_t)page * n_kv + kv_head) * page_size + place % page_size) * D;
    }

    // a lane takes two neighbouring elements of each half at a time (head sizes are multiples of 4)
    float2 lo[kMaxPairsPerLane / 2], hi[kMaxPairsPerLane / 2];
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < kMaxPairsPerLane / 2; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            lo[j] = load2(src + i);
            hi[j] = load2(src + i + half);
            ssq += lo[j].x * lo[j].x + lo[j].y * lo[j].y + hi[j].x * hi[j].x + hi[j].y * hi[j].y;
        }
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    if (w != nullptr) {
        ssq = warp_sum(ssq);
        const float scale = 1.0f / sqrtf(ssq / (float)D + eps);
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane / 2; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) {
                const float2 wl = *reinterpret_cast<const float2*>(w + i), wh = *reinterpret_cast<const float2*>(w + i + half);
                lo[j].x *= scale * wl.x; lo[j].y *= scale * wl.y;
                hi[j].x *= scale * wh.x; hi[j].y *= scale * wh.y;
            }
        }
    }
    const bool rotate = (is_q || is_k) && cos_t != nullptr;
    const float* c = rotate ? cos_t + (size_t)row_pos[row] * half : nullptr;
    const float* s = rotate ? sin_t + (size_t)row_pos[row] * half : nullptr;
#pragma unroll
    for (int j = 0; j < kMaxPairsPerLane / 2; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            float2 a = lo[j], b = hi[j];
            if (rotate) {
                const float2 cv = *reinterpret_cast<const float2*>(c + i), sv = *reinterpret_cast<const float2*>(s + i);
                a.x = lo[j].x * cv.x - hi[j].x * sv.x; a.y = lo[j].y * cv.y - hi[j].y * sv.y;
                b.x = hi[j].x * cv.x + lo[j].x * sv.x; b.y = hi[j].y * cv.y + lo[j].y * sv.y;
            }
            store2(dst + i, a);
            store2(dst + i + half, b);
        }
    }
}

// The same for a rotation of only the first R < D elements of a head (pairs i and i + R/2 for i < R/2;
// the elements from R on are normalised but not rotated; cos/sin are [max_positions, R/2]).  One warp per
// (row, head); a lane takes the elements lane, lane + 32, ... and finds each one's partner, which
// another lane holds, in the warp's shared-memory copy of the normalised head.
constexpr int kPartialWarps = 4;

template <typename T>
__global__ void qk_norm_rope_write_partial_kernel(T* __restrict__ qkv, int row_stride, int n_q, int n_kv, int D, int R,
                                                  const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                                  const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                  const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                                  const int* __restrict__ block_table, int table_width, int page_size,
                                                  int ring_tokens, int write_cache) {
    __shared__ float normed[kPartialWarps][64 * kMaxPairsPerLane];
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int head = blockIdx.y * kPartialWarps + warp;
    if (head >= n_q + 2 * n_kv) return;
    const int row = blockIdx.x;
    const bool is_q = head < n_q;
    const bool is_k = !is_q && head < n_q + n_kv;
    if (!is_q && !write_cache) return;
    T* src = qkv + (size_t)row * row_stride + (size_t)head * D;
    T* dst = src;
    const int pos = row_pos[row];
    if (!is_q) {
        const int place = place_of(pos, ring_tokens);
        const int page = block_table[(size_t)row_seq[row] * table_width + place / page_size];
        const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
        dst = (is_k ? k_cache : v_cache) + (((size_t)page * n_kv + kv_head) * page_size + place % page_size) * D;
    }
    float ssq = 0.f;
    for (int i = lane; i < D; i += 32) {
        const float v = to_float(src[i]);
        normed[warp][i] = v;
        ssq += v * v;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    if (w != nullptr) {
        ssq = warp_sum(ssq);
        const float scale = 1.0f / sqrtf(ssq / (float)D + eps);
        for (int i = lane; i < D; i += 32) normed[warp][i] *= scale * w[i];
    }
    __syncwarp();
    const bool rotate = (is_q || is_k) && cos_t != nullptr;
    const int half = R >> 1;
    for (int i = lane; i < D; i += 32) {
        float v = normed[warp][i];
        if (rotate && i < R) {
            const int pair = i < half ? i : i - half;
            const float c = cos_t[(size_t)pos * half + pair], sn = sin_t[(size_t)pos * half + pair];
            v = i < half ? v * c - normed[warp][i + half] * sn : v * c + normed[warp][i - half] * sn;
        }
        dst[i] = from_float<T>(v);
    }
}

// The same with eight lanes per head (four heads per warp) and eight neighbouring elements of each half
// of a head per lane, for head sizes that are multiples of 16 up to 256: with many rows a warp mostly
// waits for its loads, so every lane takes a 16-byte load's worth of a head (half the warps per row).
constexpr int kWideSteps = 2;  // 8 lanes x 8 elements x 2 steps cover half a head of up to 128 (one step: up to 64)

struct Oct { float v[8]; };
__device__ __forceinline__ Oct load8(const float* p) {
    const float4 f = *reinterpret_cast<const float4*>(p), g = *reinterpret_cast<const float4*>(p + 4);
    return Oct{{f.x, f.y, f.z, f.w, g.x, g.y, g.z, g.w}};
}
__device__ __forceinline__ Oct load8(const bf16* p) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.z));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.w));
    return Oct{{a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y}};
}
__device__ __forceinline__ void store8(float* p, const Oct& q) {
    *reinterpret_cast<float4*>(p) = make_float4(q.v[0], q.v[1], q.v[2], q.v[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(q.v[4], q.v[5], q.v[6], q.v[7]);
}
__device__ __forceinline__ void store8(bf16* p, const Oct& q) {
    uint4 u;
    *reinterpret_cast<__nv_bfloat162*>(&u.x) = __floats2bfloat162_rn(q.v[0], q.v[1]);
    *reinterpret_cast<__nv_bfloat162*>(&u.y) = __floats2bfloat162_rn(q.v[2], q.v[3]);
    *reinterpret_cast<__nv_bfloat162*>(&u.z) = __floats2bfloat162_rn(q.v[4], q.v[5]);
    *reinterpret_cast<__nv_bfloat162*>(&u.w) = __floats2bfloat162_rn(q.v[6], q.v[7]);
    *reinterpret_cast<uint4*>(p) = u;
}

template <typename T, int STEPS>
__global__ void qk_norm_rope_write_wide_kernel(T* __restrict__ qkv, int row_stride, int n_q, int n_kv, int D,
                                               const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                               const int* __restrict__ row_pos, const int* __restrict__ row_seq,
                                               T* __restrict__ k_cache, T* __restrict__ v_cache,
                                               const int* __restrict__ block_table, int table_width, int page_size,
                                               int ring_tokens, int write_cache) {
    pdl_launch_next();
    pdl_wait();
    const int lane = threadIdx.x & 7;
    const int head = blockIdx.y * (blockDim.x >> 3) + (threadIdx.x >> 3);
    const int row = blockIdx.x;
    const bool is_q = head < n_q;
    const bool is_k = !is_q && head < n_q + n_kv;
    // a lane that has nothing to do still takes part in the sums of its warp
    const bool active = head < n_q + 2 * n_kv && (is_q || write_cache);
    const int half = D >> 1;
    T* src = qkv + (size_t)row * row_stride + (size_t)(active ? head : 0) * D;
    const int pos = row_pos[row];

    Oct lo[STEPS], hi[STEPS];
#pragma unroll
    for (int j = 0; j < STEPS; ++j) {
        const int i = 8 * lane + 64 * j;
        if (active && i < half) {
            lo[j] = load8(src + i);
            hi[j] = load8(src + i + half);
        }
    }
    // where keys and values go: looked up after the row has been asked for, which does not wait for it
    T* dst = src;
    if (active && !is_q) {
        const int place = place_of(pos, ring_tokens);
        const int page = block_table[(size_t)row_seq[row] * table_width + place / page_size];
        const int kv_head = is_k ? head - n_q : head - n_q - n_kv;
        T* cache = is_k ? k_cache : v_cache;
        dst = cache + (((size_t)page * n_kv + kv_head) * page_size + place % page_size) * D;
    }
    const float* w = is_q ? q_w : (is_k ? k_w : nullptr);
    const bool rotate = (is_q || is_k) && cos_t != nullptr;
    float ssq = 0.f;
#pragma unroll
    for (int j = 0; j < STEPS; ++j) {
        if (active && 8 * lane + 64 * j < half) {
#pragma unroll
            for (int e = 0; e < 8; ++e) ssq += lo[j].v[e] * lo[j].v[e] + hi[j].v[e] * hi[j].v[e];
        }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) ssq += __shfl_xor_sync(0xffffffffu, ssq, o);
    if (!active) return;
    const float scale = w != nullptr ? 1.0f / sqrtf(ssq / (float)D + eps) : 1.0f;
#pragma unroll
    for (int j = 0; j < STEPS; ++j) {
        const int i = 8 * lane + 64 * j;
        if (i < half) {
            Oct a = lo[j], b = hi[j];
            if (w != nullptr) {
                const Oct wl = load8(w + i), wh = load8(w + i + half);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a.v[e] *= scale * wl.v[e];
                    b.v[e] *= scale * wh.v[e];
                }
            }
            if (rotate) {
                const Oct cv = load8(cos_t + (size_t)pos * half + i), sv = load8(sin_t + (size_t)pos * half + i);
                const Oct a0 = a, b0 = b;
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    a.v[e] = a0.v[e] * cv.v[e] - b0.v[e] * sv.v[e];
                    b.v[e] = b0.v[e] * cv.v[e] + a0.v[e] * sv.v[e];
                }
            }
            store8(dst + i, a);
            store8(dst + i + half, b);
        }
    }
}

template <typename T>
static int launch_embedding(const void* table, const int* ids, void* out, int rows, int hidden, int vocab,
                            cudaStream_t st) {
    const bool vec = hidden % Vec16<T>::n == 0 && aligned16(table) && aligned16(out);
    const int threads = 128;
    if (vec) launch(embedding_kernel<T, true>, rows, threads, 0, st, (const T*)table, ids, (T*)out, hidden, vocab);
    else launch(embedding_kernel<T, false>, rows, threads, 0, st, (const T*)table, ids, (T*)out, hidden, vocab);
    return DFI_OK;
}

template <typename T>
static int launch_gather(const void* x, const int* rows_idx, void* out, int rows, int dim, cudaStream_t st) {
    const bool vec = dim % Vec16<T>::n == 0 && aligned16(x) && aligned16(out);
    if (vec) launch(gather_rows_kernel<T, true>, rows, 128, 0, st, (const T*)x, rows_idx, (T*)out, dim);
    else launch(gather_rows_kernel<T, false>, rows, 128, 0, st, (const T*)x, rows_idx, (T*)out, dim);
    return DFI_OK;
}

template <typename T>
static int launch_rmsnorm(void* residual, const void* delta, const float* weight, void* out, int rows, int dim,
                          float eps, cudaStream_t st) {
    const bool vec = dim % Vec16<T>::n == 0 && aligned16(residual) && aligned16(out) &&
                     (delta == nullptr || aligned16(delta));
    if (vec && aligned16(weight) && rows >= 64 && dim <= 256 * kRowVectors * Vec16<T>::n) {
        // many rows (a prompt): each row is read once and kept in registers
        int t = 64;
        while (t < 256 && t * kRowVectors * Vec16<T>::n < dim) t <<= 1;
        if (delta != nullptr) launch(rmsnorm_registers_kernel<T, true>, rows, t, 0, st, (T*)residual, (const T*)delta, weight, (T*)out, dim, eps);
        else launch(rmsnorm_registers_kernel<T, false>, rows, t, 0, st, (T*)residual, (const T*)nullptr, weight, (T*)out, dim, eps);
        return DFI_OK;
    }
    int threads = 32;
    const int per = vec ? Vec16<T>::n : 1;
    while (threads < 512 && threads * per < dim) threads <<= 1;
    if (delta != nullptr) {
        if (vec) launch(rmsnorm_kernel<T, true, true>, rows, threads, 0, st, (T*)residual, (const T*)delta, weight, (T*)out, dim, eps);
        else launch(rmsnorm_kernel<T, false, true>, rows, threads, 0, st, (T*)residual, (const T*)delta, weight, (T*)out, dim, eps);
    } else {
        if (vec) launch(rmsnorm_kernel<T, true, false>, rows, threads, 0, st, (T*)residual, nullptr, weight, (T*)out, dim, eps);
        else launch(rmsnorm_kernel<T, false, false>, rows, threads, 0, st, (T*)residual, nullptr, weight, (T*)out, dim, eps);
    }
    return DFI_OK;
}

template <typename T>
static int launch_swiglu(const void* gate_up, void* out, int rows, int inter, cudaStream_t st) {
    const bool vec = inter % Vec16<T>::n == 0 && aligned16(gate_up) && aligned16(out);
    const int per = vec ? Vec16<T>::n : 1;
    const int threads = 256;
    dim3 grid((inter + threads * per - 1) / (threads * per), rows);
    if (vec) launch(swiglu_kernel<T, true>, grid, threads, 0, st, (const T*)gate_up, (T*)out, inter);
    else launch(swiglu_kernel<T, false>, grid, threads, 0, st, (const T*)gate_up, (T*)out, inter);
    return DFI_OK;
}

}  // namespace dfi

using namespace dfi;

// 1: kernels of this library are launched so that they may overlap the tail of the kernel before
// them (programmatic dependent launch); 0: plain launches.  Returns the previous setting.
DFI_EXPORT int dfi_set_pdl(int enabled) {
    const int before = pdl_enabled();
    pdl_enabled() = enabled ? 1 : 0;
    return before;
}

DFI_EXPORT int dfi_embedding(const void* table, const int* ids, void* out, int rows, int hidden, int vocab,
                             int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (hidden <= 0 || vocab <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch_embedding<float>(table, ids, out, rows, hidden, vocab, st);
    else if (dtype == DFI_DTYPE_BF16) launch_embedding<bf16>(table, ids, out, rows, hidden, vocab, st);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_scale_add(void* a, const void* b, long long n, float scale, int dtype, void* stream) {
    if (n <= 0) return DFI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
    if (dtype == DFI_DTYPE_F32) launch(scale_add_kernel<float>, blocks, 256, 0, st, (float*)a, (const float*)b, n, scale);
    else if (dtype == DFI_DTYPE_BF16) launch(scale_add_kernel<bf16>, blocks, 256, 0, st, (bf16*)a, (const bf16*)b, n, scale);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_scale_cap(float* x, long long n, float scale, float cap, void* stream) {
    if (n <= 0) return DFI_OK;
    const int blocks = (int)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
    launch(scale_cap_kernel, blocks, 256, 0, (cudaStream_t)stream, x, n, scale, cap);
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_gather_rows(const void* x, const int* rows_idx, void* out, int rows, int dim, int dtype,
                               void* stream) {
    if (rows <= 0) return DFI_OK;
    if (dim <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch_gather<float>(x, rows_idx, out, rows, dim, st);
    else if (dtype == DFI_DTYPE_BF16) launch_gather<bf16>(x, rows_idx, out, rows, dim, st);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

// delta == nullptr: out = rmsnorm(residual) * weight.  Otherwise residual += delta first (in place).
DFI_EXPORT int dfi_rmsnorm(void* residual, const void* delta, const float* weight, void* out, int rows, int dim,
                           float eps, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (dim <= 0) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch_rmsnorm<float>(residual, delta, weight, out, rows, dim, eps, st);
    else if (dtype == DFI_DTYPE_BF16) launch_rmsnorm<bf16>(residual, delta, weight, out, rows, dim, eps, st);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_swiglu(const void* gate_up, void* out, int rows, int inter, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (inter <= 0) return DFI_ERR_SHAPE;
    if (rows > 65535) return DFI_ERR_LIMIT;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == DFI_DTYPE_F32) launch_swiglu<float>(gate_up, out, rows, inter, st);
    else if (dtype == DFI_DTYPE_BF16) launch_swiglu<bf16>(gate_up, out, rows, inter, st);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}

DFI_EXPORT int dfi_qk_norm_rope_write(void* qkv, int rows, int row_stride, int n_q, int n_kv, int head_dim,
                                      const float* q_w, const float* k_w, float eps, const float* cos_t,
                                      const float* sin_t, int rotary_dim, const int* row_pos, const int* row_seq,
                                      void* k_cache, void* v_cache, const int* block_table, int table_width,
                                      int page_size, int ring_tokens, int write_cache, int dtype, void* stream) {
    if (rows <= 0) return DFI_OK;
    if (head_dim <= 0 || head_dim % 4 || head_dim > 64 * kMaxPairsPerLane) return DFI_ERR_SHAPE;
    if (row_stride % 2) return DFI_ERR_ALIGN;
    if (n_q < 0 || n_kv < 0 || page_size <= 0 || table_width <= 0) return DFI_ERR_SHAPE;
    if (cos_t != nullptr && (rotary_dim <= 0 || rotary_dim % 2 || rotary_dim > head_dim)) return DFI_ERR_SHAPE;
    cudaStream_t st = (cudaStream_t)stream;
    const int warps = 4;
    const int heads = n_q + 2 * n_kv;
    if (cos_t != nullptr && rotary_dim != head_dim) {
        // only part of each head rotates: the pairing differs from the kernels below
        dim3 grid(rows, (heads + kPartialWarps - 1) / kPartialWarps);
        if (grid.y > 65535) return DFI_ERR_LIMIT;
        if (dtype == DFI_DTYPE_F32)
            launch(qk_norm_rope_write_partial_kernel<float>, grid, kPartialWarps * 32, 0, st, (float*)qkv, row_stride, n_q,
                   n_kv, head_dim, rotary_dim, q_w, k_w, eps, cos_t, sin_t, row_pos, row_seq, (float*)k_cache,
                   (float*)v_cache, block_table, table_width, page_size, ring_tokens, write_cache);
        else if (dtype == DFI_DTYPE_BF16)
            launch(qk_norm_rope_write_partial_kernel<bf16>, grid, kPartialWarps * 32, 0, st, (bf16*)qkv, row_stride, n_q,
                   n_kv, head_dim, rotary_dim, q_w, k_w, eps, cos_t, sin_t, row_pos, row_seq, (bf16*)k_cache,
                   (bf16*)v_cache, block_table, table_width, page_size, ring_tokens, write_cache);
        else return DFI_ERR_DTYPE;
        DFI_CHECK_LAUNCH();
        return DFI_OK;
    }
    const bool wide = rows >= 64 && head_dim % 16 == 0 && head_dim <= 128 * kWideSteps && row_stride % 8 == 0 &&
                      aligned16(qkv) && aligned16(k_cache) && aligned16(v_cache) && aligned16(q_w) && aligned16(k_w) &&
                      aligned16(cos_t) && aligned16(sin_t);
    if (wide) {
        dim3 wide_grid(rows, (heads + 4 * warps - 1) / (4 * warps));
#define DFI_WIDE(TYPE, STEPS)                                                                                       \
    launch(qk_norm_rope_write_wide_kernel<TYPE, STEPS>, wide_grid, warps * 32, 0, st, (TYPE*)qkv, row_stride, n_q,       \
           n_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, row_pos, row_seq, (TYPE*)k_cache, (TYPE*)v_cache, block_table,  \
           table_width, page_size, ring_tokens, write_cache)
        if (dtype == DFI_DTYPE_F32) {
            if (head_dim <= 128) DFI_WIDE(float, 1); else DFI_WIDE(float, 2);
        } else if (dtype == DFI_DTYPE_BF16) {
            if (head_dim <= 128) DFI_WIDE(bf16, 1); else DFI_WIDE(bf16, 2);
        }
#undef DFI_WIDE
        else return DFI_ERR_DTYPE;
        DFI_CHECK_LAUNCH();
        return DFI_OK;
    }
    dim3 grid(rows, (heads + warps - 1) / warps);
    if (grid.y > 65535) return DFI_ERR_LIMIT;
    if (dtype == DFI_DTYPE_F32)
        launch(qk_norm_rope_write_kernel<float>, grid, warps * 32, 0, st, 
            (float*)qkv, row_stride, n_q, n_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, row_pos, row_seq,
            (float*)k_cache, (float*)v_cache, block_table, table_width, page_size, ring_tokens, write_cache);
    else if (dtype == DFI_DTYPE_BF16)
        launch(qk_norm_rope_write_kernel<bf16>, grid, warps * 32, 0, st, 
            (bf16*)qkv, row_stride, n_q, n_kv, head_dim, q_w, k_w, eps, cos_t, sin_t, row_pos, row_seq,
            (bf16*)k_cache, (bf16*)v_cache, block_table, table_width, page_size, ring_tokens, write_cache);
    else return DFI_ERR_DTYPE;
    DFI_CHECK_LAUNCH();
    return DFI_OK;
}
