// Shared helpers for the sm_100a kernels: element types, vector loads, reductions,
// and the convention of the C entry points.
//
// Every entry point is `extern "C" int dfi_<name>(..., void* stream)`.  It returns 0 or
// one of the DFI_ERR_* codes below and never throws, allocates or synchronises.  `dtype`
// arguments are 0 for float32 and 1 for bfloat16.  All arithmetic inside the kernels is
// float32; the storage type only decides how values are loaded and rounded on store.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define DFI_OK 0
#define DFI_ERR_DTYPE 1      // dtype code not 0 or 1
#define DFI_ERR_SHAPE 2      // a size the kernel does not take
#define DFI_ERR_ALIGN 3      // a pointer or stride that is not aligned as required
#define DFI_ERR_LAUNCH 4     // the launch itself failed (cudaGetLastError)
#define DFI_ERR_LIMIT 5      // a size beyond a stated maximum

#define DFI_DTYPE_F32 0
#define DFI_DTYPE_BF16 1

#define DFI_EXPORT extern "C" __attribute__((visibility("default")))

#define DFI_CHECK_LAUNCH()                                   \
    do {                                                     \
        if (cudaPeekAtLastError() != cudaSuccess) {          \
            cudaGetLastError();                              \
            return DFI_ERR_LAUNCH;                           \
        }                                                    \
    } while (0)

namespace dfi {

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

// Number of elements of T in one 16-byte vector.
template <typename T> struct Vec16 { static constexpr int n = 16 / sizeof(T); };

// Loads Vec16<T>::n consecutive elements (16-byte aligned) as floats.
__device__ __forceinline__ void load16(const float* p, float* out) {
    float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void load16(const bf16* p, float* out) {
    uint4 v = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(h[i]);
        out[2 * i] = f.x; out[2 * i + 1] = f.y;
    }
}
__device__ __forceinline__ void store16(float* p, const float* in) {
    *reinterpret_cast<float4*>(p) = make_float4(in[0], in[1], in[2], in[3]);
}
__device__ __forceinline__ void store16(bf16* p, const float* in) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(in[2 * i], in[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over the block; `scratch` holds at least 32 floats.  Every thread gets the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = (lane < n_warps) ? scratch[lane] : 0.f;
    return warp_sum(total);
}

// Programmatic dependent launch: a kernel launched through `launch` may begin while the kernel
// before it on the stream is still running; it must call pdl_wait() before it reads anything an
// earlier kernel wrote (or writes anything an earlier kernel reads), and may do work that depends
// on no earlier kernel (set-up, loading weights) before that.  pdl_launch_next() lets the kernel
// after this one begin.  Both are no-ops in a kernel that was launched the ordinary way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_next() { asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory"); }

inline int& pdl_enabled() {
    static int enabled = 1;
    return enabled;
}

template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attr;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

// Takes a ticket from a counter in global memory with acquire-release ordering at GPU scope.
__device__ __forceinline__ int ticket_add(int* counter) {
    int ticket;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;\n" : "=r"(ticket) : "l"(counter) : "memory");
    return ticket;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Place of position `p` in a sequence's storage: itself, or its place in the ring.
__device__ __forceinline__ int place_of(int p, int ring_tokens) { return ring_tokens > 0 ? p % ring_tokens : p; }

}  // namespace dfi
