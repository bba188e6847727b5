// dfi_skinny_gemm_static: the decode matrix product for callers that must not allocate.
//
// This entry point has no counterpart in the reference engine; it is an addition of this
// library.
//
// Who it is for.  Some programs that link this library cannot ask the CUDA runtime for
// memory at the moment they need a product: a host application that claimed the whole
// device for its own pool at start-up and forbids later driver allocations, a control
// loop that cannot afford the implicit device synchronisation that cudaMalloc and
// cudaFree may bring, or a plain C caller that has no tensor library and no allocator of
// its own to keep a workspace alive between calls.  The ordinary entry point
// (dfi_skinny_gemm) leaves the workspace to its caller; this one brings its own.
//
// How.  The workspace of the stream-K product (the partial sums of CTAs that share a row
// block, and the row blocks' arrival counters) lives in one array in the library's device
// image, fixed in size when the library is built.  Every GPU that loads the library holds
// that array (about 1.3 MB) until the process ends.  The caller passes inputs and the
// output exactly as to dfi_skinny_gemm; nothing is allocated or freed by the call, by the
// CUDA runtime or by any other library.
//
// Limits (beyond them the call returns DFI_ERR_LIMIT = 5 and launches nothing):
//     M <= DFI_STATIC_MAX_ROWS (8)        rows of activations
//     N <= DFI_STATIC_MAX_COLS (262144)   columns of the output (with swiglu: of each half of W)
// and as for dfi_skinny_gemm: K a multiple of 8, x and w 16-byte aligned, bfloat16 inputs.
//
// First call on a device.  The first call made while a given device is current looks up
// the array's device address (cudaGetSymbolAddress) and clears the counters with a
// cudaMemsetAsync on the caller's stream.  Make that first call during set-up, before any
// stream capture is begun on that stream.  Later calls on the device only launch.  Host
// threads that make their first calls at the same moment are taken one after the other
// (a lock around the set-up); the clearing is ordered before the first product only on the
// stream of the thread that did the set-up, so a second thread on another stream must
// order its first call after that one, as it must anyway (see Sharing).
//
// Sharing.  All calls on a device use the same array, and it keeps what the last call left
// in it.  The partial sums are overwritten before they are read; the counters are left at
// zero by every completed call, which is the state the next call needs.  Two calls that
// overlap on the GPU (different streams without an ordering between them) race on the
// array and give wrong results: order them on one stream or with events.
#pragma once

#define DFI_STATIC_MAX_ROWS 8
#define DFI_STATIC_MAX_COLS 262144

#ifdef __cplusplus
extern "C" {
#endif

// out[M, N] = x[M, K] . w[N, K]^T, or with swiglu != 0 and w = [gate; up] of 2N rows:
// out = silu(x . gate^T) * (x . up^T).  out_dtype: 0 float32, 1 bfloat16.  Returns 0 or a
// DFI_ERR_* code (see dfi_error_string).
int dfi_skinny_gemm_static(const void* x, const void* w, void* out, int M, int N, int K, int swiglu, int out_dtype,
                           void* stream);

// A short description of a DFI_ERR_* code.
const char* dfi_error_string(int code);

#ifdef __cplusplus
}
#endif
