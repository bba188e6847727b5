"""The allocation-free entry point of the decode matrix product, called as a C program would
call it: through its exported symbol, with raw pointers, with nothing but the inputs and the
output allocated by the caller.  Its results must be those of a plain float32 product, on the
first call on the device and on the next one (which finds the shared workspace as the first left it),
and also when calls follow each other on a stream without a wait between them.

Collected last on purpose: a run that stops at the first failure has then run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from dryft_flash_infer_b200.ops.build import CORE_SOURCES, compile_library

    lib = ctypes.CDLL(str(compile_library("dfi_core", CORE_SOURCES)))
    lib.dfi_skinny_gemm_static.restype = ctypes.c_int
    lib.dfi_skinny_gemm_static.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                           ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.dfi_error_string.restype = ctypes.c_char_p
    return lib


def _call(lib, x, w, out, swiglu):
    n = w.shape[0] // 2 if swiglu else w.shape[0]
    code = {torch.float32: 0, torch.bfloat16: 1}[out.dtype]
    return lib.dfi_skinny_gemm_static(x.data_ptr(), w.data_ptr(), out.data_ptr(), x.shape[0], n, x.shape[1],
                                      int(swiglu), code, torch.cuda.current_stream().cuda_stream)


def _float_product(x, w, swiglu):
    """What the entry point computes, in float32 by the library's plain product (nothing of this package)."""
    full = x.float() @ w.float().T
    if not swiglu:
        return full
    inter = w.shape[0] // 2
    return full[:, :inter] / (1 + torch.exp(-full[:, :inter])) * full[:, inter:]


@pytest.mark.parametrize("swiglu", [False, True])
def test_static_entry_point_matches_a_float_product_twice_in_a_row(swiglu):
    from dryft_flash_infer_b200.ops import kernels

    lib = _library()
    g = torch.Generator().manual_seed(5)
    for m, n, k in ((8, 2560, 4096), (3, 200, 96), (1, 6144, 2560)):
        rows = 2 * n if swiglu else n
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(rows, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
        want = _float_product(x, w, swiglu)
        for call in range(2):
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            rc = _call(lib, x, w, out, swiglu)
            assert rc == 0, lib.dfi_error_string(rc).decode()
            torch.cuda.synchronize()
            assert torch.allclose(out, want, atol=2e-3, rtol=1e-3), (call, float((out - want).abs().max()))
        # the ordinary entry point (the same kernel with a workspace of the caller's) gives the same numbers
        assert torch.allclose(kernels.skinny_linear(x, w, torch.float32, swiglu=swiglu), out, atol=2e-3, rtol=1e-3)
        out16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        assert _call(lib, x, w, out16, swiglu) == 0
        assert torch.allclose(out16.float(), want, atol=2e-2, rtol=1e-2)


def test_static_entry_point_called_back_to_back_without_waiting():
    """Calls of different shapes follow each other on one stream with nothing between them: each finds the
    shared workspace as the call before left it (its counters back at zero) while that call may still be
    finishing.  The last case fills the workspace to its edge: eight rows, every CTA with parts to add."""
    lib = _library()
    g = torch.Generator().manual_seed(6)
    cases = [(8, 2560, 4096, False), (1, 320, 200 * 8, True), (5, 9728, 2560, True), (8, 151936, 64, False),
             (2, 128, 8, False), (8, 19456 // 2, 2560, True), (8, 131072, 256, True)]
    held = []
    for m, n, k, swiglu in cases:
        rows = 2 * n if swiglu else n
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(rows, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
        held.append((x, w, swiglu, torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")))
    torch.cuda.synchronize()
    for _ in range(2):
        for x, w, swiglu, out in held:
            assert _call(lib, x, w, out, swiglu) == 0
    torch.cuda.synchronize()
    for x, w, swiglu, out in held:
        want = _float_product(x, w, swiglu)
        assert torch.allclose(out, want, atol=2e-3, rtol=1e-3), (tuple(x.shape), tuple(w.shape), swiglu,
                                                                  float((out - want).abs().max()))


def test_static_entry_point_refuses_what_its_workspace_cannot_hold():
    lib = _library()
    x = torch.zeros(9, 64, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(9, 64, dtype=torch.float32, device="cuda")
    rc = _call(lib, x, w, out, False)            # nine rows: one more than the workspace is built for
    assert rc == 5 and b"maximum" in lib.dfi_error_string(rc)
    rc = lib.dfi_skinny_gemm_static(x.data_ptr(), w.data_ptr(), out.data_ptr(), 8, 262145, 64, 0, 0,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 5
    torch.cuda.synchronize()
