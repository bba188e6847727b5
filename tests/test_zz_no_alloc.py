"""The allocation-free entry point of the decode matrix product, called as a C program would
call it: through its exported symbol, with raw pointers, with nothing but the inputs and the
output allocated by the caller.  Its results must be those of the ordinary entry point, on the
first call on the device and on the next one (which finds the shared workspace as the first left it).

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


@pytest.mark.parametrize("swiglu", [False, True])
def test_static_entry_point_matches_the_ordinary_one_twice_in_a_row(swiglu):
    from dryft_flash_infer_b200.ops import kernels

    lib = _library()
    g = torch.Generator().manual_seed(5)
    for m, n, k in ((8, 2560, 4096), (3, 200, 96), (1, 6144, 2560)):
        rows = 2 * n if swiglu else n
        x = torch.randn(m, k, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(rows, k, generator=g) * 0.05).to(torch.bfloat16).cuda()
        want = kernels.skinny_linear(x, w, torch.float32, swiglu=swiglu)
        for call in range(2):
            out = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            rc = _call(lib, x, w, out, swiglu)
            assert rc == 0, lib.dfi_error_string(rc).decode()
            torch.cuda.synchronize()
            assert torch.allclose(out, want, atol=2e-3, rtol=1e-3), (call, float((out - want).abs().max()))
        out16 = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        assert _call(lib, x, w, out16, swiglu) == 0
        assert torch.allclose(out16.float(), want, atol=2e-2, rtol=1e-2)


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
