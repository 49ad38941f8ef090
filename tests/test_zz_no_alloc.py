"""The entry point that allocates nothing (csrc/gemm_tc_noalloc.h), called through its
exported C symbol as a host application would call it, against the ordinary entry point.

Some users of the library may not allocate device memory when they need a product:
the device belongs to a pool of their own, or their memory budget is fixed at start,
or a cudaMalloc would stall their other streams.  For them the K split's scratch
memory is a fixed array inside the library; this test checks that the results are
the ordinary ones, twice in a row (the array keeps what the first call left), and
that sizes beyond the array are refused in words.  It runs last so that a failure
here hides no other test's result, and passes alone in a fresh process as well.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def entry_point():
    from gguf_rs_cli_b200 import native
    lib = ctypes.CDLL(native.build(verbose=False))          # the shared library itself, by its exported symbols
    fn = lib.gb_gemm_tc_noalloc
    P, L, I = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn.argtypes = [P, L, P, L, P, I, P, I, L, I, I, I, P]
    fn.restype = I
    lib.gb_last_error.restype = ctypes.c_char_p
    lib.gb_gemm_tc_noalloc_status.restype = I
    lib.gb_gemm_tc_scratch_floats.restype = L
    lib.gb_gemm_tc_scratch_floats.argtypes = [I, I, I, I]
    return lib, fn


def call_noalloc(lib, fn, x, w, bias, out):
    T, K = x.shape
    N = w.shape[0]
    code = {torch.float32: 0, torch.bfloat16: 1}
    rc = fn(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None if bias is None else bias.data_ptr(),
            0 if bias is None else code[bias.dtype], out.data_ptr(), code[out.dtype], out.stride(0), T, N, K,
            torch.cuda.current_stream().cuda_stream)
    return rc, lib.gb_last_error().decode()


@pytest.mark.parametrize("T,N,K,out_dtype", [(8, 512, 4096, torch.float32),      # K split 16 ways: the scratch is used
                                             (1, 1024, 2048, torch.bfloat16),
                                             (40, 384, 1024, torch.bfloat16),
                                             (300, 2000, 328, torch.float32)])    # no split: the scratch stays idle
def test_no_alloc_entry_point_gives_the_ordinary_result_twice(T, N, K, out_dtype):
    from gguf_rs_cli_b200 import kernels
    lib, fn = entry_point()
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    want = torch.empty(T, N, dtype=out_dtype, device=DEV)
    kernels.gemm_tc(x, w, bias, want)                        # the existing entry point, with caller-allocated scratch
    tol = 1e-5 if out_dtype == torch.float32 else 5e-3
    scale = float(want.float().abs().max())
    for attempt in (1, 2):
        out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
        before = torch.cuda.memory_allocated()
        rc, msg = call_noalloc(lib, fn, x, w, bias, out)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before       # nothing was taken from torch's pool either
        assert lib.gb_gemm_tc_noalloc_status() == 0
        err = float((out.float() - want.float()).abs().max())
        assert err <= tol * scale, f"call {attempt}: max error {err:.3e} against {scale:.3e}"


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    lib, fn = entry_point()
    T, N, K = 128, 8192 + 128, 8192                          # 65 tiles x 2 splits x 128 x 128 floats > 2 Mi floats
    assert lib.gb_gemm_tc_scratch_floats(T, N, K, lib.gb_sm_count()) > 2 * 1024 * 1024
    x = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
    rc, msg = call_noalloc(lib, fn, x, w, None, out)
    assert rc != 0 and "built-in scratch holds" in msg and "gb_gemm_tc" in msg
    rc, msg = call_noalloc(lib, fn, x[:, :100], w[:, :100], None, out)      # K = 100 is no multiple of 8
    assert rc != 0 and "multiples of 8" in msg
