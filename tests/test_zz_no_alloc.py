"""The entry point that allocates nothing (csrc/gemm_tc_noalloc.h), called through its
exported C symbol as a host application would call it, against the ordinary entry point
and against the product in 64-bit.

Some users of the library may not allocate device memory when they need a product:
the device belongs to a pool of their own, or their memory budget is fixed at start,
or a cudaMalloc would stall their other streams.  For them the K split's scratch
memory is a fixed array inside the library; this test checks that the results are
the ordinary ones, twice in a row (the array keeps what the first call left), that
the device's free memory is the same before and after (cudaMemGetInfo sees a
cudaMalloc that torch's own counters would miss), that a call may read as W what the
call before wrote, and that sizes beyond the array are refused in words.  It runs last so that a failure
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
    exact = x.double().cpu() @ w.double().cpu().t() + bias.double().cpu()
    tol = 1e-5 if out_dtype == torch.float32 else 5e-3
    scale = float(exact.abs().max())
    warm = torch.empty(T, N, dtype=out_dtype, device=DEV)
    assert call_noalloc(lib, fn, x, w, bias, warm)[0] == 0    # loads this tile width's kernel (the header says so)
    torch.cuda.synchronize()
    for attempt in (1, 2):
        out = torch.full((T, N), float("nan"), dtype=out_dtype, device=DEV)
        torch.cuda.synchronize()
        free_before, pool_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc, msg = call_noalloc(lib, fn, x, w, bias, out)
        assert rc == 0, msg
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before   # no cudaMalloc, by whomever
        assert torch.cuda.memory_allocated() == pool_before  # and nothing from torch's pool
        assert lib.gb_gemm_tc_noalloc_status() == 0
        assert torch.equal(out, want), f"call {attempt} differs from the ordinary entry point"
        err = float((out.double().cpu() - exact).abs().max())
        assert err <= tol * scale, f"call {attempt}: max error {err:.3e} against {scale:.3e}"


def test_no_alloc_call_may_read_what_the_call_before_wrote():
    """The output of one call as the W of the next on the same stream, at sizes where no tile is shared (nothing but
    the stream orders the two launches): the entry point launches the ordinary way, so the second call sees
    the first one's results."""
    lib, fn = entry_point()
    n_rows = 128 * 2 * lib.gb_sm_count()                      # one tile per resident CTA of the second call
    g = torch.Generator().manual_seed(3)
    x1 = torch.randn(n_rows, 64, generator=g).to(torch.bfloat16).to(DEV)
    w1 = (torch.randn(64, 64, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    x2 = torch.randn(8, 64, generator=g).to(torch.bfloat16).to(DEV)
    assert lib.gb_gemm_tc_scratch_floats(8, n_rows, 64, lib.gb_sm_count()) == 0
    for attempt in (1, 2):
        mid = torch.zeros(n_rows, 64, dtype=torch.bfloat16, device=DEV)
        out = torch.full((8, n_rows), float("nan"), dtype=torch.float32, device=DEV)
        assert call_noalloc(lib, fn, x1, w1, None, mid)[0] == 0
        assert call_noalloc(lib, fn, x2, mid, None, out)[0] == 0
        torch.cuda.synchronize()
        assert lib.gb_gemm_tc_noalloc_status() == 0
        exact = x2.double().cpu() @ mid.double().cpu().t()
        assert float(mid.float().abs().max()) > 0
        assert float((out.double().cpu() - exact).abs().max()) <= 1e-5 * float(exact.abs().max()), f"call {attempt}"


def test_no_alloc_entry_point_refuses_what_its_scratch_cannot_hold():
    lib, fn = entry_point()
    T, N, K = 128, 8192 + 128, 8192                          # 130 tiles shared by all resident CTAs: 2 partial tiles each
    assert lib.gb_gemm_tc_scratch_floats(T, N, K, lib.gb_sm_count()) > 2 * 1024 * 1024
    x = torch.zeros(T, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    out = torch.zeros(T, N, dtype=torch.bfloat16, device=DEV)
    rc, msg = call_noalloc(lib, fn, x, w, None, out)
    assert rc != 0 and "built-in scratch holds" in msg and "gb_gemm_tc" in msg
    rc, msg = call_noalloc(lib, fn, x[:, :100], w[:, :100], None, out)      # K = 100 is no multiple of 8
    assert rc != 0 and "multiples of 8" in msg
