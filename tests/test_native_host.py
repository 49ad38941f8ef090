"""Host-side arithmetic of the CUDA library that needs no device: how the tensor-core product cuts its work."""
from gguf_rs_cli_b200 import native


def test_product_cut_never_asks_for_more_than_the_scratch_holds_and_takes_no_tokens():
    lib = native.library()
    sms = 148
    capacity = 2 * sms * 256 * 128                      # what kernels.py allocates once
    assert lib.gb_gemm_tc_scratch_floats(0, 384, 96, sms) == 0 and lib.gb_gemm_tc_ctas(0, 384, 96, sms) == 1
    for T in (1, 7, 16, 17, 33, 64, 65, 128, 129, 300, 700, 2048):
        for N, K in ((8, 8), (384, 96), (1000, 320), (4096, 4096), (6144, 4096), (28672, 4096), (4096, 14336), (128256, 4096)):
            need, ctas = lib.gb_gemm_tc_scratch_floats(T, N, K, sms), lib.gb_gemm_tc_ctas(T, N, K, sms)
            assert 0 <= need <= capacity, (T, N, K, need)
            assert 1 <= ctas <= 2 * sms, (T, N, K, ctas)
    # a decode step of the 8B shape: the narrow products share their tiles, gate and up and the head do not
    assert lib.gb_gemm_tc_scratch_floats(8, 4096, 4096, sms) > 0 and lib.gb_gemm_tc_scratch_floats(8, 4096, 14336, sms) > 0
    assert lib.gb_gemm_tc_scratch_floats(8, 28672, 4096, sms) == 0 and lib.gb_gemm_tc_scratch_floats(8, 128256, 4096, sms) == 0


def test_the_ordinary_library_has_no_time_stamps():
    """Time stamps inside kernels belong to a second build (-DGB_STAMPS, bin/kernel_stamps); the library that
    serves refuses to be given a buffer for them."""
    import pytest
    assert not native.STAMPS
    for entry, args in (("gb_gemm_tc_set_stamps", (0, 0, 0)), ("gb_attention_decode_set_stamps", (0,))):
        with pytest.raises(native.NativeError, match="without -DGB_STAMPS"):
            native.call(entry, *args)
