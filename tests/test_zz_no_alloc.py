"""The allocation-free NVFP4 quantizer entry (mpsa_quant_nvfp4_static).

It exists for hosts that cannot hand the library a scratch buffer because they are not allowed to
allocate device memory where they call it (all memory given to their own pool at start-up, or no access
to the CUDA allocator on the request path): its scratch is an array inside the library's device image.
The test calls it through the C-ABI, twice in a row with different shapes (the second call finds the
first call's leftovers in the shared array), and demands bit-identical output to mpsa_quant_nvfp4.
This file sorts last on purpose, so that a run stopping at the first failure has run every other test."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _both(x):
    import mpsa
    from mpsa import _lib
    lib = _lib.load()
    rows, cols = x.shape
    dev = x.device
    ref_codes, ref_scales, ref_ts = mpsa.quantize_nvfp4(x)            # caller-provided scratch
    codes = torch.full_like(ref_codes, 0xAA)
    scales = torch.full_like(ref_scales, 0xAA)
    ts = torch.full((1,), -1.0, dtype=torch.float32, device=dev)
    before = torch.cuda.memory_allocated(dev)
    rc = lib.mpsa_quant_nvfp4_static(x.data_ptr(), {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[x.dtype],
                                     rows, cols, x.stride(0), 1.0, codes.data_ptr(), codes.stride(0),
                                     scales.data_ptr(), ts.data_ptr(), torch.cuda.current_stream().cuda_stream)
    _lib.check(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    return (codes, scales, ts), (ref_codes, ref_scales, ref_ts)


def test_static_scratch_entry_matches_the_allocating_one_twice_in_a_row():
    g = torch.Generator().manual_seed(77)
    # first call: many tiles, large values; second call: fewer tiles, small values - stale partial maxima of
    # the first call would inflate the second call's tensor scale if they were read
    for rows, cols, amp, dtype in ((1024, 2048, 50.0, torch.bfloat16), (200, 576, 0.01, torch.float16)):
        x = (torch.randn(rows, cols, generator=g) * amp).to(dtype).cuda()
        got, ref = _both(x)
        for a, b in zip(got, ref):
            assert torch.equal(a, b)


def test_static_scratch_entry_refuses_operands_beyond_its_limit():
    from mpsa import _lib
    lib = _lib.load()
    x = torch.zeros(16, 64, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(4096, dtype=torch.uint8, device="cuda")
    ts = torch.zeros(1, dtype=torch.float32, device="cuda")
    # 131072 x 16384 elements -> 1024 * 32 = 32768 partial maxima > 16384; refused before anything is launched
    rc = lib.mpsa_quant_nvfp4_static(x.data_ptr(), 0, 131072, 16384, 16384, 1.0, out.data_ptr(), 8192,
                                     out.data_ptr(), ts.data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    msg = _lib.last_error()
    assert "16384" in msg and "mpsa_quant_nvfp4" in msg
    with pytest.raises(ValueError):
        _lib.check(rc)
