"""Failure detection on the GPU without a fault: every wait in the kernels is bounded; when a wait runs out the kernel
records a status code, returns normally, and the host raises from the status word.  The test makes a wait run out on
purpose (a barrier that nothing arrives at, limit 2e6 cycles = about a millisecond) and checks that chain; afterwards
the same context runs an ordinary forward."""
import pytest
import torch

from oracle import mx_oracle as O

pytestmark = pytest.mark.gpu


def test_expired_wait_reports_through_the_status_word_and_the_context_survives():
    import mpsa
    from mpsa import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    ops.check_status(dev)                                   # clean to begin with
    st = ops.status_word(dev)
    for code in (3, 1):
        _lib.check(lib.mpsa_selftest_wait_timeout(st.data_ptr(), 2_000_000, code, torch.cuda.current_stream().cuda_stream))
        with pytest.raises(_lib.MpsaError, match=f"status {code}"):
            ops.check_status(dev)
        assert int(st[0]) == 0                              # check_status cleared the word
    # argument checks of the entry itself
    assert lib.mpsa_selftest_wait_timeout(None, 1000, 3, None) == -1
    assert lib.mpsa_selftest_wait_timeout(st.data_ptr(), 0, 3, None) == -1
    assert lib.mpsa_selftest_wait_timeout(st.data_ptr(), 1000, 9, None) == -1
    # the context is intact: an ordinary forward runs and matches the oracle
    q, k, v = O.make_qkv(0, 1, 2, 2, 256, 128)
    out = mpsa.attention_forward(q.cuda(), k.cuda(), v.cuda(), causal=True, out_dtype=torch.float32, check=True)
    m = O.parity_metrics(out.cpu(), O.attention_mxfp(q, k, v, causal=True))
    assert m["cos"] >= 0.9999 and m["rel_l2"] <= 1e-2, m


def test_a_recorded_failure_surfaces_at_the_next_call_without_a_synchronisation():
    """The status word lives in pinned host memory and the wrappers look at it before they launch anything: once the
    kernel that gave up has finished, the next library call raises (and clears the word) instead of running on."""
    import mpsa
    from mpsa import _lib, ops
    lib = _lib.load()
    dev = torch.device("cuda", torch.cuda.current_device())
    st = ops.status_word(dev)
    assert not st.is_cuda and st.is_pinned()
    _lib.check(lib.mpsa_selftest_wait_timeout(st.data_ptr(), 1_000_000, 2, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()                                # the failing kernel has finished; nothing read the word yet
    q, k, v = (t.cuda() for t in O.make_qkv(1, 1, 2, 2, 128, 128))
    with pytest.raises(_lib.MpsaError, match="status 2"):
        mpsa.attention_forward(q, k, v, causal=True)        # raises before launching its forward
    mpsa.attention_forward(q, k, v, causal=True, check=True)
