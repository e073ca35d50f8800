"""Failure detection on the GPU in the one form that cannot hurt it: a wait that is allowed to run out.

Every wait inside the tensor-core kernels is bounded (about a second); a wait that runs out records a code in a status
word, the kernel ends normally, and the host is told at its next call into the library (RINGRNN_ERR_DEVICE) -- where the
reference would have printed and exited on the spot (cpp/cuda_common.cuh:30-39).  The self-test entry point runs the
same wait routine on a barrier nobody will ever complete, with a limit of a fraction of a millisecond.  Nothing here
faults, traps or spins without a bound, and the context stays usable (the last test runs the operator afterwards).
"""
import ctypes as C

import pytest
import torch

from rnn_train_ring_attractor_b200 import _lib

pytestmark = pytest.mark.gpu


def _drain():
    torch.cuda.synchronize()
    _lib.lib().ringrnn_device_status(None)


def test_a_wait_that_runs_out_sets_the_status_word_and_the_kernel_returns():
    L = _lib.lib()
    _drain()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.ringrnn_selftest_wait(200000, 4242, status.data_ptr(), None) == 0   # ~0.1 ms of cycles
    torch.cuda.synchronize()                                                     # returns: the kernel ended normally
    assert int(status[0]) == 4242
    code = C.c_int(0)
    assert L.ringrnn_device_status(C.byref(code)) == _lib.ERR_DEVICE and code.value == 4242
    assert L.ringrnn_device_status(C.byref(code)) == 0 and code.value == 0       # reading cleared the report


def test_the_next_operator_call_reports_the_earlier_failure():
    """No synchronisation on the reporting path: the status word reaches the host behind the kernel, and the next
    forward call -- through the Python surface -- raises RingRnnError(6) instead of launching."""
    from rnn_train_ring_attractor_b200.ring_rnn_cuda import ring_rnn_cuda_func
    L = _lib.lib()
    _drain()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert L.ringrnn_selftest_wait(200000, 77, status.data_ptr(), None) == 0
    torch.cuda.synchronize()
    g = torch.Generator().manual_seed(0)
    A = torch.rand(4, 3, 2, generator=g).cuda()
    Wa = (torch.randn(2, 16, 16, generator=g) * 0.1).cuda()
    Wo = (torch.randn(16, 16, generator=g) * 0.1).cuda()
    r0 = torch.rand(4, 16, generator=g).cuda()
    with pytest.raises(_lib.RingRnnError) as e:
        ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.1, "tanh")
    assert e.value.status == _lib.ERR_DEVICE and "77" in str(e.value)
    # reported once; the context is intact and the operator works
    out = ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.1, "tanh")
    torch.cuda.synchronize()
    assert torch.isfinite(out).all()
    _lib.raise_if_device_error()


def test_a_nonzero_status_word_makes_later_waits_give_up_at_once():
    """A caller-supplied status word that is not zero: every slow-path wait of kernels that share it is abandoned
    (documented in include/ringrnn.h); the wait self-test returns immediately and keeps the first code."""
    L = _lib.lib()
    _drain()
    status = torch.full((1,), 5, dtype=torch.int32, device="cuda")
    assert L.ringrnn_selftest_wait(4000000000, 9, status.data_ptr(), None) == 0  # would be ~2 s if it really waited
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    assert L.ringrnn_selftest_wait(4000000000, 9, status.data_ptr(), None) == 0
    e1.record()
    torch.cuda.synchronize()
    assert e0.elapsed_time(e1) < 100.0
    assert int(status[0]) == 5
    assert L.ringrnn_device_status(None) == _lib.ERR_DEVICE
    _drain()
