"""The allocation-free loss entry point, ringrnn_angle_loss_static.

Some hosts cannot allocate device memory at the point where they need the loss -- their framework's pool owns
the whole GPU, or they sit in a loop that cannot take the device-wide stall of an allocation -- so this variant
keeps its per-sample scratch in an array inside the library.  It must give exactly what ringrnn_angle_loss
gives with caller scratch, on back-to-back calls that reuse the shared array with different batch sizes (the
array keeps the previous call's contents), and it must refuse batches beyond its fixed capacity.

Collected last on purpose (file name), so a run that stops at the first failure has already run the rest.
"""
import math

import pytest
import torch

from rnn_train_ring_attractor_b200 import _lib

pytestmark = pytest.mark.gpu

TOL = 1e-6  # both entry points run the same kernels; the fp32-mode bound of the other tests is 1e-4


def _inputs(B, T, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(B, T, device="cuda", generator=g)
    y = torch.randn(B, T, device="cuda", generator=g)
    ta = torch.rand(B, T, device="cuda", generator=g) * 10 + 1
    target = torch.rand(B, T, device="cuda", generator=g) * 2 * math.pi
    return x, y, ta, target


def _call(static, B, T, ins, poison):
    L = _lib.lib()
    x, y, ta, target = ins
    outs = [torch.full((B, T), float("nan"), device="cuda") for _ in range(4)]  # coef_x, coef_y, coef_s, decoded
    parts = torch.full((2,), float("nan"), device="cuda")
    args = [B, T, x.data_ptr(), y.data_ptr(), ta.data_ptr(), target.data_ptr(), 0.2, 1.0 / (B * T)]
    args += [o.data_ptr() for o in outs] + [parts.data_ptr()]
    if static:
        rc = L.ringrnn_angle_loss_static(*args, None)
    else:
        scratch = torch.full((2 * B,), poison, device="cuda")
        rc = L.ringrnn_angle_loss(*args, scratch.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0, L.ringrnn_strerror(rc)
    return outs + [parts]


def _close(a, b):
    return float((a.double() - b.double()).norm()) <= TOL * max(float(b.double().norm()), 1e-30)


def test_static_scratch_matches_caller_scratch_on_consecutive_calls():
    # a large batch first, then a smaller one: the second call runs over the leftovers of the first
    for B, T, seed in ((700, 33, 1), (96, 57, 2), (700, 33, 1)):
        ins = _inputs(B, T, seed)
        want = _call(False, B, T, ins, float("nan"))
        got = _call(True, B, T, ins, None)
        for g, w in zip(got, want):
            assert torch.isfinite(g).all()
            assert _close(g, w)


def test_static_scratch_at_its_capacity_and_without_allocating():
    """B == RINGRNN_STATIC_LOSS_MAX_B exactly (the last valid entries of the built-in array), compared with caller
    scratch; and the reason the entry point exists: with its outputs in place, a call takes no device memory -- neither
    from the driver (free bytes unchanged) nor from torch's pool."""
    L = _lib.lib()
    B, T = _lib.STATIC_LOSS_MAX_B, 2
    ins = _inputs(B, T, 3)
    want = _call(False, B, T, ins, float("nan"))
    got = _call(True, B, T, ins, None)  # also the first-call set-up, if this test runs alone
    for g, w in zip(got, want):
        assert torch.isfinite(g).all() and _close(g, w)
    # second call with preallocated outputs: nothing may be allocated
    x, y, ta, target = ins
    outs = [torch.empty(B, T, device="cuda") for _ in range(4)]
    parts = torch.empty(2, device="cuda")
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    alloc0, reserved0 = torch.cuda.memory_allocated(), torch.cuda.memory_reserved()
    rc = L.ringrnn_angle_loss_static(B, T, x.data_ptr(), y.data_ptr(), ta.data_ptr(), target.data_ptr(), 0.2,
                                     1.0 / (B * T), *[o.data_ptr() for o in outs], parts.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0, "the call changed the device's free memory"
    assert torch.cuda.memory_allocated() == alloc0 and torch.cuda.memory_reserved() == reserved0
    for g, w in zip(outs + [parts], want):
        assert _close(g, w)


def test_static_scratch_rejects_oversize_and_bad_arguments():
    L = _lib.lib()
    too_big = _lib.STATIC_LOSS_MAX_B + 1
    assert L.ringrnn_angle_loss_static(too_big, 4, 1, 1, 1, 1, 0.2, 1.0, 1, 1, 1, None, 1, None) == _lib.ERR_TOO_LARGE
    assert b"built-in scratch" in L.ringrnn_strerror(_lib.ERR_TOO_LARGE)
    assert L.ringrnn_angle_loss_static(0, 4, 1, 1, 1, 1, 0.2, 1.0, 1, 1, 1, None, 1, None) == 2
    assert L.ringrnn_angle_loss_static(8, 4, None, 1, 1, 1, 0.2, 1.0, 1, 1, 1, None, 1, None) == 1
