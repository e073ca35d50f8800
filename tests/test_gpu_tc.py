"""The tcgen05 / TMA building blocks of the bf16 mode, checked in isolation through the library self-test."""
import ctypes as C

import pytest
import torch

from rnn_train_ring_attractor_b200 import _lib

pytestmark = pytest.mark.gpu


def _run(mn_major, M, N, K, nsplit, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if mn_major:
        A = torch.randn(K, M, device="cuda", generator=g).bfloat16()
        B = torch.randn(K, N, device="cuda", generator=g).bfloat16()
        ref = A.float().t() @ B.float()
    else:
        A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
        B = torch.randn(N, K, device="cuda", generator=g).bfloat16()
        ref = A.float() @ B.float().t()
    partial = torch.full((nsplit, M, N), float("nan"), device="cuda")
    out = torch.full((M, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().ringrnn_selftest_gemm(mn_major, A.data_ptr(), B.data_ptr(), partial.data_ptr(), out.data_ptr(),
                                          M, N, K, nsplit, status.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0, _lib.lib().ringrnn_strerror(rc)
    assert int(status) == 0, f"device wait ran out, code {int(status)}"
    return out, ref


CASES = [(128, 128, 64, 1), (128, 256, 256, 1), (256, 512, 1000, 3), (384, 256, 4096, 5), (128, 128, 40, 1)]


@pytest.mark.parametrize("mn_major", [0, 1], ids=["k_major", "mn_major"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: "M%d-N%d-K%d-s%d" % c)
def test_tensor_core_gemm(mn_major, case):
    M, N, K, nsplit = case
    out, ref = _run(mn_major, M, N, K, nsplit)
    err = float((out - ref).norm() / ref.norm())
    if not err < 1e-5:
        bad = (out - ref).abs()
        idx = int(bad.flatten().argmax())
        print("worst", idx // N, idx % N, float(out.flatten()[idx]), float(ref.flatten()[idx]))
        print("rows with error", (bad.max(dim=1)[0] > 1e-2).nonzero().flatten()[:16].tolist())
        print("cols with error", (bad.max(dim=0)[0] > 1e-2).nonzero().flatten()[:16].tolist())
    assert err < 1e-5


PAIR_CASES = [(256, 128, 64), (256, 256, 512), (512, 224, 512), (1024, 448, 1000)]


@pytest.mark.parametrize("case", PAIR_CASES, ids=lambda c: "M%d-N%d-K%d" % c)
def test_tensor_core_gemm_cta_pair(case):
    """cta_group::2 building blocks: pair TMEM allocation, pair MMA, commit to both CTAs, TMA crediting the even CTA."""
    M, N, K = case
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.randn(M, K, device="cuda", generator=g).bfloat16()
    B = torch.randn(N, K, device="cuda", generator=g).bfloat16()
    ref = A.float() @ B.float().t()
    out = torch.full((M, N), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().ringrnn_selftest_gemm(2, A.data_ptr(), B.data_ptr(), out.data_ptr(), out.data_ptr(), M, N, K, 1,
                                          status.data_ptr(), None)
    torch.cuda.synchronize()
    assert rc == 0, _lib.lib().ringrnn_strerror(rc)
    assert int(status) == 0, f"device wait ran out, code {int(status)}"
    err = float((out - ref).norm() / ref.norm())
    if not err < 1e-5:
        bad = (out - ref).abs()
        print("rows with error", (bad.max(dim=1)[0] > 1e-2).nonzero().flatten()[:16].tolist())
        print("cols with error", (bad.max(dim=0)[0] > 1e-2).nonzero().flatten()[:16].tolist())
    assert err < 1e-5
