"""Host-side checks that need no GPU: the C-ABI library loads, exports everything include/ringrnn.h
declares, validates arguments before touching CUDA, and sizes its buffers sanely."""
import ctypes as C
import os
import re

import pytest

from rnn_train_ring_attractor_b200 import _lib
from rnn_train_ring_attractor_b200.build import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    build()
    return _lib.lib()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ringrnn.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ringrnn_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_all_exported(L):
    names = declared_functions()
    assert "ringrnn_fwd" in names and "ringrnn_bwd" in names and len(names) >= 9
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/ringrnn.h but not exported"
    assert sorted(_lib.SYMBOLS) == names, "ctypes table and header disagree"


def test_version_and_strerror(L):
    assert L.ringrnn_version() >= 100
    assert L.ringrnn_strerror(0) == b"ok"
    for code in range(1, 8):
        assert len(L.ringrnn_strerror(code)) > 3
    assert L.ringrnn_strerror(99) == b"unknown status"


def _problem(**kw):
    d = dict(B=8, T=5, N=24, a_dim=2, act=2, prec=0, J0=-0.1, J1=0.1, alpha=0.1, A=1, Wa=1, Wo=1, r_init=1)
    d.update(kw)
    return _lib.make_problem(d["B"], d["T"], d["N"], d["a_dim"], d["act"], d["prec"], d["J0"], d["J1"], d["alpha"],
                             d["A"], d["Wa"], d["Wo"], d["r_init"], d.get("active"), d.get("ckpt_every", 0))


def test_argument_validation_returns_status_not_exit(L):
    assert L.ringrnn_fwd(None, None) == 1
    assert L.ringrnn_bwd(None, None) == 1
    a = _lib.FwdArgs()
    a.p = _problem(B=0)
    assert L.ringrnn_fwd(C.byref(a), None) == 2  # shape
    a.p = _problem(act=7)
    assert L.ringrnn_fwd(C.byref(a), None) == 1  # bad activation code
    a.p = _problem(A=None)
    assert L.ringrnn_fwd(C.byref(a), None) == 1  # null tensor
    a.p = _problem()
    assert L.ringrnn_fwd(C.byref(a), None) == 1  # nothing to produce
    a.bump_history = 1
    assert L.ringrnn_fwd(C.byref(a), None) == 3  # no workspace
    b = _lib.BwdArgs()
    b.p = _problem()
    assert L.ringrnn_bwd(C.byref(b), None) == 1  # no grad outputs
    b.grad_Wa, b.grad_Wo = 1, 1
    assert L.ringrnn_bwd(C.byref(b), None) == 1  # no cotangent source
    b.grad_output = 1
    b.bump_history = 1
    assert L.ringrnn_bwd(C.byref(b), None) == 3  # no workspace
    a.p = _problem(active=[0, 5])
    assert L.ringrnn_fwd(C.byref(a), None) == 1  # active column out of range
    assert L.ringrnn_angle_loss(0, 4, 1, 1, 1, 1, 0.2, 1.0, 1, 1, 1, None, 1, 1, None) == 2
    assert L.ringrnn_angle_loss(4, 4, None, 1, 1, 1, 0.2, 1.0, 1, 1, 1, None, 1, 1, None) == 1


def test_workspace_sizes(L):
    p = _problem(B=128, T=120, N=120)
    fwd = L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 1)
    assert fwd >= 3 * 120 * 120 * 4
    assert L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_SAVED, 1) == 0
    assert L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_SAVED, 0) >= 120 * 128 * 120 * 4
    bwd = L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_BWD, 1)
    assert bwd >= 120 * 128 * 120 * 4 + 3 * 120 * 120 * 4
    bad = _problem(N=-3)
    assert L.ringrnn_workspace_bytes(C.byref(bad), _lib.WS_FWD, 1) == C.c_size_t(-1).value
    assert L.ringrnn_workspace_bytes(None, _lib.WS_FWD, 1) == C.c_size_t(-1).value
    assert L.ringrnn_workspace_bytes(C.byref(p), 9, 1) == C.c_size_t(-1).value
    pa = _problem(a_dim=16, active=[0, 1])
    pf = _problem(a_dim=16)
    assert L.ringrnn_workspace_bytes(C.byref(pa), _lib.WS_FWD, 1) < L.ringrnn_workspace_bytes(C.byref(pf), _lib.WS_FWD, 1)


def test_bf16_mode_sizes_every_shape_and_checkpoints_shrink_the_saved_state(L):
    """bf16 mode takes any shape with up to 64 active action columns (persistent kernels or one GEMM per timestep);
    checkpoints replace the per-step saved tensors by T/K states."""
    unsupported = C.c_size_t(-1).value
    for N, a_dim, B in ((120, 2, 128), (512, 2, 4096), (1024, 2, 1024), (512, 16, 4096), (512, 16, 256),
                        (1024, 16, 256), (2048, 64, 256), (1100, 3, 40)):
        p = _problem(B=B, T=20, N=N, a_dim=a_dim, prec=1)
        sizes = [L.ringrnn_workspace_bytes(C.byref(p), w, 0) for w in (_lib.WS_FWD, _lib.WS_SAVED, _lib.WS_BWD)]
        assert all(0 < x != unsupported for x in sizes), (N, a_dim, B, sizes)
    too_wide = _problem(B=8, T=4, N=64, a_dim=80, prec=1)   # more than RINGRNN_MAX_ACTIVE columns
    assert L.ringrnn_workspace_bytes(C.byref(too_wide), _lib.WS_FWD, 0) == unsupported
    keep = _problem(B=1024, T=2000, N=1024, prec=1)
    ckpt = _problem(B=1024, T=2000, N=1024, prec=1, ckpt_every=64)
    s_keep = L.ringrnn_workspace_bytes(C.byref(keep), _lib.WS_SAVED, 0)
    s_ckpt = L.ringrnn_workspace_bytes(C.byref(ckpt), _lib.WS_SAVED, 0)
    assert s_keep >= 2 * 2000 * 1024 * 1024 * 2              # two bf16 tensors of T*B*N
    assert 32 * 1024 * 1024 * 4 <= s_ckpt < s_keep // 50     # ceil(2000/64) = 32 fp32 states of B*N
    w_keep = L.ringrnn_workspace_bytes(C.byref(keep), _lib.WS_BWD, 0)
    w_ckpt = L.ringrnn_workspace_bytes(C.byref(ckpt), _lib.WS_BWD, 0)
    assert w_ckpt < w_keep // 10                             # one stretch of 64 steps instead of all 2000
    bad = _problem(prec=1, ckpt_every=-1)
    assert L.ringrnn_workspace_bytes(C.byref(bad), _lib.WS_FWD, 0) == unsupported
    same = _problem(B=64, T=16, N=128, prec=1, ckpt_every=16)  # K >= T: nothing to checkpoint
    base = _problem(B=64, T=16, N=128, prec=1)
    assert L.ringrnn_workspace_bytes(C.byref(same), _lib.WS_SAVED, 0) == L.ringrnn_workspace_bytes(C.byref(base), _lib.WS_SAVED, 0)


def test_clip_adam_validates_arguments(L):
    assert L.ringrnn_clip_adam(None, 1, 1, 1, 10, 1e-3, 0.9, 0.999, 1e-8, 1, 1.0, 1, None) == 1
    assert L.ringrnn_clip_adam(1, 1, 1, 1, 10, 1e-3, 0.9, 0.999, 1e-8, 0, 1.0, 1, None) == 1   # steps count from 1
    assert L.ringrnn_clip_adam(1, 1, 1, 1, 0, 1e-3, 0.9, 0.999, 1e-8, 1, 1.0, 1, None) == 0    # nothing to do


def test_python_surface_mirrors_reference_names():
    import cpp.ring_rnn_cuda as m
    import cpp.rnn_cuda as r
    assert hasattr(m, "torch") and hasattr(m, "Function")  # leak through the star import, as the reference
    assert not hasattr(m, "__all__")
    assert callable(m.ring_rnn_cuda_func) and issubclass(m.RingRnnCudaFunc, m.Function)
    assert hasattr(r.fwd_cuda, "fwd") and hasattr(r.bwd_cuda, "bwd")
    import inspect
    sig = inspect.signature(m.ring_rnn_cuda_func)
    assert list(sig.parameters) == ["action_signal", "Wa", "J0", "J1", "Wo", "r_init", "alpha", "activation"]
    assert sig.parameters["activation"].default == "relu"


def test_operator_refuses_cpu_tensors_loudly():
    import torch
    import cpp.ring_rnn_cuda as m
    A = torch.zeros(2, 3, 2)
    Wa = torch.zeros(2, 4, 4)
    Wo = torch.zeros(4, 4)
    r0 = torch.zeros(2, 4)
    with pytest.raises(ValueError):
        m.ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.1, "swish")
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        m.ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.1, "tanh")


def test_documented_binding_matches_the_real_struct():
    """The integration guide prints the ctypes Problem structure a maintainer would paste into the reference: its field
    list must be the one the library is built with (a short structure hands check_problem garbage)."""
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    block = text[text.index("class Problem(C.Structure)"):]
    block = block[:block.index("def fwd(")]
    documented = re.findall(r'\("([A-Za-z0-9_]+)",\s*C\.', block)
    assert documented == [f[0] for f in _lib.Problem._fields_]
    # and the header declares the same members in the same order
    hdr = open(os.path.join(ROOT, "include", "ringrnn.h")).read()
    body = hdr[hdr.index("typedef struct RingRnnProblem {"):hdr.index("} RingRnnProblem;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    members = re.findall(r"([A-Za-z_][A-Za-z0-9_]*)\s*(?:\[[^\]]*\])?\s*[,;]", body.split("{", 1)[1])
    assert members == [f[0] for f in _lib.Problem._fields_], members


def test_more_than_64_action_columns_only_in_fp32_mode(L):
    """The reference's entry points take any a_dim (cpp/fwd.cu:21-50).  Here "all columns" (n_active < 0) with
    a_dim > RINGRNN_MAX_ACTIVE is a valid fp32-mode problem and an unsupported bf16-mode one."""
    p = _problem(a_dim=80, prec=0)
    assert p.n_active == -1
    assert L.ringrnn_workspace_bytes(C.byref(p), 0, 1) not in (0, C.c_size_t(-1).value)
    assert L.ringrnn_workspace_bytes(C.byref(p), 2, 1) != C.c_size_t(-1).value
    p16 = _problem(a_dim=80, prec=1)
    assert L.ringrnn_workspace_bytes(C.byref(p16), 0, 1) == C.c_size_t(-1).value
    a = _lib.FwdArgs()
    a.p = p16
    a.bump_history = 1
    assert L.ringrnn_fwd(C.byref(a), None) == _lib.ERR_UNSUPPORTED
    # an explicit list cannot name more than 64 columns; a longer list must be all of them
    q = _problem(a_dim=80, prec=0, active=list(range(80)))
    assert q.n_active == -1
    with pytest.raises(ValueError):
        _problem(a_dim=80, prec=0, active=list(range(70)))


def test_device_status_surface_without_a_gpu(L):
    """Nothing has been launched: no deferred failure to report, and reading the report is not an error."""
    code = C.c_int(123)
    assert L.ringrnn_device_status(C.byref(code)) == 0 and code.value == 0
    assert L.ringrnn_device_status(None) == 0
    assert L.ringrnn_selftest_wait(1000, 7, None, None) == 1      # no status word
    assert L.ringrnn_selftest_wait(-1, 7, 1, None) == 1           # negative limit
    assert L.ringrnn_selftest_wait(1000, 0, 1, None) == 1         # code 0 would be indistinguishable from success
    _lib.raise_if_device_error()


def test_generate_trials_validates_arguments(L):
    ratios = (C.c_float * 3)(0.2, 0.5, 0.8)
    ok = [8, 10, 16, 2, 1, 0, 0.3, 0.3, 0.1, ratios, 3, 0, 4.0, 1, 1, 1, 1, None]

    def call(**kw):
        a = list(ok)
        for i, v in kw.items():
            a[int(i[1:])] = v
        return L.ringrnn_generate_trials(*a)

    assert call(_0=0) == 2            # no trials
    assert call(_13=None) == 1        # A missing
    assert call(_10=9) == 1           # more zero-ratios than the library holds
    assert call(_6=0.0) == 1          # max_av must be positive
    assert call(_11=2) == 1           # unknown bump kind
    assert call(_16=None) == 1        # r_init without the theta0 scratch
    bad = (C.c_float * 3)(0.2, 1.5, 0.8)
    assert call(_9=bad) == 1          # a zero-ratio outside [0, 1]
