"""The reference's raw extension objects (cpp/rnn_cuda.py:59-91): `fwd_cuda.fwd(...)`, `bwd_cuda.bwd(...)`.

Keyword names follow the pybind definitions (cpp/fwd.cpp:49-55, cpp/bwd.cpp:101-123), because
legacy/bwd_fp32.py calls them directly.  Nothing is compiled at import; the calls go to libringrnn.so's
reference-signature entry points in fp32 mode.  The reference's scratch tensors and cuBLAS handle are
accepted and ignored.  Like the reference kernels, `bwd` accumulates into grad_Wa / grad_Wo, which the
caller zero-fills first (cpp/ring_rnn_cuda.py:98-99).
"""
import ctypes as C

import torch

from . import _lib
from .ring_rnn_cuda import _check_tensor, _scratch


def _problem(A, Wa, alpha, activation_type, J0, J1, Wo, r_init):
    B, T, a_dim = A.shape
    N = Wa.shape[1]
    return _lib.make_problem(B, T, N, a_dim, int(activation_type), _lib.PREC["fp32"], J0, J1, alpha,
                             A.data_ptr(), Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(), None)


class _Fwd:
    @staticmethod
    def fwd(A, Wa, J0, J1, Wo, r_init, bump_history, alpha, activation_type):
        for name, t in (("A", A), ("Wa", Wa), ("Wo", Wo), ("r_init", r_init), ("bump_history", bump_history)):
            _check_tensor(name, t)
        B, T, a_dim = A.shape
        N = Wa.shape[1]
        L = _lib.lib()
        with torch.cuda.device(A.device):
            p = _problem(A, Wa, alpha, activation_type, J0, J1, Wo, r_init)
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 1), A.device)
            _lib.check(L.ringrnn_fwd_cuda(A.data_ptr(), Wa.data_ptr(), float(J0), float(J1), Wo.data_ptr(),
                                          r_init.data_ptr(), bump_history.data_ptr(), float(alpha), N, a_dim, T, B,
                                          int(activation_type), _lib.PREC["fp32"], None, 0, ws.data_ptr(), ws.numel(),
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream)))


class _Bwd:
    @staticmethod
    def bwd(grad_output, A, Wa, J0, J1, Wo, bump_history, re_history, r_init, grad_Wa, grad_Wo, alpha,
            activation_type, grad_r=None, W_eff_temp=None, grad_re_temp=None, grad_W_eff_temp_bf16=None,
            A_t_temp_bf16=None, grad_re_temp_T=None, cublas_handle=None):
        for name, t in (("grad_output", grad_output), ("A", A), ("Wa", Wa), ("Wo", Wo), ("bump_history", bump_history),
                        ("r_init", r_init), ("grad_Wa", grad_Wa), ("grad_Wo", grad_Wo)):
            _check_tensor(name, t)
        B, T, a_dim = A.shape
        N = Wa.shape[1]
        L = _lib.lib()
        with torch.cuda.device(A.device):
            p = _problem(A, Wa, alpha, activation_type, J0, J1, Wo, r_init)
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_BWD, 1), A.device)
            gWa = torch.empty_like(grad_Wa)
            gWo = torch.empty_like(grad_Wo)
            _lib.check(L.ringrnn_bwd_cuda(grad_output.data_ptr(), A.data_ptr(), Wa.data_ptr(), float(J0), float(J1),
                                          Wo.data_ptr(), bump_history.data_ptr(), r_init.data_ptr(), gWa.data_ptr(),
                                          gWo.data_ptr(), float(alpha), N, a_dim, T, B, int(activation_type),
                                          _lib.PREC["fp32"], None, 0, ws.data_ptr(), ws.numel(),
                                          C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            grad_Wa.add_(gWa)
            grad_Wo.add_(gWo)


fwd_cuda = _Fwd()
bwd_cuda = _Bwd()
