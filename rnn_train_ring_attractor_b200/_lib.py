"""ctypes binding of libringrnn.so (the declarations of include/ringrnn.h).

The library is loaded on first use, so importing the package works on a host without a GPU; any
attempt to run the operator without the built library raises -- there is no CPU or eager fallback.
"""
import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libringrnn.so")

MAX_ACTIVE = 64
ACT = {"relu": 0, "gelu": 1, "tanh": 2, "silu": 3}  # cpp/ring_rnn_cuda.py:63
PREC = {"fp32": 0, "bf16": 1}
WS_FWD, WS_SAVED, WS_BWD = 0, 1, 2
ERR_UNSUPPORTED = 5
ERR_DEVICE = 6
ERR_TOO_LARGE = 7
STATIC_LOSS_MAX_B = 65536

c_float_p = C.c_void_p


class Problem(C.Structure):
    _fields_ = [("B", C.c_int), ("T", C.c_int), ("N", C.c_int), ("a_dim", C.c_int),
                ("activation", C.c_int), ("precision", C.c_int),
                ("J0", C.c_float), ("J1", C.c_float), ("alpha", C.c_float),
                ("A", C.c_void_p), ("Wa", C.c_void_p), ("Wo", C.c_void_p), ("r_init", C.c_void_p),
                ("n_active", C.c_int), ("active_cols", C.c_int * MAX_ACTIVE), ("ckpt_every", C.c_int)]


class FwdArgs(C.Structure):
    _fields_ = [("p", Problem), ("bump_history", C.c_void_p), ("saved", C.c_void_p), ("saved_bytes", C.c_size_t),
                ("dec_x", C.c_void_p), ("dec_y", C.c_void_p), ("dec_ta", C.c_void_p),
                ("dec_u", C.c_void_p), ("dec_v", C.c_void_p), ("final_state", C.c_void_p),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p)]


class BwdArgs(C.Structure):
    _fields_ = [("p", Problem), ("grad_output", C.c_void_p), ("coef_x", C.c_void_p), ("coef_y", C.c_void_p),
                ("coef_s", C.c_void_p), ("dec_u", C.c_void_p), ("dec_v", C.c_void_p),
                ("bump_history", C.c_void_p), ("saved", C.c_void_p), ("saved_bytes", C.c_size_t),
                ("grad_Wa", C.c_void_p), ("grad_Wo", C.c_void_p), ("grad_J", C.c_void_p),
                ("grad_r_init", C.c_void_p), ("grad_A", C.c_void_p), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_size_t), ("status", C.c_void_p)]


# every symbol include/ringrnn.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "ringrnn_version": (C.c_int, []),
    "ringrnn_strerror": (C.c_char_p, [C.c_int]),
    "ringrnn_last_cuda_error": (C.c_int, []),
    "ringrnn_last_cuda_error_string": (C.c_char_p, []),
    "ringrnn_workspace_bytes": (C.c_size_t, [C.POINTER(Problem), C.c_int, C.c_int]),
    "ringrnn_fwd": (C.c_int, [C.POINTER(FwdArgs), C.c_void_p]),
    "ringrnn_bwd": (C.c_int, [C.POINTER(BwdArgs), C.c_void_p]),
    "ringrnn_fwd_cuda": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p,
                                   C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "ringrnn_bwd_cuda": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int,
                                   C.c_int, C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]),
    "ringrnn_angle_loss": (C.c_int, [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                     C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                     C.c_void_p, C.c_void_p]),
    "ringrnn_angle_loss_static": (C.c_int, [C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_float, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                            C.c_void_p, C.c_void_p]),
    "ringrnn_generate_trials": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_ulonglong, C.c_longlong, C.c_float,
                                          C.c_float, C.c_float, C.POINTER(C.c_float), C.c_int, C.c_int, C.c_float,
                                          C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ringrnn_clip_adam": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_float, C.c_float,
                                    C.c_float, C.c_float, C.c_int, C.c_float, C.c_void_p, C.c_void_p]),
    "ringrnn_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "ringrnn_last_device_code": (C.c_int, []),
    "ringrnn_selftest_wait": (C.c_int, [C.c_longlong, C.c_int, C.c_void_p, C.c_void_p]),
    "ringrnn_launch_count": (C.c_longlong, []),
    "ringrnn_timing_slots": (C.c_int, []),
    "ringrnn_timing_name": (C.c_char_p, [C.c_int]),
    "ringrnn_timing_enable": (C.c_int, [C.c_int]),
    "ringrnn_timing_read": (C.c_int, [C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "ringrnn_timing_reset": (C.c_int, []),
    "ringrnn_selftest_gemm": (C.c_int, [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int,
                                        C.c_longlong, C.c_int, C.c_void_p, C.c_void_p]),
}

_lib = None


class RingRnnError(RuntimeError):
    def __init__(self, status, text):
        super().__init__(f"libringrnn status {status}: {text}")
        self.status = status


def lib():
    """The loaded library; raises if it has not been built (python -m rnn_train_ring_attractor_b200.build)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m rnn_train_ring_attractor_b200.build` "
                               "(there is no fallback path)")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status):
    if status != 0:
        L = lib()
        text = L.ringrnn_strerror(status).decode()
        if status == 4:
            text += ": " + L.ringrnn_last_cuda_error_string().decode()
        if status == ERR_DEVICE:
            text += (f" (kernel code {L.ringrnn_last_device_code()}): the results of the launches before this call are "
                     "invalid")
        raise RingRnnError(status, text)


def raise_if_device_error():
    """Raise RingRnnError(6) if a bf16-mode launch whose status word has reached the host abandoned a bounded wait.
    Never synchronises: call it right after a synchronisation of your own (the read-back of a loss, say) to cover
    everything launched before it.  The library makes the same check on entry to every forward / backward call."""
    check(lib().ringrnn_device_status(None))


def make_problem(B, T, N, a_dim, act, prec, J0, J1, alpha, A, Wa, Wo, r_init, active=None, ckpt_every=0):
    p = Problem()
    p.ckpt_every = int(ckpt_every)
    p.B, p.T, p.N, p.a_dim = B, T, N, a_dim
    p.activation, p.precision = act, prec
    p.J0, p.J1, p.alpha = float(J0), float(J1), float(alpha)
    p.A, p.Wa, p.Wo, p.r_init = A, Wa, Wo, r_init
    if active is None or len(active) > MAX_ACTIVE:
        # all columns (the list holds MAX_ACTIVE entries; beyond that only "all" can be expressed, fp32 mode only)
        if active is not None and len(active) != a_dim:
            raise ValueError(f"more than {MAX_ACTIVE} active action columns must be all {a_dim} of them")
        p.n_active = -1
    else:
        p.n_active = len(active)
        for k, c in enumerate(active):
            p.active_cols[k] = int(c)
    return p


def timing_snapshot():
    """{kernel class: (total ms, launches)} recorded since the last reset (synchronises the events)."""
    L = lib()
    out = {}
    for slot in range(L.ringrnn_timing_slots()):
        ms, n = C.c_float(0), C.c_int(0)
        check(L.ringrnn_timing_read(slot, C.byref(ms), C.byref(n)))
        out[L.ringrnn_timing_name(slot).decode()] = (ms.value, n.value)
    return out


CHECK_DEVICE_STATUS = os.environ.get("RINGRNN_CHECK", "0") == "1"


def check_device_status(workspace, what):
    """With RINGRNN_CHECK=1: synchronise and raise at once if a bf16-mode kernel abandoned a bounded wait (the first
    word of its scratch buffer is the status word).  Without it the failure is reported by the NEXT library call or
    by raise_if_device_error(), with no synchronisation (the status word travels to the host behind the kernels)."""
    if not CHECK_DEVICE_STATUS:
        return
    import torch
    torch.cuda.synchronize()
    code = int(workspace[:4].view(torch.int32)[0])
    if code != 0:
        raise RingRnnError(6, f"{what}: a bounded device-side wait ran out (code {code})")
