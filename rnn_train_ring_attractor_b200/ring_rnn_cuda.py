"""The reference's operator surface (cpp/ring_rnn_cuda.py:18-144) on top of libringrnn.so.

Same names, argument order, return layout and error behaviour:
  ring_rnn_cuda_func(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation='relu') -> bump_history[T,B,N]
  RingRnnCudaFunc.forward(ctx, action_signal, Wa, J0, J1, Wo, r_init, alpha, activation_name)
  RingRnnCudaFunc.backward(ctx, grad_output) -> 8-tuple, gradients for Wa and Wo

`torch` and `Function` stay in this module's namespace on purpose: the reference's training script
obtains `torch` through `from cpp.ring_rnn_cuda import *` (train_general_ring_no_gain.py:1-19).

Extensions beyond the reference (all optional): J0 / J1 may be 0-dim tensors that require grad (their
gradients are then returned instead of None), and r_init and action_signal receive their gradients when they
require them (the reference returns None for all four, cpp/ring_rnn_cuda.py:144).  The action-signal gradient is
what the gain-network models (train/train_ring_attractor.py:131-146) need to train their gain MLPs through the op.
Arithmetic mode: `set_precision("bf16" | "fp32" | "auto")` or the RINGRNN_PRECISION environment variable;
"auto" takes the bf16 tensor-core path whenever it supports the shape, else the fp32 path, which is the
reference's own dispatch rule in spirit (cpp/fwd.cu:36).
"""
import contextlib
import ctypes as C
import os
import weakref

import torch
from torch.autograd import Function

from . import _lib


@contextlib.contextmanager
def nvtx_range(name):
    """NVTX range around a library call (the reference brackets its fwd/bwd the same way for its profiles,
    legacy/bwd_fp32.py:705-740); a no-op when torch has no CUDA runtime to push to."""
    pushed = False
    try:
        torch.cuda.nvtx.range_push(name)
        pushed = True
    except Exception:
        pass
    try:
        yield
    finally:
        if pushed:
            torch.cuda.nvtx.range_pop()

_precision = os.environ.get("RINGRNN_PRECISION", "auto")


def set_precision(mode):
    """Select the arithmetic mode of subsequent calls: "bf16", "fp32" or "auto"."""
    global _precision
    if mode not in ("bf16", "fp32", "auto"):
        raise ValueError("precision must be 'bf16', 'fp32' or 'auto'")
    _precision = mode


def get_precision():
    return _precision


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _scalar(x):
    return float(x.detach()) if torch.is_tensor(x) else float(x)


def _check_tensor(name, t):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (the operator has no CPU path)")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")  # TORCH_CHECK of cpp/fwd.cpp:31-35


_active_cache = {}  # id(tensor) -> (weakref, _version, columns)


def active_columns(action_signal):
    """Columns of A that are not identically zero.  The root training script pads [L, R] to 16 columns
    with zeros (train_general_ring_no_gain.py:200-223); their matrices cannot influence the result and
    their gradients are exactly zero, so both directions skip them.

    Finding them costs one small device->host read (a synchronisation), so the answer is remembered per tensor
    OBJECT and version counter: a signal that is passed again unchanged (evaluation loops, benchmarks) is not read
    twice, while a new tensor -- even one that reuses the freed memory of an old one -- or an in-place update is.
    More than MAX_ACTIVE non-zero columns: all columns are reported (only "all" can be expressed beyond the list)."""
    a_dim = action_signal.shape[2]
    if a_dim <= 2:
        return list(range(a_dim))
    key = id(action_signal)
    hit = _active_cache.get(key)
    if hit is not None and hit[0]() is action_signal and hit[1] == action_signal._version:
        return hit[2]
    flags = (action_signal != 0).flatten(0, 1).any(dim=0)
    cols = torch.nonzero(flags).flatten().tolist()
    if len(cols) > _lib.MAX_ACTIVE:
        cols = list(range(a_dim))
    try:
        ref = weakref.ref(action_signal, lambda _r, k=key: _active_cache.pop(k, None))
        _active_cache[key] = (ref, action_signal._version, cols)
    except TypeError:
        pass
    return cols


def choose_precision(B, T, N, a_dim, act_code, n_active, requested=None):
    """Resolve "auto": bf16 when libringrnn supports the shape in that mode, else fp32."""
    mode = requested or _precision
    if mode == "fp32":
        return _lib.PREC["fp32"]
    ok = n_active <= _lib.MAX_ACTIVE  # the tensor-core kernels take at most that many active columns
    if ok:
        p = _lib.Problem()
        p.B, p.T, p.N, p.a_dim, p.activation, p.precision = B, T, N, a_dim, act_code, _lib.PREC["bf16"]
        p.n_active = n_active
        for k in range(max(n_active, 0)):
            p.active_cols[k] = k
        ok = _lib.lib().ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 1) != C.c_size_t(-1).value
    if ok:
        return _lib.PREC["bf16"]
    if mode == "bf16":
        raise RuntimeError("bf16 mode does not support this shape "
                           f"(B={B}, T={T}, N={N}, active action columns={n_active})")
    return _lib.PREC["fp32"]


def _scratch(nbytes, device):
    return torch.empty(max(int(nbytes), 16), dtype=torch.uint8, device=device)


def ring_rnn_cuda_func(
        action_signal,
        Wa,
        J0,
        J1,
        Wo,
        r_init,
        alpha,
        activation='relu',
):
    """Ring RNN forward pass (same contract as the reference's function of this name).

    action_signal (B,T,a) ; Wa (a,N,N) ; J0, J1 scalars ; Wo (N,N) ; r_init (B,N) ; alpha float ;
    activation in {'relu','gelu','tanh','silu'}.  Returns bump_history (T,B,N).
    """
    return RingRnnCudaFunc.apply(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation)


class RingRnnCudaFunc(Function):
    @staticmethod
    def forward(ctx, action_signal, Wa, J0, J1, Wo, r_init, alpha, activation_name):
        batch_size, seq_len, a_dim = action_signal.shape
        N = Wa.shape[1]
        activation_map = _lib.ACT
        if activation_name not in activation_map:
            raise ValueError(f"Invalid activation '{activation_name}'. Must be one of {list(activation_map.keys())}.")
        act = activation_map[activation_name]
        action_signal, Wa, Wo, r_init = (action_signal.detach(), Wa.detach(), Wo.detach(), r_init.detach())
        for name, t in (("A", action_signal), ("Wa", Wa), ("Wo", Wo), ("r_init", r_init)):
            _check_tensor(name, t)
        if Wa.shape != (a_dim, N, N) or Wo.shape != (N, N) or r_init.shape != (batch_size, N):
            raise RuntimeError("shape mismatch between action_signal, Wa, Wo and r_init")
        dev = action_signal.device
        # zero columns may be skipped only if nobody asks for the gradient with respect to the action signal
        active = list(range(a_dim)) if ctx.needs_input_grad[0] else active_columns(action_signal)
        prec = choose_precision(batch_size, seq_len, N, a_dim, act, len(active))
        L = _lib.lib()
        with torch.cuda.device(dev), nvtx_range("ringrnn_fwd"):
            p = _lib.make_problem(batch_size, seq_len, N, a_dim, act, prec, _scalar(J0), _scalar(J1), alpha,
                                  action_signal.data_ptr(), Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(), active)
            bump_history = torch.empty(seq_len, batch_size, N, device=dev, dtype=action_signal.dtype)
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 1), dev)
            saved = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_SAVED, 1), dev)
            a = _lib.FwdArgs()
            a.p = p
            a.bump_history = bump_history.data_ptr()
            a.saved, a.saved_bytes = saved.data_ptr(), saved.numel()
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            _lib.check(L.ringrnn_fwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            if prec == _lib.PREC["bf16"]:
                _lib.check_device_status(ws, "forward")
        ctx.save_for_backward(action_signal, Wa, Wo, bump_history, r_init, saved)
        ctx.J0 = J0
        ctx.J1 = J1
        ctx.alpha = alpha
        ctx.activation_name = activation_name
        ctx.active = active
        ctx.prec = prec
        return bump_history

    @staticmethod
    def backward(ctx, grad_output):
        action_signal, Wa, Wo, bump_history, r_init, saved = ctx.saved_tensors
        batch_size, seq_len, a_dim = action_signal.shape
        N = Wa.shape[1]
        act = _lib.ACT[ctx.activation_name]
        dev = grad_output.device
        grad_output_ctg = grad_output.contiguous()  # arrives as a permuted view from the model's decode
        want_j = any(torch.is_tensor(j) and j.requires_grad for j in (ctx.J0, ctx.J1))
        want_r = ctx.needs_input_grad[5]
        want_a = ctx.needs_input_grad[0]
        L = _lib.lib()
        with torch.cuda.device(dev), nvtx_range("ringrnn_bwd"):
            p = _lib.make_problem(batch_size, seq_len, N, a_dim, act, ctx.prec, _scalar(ctx.J0), _scalar(ctx.J1),
                                  ctx.alpha, action_signal.data_ptr(), Wa.data_ptr(), Wo.data_ptr(),
                                  r_init.data_ptr(), ctx.active)
            grad_Wa = torch.empty_like(Wa)
            grad_Wo = torch.empty_like(Wo)
            grad_J = torch.empty(2, device=dev, dtype=torch.float32) if want_j else None
            grad_r = torch.empty_like(r_init) if want_r else None
            grad_a = torch.empty_like(action_signal) if want_a else None
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_BWD, 1), dev)
            a = _lib.BwdArgs()
            a.p = p
            a.grad_A = None if grad_a is None else grad_a.data_ptr()
            a.grad_output = grad_output_ctg.data_ptr()
            a.bump_history = bump_history.data_ptr()
            a.saved, a.saved_bytes = saved.data_ptr(), saved.numel()
            a.grad_Wa, a.grad_Wo = grad_Wa.data_ptr(), grad_Wo.data_ptr()
            a.grad_J = None if grad_J is None else grad_J.data_ptr()
            a.grad_r_init = None if grad_r is None else grad_r.data_ptr()
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            _lib.check(L.ringrnn_bwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            if ctx.prec == _lib.PREC["bf16"]:
                _lib.check_device_status(ws, "backward")
        gJ0 = grad_J[0].reshape(ctx.J0.shape) if (torch.is_tensor(ctx.J0) and ctx.J0.requires_grad) else None
        gJ1 = grad_J[1].reshape(ctx.J1.shape) if (torch.is_tensor(ctx.J1) and ctx.J1.requires_grad) else None
        return grad_a, grad_Wa, gJ0, gJ1, grad_Wo, grad_r, None, None
