"""Loss-fused surface: forward + decode + loss + backward-through-time without a [T,B,N] fp32 tensor.

The reference's training step materialises bump_history[T,B,N], multiplies it by W_delta7, normalises by
the row maximum, and feeds two losses (train_general_ring_no_gain.py:101-116, :327-330).  Here the
forward kernel emits, per (sample, step), only x = r.u, y = r.v and ta = sum|r|
(u = W_delta7 cos(phi), v = W_delta7 sin(phi), phi = linspace(0, 2pi, N) as
train/train_ring_attractor.py:197); `ringrnn_angle_loss` turns them into the loss and the coefficients of
its closed-form gradient, and the reverse-time kernel injects that gradient.  What backward needs is kept
in the library's own saved-state buffer.
"""
import ctypes as C
import math

import torch
from torch.autograd import Function

from . import _lib
from .ring_rnn_cuda import _check_tensor, _scalar, _scratch, active_columns, choose_precision, nvtx_range

_decode_cache = {}


def decode_vectors(N, device):
    """u, v [N] fp32 on `device` (computed in float64 once per (N, device))."""
    key = (N, str(device))
    if key not in _decode_cache:
        idx = torch.arange(N, dtype=torch.float64)
        W = torch.cos(2 * math.pi * (idx[:, None] - idx[None, :]) / N)
        phi = torch.linspace(0, 2 * math.pi, N, dtype=torch.float64)
        u = (W @ torch.cos(phi)).float().to(device)
        v = (W @ torch.sin(phi)).float().to(device)
        _decode_cache[key] = (u, v)
    return _decode_cache[key]


class RingRnnFusedFunc(Function):
    """apply(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation, target_angle, bump_weight, inv_count,
    precision, grad_buffer, ckpt_every) -> (loss, loss_parts[2], decoded[B,T], final_state[B,N])"""

    @staticmethod
    def forward(ctx, action_signal, Wa, J0, J1, Wo, r_init, alpha, activation_name, target, bump_weight,
                inv_count, precision, grad_buffer, ckpt_every=0):
        B, T, a_dim = action_signal.shape
        N = Wa.shape[1]
        if activation_name not in _lib.ACT:
            raise ValueError(f"Invalid activation '{activation_name}'. Must be one of {list(_lib.ACT.keys())}.")
        act = _lib.ACT[activation_name]
        action_signal, Wa, Wo, r_init, target = (t.detach() for t in (action_signal, Wa, Wo, r_init, target))
        for name, t in (("A", action_signal), ("Wa", Wa), ("Wo", Wo), ("r_init", r_init), ("target_angle", target)):
            _check_tensor(name, t)
        if target.shape != (B, T):
            raise RuntimeError("target_angle must be (batch, seq_len)")
        dev = action_signal.device
        active = list(range(a_dim)) if ctx.needs_input_grad[0] else active_columns(action_signal)
        prec = choose_precision(B, T, N, a_dim, act, len(active), precision)
        if inv_count is None:
            inv_count = 1.0 / (B * T)
        u, v = decode_vectors(N, dev)
        L = _lib.lib()
        with torch.cuda.device(dev), nvtx_range("ringrnn_fused_fwd"):
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            p = _lib.make_problem(B, T, N, a_dim, act, prec, _scalar(J0), _scalar(J1), alpha,
                                  action_signal.data_ptr(), Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(), active,
                                  ckpt_every=ckpt_every)
            scal = torch.empty(6, B, T, device=dev, dtype=torch.float32)  # x, y, ta, coef_x, coef_y, coef_s
            decoded = torch.empty(B, T, device=dev, dtype=torch.float32)
            final_state = torch.empty(B, N, device=dev, dtype=torch.float32)
            parts = torch.empty(2, device=dev, dtype=torch.float32)
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 0), dev)
            saved = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_SAVED, 0), dev)
            a = _lib.FwdArgs()
            a.p = p
            a.saved, a.saved_bytes = saved.data_ptr(), saved.numel()
            a.dec_x, a.dec_y, a.dec_ta = scal[0].data_ptr(), scal[1].data_ptr(), scal[2].data_ptr()
            a.dec_u, a.dec_v = u.data_ptr(), v.data_ptr()
            a.final_state = final_state.data_ptr()
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            _lib.check(L.ringrnn_fwd(C.byref(a), stream))
            if prec == _lib.PREC["bf16"]:
                _lib.check_device_status(ws, "forward")
            red = torch.empty(2 * B, device=dev, dtype=torch.float32)
            _lib.check(L.ringrnn_angle_loss(B, T, scal[0].data_ptr(), scal[1].data_ptr(), scal[2].data_ptr(),
                                            target.data_ptr(), float(bump_weight), float(inv_count),
                                            scal[3].data_ptr(), scal[4].data_ptr(), scal[5].data_ptr(),
                                            decoded.data_ptr(), parts.data_ptr(), red.data_ptr(), stream))
            loss = parts[0] + bump_weight * parts[1]
        ctx.save_for_backward(action_signal, Wa, Wo, r_init, saved, scal, u, v)
        ctx.J0, ctx.J1, ctx.alpha, ctx.act, ctx.active, ctx.prec = J0, J1, alpha, act, active, prec
        ctx.grad_buffer = grad_buffer
        ctx.ckpt_every = ckpt_every
        ctx.mark_non_differentiable(parts, decoded, final_state)
        return loss, parts, decoded, final_state

    @staticmethod
    def backward(ctx, g_loss, _gp, _gd, _gf):
        action_signal, Wa, Wo, r_init, saved, scal, u, v = ctx.saved_tensors
        B, T, a_dim = action_signal.shape
        N = Wa.shape[1]
        dev = action_signal.device
        want_j = any(torch.is_tensor(j) and j.requires_grad for j in (ctx.J0, ctx.J1)) or ctx.grad_buffer is not None
        want_r = ctx.needs_input_grad[5]
        want_a = ctx.needs_input_grad[0]
        L = _lib.lib()
        with torch.cuda.device(dev), nvtx_range("ringrnn_fused_bwd"):
            p = _lib.make_problem(B, T, N, a_dim, ctx.act, ctx.prec, _scalar(ctx.J0), _scalar(ctx.J1), ctx.alpha,
                                  action_signal.data_ptr(), Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(),
                                  ctx.active, ckpt_every=ctx.ckpt_every)
            if ctx.grad_buffer is not None:
                # one contiguous buffer [Wo | Wa | dJ0 dJ1] so a data-parallel step all-reduces it in one call
                buf = ctx.grad_buffer
                grad_Wo = buf[:N * N].view(N, N)
                grad_Wa = buf[N * N:(1 + a_dim) * N * N].view(a_dim, N, N)
                grad_J = buf[(1 + a_dim) * N * N:(1 + a_dim) * N * N + 2]
            else:
                grad_Wa = torch.empty_like(Wa)
                grad_Wo = torch.empty_like(Wo)
                grad_J = torch.empty(2, device=dev, dtype=torch.float32) if want_j else None
            grad_r = torch.empty_like(r_init) if want_r else None
            grad_a = torch.empty_like(action_signal) if want_a else None
            ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_BWD, 0), dev)
            a = _lib.BwdArgs()
            a.p = p
            a.grad_A = None if grad_a is None else grad_a.data_ptr()
            a.coef_x, a.coef_y, a.coef_s = scal[3].data_ptr(), scal[4].data_ptr(), scal[5].data_ptr()
            a.dec_u, a.dec_v = u.data_ptr(), v.data_ptr()
            a.saved, a.saved_bytes = saved.data_ptr(), saved.numel()
            a.grad_Wa, a.grad_Wo = grad_Wa.data_ptr(), grad_Wo.data_ptr()
            a.grad_J = None if grad_J is None else grad_J.data_ptr()
            a.grad_r_init = None if grad_r is None else grad_r.data_ptr()
            a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
            _lib.check(L.ringrnn_bwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
            if ctx.prec == _lib.PREC["bf16"]:
                _lib.check_device_status(ws, "backward")
            if ctx.grad_buffer is not None:
                ctx.grad_buffer[:(1 + a_dim) * N * N + 2].mul_(g_loss)
            else:
                grad_Wa.mul_(g_loss)
                grad_Wo.mul_(g_loss)
                if grad_J is not None:
                    grad_J.mul_(g_loss)
            if grad_r is not None:
                grad_r.mul_(g_loss)
            if grad_a is not None:
                grad_a.mul_(g_loss)
        gJ0 = grad_J[0].reshape(ctx.J0.shape) if (torch.is_tensor(ctx.J0) and ctx.J0.requires_grad) else None
        gJ1 = grad_J[1].reshape(ctx.J1.shape) if (torch.is_tensor(ctx.J1) and ctx.J1.requires_grad) else None
        return (grad_a, grad_Wa, gJ0, gJ1, grad_Wo, grad_r, None, None, None, None, None, None, None, None)


def ring_rnn_fused(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation, target_angle, bump_weight=0.2,
                   inv_count=None, precision=None, grad_buffer=None, ckpt_every=0):
    """One fused training forward: returns (loss, loss_parts, decoded_angle[B,T], final_state[B,N]).

    loss = mean(2 - 2cos(decoded - target)) + bump_weight * mean((ta_t - ta_0)^2), the total of
    train_general_ring_no_gain.py:327-330.  `inv_count` (default 1/(B*T)) lets a data-parallel caller
    normalise by the global batch.  `grad_buffer`: optional flat fp32 tensor of (1+a)*N*N+2 elements that
    receives [dWo | dWa | dJ0 dJ1] contiguously during backward.  `ckpt_every` = K > 0 keeps only the fp32 state
    every K steps (the "state checkpoints every 64 steps and recompute in backward" of the long-sequence
    configuration): T/K states of B*N floats instead of two bf16 tensors of T*B*N, for one extra forward pass.
    """
    return RingRnnFusedFunc.apply(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation, target_angle,
                                  bump_weight, inv_count, precision, grad_buffer, ckpt_every)


def ring_rnn_rollout(action_signal, Wa, J0, J1, Wo, r_init, alpha, activation, precision=None):
    """Forward-only rollout: (decoded_angle[B,T] in [0,2pi), final_state[B,N]); no history, nothing saved."""
    B, T, a_dim = action_signal.shape
    N = Wa.shape[1]
    if activation not in _lib.ACT:
        raise ValueError(f"Invalid activation '{activation}'. Must be one of {list(_lib.ACT.keys())}.")
    act = _lib.ACT[activation]
    for name, t in (("A", action_signal), ("Wa", Wa), ("Wo", Wo), ("r_init", r_init)):
        _check_tensor(name, t)
    dev = action_signal.device
    active = active_columns(action_signal)
    prec = choose_precision(B, T, N, a_dim, act, len(active), precision)
    u, v = decode_vectors(N, dev)
    L = _lib.lib()
    with torch.cuda.device(dev), torch.no_grad(), nvtx_range("ringrnn_rollout"):
        p = _lib.make_problem(B, T, N, a_dim, act, prec, _scalar(J0), _scalar(J1), alpha, action_signal.data_ptr(),
                              Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(), active)
        xy = torch.empty(2, B, T, device=dev, dtype=torch.float32)
        final_state = torch.empty(B, N, device=dev, dtype=torch.float32)
        ws = _scratch(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, 0), dev)
        a = _lib.FwdArgs()
        a.p = p
        a.dec_x, a.dec_y = xy[0].data_ptr(), xy[1].data_ptr()
        a.dec_u, a.dec_v = u.data_ptr(), v.data_ptr()
        a.final_state = final_state.data_ptr()
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        _lib.check(L.ringrnn_fwd(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        decoded = torch.remainder(torch.atan2(xy[1], xy[0]) + 2 * math.pi, 2 * math.pi)
    return decoded, final_state
