"""Helpers shared by the GPU parity tests: direct C-ABI calls with canary-padded, NaN-poisoned buffers."""
import ctypes as C
import math

import torch

from rnn_train_ring_attractor_b200 import _lib
from rnn_train_ring_attractor_b200.fused import decode_vectors

CANARY = 12345.0
PAD = 64  # floats of canary on each side of every output


def padded(shape, device="cuda"):
    """A tensor surrounded by canary values; returns (view, backing)."""
    n = int(math.prod(shape))
    back = torch.full((n + 2 * PAD,), CANARY, device=device, dtype=torch.float32)
    back[PAD:PAD + n] = float("nan")
    return back[PAD:PAD + n].view(*shape), back


def canaries_intact(back):
    return bool((back[:PAD] == CANARY).all()) and bool((back[-PAD:] == CANARY).all())


def poisoned_bytes(nbytes, device="cuda"):
    """Scratch filled with 0xFF bytes (NaN as fp32 / bf16): a kernel that reads it uninitialised shows NaN."""
    return torch.full((max(int(nbytes), 16),), 255, dtype=torch.uint8, device=device)


def problem(A, Wa, Wo, r_init, J0, J1, alpha, act, prec, active=None, ckpt_every=0):
    B, T, a = A.shape
    return _lib.make_problem(B, T, Wa.shape[1], a, _lib.ACT[act], _lib.PREC[prec], J0, J1, alpha, A.data_ptr(),
                             Wa.data_ptr(), Wo.data_ptr(), r_init.data_ptr(), active, ckpt_every=ckpt_every)


def run_forward(A, Wa, Wo, r_init, J0, J1, alpha, act, prec="fp32", active=None, history=True, decode=False,
                save=True, ckpt_every=0):
    """Calls ringrnn_fwd through the C ABI.  Returns dict(hist, saved, dec(x,y,ta), final, backs)."""
    L = _lib.lib()
    B, T, a = A.shape
    N = Wa.shape[1]
    p = problem(A, Wa, Wo, r_init, J0, J1, alpha, act, prec, active, ckpt_every)
    out = {"backs": []}
    args = _lib.FwdArgs()
    args.p = p
    if history:
        out["hist"], back = padded((T, B, N))
        out["backs"].append(back)
        args.bump_history = out["hist"].data_ptr()
    ws = poisoned_bytes(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_FWD, int(history)))
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    if save:
        out["saved"] = poisoned_bytes(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_SAVED, int(history)))
        args.saved, args.saved_bytes = out["saved"].data_ptr(), out["saved"].numel()
    if decode:
        u, v = decode_vectors(N, A.device)
        out["u"], out["v"] = u, v
        for k in ("x", "y", "ta"):
            out[k], back = padded((B, T))
            out["backs"].append(back)
        args.dec_x, args.dec_y, args.dec_ta = out["x"].data_ptr(), out["y"].data_ptr(), out["ta"].data_ptr()
        args.dec_u, args.dec_v = u.data_ptr(), v.data_ptr()
    out["final"], back = padded((B, N))
    out["backs"].append(back)
    args.final_state = out["final"].data_ptr()
    _lib.check(L.ringrnn_fwd(C.byref(args), None))
    torch.cuda.synchronize()
    out["ws"] = ws
    if prec == "bf16":  # first word of the scratch: non-zero if a bounded device-side wait ran out
        assert int(ws[:4].view(torch.int32)[0]) == 0, "forward kernel reported an abandoned wait"
    return out


def run_backward(A, Wa, Wo, r_init, J0, J1, alpha, act, fwd, grad_output=None, coefs=None, prec="fp32",
                 active=None, ckpt_every=0):
    """Calls ringrnn_bwd through the C ABI.  `fwd` is run_forward's result.  Returns dict of gradients."""
    L = _lib.lib()
    B, T, a = A.shape
    N = Wa.shape[1]
    p = problem(A, Wa, Wo, r_init, J0, J1, alpha, act, prec, active, ckpt_every)
    args = _lib.BwdArgs()
    args.p = p
    out = {"backs": []}
    for name, shape in (("dWa", (a, N, N)), ("dWo", (N, N)), ("dJ", (2,)), ("dr_init", (B, N)), ("dA", (B, T, a))):
        out[name], back = padded(shape)
        out["backs"].append(back)
    args.grad_Wa, args.grad_Wo = out["dWa"].data_ptr(), out["dWo"].data_ptr()
    args.grad_J, args.grad_r_init = out["dJ"].data_ptr(), out["dr_init"].data_ptr()
    args.grad_A = out["dA"].data_ptr()
    if grad_output is not None:
        args.grad_output = grad_output.data_ptr()
    if coefs is not None:
        args.coef_x, args.coef_y, args.coef_s = (c.data_ptr() for c in coefs)
        args.dec_u, args.dec_v = fwd["u"].data_ptr(), fwd["v"].data_ptr()
    has_hist = "hist" in fwd
    if has_hist:
        args.bump_history = fwd["hist"].data_ptr()
    if "saved" in fwd:
        args.saved, args.saved_bytes = fwd["saved"].data_ptr(), fwd["saved"].numel()
    ws = poisoned_bytes(L.ringrnn_workspace_bytes(C.byref(p), _lib.WS_BWD, int(has_hist)))
    args.workspace, args.workspace_bytes = ws.data_ptr(), ws.numel()
    _lib.check(L.ringrnn_bwd(C.byref(args), None))
    torch.cuda.synchronize()
    if prec == "bf16":
        assert int(ws[:4].view(torch.int32)[0]) == 0, "backward kernel reported an abandoned wait"
    return out


def angle_loss(x, y, ta, target, bump_weight, inv_count):
    L = _lib.lib()
    B, T = x.shape
    coefs = [torch.full((B, T), float("nan"), device=x.device) for _ in range(3)]
    decoded = torch.empty(B, T, device=x.device)
    parts = torch.empty(2, device=x.device)
    scratch = torch.empty(2 * B, device=x.device)
    _lib.check(L.ringrnn_angle_loss(B, T, x.data_ptr(), y.data_ptr(), ta.data_ptr(), target.data_ptr(),
                                    bump_weight, inv_count, coefs[0].data_ptr(), coefs[1].data_ptr(),
                                    coefs[2].data_ptr(), decoded.data_ptr(), parts.data_ptr(), scratch.data_ptr(),
                                    None))
    torch.cuda.synchronize()
    return coefs, decoded, parts
