"""The benchmark configurations at their OWN horizon and weights, CUDA path vs the CPU oracle through the C ABI.

The sweep in test_gpu_parity.py covers shapes at short horizons; the cases here run the full number of steps of each
named configuration on a sub-batch the oracle finishes in seconds (every sample's recurrence is independent and the
weight gradients are sums over samples, so a sub-batch exercises exactly the per-sample arithmetic of the full batch):

  C2  N=256,  T=256,  relu, randn*0.01 weights            (B=32)
  C3  N=512,  T=512,  gelu, randn*0.01 weights            (B=128)
  C4  N=1024, T=2000, tanh, max_av=0.05*pi, keeping every step and with state checkpoints every 64 steps (B=16)
  C5  N=120,  T=4000, tanh, ideal cosine weights, forward rollout with per-step decode (B=64)

Tolerances: rel = ||x - ref||_F / ||ref||_F <= 1e-2 in bf16 mode, 1e-4 in fp32 mode, against the oracle evaluated in
double precision, plus the distance between the oracle's own fp32 and fp64 evaluations of the same quantity (what two
correct fp32 implementations may differ by).  What the configurations, as given, do to these quantities:
  * C2: with J0 = -0.1 and weights of size 0.01 the pre-activation is J0*sum(r) < 0 for every neuron at every step:
    relu never fires, the state decays as 0.9^t and every weight gradient is exactly zero -- in the oracle and here.
  * C3: the population-mean mode has loop gain alpha*J0*N*F' = -5.1*F' > 1 in magnitude: the oracle's fp32 and fp64
    histories part after about 30 steps (rel 7e-3 at t=31, 0.16 at t=63), and bf16 operand rounding, 2^15 times
    coarser, is amplified by the same dynamics that much sooner.  Compared: the first steps to the plain tolerance,
    every later step to a bound scaled by the oracle's own measured amplification while that bound says anything,
    the loss at the full horizon, and gradients at horizons 8/16/24.
  * C4: tanh saturates (J0*sum(r) ~ -20), F' = 1 - tanh^2 underflows and the weight gradients are rounding noise of
    the fp32 evaluation (oracle fp32 vs fp64: 0.4-0.6); history, decode and loss are well conditioned and compared
    tightly; long-horizon GRADIENT parity is pinned by the persistent-state cases at the end of this file.
Every comparison reports its achieved error (conftest.report_achieved), printed after the run.
"""
import math

import pytest
import torch

from oracle import ring_oracle as orc

pytestmark = pytest.mark.gpu

TOL = {"fp32": 1e-4, "bf16": 1e-2}


def _dev(*ts):
    return [t.cuda().contiguous() for t in ts]


_ORACLE_CACHE = {}


def _case_and_oracle(N, B, T, act, **kw):
    """make_case + _oracle, computed once per configuration (the N=1024, T=2000 oracle takes 20 s of CPU)."""
    key = (N, B, T, act, tuple(sorted(kw.items())))
    if key not in _ORACLE_CACHE:
        case = orc.make_case(N, B, T, act, seed=0, **kw)
        _ORACLE_CACHE[key] = (case, _oracle(case))
    return _ORACLE_CACHE[key]


def _oracle(case):
    """fp32 and fp64 evaluations of the oracle's training step + decode scalars of the fp64 one."""
    l32, dWo32, dWa32, h32 = orc.train_step_ref(case, lean=True)
    l64, dWo64, dWa64, h64 = orc.train_step_ref(case, lean=True, dtype=torch.float64)
    _, x, y, ta, _ = orc.fused_loss_terms(h64, case.target.double())
    _, x32, y32, ta32, _ = orc.fused_loss_terms(h32, case.target)
    noise = dict(loss=abs(float(l32) - float(l64)) / max(1.0, abs(float(l64))), dWo=orc.rel_err(dWo32, dWo64),
                 dWa=orc.rel_err(dWa32, dWa64), x=orc.rel_err(x32, x), y=orc.rel_err(y32, y), ta=orc.rel_err(ta32, ta),
                 final=orc.rel_err(h32[-1], h64[-1]))
    return dict(loss=float(l64), dWo=dWo64, dWa=dWa64, hist=h64, hist32=h32, x=x, y=y, ta=ta, noise=noise)


def _fused_step(case, prec, ckpt_every=0):
    """forward (decode scalars, no history) -> angle loss -> backward, all through the C ABI."""
    from gpu_helpers import angle_loss, run_backward, run_forward
    A, Wa, Wo, r0, tgt = _dev(case.A, case.Wa, case.Wo, case.r_init, case.target)
    B, T, _ = case.A.shape
    f = run_forward(A, Wa, Wo, r0, case.J0, case.J1, case.alpha, case.act, prec, history=False, decode=True,
                    ckpt_every=ckpt_every)
    coefs, decoded, parts = angle_loss(f["x"], f["y"], f["ta"], tgt, 0.2, 1.0 / (B * T))
    b = run_backward(A, Wa, Wo, r0, case.J0, case.J1, case.alpha, case.act, f, coefs=coefs, prec=prec,
                     ckpt_every=ckpt_every)
    return dict(x=f["x"], y=f["y"], ta=f["ta"], final=f["final"], decoded=decoded, loss=float(parts[0] + 0.2 * parts[1]),
                dWo=b["dWo"], dWa=b["dWa"], dJ=b["dJ"])


def _check_forward_side(got, ref, prec, achieved, label):
    tol, n = TOL[prec], ref["noise"]
    itol = tol if prec == "fp32" else 2 * tol  # per-(sample, step) intermediates of the loss
    e = dict(x=orc.rel_err(got["x"], ref["x"]), y=orc.rel_err(got["y"], ref["y"]), ta=orc.rel_err(got["ta"], ref["ta"]),
             final=orc.rel_err(got["final"], ref["hist"][-1]),
             loss=abs(got["loss"] - ref["loss"]) / max(1.0, abs(ref["loss"])))
    achieved(f"{label} {prec}", **e)
    assert e["x"] < itol + n["x"] and e["y"] < itol + n["y"] and e["ta"] < itol + n["ta"], (prec, e)
    assert e["final"] < tol + n["final"], (prec, e)
    assert e["loss"] < tol + n["loss"], (prec, e)
    return e


def _check_dj(got, ref, case, prec, achieved, label):
    """dJ0 = sum_ij G_ij and dJ1 = <G, Wo> with G = dWo / J1: relative to the oracle's value when the sum does not cancel
    (|sum| at least 1e-2 of the sum of magnitudes), else against the magnitude of the terms."""
    G = ref["dWo"] / case.J1
    want0, want1 = float(G.sum()), float((G * case.Wo.double()).sum())
    mag0, mag1 = float(G.abs().sum()), float((G * case.Wo.double()).abs().sum())
    e0, e1 = abs(float(got["dJ"][0]) - want0), abs(float(got["dJ"][1]) - want1)
    tol = TOL[prec] + ref["noise"]["dWo"]
    achieved(f"{label} {prec} dJ", dJ0_rel=e0 / max(abs(want0), 1e-30), dJ1_rel=e1 / max(abs(want1), 1e-30),
             cancel0=abs(want0) / max(mag0, 1e-30), cancel1=abs(want1) / max(mag1, 1e-30))
    for e, want, mag in ((e0, want0, mag0), (e1, want1, mag1)):
        if mag == 0.0:
            assert e == 0.0
        elif abs(want) >= 1e-2 * mag:
            assert e < tol * abs(want) * 3, (prec, e, want)  # three rounding sources: delta, the state, Wo in bf16
        else:
            assert e < tol * mag, (prec, e, want, mag)


@pytest.mark.parametrize("prec", ["bf16", "fp32"])
def test_config_c2_full_horizon(prec, achieved):
    """N=256, T=256, relu as configured (B=32 of the 1024)."""
    case, ref = _case_and_oracle(256, 32, 256, "relu")
    got = _fused_step(case, prec)
    _check_forward_side(got, ref, prec, achieved, "C2 N=256 T=256 relu")
    # relu never fires in this configuration: the oracle's gradients are exactly zero, and so must ours be
    assert float(ref["dWo"].abs().max()) == 0.0 and float(ref["dWa"].abs().max()) == 0.0
    assert float(got["dWo"].abs().max()) == 0.0 and float(got["dWa"].abs().max()) == 0.0
    dec = orc.decode_angle(ref["hist"]).float()
    err = float(orc.angular_error(got["decoded"].cpu(), dec).mean())
    achieved(f"C2 {prec} decoded angle", mean_abs_rad=err)
    assert err < 10 * TOL[prec]


# How far a rounding error of relative size eps grows along a trajectory is a property of the SYSTEM, which the oracle
# measures on itself: its fp32 evaluation (rounding 2^-24) ends up `noise` away from its fp64 evaluation.  The same
# dynamics amplify the bf16 operand rounding of the tensor-core mode (2^-9) by the same factor, so a comparison in a
# badly conditioned configuration is bounded by  tol + noise * (eps_mode / 2^-24)  and carries information only while
# that bound is small.
AMPLIFIED = {"fp32": 1.0, "bf16": 2.0 ** 15}


def test_config_c3_full_horizon(achieved):
    """N=512, T=512, gelu as configured (B=128 of the 4096): bf16 mode against the library's fp32 mode and the oracle.
    Per step, the history is held to tol + the oracle's own fp32-vs-fp64 distance at that step scaled to the mode's
    rounding, for as long as that bound stays below 0.5; the first 8 steps to the plain tolerance; the loss at the
    full horizon to the plain tolerance (it averages 65536 (sample, step) pairs and does not inherit the divergence of
    single trajectories)."""
    from gpu_helpers import angle_loss, run_forward
    N, B, T = 512, 128, 512
    case = orc.make_case(N, B, T, "gelu", seed=0)
    h32 = orc.ring_forward_lean(case.A, case.Wa, case.J0, case.J1, case.Wo, case.r_init, case.alpha, "gelu")
    h64 = orc.ring_forward_lean(case.A.double(), case.Wa.double(), case.J0, case.J1, case.Wo.double(),
                                case.r_init.double(), case.alpha, "gelu")
    noise = [orc.rel_err(h32[t], h64[t]) for t in range(T)]
    l32 = float(orc.training_loss_ref(h32, case.target))
    l64 = float(orc.training_loss_ref(h64, case.target.double()))
    A, Wa, Wo, r0, tgt = _dev(case.A, case.Wa, case.Wo, case.r_init, case.target)
    losses = {}
    for prec in ("bf16", "fp32"):
        tol = TOL[prec]
        f = run_forward(A, Wa, Wo, r0, case.J0, case.J1, case.alpha, "gelu", prec, history=True, decode=True, save=False)
        rel = [orc.rel_err(f["hist"][t], h64[t]) for t in range(T)]
        # (factor 4: two fp32 evaluations with different summation orders do not sit at the same distance from fp64)
        bound = [tol + 4 * noise[t] * AMPLIFIED[prec] for t in range(T)]
        informative = next((t for t in range(T) if bound[t] >= 0.5), T)   # steps before this one carry information
        crossed = next((t for t in range(T) if rel[t] >= tol), T)         # first step beyond the plain tolerance
        _, _, parts = angle_loss(f["x"], f["y"], f["ta"], tgt, 0.2, 1.0 / (B * T))
        losses[prec] = float(parts[0] + 0.2 * parts[1])
        e_loss = abs(losses[prec] - l64) / abs(l64)
        achieved(f"C3 N=512 T=512 gelu {prec}", hist_rel_first_8_steps=max(rel[:8]), steps_within_plain_tolerance=crossed,
                 steps_with_informative_bound=informative,
                 worst_ratio_to_bound=max(rel[t] / bound[t] for t in range(informative)),
                 oracle_fp32_vs_fp64_reaches_1e_3_at_step=next((t for t in range(T) if noise[t] >= 1e-3), T),
                 loss=losses[prec], loss_rel=e_loss, oracle_loss_fp32_vs_fp64=abs(l32 - l64) / abs(l64))
        assert max(rel[:8]) < tol, (prec, rel[:8])
        assert all(rel[t] < bound[t] for t in range(informative)), prec
        assert e_loss < tol + abs(l32 - l64) / abs(l64), (prec, losses[prec], l64)
    assert abs(losses["bf16"] - losses["fp32"]) / abs(losses["fp32"]) < TOL["bf16"]


@pytest.mark.parametrize("T", [8, 16, 24])
def test_config_c3_gradients_up_to_the_conditioning_horizon(T, achieved):
    """C3's weights, gelu, N=512: loss and weight gradients at growing horizons, in both modes, bounded as explained at
    AMPLIFIED (the oracle's fp32-vs-fp64 gradient distance is 6e-6 at T=8 and 2e-2 at T=32)."""
    case, ref = _case_and_oracle(512, 128, T, "gelu")
    for prec in ("bf16", "fp32"):
        got = _fused_step(case, prec)
        _check_forward_side(got, ref, prec, achieved, f"C3-weights T={T}")
        e = dict(dWo=orc.rel_err(got["dWo"], ref["dWo"]), dWa=orc.rel_err(got["dWa"], ref["dWa"]))
        bound = {k: TOL[prec] + ref["noise"][k] * AMPLIFIED[prec] for k in ("dWo", "dWa")}
        achieved(f"C3-weights T={T} {prec} gradients", oracle_noise_dWo=ref["noise"]["dWo"], bound_dWo=bound["dWo"], **e)
        assert e["dWo"] < bound["dWo"] and e["dWa"] < bound["dWa"], (prec, e, bound)
        if T == 8:  # arithmetic level: the plain tolerance, and the J gradients relatively
            assert e["dWo"] < TOL[prec] and e["dWa"] < TOL[prec], (prec, e)
            _check_dj(got, ref, case, prec, achieved, f"C3-weights T={T}")


@pytest.mark.parametrize("ckpt", [0, 64])
def test_config_c4_full_horizon(ckpt, achieved):
    """N=1024, T=2000, tanh, max_av = 0.05*pi as configured (B=16 of the 8192), keeping every step and with state
    checkpoints every 64 steps + recompute in backward -- both against the oracle."""
    case, ref = _case_and_oracle(1024, 16, 2000, "tanh", max_av=0.05 * math.pi)
    label = f"C4 N=1024 T=2000 tanh ckpt={ckpt}"
    got = _fused_step(case, "bf16", ckpt_every=ckpt)
    _check_forward_side(got, ref, "bf16", achieved, label)
    e = dict(dWo=orc.rel_err(got["dWo"], ref["dWo"]), dWa=orc.rel_err(got["dWa"], ref["dWa"]))
    achieved(label + " gradients", oracle_noise_dWo=ref["noise"]["dWo"], oracle_noise_dWa=ref["noise"]["dWa"],
             ref_norm_dWo=float(ref["dWo"].norm()), got_norm_dWo=float(got["dWo"].norm()), **e)
    # saturated tanh: the gradients are rounding noise of F' = 1 - tanh^2 (see the module docstring) and their size
    # (|dWo| ~ 0.2 beside a loss of 4487) is itself the result; the bound, a small multiple of the oracle's own
    # fp32-vs-fp64 distance, only excludes gross errors of sign or scale
    assert e["dWo"] < TOL["bf16"] + 2.5 * ref["noise"]["dWo"] and e["dWa"] < TOL["bf16"] + 2.5 * ref["noise"]["dWa"], e
    assert float(got["dWo"].norm()) < 4 * float(ref["dWo"].norm()) and torch.isfinite(got["dWo"]).all()
    if ckpt == 0:  # the fp32 mode on the same inputs (one CTA: slow, once is enough)
        got32 = _fused_step(case, "fp32")
        _check_forward_side(got32, ref, "fp32", achieved, label)


@pytest.mark.parametrize("prec", ["bf16", "fp32"])
def test_config_c5_rollout_full_horizon(prec, achieved):
    """N=120, T=4000, tanh, ideal cosine weights, forward only (B=64 of the 65536): decoded angle at every step and the
    final state against the oracle."""
    from gpu_helpers import run_forward
    N, B, T = 120, 64, 4000
    case = orc.make_case(N, B, T, "tanh", seed=0, weights="ideal")
    with torch.no_grad():
        h64 = orc.ring_forward_lean(case.A.double(), case.Wa.double(), case.J0, case.J1, case.Wo.double(),
                                    case.r_init.double(), case.alpha, "tanh")
        h32 = orc.ring_forward_lean(case.A, case.Wa, case.J0, case.J1, case.Wo, case.r_init, case.alpha, "tanh")
    dec64, dec32 = orc.decode_angle(h64), orc.decode_angle(h32)
    A, Wa, Wo, r0 = _dev(case.A, case.Wa, case.Wo, case.r_init)
    f = run_forward(A, Wa, Wo, r0, case.J0, case.J1, case.alpha, "tanh", prec, history=False, decode=True, save=False)
    dec = torch.remainder(torch.atan2(f["y"], f["x"]) + 2 * math.pi, 2 * math.pi).cpu()
    err = orc.angular_error(dec.double(), dec64)
    noise = orc.angular_error(dec32.double(), dec64)
    e_final = orc.rel_err(f["final"], h64[-1])
    # error against the integrated target: the ideal-weight model's own drift, the same in the oracle
    drift_ours = float(orc.angular_error(dec.double(), case.target.double()).mean())
    drift_ref = float(orc.angular_error(dec64, case.target.double()).mean())
    achieved(f"C5 N=120 T=4000 tanh ideal weights {prec}", decoded_mean_abs_rad=float(err.mean()),
             decoded_max_abs_rad=float(err.max()), oracle_fp32_vs_fp64_max_rad=float(noise.max()), final_state=e_final,
             error_vs_target_ours_rad=drift_ours, error_vs_target_oracle_rad=drift_ref)
    assert float(err.mean()) < TOL[prec] + float(noise.mean())
    assert float(err.max()) < 10 * TOL[prec] + float(noise.max())
    assert e_final < TOL[prec] + orc.rel_err(h32[-1], h64[-1])
    assert abs(drift_ours - drift_ref) < 10 * TOL[prec]


# Long horizons with a state that persists: the ideal cosine weights with tanh keep a saturated bump alive for the whole
# sequence (|r| -> 1), so every step's rounding of the bf16 operands enters the result.  The forward side (decode
# scalars, final state, loss) is held to the plain tolerance.  The gradients of this model are badly conditioned at these
# sizes -- J1*Wo has eigenvalue J1*N/2 >> 1 wherever tanh is not saturated -- and the oracle measures by how much: its
# own fp32 and fp64 gradients differ by 1e-5 (N=256, T=256), 1e-3 (N=512, T=512), 6e-2 (N=1024, T=2000), i.e. rounding at
# 2^-24 is amplified 1e2 .. 1e6 times.  They are bounded as explained at AMPLIFIED and asserted where that bound says
# something (< 0.5); elsewhere the achieved distance is reported.  (With the benchmark constants J0 = -0.1, J1 = 0.1
# there is no long-horizon regime with well-conditioned gradients at N >= 256: the state either dies out, saturates or
# is chaotic; the well-conditioned long case is the CPU-runnable configuration N=120, T=120 in test_gpu_parity.py.)
@pytest.mark.parametrize("cfg", [(256, 32, 256, 0.1, 0), (512, 32, 512, 0.1, 0), (1024, 16, 2000, 0.05, 0),
                                 (1024, 16, 2000, 0.05, 64)], ids=lambda c: "N%d-B%d-T%d-av%s-ckpt%d" % c)
def test_long_horizon_gradients_with_persistent_state(cfg, achieved):
    N, B, T, mav, ckpt = cfg
    case, ref = _case_and_oracle(N, B, T, "tanh", max_av=mav * math.pi, weights="ideal")
    label = f"ideal-weights tanh N={N} T={T} ckpt={ckpt}"
    for prec in (("bf16",) if (ckpt or N == 1024) else ("bf16", "fp32")):
        got = _fused_step(case, prec, ckpt_every=ckpt)
        _check_forward_side(got, ref, prec, achieved, label)
        e = dict(dWo=orc.rel_err(got["dWo"], ref["dWo"]), dWa=orc.rel_err(got["dWa"], ref["dWa"]))
        bound = {k: TOL[prec] + ref["noise"][k] * AMPLIFIED[prec] for k in ("dWo", "dWa")}
        achieved(f"{label} {prec} gradients", oracle_noise_dWo=ref["noise"]["dWo"], oracle_noise_dWa=ref["noise"]["dWa"],
                 bound_dWo=bound["dWo"], **e)
        assert torch.isfinite(got["dWo"]).all() and torch.isfinite(got["dWa"]).all()
        for k in ("dWo", "dWa"):
            if bound[k] < 0.5:
                assert e[k] < bound[k], (prec, k, e, bound)


# The reference's own J0 = -0.1 on the shapes of the sweep whose random cases scale it down (N > 128): short horizons,
# where the unstable population-mean mode has not yet amplified rounding differences.
@pytest.mark.parametrize("shape", [(256, 130, 4, 2, "gelu"), (512, 260, 4, 2, "gelu"), (384, 700, 3, 2, "tanh"),
                                   (1024, 130, 4, 2, "gelu"), (640, 300, 3, 2, "tanh"), (512, 4352, 3, 2, "tanh"),
                                   (512, 1030, 3, 16, "gelu"), (256, 1100, 3, 5, "silu"), (1152, 40, 3, 2, "gelu")],
                         ids=lambda s: "N%d-B%d-T%d-a%d-%s" % s)
def test_reference_j0_on_the_large_shapes(shape, achieved):
    from gpu_helpers import run_backward, run_forward
    from test_gpu_parity import _modes_for, random_case
    N, B, T, a_dim, act = shape
    A, Wa, Wo, r0, _, J1, alpha, act = random_case(N, B, T, a_dim, act, seed=N + B + T)
    J0 = -0.1
    h64 = orc.ring_forward_lean(A.double(), Wa.double(), J0, J1, Wo.double(), r0.double(), alpha, act)
    g = torch.Generator().manual_seed(99)
    cot = torch.randn(T, B, N, generator=g)
    ref = orc.ring_backward_manual(cot.double(), A.double(), Wa.double(), J0, J1, Wo.double(), h64, r0.double(), alpha, act)
    h32 = orc.ring_forward_lean(A, Wa, J0, J1, Wo, r0, alpha, act)
    ref32 = orc.ring_backward_manual(cot, A, Wa, J0, J1, Wo, h32, r0, alpha, act)
    noise = {k: orc.rel_err(ref32[k], ref[k]) for k in ("dWo", "dWa")}
    noise["hist"] = orc.rel_err(h32, h64)
    dA, dWa_, dWo_, dr0, dcot = _dev(A, Wa, Wo, r0, cot)
    for prec in _modes_for(N, B, T, a_dim, a_dim):
        tol = TOL[prec]
        f = run_forward(dA, dWa_, dWo_, dr0, J0, J1, alpha, act, prec, history=True)
        b = run_backward(dA, dWa_, dWo_, dr0, J0, J1, alpha, act, f, grad_output=dcot, prec=prec)
        e = dict(hist=orc.rel_err(f["hist"], h64), dWo=orc.rel_err(b["dWo"], ref["dWo"]), dWa=orc.rel_err(b["dWa"], ref["dWa"]))
        achieved("J0=-0.1 N%d-B%d-T%d-a%d-%s %s" % (shape + (prec,)), **e)
        # J0 = -0.1 at N >= 512 is the unstable regime (see AMPLIFIED): already after these few steps the oracle's fp32
        # evaluation is several times its usual 2e-7 away from fp64, and bf16 operand rounding grows alike
        amp = AMPLIFIED[prec]
        assert e["hist"] < tol + noise["hist"] * amp and e["dWo"] < tol + noise["dWo"] * amp and \
            e["dWa"] < tol + noise["dWa"] * amp, (prec, e, noise)
