"""Trials generated on the device (ringrnn_generate_trials) against the properties and statistics of the reference's
host generator (utils/generate_av_integration_data.py:11-58; its output is pinned bit for bit by tests/golden and
test_inputs_cpu.py -- the device generator draws from another random stream, so it is held to the generator's
construction rules exactly and to its distribution statistically), and as the feed of the fused operator."""
import math

import pytest
import torch

from oracle import ring_oracle as orc

pytestmark = pytest.mark.gpu


def test_construction_rules_hold_exactly():
    from rnn_train_ring_attractor_b200.inputs import generate_on_device
    B, T, N, max_av = 4096, 200, 120, 0.1 * math.pi
    d = generate_on_device(B, T, N, seed=5, max_av=max_av, action_dim=16)
    A, target, r0 = d["A"].cpu(), d["target"].cpu(), d["r_init"].cpu()
    L, R = A[:, :, 0], A[:, :, 1]
    assert float((L * R).abs().max()) == 0.0                      # L * R == 0 always
    assert float(A[:, :, 2:].abs().max()) == 0.0                  # zero padding beyond the two columns
    assert float(A.min()) >= 0.0 and float(A.max()) <= 1.0        # divided by max_av
    av = (R - L) * max_av
    n0, rest = int(T * 0.1), T - int(T * 0.1)
    assert float(av[:, :n0].abs().max()) == 0.0                   # the first 10 % of steps are zero
    counts = (av != 0).sum(dim=1)
    allowed = sorted(rest - int(rest * r) for r in (0.2, 0.5, 0.8))
    # an EXACT count of kept steps, one per ratio (a kept step whose drawn value is exactly 0.0 -- probability 2^-24 per
    # draw, in the reference's generator too -- shows as one fewer non-zero step: tolerated for a handful of trials)
    assert set(allowed) <= set(counts.tolist())
    off = [c for c in counts.tolist() if c not in allowed]
    assert len(off) <= 3 and all(c + 1 in allowed for c in off), off
    # the target lags by one step and integrates the velocity
    theta0 = target[:, 0]
    assert float(theta0.min()) >= 0.0 and float(theta0.max()) < 2 * math.pi
    want = (theta0[:, None].double() + torch.cumsum(av[:, :-1].double(), dim=1)) % (2 * math.pi)
    assert float(orc.angular_error(target[:, 1:].double(), want).max()) < 2e-4
    # initial bump of the benchmark configurations
    assert torch.allclose(r0, orc.initial_bump_von_mises(theta0, N), atol=2e-6)
    g = generate_on_device(64, T, 48, seed=5, bump="gaussian", scale=1.0)
    assert torch.allclose(g["r_init"].cpu(), orc.initial_bump_gaussian(g["target"][:, 0].cpu(), 48), atol=2e-6)
    assert abs(float(g["A"].max()) - max_av) < 0.02 * max_av      # scale 1: the reference script's un-normalised L / R


def test_distribution_matches_the_host_generator():
    from rnn_train_ring_attractor_b200.inputs import generate_av, generate_on_device
    B, T, max_av = 20000, 100, 0.1 * math.pi
    d = generate_on_device(B, T, 16, seed=11, max_av=max_av)
    av = ((d["A"][:, :, 1] - d["A"][:, :, 0]) * max_av).cpu()
    ref_av, ref_angle = generate_av(B, T, max_av=max_av, generator=torch.Generator().manual_seed(11))
    n0 = int(T * 0.1)
    # each zero-ratio is drawn for a third of the trials
    for x in (av, ref_av):
        frac = torch.bincount((x != 0).sum(dim=1), minlength=T + 1).float() / B
        assert all(abs(float(f) - 1 / 3) < 0.02 for f in frac[frac > 0])
    # non-zero values are U(-max_av, max_av): moments against the host generator's and the exact ones
    nz, ref_nz = av[av != 0], ref_av[ref_av != 0]
    assert abs(float(nz.mean())) < 0.01 * max_av and abs(float(nz.abs().mean()) - max_av / 2) < 0.01 * max_av
    assert abs(float(nz.var()) - max_av ** 2 / 3) < 0.02 * max_av ** 2 / 3
    assert abs(float(nz.var()) - float(ref_nz.var())) < 0.03 * float(ref_nz.var())
    # the non-zero positions are uniform over the steps after the zero start: per-step occupancy is flat
    occ, ref_occ = (av[:, n0:] != 0).float().mean(dim=0), (ref_av[:, n0:] != 0).float().mean(dim=0)
    assert float((occ - occ.mean()).abs().max()) < 0.02 and abs(float(occ.mean()) - float(ref_occ.mean())) < 0.01
    # theta0 is uniform on [0, 2pi)
    th = d["target"][:, 0].cpu()
    assert abs(float(th.mean()) - math.pi) < 0.05 and abs(float(th.var()) - (2 * math.pi) ** 2 / 12) < 0.1


def test_trials_do_not_depend_on_the_batch_they_are_generated_in():
    from rnn_train_ring_attractor_b200.inputs import generate_on_device
    full = generate_on_device(64, 50, 24, seed=3)
    part = generate_on_device(16, 50, 24, seed=3, first_trial=32)   # rows 32..47 of the same global batch
    for k in ("A", "target", "r_init"):
        assert torch.equal(part[k], full[k][32:48])
    other = generate_on_device(64, 50, 24, seed=4)
    assert not torch.equal(other["A"], full["A"])


def test_device_generated_trials_feed_the_fused_operator():
    """One fused training step on device-generated inputs against the oracle on the same tensors."""
    from rnn_train_ring_attractor_b200.fused import ring_rnn_fused
    from rnn_train_ring_attractor_b200.inputs import benchmark_inputs, generate_on_device
    N, B, T = 64, 96, 30
    d = generate_on_device(B, T, N, seed=9)
    w = benchmark_inputs(N, 1, 2, seed=0)
    Wa = w["Wa"].cuda().requires_grad_(True)
    Wo = w["Wo"].cuda().requires_grad_(True)
    loss, _, _, _ = ring_rnn_fused(d["A"], Wa, -0.1, 0.1, Wo, d["r_init"], 0.1, "tanh", d["target"], precision="fp32")
    loss.backward()
    case = orc.RingCase(A=d["A"].cpu(), Wa=w["Wa"], Wo=w["Wo"], r_init=d["r_init"].cpu(), target=d["target"].cpu(),
                        J0=-0.1, J1=0.1, alpha=0.1, act="tanh")
    ref_loss, ref_dWo, ref_dWa, _ = orc.train_step_ref(case, lean=True)
    assert abs(float(loss) - float(ref_loss)) < 1e-4 * max(1.0, abs(float(ref_loss)))
    assert orc.rel_err(Wo.grad, ref_dWo) < 1e-4 and orc.rel_err(Wa.grad, ref_dWa) < 1e-4
