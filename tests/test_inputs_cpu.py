"""The PRODUCT input generator (rnn_train_ring_attractor_b200/inputs.py) against the committed outputs of the
unmodified reference generator (tests/golden/ref_generator*.npz, made by tests/golden/make_golden.py from
utils/generate_av_integration_data.py:11-58) and of the reference's initial bump and action signal.  The oracle's own
copy is held to the same files in test_oracle.py; this file makes sure the copy that feeds the kernels cannot drift."""
import math
import os

import numpy as np
import pytest
import torch

from rnn_train_ring_attractor_b200 import inputs

GOLD = os.path.join(os.path.dirname(__file__), "golden")


def _gold(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k].item()) for k in z.files}


@pytest.mark.parametrize("name", ["ref_generator", "ref_generator_slow"])
def test_product_generator_matches_reference_bit_for_bit(name):
    g = _gold(name)
    torch.manual_seed(int(g["seed"]))
    av, angle = inputs.generate_av(int(g["B"]), int(g["T"]), max_av=float(g["max_av"]))
    assert torch.equal(av, g["av"])
    assert torch.equal(angle, g["angle"])


def test_product_initial_bump_and_action_signal_match_reference():
    g = _gold("ref_tanh_n24")
    assert torch.equal(inputs.initial_bump_gaussian(g["angle"][:, 0], 24), g["r_init"])
    assert torch.equal(inputs.av_to_action_signal(g["av"]), g["A"])


def test_generator_invariants():
    """What the reference generator guarantees by construction (utils/generate_av_integration_data.py:28-56): an exact
    count of non-zero steps per trial, zeros over the first 10 %, L*R == 0, and a target that lags by one step."""
    gen = torch.Generator().manual_seed(3)
    B, T, max_av = 64, 200, 0.1 * math.pi
    av, angle = inputs.generate_av(B, T, max_av=max_av, generator=gen)
    n0, rest = int(T * 0.1), T - int(T * 0.1)
    assert (av[:, :n0] == 0).all()
    allowed = {rest - int(rest * r) for r in (0.2, 0.5, 0.8)}
    assert set((av != 0).sum(dim=1).tolist()) <= allowed
    assert float(av.abs().max()) <= max_av
    A = inputs.av_to_action_signal(av, max_av)
    assert float((A[:, :, 0] * A[:, :, 1]).abs().max()) == 0.0 and float(A.max()) <= 1.0 + 1e-6
    want = (angle[:, :1] + torch.cumsum(av[:, :-1], dim=1)) % (2 * math.pi)
    d = (angle[:, 1:] - want).abs()
    assert float(torch.minimum(d, 2 * math.pi - d).max()) < 1e-4


def test_benchmark_inputs_follow_the_named_configuration():
    """Weights randn*0.01 drawn Wo, Wl, Wr from seed 0; J0 = -0.1, J1 = 0.1; von-Mises bump kappa = 4 over
    phi_i = 2*pi*i/N; the same weights as the oracle's make_case draws for the parity tests."""
    from oracle import ring_oracle as orc
    N, B, T = 40, 12, 30
    d = inputs.benchmark_inputs(N, B, T, seed=0)
    g = torch.Generator().manual_seed(0)
    Wo = torch.randn(N, N, generator=g) * 0.01
    Wl = torch.randn(N, N, generator=g) * 0.01
    Wr = torch.randn(N, N, generator=g) * 0.01
    assert torch.equal(d["Wo"], Wo) and torch.equal(d["Wa"][0], Wl) and torch.equal(d["Wa"][1], Wr)
    case = orc.make_case(N, B, T, "tanh", seed=0)
    assert torch.equal(case.Wo, Wo) and torch.equal(case.Wa[0], Wl) and torch.equal(case.Wa[1], Wr)
    assert d["J0"] == -0.1 and d["J1"] == 0.1
    phi = 2 * math.pi * torch.arange(N, dtype=torch.float32) / N
    assert torch.allclose(d["r_init"], torch.exp(4.0 * (torch.cos(phi[None] - d["target"][:, :1]) - 1.0)))
    ideal = inputs.benchmark_inputs(N, B, T, seed=0, weights="ideal")
    Wo_i, Wl_i, Wr_i = orc.ideal_weights(N)
    assert torch.equal(ideal["Wo"], Wo_i) and torch.equal(ideal["Wa"][0], Wl_i) and torch.equal(ideal["Wa"][1], Wr_i)
