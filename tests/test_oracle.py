"""The oracle against outputs of the unmodified reference (tests/golden/*.npz)."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle import ring_oracle as orc

GOLD = os.path.join(os.path.dirname(__file__), "golden")
MODEL_CASES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLD, "ref_*_n*.npz")))


def load(name):
    z = np.load(os.path.join(GOLD, name + ".npz"))
    return {k: (torch.from_numpy(z[k]) if z[k].ndim else z[k].item()) for k in z.files}


def test_fixtures_present():
    assert len(MODEL_CASES) == 4


@pytest.mark.parametrize("name", MODEL_CASES)
def test_forward_matches_reference(name):
    g = load(name)
    hist = orc.ring_forward_ref(g["A"], g["Wa"], g["J0"], g["J1"], g["Wo"], g["r_init"], g["alpha"], g["act"])
    # same op sequence as the reference model on the same torch build: bit-equal
    assert torch.equal(hist.permute(1, 0, 2), g["bump"])
    lean = orc.ring_forward_lean(g["A"], g["Wa"], g["J0"], g["J1"], g["Wo"], g["r_init"], g["alpha"], g["act"])
    assert orc.rel_err(lean, hist) < 2e-6
    wave = orc.decode_normalised(hist.permute(1, 0, 2))
    assert torch.allclose(wave, g["wave"], rtol=0, atol=1e-6)


@pytest.mark.parametrize("name", MODEL_CASES)
def test_losses_and_autograd_match_reference(name):
    g = load(name)
    Wa = g["Wa"].clone().requires_grad_(True)
    Wo = g["Wo"].clone().requires_grad_(True)
    hist = orc.ring_forward_ref(g["A"], Wa, g["J0"], g["J1"], Wo, g["r_init"], g["alpha"], g["act"])
    bump = hist.permute(1, 0, 2)
    lc = orc.cosine_similarity_loss(orc.decode_normalised(bump), g["angle"])
    la = orc.bump_amplitude_loss(bump)
    assert abs(float(lc.detach()) - float(g["loss_cos"])) <= 1e-6 * max(1.0, abs(float(g["loss_cos"])))
    assert abs(float(la.detach()) - float(g["loss_amp"])) <= 1e-6 * max(1.0, abs(float(g["loss_amp"])))
    (lc + 0.2 * la).backward()
    assert orc.rel_err(Wo.grad, g["dWo"]) < 1e-5
    assert orc.rel_err(Wa.grad, g["dWa"]) < 1e-5


@pytest.mark.parametrize("name", MODEL_CASES)
def test_manual_bptt_matches_reference(name):
    g = load(name)
    hist = g["bump"].permute(1, 0, 2).contiguous()
    cot = g["cot"].permute(1, 0, 2).contiguous()
    out = orc.ring_backward_manual(cot.double(), g["A"].double(), g["Wa"].double(), g["J0"], g["J1"], g["Wo"].double(),
                                   hist.double(), g["r_init"].double(), g["alpha"], g["act"])
    assert orc.rel_err(out["dWo"], g["dWo_cot"]) < 2e-5
    assert orc.rel_err(out["dWa"], g["dWa_cot"]) < 2e-5


@pytest.mark.parametrize("act", orc.ACTIVATIONS)
def test_manual_bptt_matches_autograd_fp64(act):
    torch.manual_seed(11)
    B, T, N, a = 5, 7, 12, 3
    A = torch.rand(B, T, a, dtype=torch.float64, requires_grad=True)
    Wa = (torch.randn(a, N, N, dtype=torch.float64) / math.sqrt(N)).requires_grad_(True)
    Wo = (torch.randn(N, N, dtype=torch.float64) / math.sqrt(N)).requires_grad_(True)
    J0 = torch.tensor(-0.1, dtype=torch.float64, requires_grad=True)
    J1 = torch.tensor(0.1, dtype=torch.float64, requires_grad=True)
    r0 = torch.rand(B, N, dtype=torch.float64, requires_grad=True)
    hist = orc.ring_forward_ref(A, Wa, J0, J1, Wo, r0, 0.1, act)
    cot = torch.randn(T, B, N, dtype=torch.float64)
    (hist * cot).sum().backward()
    out = orc.ring_backward_manual(cot, A.detach(), Wa.detach(), float(J0), float(J1), Wo.detach(), hist.detach(),
                                   r0.detach(), 0.1, act)
    for key, ref in (("dWo", Wo.grad), ("dWa", Wa.grad), ("dJ0", J0.grad), ("dJ1", J1.grad), ("dA", A.grad),
                     ("dr_init", r0.grad)):
        assert orc.rel_err(out[key], ref) < 1e-12, key


@pytest.mark.parametrize("act", ["tanh", "gelu"])
def test_activation_grad_matches_autograd(act):
    x = torch.linspace(-4, 4, 101, dtype=torch.float64, requires_grad=True)
    orc.activation(x, act).sum().backward()
    assert torch.allclose(orc.activation_grad(x.detach(), act), x.grad, atol=1e-12)


@pytest.mark.parametrize("name", MODEL_CASES)
def test_fused_loss_terms_match_reference(name):
    g = load(name)
    hist = g["bump"].permute(1, 0, 2).contiguous().double().requires_grad_(True)
    angle = g["angle"].double()
    loss_ref = orc.training_loss_ref(hist, angle)
    loss_ref.backward()
    loss, x, y, ta, grad = orc.fused_loss_terms(hist.detach(), angle)
    assert abs(float(loss) - float(loss_ref)) < 1e-12
    assert abs(float(loss) - float(g["loss"])) < 1e-5 * max(1.0, abs(float(g["loss"])))
    assert orc.rel_err(grad, hist.grad) < 1e-10
    dec = orc.decode_angle(hist.detach())
    assert float(orc.angular_error(dec, g["decoded"].double()).max()) < 1e-5


@pytest.mark.parametrize("name", ["ref_generator", "ref_generator_slow"])
def test_generator_matches_reference(name):
    g = load(name)
    torch.manual_seed(int(g["seed"]))
    av, angle = orc.generate_av(int(g["B"]), int(g["T"]), max_av=float(g["max_av"]))
    assert torch.equal(av, g["av"])
    assert torch.equal(angle, g["angle"])


def test_initial_bump_and_action_signal_match_reference():
    g = load("ref_tanh_n24")
    assert torch.equal(orc.initial_bump_gaussian(g["angle"][:, 0], 24), g["r_init"])
    assert torch.equal(orc.av_to_action_signal(g["av"]), g["A"])


def test_make_case_is_deterministic_and_well_formed():
    c1 = orc.make_case(24, 6, 20, "tanh", seed=0)
    c2 = orc.make_case(24, 6, 20, "tanh", seed=0)
    assert torch.equal(c1.A, c2.A) and torch.equal(c1.Wo, c2.Wo)
    assert float((c1.A[:, :, 0] * c1.A[:, :, 1]).abs().max()) == 0.0  # L*R == 0
    assert float(c1.A.max()) <= 1.0 + 1e-6
    assert (c1.A[:, :2, :] == 0).all()  # first 10% of steps are zero
    loss, dWo, dWa, hist = orc.train_step_ref(c1)
    loss2, dWo2, dWa2, _ = orc.train_step_ref(c1, lean=True)
    assert abs(float(loss) - float(loss2)) < 1e-5
    assert orc.rel_err(dWo2, dWo) < 1e-4 and orc.rel_err(dWa2, dWa) < 1e-4


def test_ideal_weights_integrate_heading():
    # the reference's sanity check (train/train_ring_attractor.py:327-348) in spirit: ideal cosine
    # weights keep a bump alive; the decode follows it
    Wo, Wl, Wr = orc.ideal_weights(120)
    assert torch.allclose(Wo, Wo.t(), atol=1e-6)
    assert torch.allclose(Wl[:, :-1], Wo[:, 1:])
    assert torch.allclose(Wr[:, 1:], Wo[:, :-1])
