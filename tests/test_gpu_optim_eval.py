"""Device-side optimizer step, training-state files and the angular-error evaluation, against PyTorch / the oracle."""
import math
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from oracle import ring_oracle as orc  # noqa: E402

pytestmark = pytest.mark.gpu


def _torch_reference_steps(p0, grads, lr, betas, eps, max_norm):
    """clip_grad_norm_ + Adam as the reference training loop applies them (train_general_ring_no_gain.py:335-336)."""
    p = torch.nn.Parameter(p0.clone().double())
    opt = torch.optim.Adam([p], lr=lr, betas=betas, eps=eps)
    norms = []
    for g in grads:
        p.grad = g.clone().double()
        norms.append(float(torch.nn.utils.clip_grad_norm_([p], max_norm)))
        opt.step()
    return p.detach(), norms


@pytest.mark.parametrize("n,max_norm", [(1000, 1.0), (3 * 120 * 120 + 2, 1.0), (70001, 0.0)])
def test_clip_adam_matches_torch(n, max_norm):
    from rnn_train_ring_attractor_b200.optim import FusedClipAdam
    g = torch.Generator().manual_seed(n)
    p0 = torch.randn(n, generator=g)
    grads = [torch.randn(n, generator=g) * s for s in (0.5, 3.0, 0.01, 1.0)]  # norms above and below the clip level
    ref_clip = max_norm if max_norm > 0 else 1e30
    ref, ref_norms = _torch_reference_steps(p0, grads, 1e-3, (0.9, 0.999), 1e-8, ref_clip)
    flat = p0.cuda()
    opt = FusedClipAdam(flat, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, max_norm=max_norm, train_J=True)  # every element
    for gi, rn in zip(grads, ref_norms):
        norm = opt.step(gi.cuda())
        assert abs(float(norm) - rn) < 1e-5 * rn
    assert orc.rel_err(flat, ref) < 1e-6
    assert float((flat.cpu().double() - ref).abs().max()) < 1e-6
    # the UPDATE itself (not hidden behind the size of the parameters): fp32 arithmetic against torch's double
    assert orc.rel_err(flat.cpu().double() - p0.double(), ref - p0.double()) < 1e-4


def test_clip_adam_leaves_j0_j1_alone_by_default():
    """In the reference J0 and J1 are plain floats (train_general_ring_no_gain.py:47-48): model.parameters() is
    {Wo, Wa}.  With the flat [Wo | Wa | J0 J1] buffer the default step must neither move the two trailing elements nor
    count their gradients in the clip norm."""
    from rnn_train_ring_attractor_b200.optim import FusedClipAdam
    n = 3 * 16 * 16 + 2
    g = torch.Generator().manual_seed(1)
    p0 = torch.randn(n, generator=g)
    grads = [torch.randn(n, generator=g) * s for s in (2.0, 0.1)]
    for gr in grads:
        gr[-2:] = 1e4  # dJ0 = sum_ij G_ij is large in practice: it must not shrink the Wo / Wa updates
    ref, ref_norms = _torch_reference_steps(p0[:-2], [gr[:-2] for gr in grads], 1e-3, (0.9, 0.999), 1e-8, 1.0)
    flat = p0.cuda()
    opt = FusedClipAdam(flat)
    for gi, rn in zip(grads, ref_norms):
        assert abs(float(opt.step(gi.cuda())) - rn) < 1e-5 * rn
    assert torch.equal(flat[-2:].cpu(), p0[-2:])
    assert orc.rel_err(flat[:-2].cpu().double() - p0[:-2].double(), ref - p0[:-2].double()) < 1e-4


def test_training_steps_follow_the_reference_loop():
    """K steps of fused forward + loss + backward (dp.train_step) + FusedClipAdam against the oracle's reference-shaped
    loop: autograd, clip_grad_norm_(1.0) and torch.optim.Adam on {Wo, Wa}, J0 / J1 fixed
    (train_general_ring_no_gain.py:312-336)."""
    from rnn_train_ring_attractor_b200 import dp
    from rnn_train_ring_attractor_b200.optim import FlatRingParams, FusedClipAdam
    N, B, T, K = 48, 24, 20, 4
    case = orc.make_case(N, B, T, "tanh", seed=2)
    Wo = case.Wo.clone().requires_grad_(True)
    Wa = case.Wa.clone().requires_grad_(True)
    opt_ref = torch.optim.Adam([Wo, Wa], lr=1e-3)
    ref_losses = []
    for _ in range(K):
        hist = orc.ring_forward_ref(case.A, Wa, case.J0, case.J1, Wo, case.r_init, case.alpha, case.act)
        loss = orc.training_loss_ref(hist, case.target)
        opt_ref.zero_grad()
        loss.backward()
        torch.nn.utils.clip_grad_norm_([Wo, Wa], 1.0)
        opt_ref.step()
        ref_losses.append(float(loss))
    params = FlatRingParams(case.Wo.cuda(), case.Wa.cuda(), case.J0, case.J1)
    opt = FusedClipAdam(params.flat)
    ins = tuple(t.cuda() for t in (case.A, case.r_init, case.target))
    buf = torch.empty(dp.grad_buffer_numel(N, 2), dtype=torch.float32, device="cuda")
    losses = []
    for _ in range(K):
        fn = dp.fused_step_fn(params.Wa, case.J0, case.J1, params.Wo, case.alpha, case.act, precision="fp32")
        loss, _ = dp.train_step(fn, ins, N, 2, B, T, buf=buf)
        opt.step(buf[:params.flat.numel()])
        losses.append(float(loss))
    for a, b in zip(losses, ref_losses):
        assert abs(a - b) < 1e-4 * max(1.0, abs(b)), (losses, ref_losses)
    assert orc.rel_err(params.Wo, Wo) < 1e-5 and orc.rel_err(params.Wa, Wa) < 1e-5
    # the update, not just the weights: K steps of lr 1e-3 move every weight by up to K * 1e-3
    assert orc.rel_err(params.Wo.cpu() - case.Wo, Wo.detach() - case.Wo) < 1e-3
    assert abs(float(params.J[0]) - case.J0) < 1e-7 and abs(float(params.J[1]) - case.J1) < 1e-7


def test_flat_params_views_and_state_roundtrip(tmp_path):
    from rnn_train_ring_attractor_b200.optim import (FlatRingParams, FusedClipAdam, load_training_state,
                                                     save_training_state)
    N, a = 24, 2
    g = torch.Generator().manual_seed(5)
    Wo, Wa = torch.randn(N, N, generator=g).cuda(), torch.randn(a, N, N, generator=g).cuda()
    params = FlatRingParams(Wo, Wa, -0.1, 0.1)
    assert torch.equal(params.Wo, Wo) and torch.equal(params.Wa, Wa)
    assert params.flat.numel() == (1 + a) * N * N + 2 and abs(float(params.J[0]) + 0.1) < 1e-7
    opt = FusedClipAdam(params.flat)
    grads = [torch.randn(params.flat.numel(), generator=g).cuda() for _ in range(3)]
    opt.step(grads[0])
    path = str(tmp_path / "state.pt")
    save_training_state(path, params, opt, step=1, extra={"loss": 0.5})
    opt.step(grads[1])
    opt.step(grads[2])
    expect = params.flat.clone()
    # resume from the file and replay the same two steps: identical bits
    params2 = FlatRingParams(torch.zeros_like(Wo), torch.zeros_like(Wa), 0.0, 0.0)
    opt2 = FusedClipAdam(params2.flat)
    step, extra = load_training_state(path, params2, opt2)
    assert step == 1 and extra["loss"] == 0.5
    opt2.step(grads[1])
    opt2.step(grads[2])
    assert torch.equal(params2.flat, expect)
    # views stay attached to the flat buffer: the operator sees the updated weights without a copy
    assert params2.Wo.data_ptr() == params2.flat.data_ptr()


def test_evaluation_matches_oracle_statistics():
    """The 200 x 500 evaluation of compare/compare_models_fair.py:120-175 on the fused forward (a smaller instance),
    against the oracle's forward + decode on the same trials."""
    from rnn_train_ring_attractor_b200.evaluate import angular_error, evaluate_angular_error
    from rnn_train_ring_attractor_b200.inputs import (av_to_action_signal, generate_av, ideal_weights,
                                                      initial_bump_gaussian)
    N, n_trials, T, batch, seed = 64, 24, 60, 8, 7
    Wo, Wl, Wr = ideal_weights(N)
    Wa = torch.stack([Wl, Wr]).contiguous()
    J0, J1, alpha, act, max_av = -0.1, 0.1, 0.1, "tanh", 0.1 * math.pi
    for prec, tol in (("fp32", 1e-4), ("bf16", 2e-2)):
        out = evaluate_angular_error(Wa.cuda(), J0, J1, Wo.cuda(), alpha, act, n_trials=n_trials, seq_len=T, batch=batch,
                                     seed=seed, max_av=max_av, precision=prec)
        g = torch.Generator().manual_seed(seed)
        errs = []
        for _ in range(n_trials // batch):
            av, angle = generate_av(batch, T, max_av=max_av, generator=g)
            A = av_to_action_signal(av, max_av)
            hist = orc.ring_forward_lean(A.double(), Wa.double(), J0, J1, Wo.double(),
                                         initial_bump_gaussian(angle[:, 0], N).double(), alpha, act)
            errs.append(angular_error(orc.decode_angle(hist).float(), angle))
        e = torch.cat(errs)
        assert out["errors"].shape == (n_trials, T)
        assert abs(out["mean"] - float(e.mean())) < tol
        assert abs(out["final_mean"] - float(e[:, -1].mean())) < 5 * tol
        assert abs(out["std"] - float(e.std())) < 5 * tol
