"""Acceptance run: the reference's own root training script, UNCHANGED, on this library's operator.

train_general_ring_no_gain.py (the only script of the reference that calls the CUDA operator) is imported from a copy of
the reference with this repository in front of it on sys.path, so that its `from cpp.ring_rnn_cuda import *` (:19)
resolves to this repository's `cpp` package while `train.*` and `utils.*` stay the reference's.  Its model class
GeneralizedRingAttractorNoGain (:21-118: keyword call of ring_rnn_cuda_func at :101-111, alpha = 0.15, float J0 / J1,
the default 16 action columns of which 14 are zero padding, `.clone()`s, permute + W_delta7 + max-normalise) then runs
the body of the script's training loop (:312-336) for a few steps, and the loss trajectory is compared with the
reference's pure-PyTorch twin of the same model (train/train_general_ring_no_gain.py:21-137) on the CPU, step by step,
both models starting from the same weights and seeing the same batches.

Where the reference lives: $RINGRNN_REFERENCE_DIR, else baseline/_ref under the repository root (git-ignored; the build
step copies the reference's Python sources there when a checkout is available).  Skipped, with that reason, if neither
holds the script.
"""
import importlib
import os
import sys
import types

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_dir():
    for d in (os.environ.get("RINGRNN_REFERENCE_DIR"), os.path.join(ROOT, "baseline", "_ref")):
        if d and os.path.isfile(os.path.join(d, "train_general_ring_no_gain.py")):
            return d
    return None


@pytest.fixture(scope="module")
def reference_modules():
    ref = _reference_dir()
    if ref is None:
        pytest.skip("no copy of the reference (train_general_ring_no_gain.py) in $RINGRNN_REFERENCE_DIR or baseline/_ref")
    saved_path, saved_mods = list(sys.path), set(sys.modules)
    try:
        import matplotlib.pyplot  # noqa: F401
    except Exception:  # the scripts import it at module top and only use it for plots
        mpl = types.ModuleType("matplotlib")
        mpl.pyplot = types.ModuleType("matplotlib.pyplot")
        sys.modules.setdefault("matplotlib", mpl)
        sys.modules.setdefault("matplotlib.pyplot", mpl.pyplot)
    for name in [m for m in sys.modules if m == "cpp" or m.startswith("cpp.")]:
        if not getattr(sys.modules[name], "__file__", "").startswith(ROOT):
            del sys.modules[name]
    sys.path[:0] = [ROOT, ref, os.path.join(ref, "train")]
    script = importlib.import_module("train_general_ring_no_gain")            # the root script
    twin = importlib.import_module("train.train_general_ring_no_gain")        # its pure-PyTorch twin
    yield script, twin, ref
    sys.path[:] = saved_path
    for name in set(sys.modules) - saved_mods:
        if name.startswith(("train", "utils", "matplotlib")):
            del sys.modules[name]


@pytest.mark.parametrize("mode,tol", [("fp32", 1e-4), ("auto", 1e-2)])
def test_reference_training_script_runs_unchanged_on_the_operator(reference_modules, mode, tol, achieved):
    script, twin, ref = reference_modules
    import cpp.ring_rnn_cuda as ours
    assert os.path.abspath(script.__file__) == os.path.join(os.path.abspath(ref), "train_general_ring_no_gain.py")
    assert script.ring_rnn_cuda_func is ours.ring_rnn_cuda_func, "the script did not pick up this repository's operator"
    assert ours.ring_rnn_cuda_func.__module__.startswith("rnn_train_ring_attractor_b200")
    assert script.torch is torch  # the script gets `torch` through the star import (it never imports it itself)

    N, action_dim, B, T, steps = 64, 16, 32, 40, 6
    torch.manual_seed(0)
    model = script.GeneralizedRingAttractorNoGain(num_neurons=N, action_dim=action_dim, tau=10, dt=1, activation="gelu",
                                                  initialization="random").to("cuda")
    cpu_model = twin.GeneralizedRingAttractorNoGain(num_neurons=N, action_dim=action_dim, tau=10, dt=1, activation="gelu",
                                                    initialization="random")
    with torch.no_grad():
        cpu_model.Wo.copy_(model.Wo.cpu())
        cpu_model.Wa.copy_(model.Wa.cpu())
    dataset = script.AVIntegrationDataset(num_samples=steps * B, seq_len=T, zero_padding_start_ratio=0.1,
                                          zero_ratios_in_rest=[0.2, 0.5, 0.8], device="cuda", fast_mode=True)
    opt = torch.optim.Adam(model.parameters(), lr=1e-3)
    cpu_opt = torch.optim.Adam(cpu_model.parameters(), lr=1e-3)
    ours.set_precision(mode)
    got, want = [], []
    try:
        for _ in range(steps):
            # ---- body of the script's loop, train_general_ring_no_gain.py:312-336, its own functions throughout
            av_signal, target_angle = dataset.generate_batch(B)
            action_signal = script.av_to_action_signal_ND(av_signal, action_dim)
            r_init = script.create_initial_bump(target_angle[:, 0], N, device="cuda")
            predicted_cosine_wave, bump_activity = model(action_signal, r_init=r_init)
            loss = script.cosine_similarity_loss(predicted_cosine_wave, target_angle)
            bump_loss = script.bump_amplitude_loss(bump_activity)
            total_loss = loss + 0.2 * bump_loss
            opt.zero_grad()
            total_loss.backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
            got.append(total_loss.item())
            # ---- the same step of the pure-PyTorch twin on the CPU, same batch
            pw, ba = cpu_model(action_signal.cpu(), r_init=r_init.cpu())
            cpu_total = script.cosine_similarity_loss(pw, target_angle.cpu()) + 0.2 * script.bump_amplitude_loss(ba)
            cpu_opt.zero_grad()
            cpu_total.backward()
            torch.nn.utils.clip_grad_norm_(cpu_model.parameters(), 1.0)
            cpu_opt.step()
            want.append(cpu_total.item())
    finally:
        ours.set_precision("auto")
    worst = max(abs(a - b) / max(1.0, abs(b)) for a, b in zip(got, want))
    w_err = float((model.Wo.detach().cpu() - cpu_model.Wo.detach()).norm() / cpu_model.Wo.detach().norm())
    achieved(f"reference script on the operator, mode {mode}", loss_rel_worst_step=worst, Wo_after_steps=w_err,
             first_loss=got[0], last_loss=got[-1])
    assert worst < tol, (got, want)
    assert w_err < 10 * tol
    # the 14 zero-padded action columns: their matrices receive exactly zero gradient, as in the twin
    assert float(model.Wa.grad[2:].abs().max()) == 0.0 and float(cpu_model.Wa.grad[2:].abs().max()) == 0.0
