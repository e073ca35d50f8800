"""Angular-error evaluation of a ring-attractor parameter set on held-out synthetic trials, on the fused forward.

Follows the evaluation block of compare/compare_models_fair.py:120-175: 200 test sequences of 500 steps in batches of
50, initial Gaussian bump at the first target angle, decoded angle from the population vector, circular error, and the
four statistics the script prints (mean, std, max, mean error at the final step).
"""
import math

import torch

from .fused import ring_rnn_rollout
from .inputs import av_to_action_signal, generate_av, initial_bump_gaussian


def angular_error(pred, target):
    """Circular |pred - target| in [0, pi] (compare/compare_models_fair.py:15-20)."""
    d = torch.abs(pred - target) % (2 * math.pi)
    return torch.minimum(d, 2 * math.pi - d)


def evaluate_angular_error(Wa, J0, J1, Wo, alpha, activation, n_trials=200, seq_len=500, batch=50, seed=123,
                           max_av=0.1 * math.pi, precision=None):
    """dict(mean, std, max, final_mean, errors[n_trials, seq_len]) in radians for the given weights (device tensors)."""
    dev = Wo.device
    N = Wo.shape[0]
    g = torch.Generator().manual_seed(seed)
    errs = []
    for _ in range((n_trials + batch - 1) // batch):
        av, angle = generate_av(batch, seq_len, max_av=max_av, generator=g)
        A = av_to_action_signal(av, max_av).to(dev)
        r0 = initial_bump_gaussian(angle[:, 0], N).to(dev)
        decoded, _ = ring_rnn_rollout(A, Wa, J0, J1, Wo, r0, alpha, activation, precision=precision)
        errs.append(angular_error(decoded, angle.to(dev)))
    e = torch.cat(errs, dim=0)[:n_trials]
    return {"mean": float(e.mean()), "std": float(e.std()), "max": float(e.max()), "final_mean": float(e[:, -1].mean()),
            "errors": e}
