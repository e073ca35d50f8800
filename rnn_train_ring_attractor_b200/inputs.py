"""Seeded synthetic inputs of the angular-velocity integration task, on any torch device.

Counterparts in the reference: the trial generator (utils/generate_av_integration_data.py:11-58), the
[L, R] action signal (train_general_ring_no_gain.py:176-188, :200-223) and the initial bump
(train/train_ring_attractor.py:21-52).  The benchmark configurations use L/R scaled by 1/max_av, weights
randn*0.01 and a von-Mises initial bump exp(kappa*(cos(phi_i - theta0) - 1)), kappa = 4.
"""
import math

import torch


def generate_av(num_trials, seq_len, zero_padding_start_ratio=0.1, zero_ratios_in_rest=(0.2, 0.5, 0.8),
                max_av=0.1 * math.pi, device="cpu", generator=None):
    """(av[num_trials, seq_len], angle[num_trials, seq_len]).  The first 10% of steps are zero; of the rest an
    exact count of floor(len*ratio) steps (ratio drawn per trial) is zeroed; the others are U(-max_av, max_av).
    angle[:, 0] = theta0 ~ U(0, 2pi) and angle[:, t] = theta0 + sum(av[:, :t]) mod 2pi (one-step lag)."""
    kw = dict(device=device, generator=generator)
    av = torch.zeros(num_trials, seq_len, device=device)
    n0 = int(seq_len * zero_padding_start_ratio)
    rest = seq_len - n0
    theta0 = torch.rand(num_trials, **kw) * 2 * math.pi
    ridx = torch.randint(0, len(zero_ratios_in_rest), (num_trials,), **kw)
    ratios = torch.tensor(list(zero_ratios_in_rest), device=device)[ridx]
    keep = rest - (rest * ratios).long()
    if rest > 0:
        vals = (torch.rand(num_trials, rest, **kw) - 0.5) * 2 * max_av
        rank = torch.rand(num_trials, rest, **kw).argsort(dim=1)
        av[:, n0:] = vals * (rank < keep[:, None]).float()
    angle = torch.zeros(num_trials, seq_len, device=device)
    angle[:, 0] = theta0
    angle[:, 1:] = (theta0[:, None] + torch.cumsum(av[:, :-1], dim=1)) % (2 * math.pi)
    return av, angle


def av_to_action_signal(av, scale=1.0, action_dim=2):
    """[relu(-av), relu(av), 0, ...] / scale as a contiguous [B, T, action_dim] tensor."""
    A = torch.zeros(av.shape[0], av.shape[1], action_dim, dtype=av.dtype, device=av.device)
    A[:, :, 0] = torch.relu(-av) / scale
    A[:, :, 1] = torch.relu(av) / scale
    return A


def initial_bump_gaussian(theta0, N, width_factor=10):
    """The reference's unit-norm Gaussian bump of width N/width_factor centred at theta0 on the ring."""
    c = (theta0 * N / (2 * math.pi))[:, None]
    idx = torch.arange(N, device=theta0.device)[None, :]
    d = torch.minimum((idx - c).abs(), N - (idx - c).abs())
    b = torch.exp(-(d ** 2) / (2 * (N / width_factor) ** 2))
    return b / b.norm(dim=1, keepdim=True)


def initial_bump_von_mises(theta0, N, kappa=4.0):
    phi = 2 * math.pi * torch.arange(N, dtype=torch.float32, device=theta0.device) / N
    return torch.exp(kappa * (torch.cos(phi[None, :] - theta0[:, None]) - 1.0))


def ideal_weights(N, device="cpu"):
    """Wo_ij = cos(2pi(i-j)/N); Wl, Wr = the same profile shifted by -1 / +1 neuron."""
    idx = torch.arange(N, dtype=torch.float32, device=device)
    Wo = torch.cos(2 * math.pi * (idx[:, None] - idx[None, :]) / N)
    return Wo, torch.roll(Wo, -1, 1).contiguous(), torch.roll(Wo, 1, 1).contiguous()


def benchmark_inputs(N, B, T, seed=0, max_av=0.1 * math.pi, weights="randn0.01", device="cpu"):
    """dict(A, Wa, Wo, r_init, target, J0, J1) for one benchmark configuration, generated on CPU from `seed`."""
    g = torch.Generator().manual_seed(seed)
    if weights == "ideal":
        Wo, Wl, Wr = ideal_weights(N)
    else:
        Wo = torch.randn(N, N, generator=g) * 0.01
        Wl = torch.randn(N, N, generator=g) * 0.01
        Wr = torch.randn(N, N, generator=g) * 0.01
    av, angle = generate_av(B, T, max_av=max_av, generator=g)
    out = dict(A=av_to_action_signal(av, max_av), Wa=torch.stack([Wl, Wr]).contiguous(), Wo=Wo,
               r_init=initial_bump_von_mises(angle[:, 0], N), target=angle)
    out = {k: v.to(device) for k, v in out.items()}
    out.update(J0=-0.1, J1=0.1)
    return out
