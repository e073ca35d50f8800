"""CPU oracle for the ring-attractor recurrent forward / backward-through-time path.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain torch-on-CPU code, what the
reference computes for this path; it exists to check the CUDA kernels and to serve as the
timed CPU baseline.  Nothing in the product package imports it, and the product path never
falls back to it.

Parity status: pinned.  ``tests/golden/*.npz`` hold outputs of the *unmodified* reference
modules (``train/train_general_ring_no_gain.py`` model + ``train/train_ring_attractor.py``
losses + ``utils/generate_av_integration_data.py`` generator) run on seeded inputs by
``tests/golden/make_golden.py``; ``tests/test_oracle.py`` checks every function below against
those files.  The reference itself ships no golden vectors or known-answer tests.

Reference map (file:line are paths inside the reference project):

* activation / derivative ............ cpp/cuda_common.cuh:56-89, train/train_ring_attractor.py:10-18,
                                        legacy/bwd_fp32.py:433-461
* forward recurrence .................. train/train_general_ring_no_gain.py:102-128 (W_eff materialised),
                                        cpp/ring_rnn_cuda.py:55-86 (output layout [T,B,N])
* backward through time ............... legacy/bwd_fp32.py:86-109, cpp/kernels/bwd_mixed_precision_aggressive.cuh:254-268,
                                        :310-317, :607-620
* decode and losses ................... train_general_ring_no_gain.py:113-116, train/train_ring_attractor.py:190-220,
                                        :257-272, :275-298
* inputs .............................. utils/generate_av_integration_data.py:11-58, train_general_ring_no_gain.py:176-188,
                                        train/train_ring_attractor.py:21-52
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

ACTIVATIONS = ("relu", "gelu", "tanh", "silu")  # enum order of cpp/cuda_common.cuh:56


# --------------------------------------------------------------------------- activations
def activation(x: torch.Tensor, name: str) -> torch.Tensor:
    """F(x).  relu / exact-erf gelu / tanh as train/train_ring_attractor.py:10-18; silu as
    cpp/cuda_common.cuh:64-66 (x * sigmoid(x))."""
    if name == "relu":
        return torch.relu(x)
    if name == "gelu":
        return torch.nn.functional.gelu(x)
    if name == "tanh":
        return torch.tanh(x)
    if name == "silu":
        return x * torch.sigmoid(x)
    raise ValueError(f"Invalid activation '{name}'. Must be one of {list(ACTIVATIONS)}.")


def activation_grad(x: torch.Tensor, name: str) -> torch.Tensor:
    """F'(x) as cpp/cuda_common.cuh:72-89: relu -> [x>0]; gelu -> Phi(x) + x*phi(x);
    silu -> s*(1 + x*(1-s)); tanh -> 1 - tanh^2."""
    if name == "relu":
        return (x > 0).to(x.dtype)
    if name == "gelu":
        cdf = 0.5 * (1.0 + torch.erf(x / math.sqrt(2.0)))
        pdf = torch.exp(-0.5 * x * x) / math.sqrt(2.0 * math.pi)
        return cdf + x * pdf
    if name == "tanh":
        return 1.0 - torch.tanh(x) ** 2
    if name == "silu":
        s = torch.sigmoid(x)
        return s * (1.0 + x * (1.0 - s))
    raise ValueError(f"Invalid activation '{name}'. Must be one of {list(ACTIVATIONS)}.")


# --------------------------------------------------------------------------- forward
def ring_forward_ref(A, Wa, J0, J1, Wo, r_init, alpha, act="relu"):
    """Reference-shaped forward: materialises W_eff[B,N,N] every step.

    Follows train/train_general_ring_no_gain.py:102-128 with ``alpha`` as a parameter (the
    reference hard-codes 0.15 at :125).  Returns ``bump_history[T,B,N]`` in the layout the
    CUDA operator uses (cpp/ring_rnn_cuda.py:62).  Differentiable through autograd.
    """
    B, T, a = A.shape
    r = r_init
    out = []
    for t in range(T):
        A_t = A[:, t, :]
        Wa_weighted = torch.sum(A_t[:, :, None, None] * Wa[None], dim=1)
        W_eff = J0 + J1 * Wo + Wa_weighted
        re = (W_eff @ r.unsqueeze(2)).squeeze(2)
        r = r * (1 - alpha) + activation(re, act) * alpha
        out.append(r)
    return torch.stack(out, dim=0)


def ring_forward_lean(A, Wa, J0, J1, Wo, r_init, alpha, act="relu"):
    """Same recurrence without W_eff:  re = J0*sum_j r + J1*(r Wo^T) + sum_k A_k*(r Wa_k^T).

    Memory O(B*N) per step instead of O(B*N^2); used where the reference formulation does not
    fit in host RAM.  Equal to :func:`ring_forward_ref` up to fp32 summation order.
    """
    B, T, a = A.shape
    r = r_init
    out = []
    for t in range(T):
        re = J0 * r.sum(dim=1, keepdim=True) + J1 * (r @ Wo.t())
        for k in range(a):
            re = re + A[:, t, k:k + 1] * (r @ Wa[k].t())
        r = r * (1 - alpha) + activation(re, act) * alpha
        out.append(r)
    return torch.stack(out, dim=0)


def ring_backward_manual(grad_out, A, Wa, J0, J1, Wo, hist, r_init, alpha, act="relu"):
    """Hand-written BPTT (no autograd), the recurrence of legacy/bwd_fp32.py:86-109.

    ``grad_out`` and ``hist`` are [T,B,N].  Returns a dict with dWa, dWo (what the reference
    returns, cpp/ring_rnn_cuda.py:144) plus dJ0, dJ1, dA and dr_init, which the reference
    does not compute.
    """
    T, B, N = hist.shape
    a = A.shape[2]
    dWa = torch.zeros_like(Wa)
    dWo = torch.zeros_like(Wo)
    dA = torch.zeros_like(A)
    dJ0 = torch.zeros((), dtype=hist.dtype)
    dJ1 = torch.zeros((), dtype=hist.dtype)
    carry = torch.zeros(B, N, dtype=hist.dtype)
    for t in reversed(range(T)):
        r_prev = r_init if t == 0 else hist[t - 1]
        yo = r_prev @ Wo.t()
        ya = [r_prev @ Wa[k].t() for k in range(a)]
        re = J0 * r_prev.sum(dim=1, keepdim=True) + J1 * yo
        for k in range(a):
            re = re + A[:, t, k:k + 1] * ya[k]
        g = grad_out[t] + carry
        delta = alpha * activation_grad(re, act) * g
        G = delta.t() @ r_prev
        dWo += J1 * G
        dJ0 += G.sum()
        dJ1 += (G * Wo).sum()
        carry = (1 - alpha) * g + J0 * delta.sum(dim=1, keepdim=True) + J1 * (delta @ Wo)
        for k in range(a):
            sd = A[:, t, k:k + 1] * delta
            dWa[k] += sd.t() @ r_prev
            dA[:, t, k] = (delta * ya[k]).sum(dim=1)
            carry = carry + sd @ Wa[k]
    return {"dWa": dWa, "dWo": dWo, "dJ0": dJ0, "dJ1": dJ1, "dA": dA, "dr_init": carry}


# --------------------------------------------------------------------------- decode + losses
def w_delta7(N, dtype=torch.float32):
    """cos(2*pi*(i-j)/N), train/train_general_ring_no_gain.py:39-43."""
    idx = torch.arange(N, dtype=torch.float32)
    return torch.cos(2 * math.pi * (idx[:, None] - idx[None, :]) / N).to(dtype)


def preferred_angles(N, dtype=torch.float32):
    """linspace(0, 2*pi, N) -- both endpoints included (train/train_ring_attractor.py:197)."""
    return torch.linspace(0, 2 * math.pi, N).to(dtype)


def decode_normalised(hist_btn):
    """r @ W_delta7 divided by its per-(b,t) max; train_general_ring_no_gain.py:113-116."""
    N = hist_btn.shape[-1]
    rd = hist_btn @ w_delta7(N, hist_btn.dtype)
    return rd / rd.max(dim=2, keepdim=True)[0]


def cosine_similarity_loss(pred_wave, true_angle):
    """train/train_ring_attractor.py:190-220."""
    phi = preferred_angles(pred_wave.shape[-1], pred_wave.dtype)
    px = torch.sum(pred_wave * torch.cos(phi), dim=-1)
    py = torch.sum(pred_wave * torch.sin(phi), dim=-1)
    th = torch.atan2(py, px)
    return torch.mean((torch.cos(th) - torch.cos(true_angle)) ** 2 + (torch.sin(th) - torch.sin(true_angle)) ** 2)


def bump_amplitude_loss(bump_btn):
    """train/train_ring_attractor.py:275-298 with target_amplitude=None."""
    ta = bump_btn.abs().sum(dim=2)
    return torch.mean((ta - ta[:, 0:1]) ** 2)


def training_loss_ref(hist_tbn, true_angle, bump_weight=0.2):
    """The loss of train_general_ring_no_gain.py:327-330 on a [T,B,N] history."""
    bump = hist_tbn.permute(1, 0, 2)
    return cosine_similarity_loss(decode_normalised(bump), true_angle) + bump_weight * bump_amplitude_loss(bump)


def decode_vectors(N, dtype=torch.float32):
    """u = W_delta7 @ cos(phi), v = W_delta7 @ sin(phi): the decode collapses to x=r.u, y=r.v
    because atan2 ignores the positive 1/max scale."""
    phi = preferred_angles(N, torch.float64)
    W = w_delta7(N, torch.float64)
    return (W @ torch.cos(phi)).to(dtype), (W @ torch.sin(phi)).to(dtype)


def fused_loss_terms(hist_tbn, true_angle, bump_weight=0.2):
    """Two-dot-product restatement of :func:`training_loss_ref`.

    Returns (loss, x[B,T], y[B,T], ta[B,T], dloss/dhist[T,B,N]) -- the gradient in closed form:
    d/dr_t = k*(x*v - y*u) + c_t*sign(r_t),  k = 2 sin(th-th*)/(x^2+y^2)/(B*T),
    c_t = 2w(ta_t-ta_0)/(B*T) for t>=1 and -2w*sum_t(ta_t-ta_0)/(B*T) at t=0.
    """
    T, B, N = hist_tbn.shape
    u, v = decode_vectors(N, hist_tbn.dtype)
    x = (hist_tbn @ u).t()
    y = (hist_tbn @ v).t()
    ta = hist_tbn.abs().sum(dim=2).t()
    th = torch.atan2(y, x)
    d = th - true_angle
    loss_cos = torch.mean(2.0 - 2.0 * torch.cos(d))
    dev = ta - ta[:, 0:1]
    loss_amp = torch.mean(dev ** 2)
    k = 2.0 * torch.sin(d) / (x * x + y * y) / (B * T)
    c = 2.0 * bump_weight * dev / (B * T)
    c[:, 0] = -c[:, 1:].sum(dim=1)
    g = (k * x).t()[:, :, None] * v - (k * y).t()[:, :, None] * u + c.t()[:, :, None] * torch.sign(hist_tbn)
    return loss_cos + bump_weight * loss_amp, x, y, ta, g


def decode_angle(hist_tbn):
    """Population-vector angle in [0, 2*pi), train/train_ring_attractor.py:257-272, applied to
    the max-normalised cosine wave (equivalently to x=r.u, y=r.v).  Returns [B,T]."""
    u, v = decode_vectors(hist_tbn.shape[-1], hist_tbn.dtype)
    th = torch.atan2(hist_tbn @ v, hist_tbn @ u).t()
    return (th + 2 * math.pi) % (2 * math.pi)


def angular_error(a, b):
    """Circular |a-b|, compare/compare_models_fair.py:15-20."""
    d = torch.abs(a - b) % (2 * math.pi)
    return torch.minimum(d, 2 * math.pi - d)


# --------------------------------------------------------------------------- inputs
def generate_av(num_trials, seq_len, zero_padding_start_ratio=0.1, zero_ratios_in_rest=(0.2, 0.5, 0.8),
                max_av=0.1 * math.pi):
    """Angular-velocity trials + integrated target angle, utils/generate_av_integration_data.py:11-58.

    Draw order (it fixes the seeded stream): theta0 ~ U(0,2pi); ratio index ~ randint; values ~ U;
    ranks ~ argsort(U).  An exact count of ``len_rest - floor(len_rest*ratio)`` steps stays non-zero;
    target[:, 0] = theta0 and target[:, 1:] = (theta0 + cumsum(av[:, :-1])) mod 2pi.
    """
    av = torch.zeros(num_trials, seq_len)
    n0 = int(seq_len * zero_padding_start_ratio)
    rest = seq_len - n0
    theta0 = torch.rand(num_trials) * 2 * math.pi
    ridx = torch.randint(0, len(zero_ratios_in_rest), (num_trials,))
    ratios = torch.tensor(list(zero_ratios_in_rest))[ridx]
    keep = rest - (rest * ratios).long()
    if rest > 0:
        vals = (torch.rand(num_trials, rest) - 0.5) * 2 * max_av
        rank = torch.rand(num_trials, rest).argsort(dim=1)
        av[:, n0:] = vals * (rank < keep[:, None]).float()
    angle = torch.zeros(num_trials, seq_len)
    angle[:, 0] = theta0
    angle[:, 1:] = (theta0[:, None] + torch.cumsum(av[:, :-1], dim=1)) % (2 * math.pi)
    return av, angle


def av_to_action_signal(av, scale=1.0, action_dim=2):
    """[L, R, 0...] = [relu(-av), relu(av)] / scale  (train_general_ring_no_gain.py:176-188, :200-223)."""
    A = torch.zeros(av.shape[0], av.shape[1], action_dim, dtype=av.dtype)
    A[:, :, 0] = torch.relu(-av) / scale
    A[:, :, 1] = torch.relu(av) / scale
    return A


def initial_bump_gaussian(theta0, N, width_factor=10):
    """Unit-norm Gaussian bump on the ring, train/train_ring_attractor.py:21-52."""
    c = (theta0 * N / (2 * math.pi))[:, None]
    idx = torch.arange(N)[None, :]
    d = torch.minimum((idx - c).abs(), N - (idx - c).abs())
    b = torch.exp(-(d ** 2) / (2 * (N / width_factor) ** 2))
    return b / b.norm(dim=1, keepdim=True)


def initial_bump_von_mises(theta0, N, kappa=4.0):
    """exp(kappa*(cos(phi_i - theta0) - 1)) with phi_i = 2*pi*i/N (the benchmark configs' initial state)."""
    phi = 2 * math.pi * torch.arange(N, dtype=torch.float32) / N
    return torch.exp(kappa * (torch.cos(phi[None, :] - theta0[:, None]) - 1.0))


def ideal_weights(N):
    """Wo_ij = cos(phi_i - phi_j); Wl / Wr the same profile shifted by -1 / +1 neuron."""
    Wo = w_delta7(N)
    return Wo, torch.roll(Wo, shifts=-1, dims=1).contiguous(), torch.roll(Wo, shifts=1, dims=1).contiguous()


@dataclass
class RingCase:
    """One seeded problem instance (all tensors fp32 on CPU)."""
    A: torch.Tensor
    Wa: torch.Tensor
    Wo: torch.Tensor
    r_init: torch.Tensor
    target: torch.Tensor
    J0: float
    J1: float
    alpha: float
    act: str


def make_case(N, B, T, act, seed=0, alpha=0.1, max_av=0.1 * math.pi, weights="randn0.01", action_dim=2):
    """Benchmark-config inputs: weights Wo,Wl,Wr = randn*0.01 drawn in that order from ``seed`` (or the
    ideal cosine weights), J0=-0.1, J1=0.1, L/R divided by max_av, von-Mises initial bump (kappa=4)."""
    g = torch.Generator().manual_seed(seed)
    if weights == "randn0.01":
        Wo = torch.randn(N, N, generator=g) * 0.01
        Wl = torch.randn(N, N, generator=g) * 0.01
        Wr = torch.randn(N, N, generator=g) * 0.01
    elif weights == "ideal":
        Wo, Wl, Wr = ideal_weights(N)
    else:
        raise ValueError(weights)
    state = torch.random.get_rng_state()
    torch.manual_seed(seed + 1)
    av, angle = generate_av(B, T, max_av=max_av)
    torch.random.set_rng_state(state)
    Wa = torch.zeros(action_dim, N, N)
    Wa[0], Wa[1] = Wl, Wr
    return RingCase(A=av_to_action_signal(av, max_av, action_dim), Wa=Wa, Wo=Wo,
                    r_init=initial_bump_von_mises(angle[:, 0], N), target=angle,
                    J0=-0.1, J1=0.1, alpha=alpha, act=act)


def train_step_ref(case: RingCase, lean=False, bump_weight=0.2, dtype=None):
    """One fwd + loss + bwd of the reference PyTorch path on CPU.  Returns (loss, dWo, dWa, hist).
    `dtype=torch.float64` evaluates the same step in double precision (the arbiter when two fp32 evaluations differ)."""
    cast = (lambda t: t.to(dtype)) if dtype is not None else (lambda t: t)
    Wa = cast(case.Wa).clone().requires_grad_(True)
    Wo = cast(case.Wo).clone().requires_grad_(True)
    fwd = ring_forward_lean if lean else ring_forward_ref
    hist = fwd(cast(case.A), Wa, case.J0, case.J1, Wo, cast(case.r_init), case.alpha, case.act)
    loss = training_loss_ref(hist, cast(case.target), bump_weight)
    loss.backward()
    return loss.detach(), Wo.grad, Wa.grad, hist.detach()


def rel_err(x, y, eps=1e-30):
    """||x-y||_F / max(||y||_F, eps): the tolerance definition used by every parity test."""
    x = x.detach().double().cpu()
    y = y.detach().double().cpu()
    return float((x - y).norm() / max(float(y.norm()), eps))
