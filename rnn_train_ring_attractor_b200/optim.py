"""Device-side optimizer step and training-state files for the ring-attractor parameters.

The reference training loop (train_general_ring_no_gain.py:331-344) calls, per step,
``torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)`` and ``torch.optim.Adam.step()`` on four separate
parameter tensors and reads the loss back with ``.item()``.  Here the parameters live in ONE contiguous fp32 buffer with
the layout of the data-parallel gradient buffer (``[Wo | Wa | J0 J1]``, dp.py), so the all-reduced gradient can be
applied by a single fused kernel (``ringrnn_clip_adam``) without any host synchronisation.  As in the reference, only
Wo and Wa are trained unless asked otherwise; J0 and J1 ride along in the buffer as constants.
"""
import ctypes as C

import torch

from . import _lib


class FlatRingParams:
    """Wo [N,N], Wa [a,N,N], J0, J1 as views into one flat fp32 buffer ``flat`` = [Wo | Wa | J0 J1]."""

    def __init__(self, Wo, Wa, J0, J1):
        N, a = Wo.shape[0], Wa.shape[0]
        dev = Wo.device
        self.N, self.a_dim = N, a
        self.flat = torch.empty((1 + a) * N * N + 2, dtype=torch.float32, device=dev)
        self.flat[:N * N].copy_(Wo.detach().reshape(-1))
        self.flat[N * N:(1 + a) * N * N].copy_(Wa.detach().reshape(-1))
        self.flat[-2] = float(J0)
        self.flat[-1] = float(J1)

    @property
    def Wo(self):
        return self.flat[:self.N * self.N].view(self.N, self.N)

    @property
    def Wa(self):
        return self.flat[self.N * self.N:(1 + self.a_dim) * self.N * self.N].view(self.a_dim, self.N, self.N)

    @property
    def J(self):
        """[J0, J1] as a 2-element device view."""
        return self.flat[-2:]


class FusedClipAdam:
    """clip_grad_norm_(max_norm) + Adam(lr, betas, eps) on a flat parameter buffer, one library call per step.

    Defaults follow the reference (Adam lr 1e-3, clip 1.0: train_general_ring_no_gain.py:312, :335).  In the reference
    J0 and J1 are plain floats (train_general_ring_no_gain.py:47-48): model.parameters() is {Wo, Wa}, so neither the
    clip norm nor the update sees them.  The same holds here by default: when the buffer has the [Wo | Wa | J0 J1]
    layout (`n_fixed_tail` = 2 trailing elements), the norm and the update cover Wo and Wa only and J0, J1 keep their
    values.  `train_J=True` opts into training them as well (their gradients then enter the clip norm).
    """

    def __init__(self, flat_params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, max_norm=1.0, train_J=False, n_fixed_tail=2):
        if flat_params.dtype != torch.float32 or not flat_params.is_cuda or not flat_params.is_contiguous():
            raise ValueError("flat_params must be a contiguous fp32 CUDA tensor")
        self.params = flat_params
        self.train_J = bool(train_J)
        self.n_updated = flat_params.numel() - (0 if train_J else int(n_fixed_tail))
        self.lr, self.betas, self.eps, self.max_norm = lr, betas, eps, max_norm
        self.exp_avg = torch.zeros_like(flat_params)
        self.exp_avg_sq = torch.zeros_like(flat_params)
        self.step_count = 0
        self._scratch = torch.zeros(129, dtype=torch.float64, device=flat_params.device)

    def step(self, flat_grads):
        """Applies one update; returns a 0-dim device tensor holding the unclipped gradient norm of the updated
        elements (no sync)."""
        if flat_grads.shape != self.params.shape or flat_grads.dtype != torch.float32 or not flat_grads.is_contiguous():
            raise ValueError("flat_grads must match the parameter buffer (contiguous fp32)")
        self.step_count += 1
        with torch.cuda.device(self.params.device):
            stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            _lib.check(_lib.lib().ringrnn_clip_adam(
                self.params.data_ptr(), flat_grads.data_ptr(), self.exp_avg.data_ptr(), self.exp_avg_sq.data_ptr(),
                self.n_updated, self.lr, self.betas[0], self.betas[1], self.eps, self.step_count, self.max_norm,
                self._scratch.data_ptr(), stream))
        return self._scratch[128]

    def state_dict(self):
        return {"exp_avg": self.exp_avg, "exp_avg_sq": self.exp_avg_sq, "step": self.step_count, "lr": self.lr,
                "betas": self.betas, "eps": self.eps, "max_norm": self.max_norm}

    def load_state_dict(self, sd):
        self.exp_avg.copy_(sd["exp_avg"])
        self.exp_avg_sq.copy_(sd["exp_avg_sq"])
        self.step_count = int(sd["step"])
        self.lr, self.betas, self.eps, self.max_norm = sd["lr"], tuple(sd["betas"]), sd["eps"], sd["max_norm"]


def save_training_state(path, params, optimizer, step, extra=None):
    """One file with the flat parameters, the optimizer moments and the step counter (the reference keeps only
    ``model.state_dict()`` of its best model in memory, train_ring_attractor.py:441-444)."""
    torch.save({"flat": params.flat.cpu(), "N": params.N, "a_dim": params.a_dim,
                "optimizer": {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in optimizer.state_dict().items()},
                "step": int(step), "extra": extra or {}}, path)


def load_training_state(path, params, optimizer):
    """Restores what save_training_state wrote into existing objects; returns (step, extra)."""
    sd = torch.load(path, map_location="cpu")
    if sd["N"] != params.N or sd["a_dim"] != params.a_dim:
        raise ValueError("training state was saved for a different shape")
    params.flat.copy_(sd["flat"])
    optimizer.load_state_dict({k: (v.to(params.flat.device) if torch.is_tensor(v) else v)
                               for k, v in sd["optimizer"].items()})
    return sd["step"], sd["extra"]
