"""Data-parallel training step: the batch is sharded evenly over ranks, weights are replicated, and the only
exchange is one sum all-reduce per step of a contiguous fp32 buffer [dWo | dWa | dJ0 dJ1 | loss parts].

The reference is single-process; samples never interact in the recurrence and only the weight gradients
(legacy/bwd_fp32.py:104-107) and the mean-reduced losses sum over the batch, which is what makes this the
whole multi-GPU story.  Works on any torch.distributed backend (NCCL on GPUs; gloo in the CPU tests, which
exercise the sharding and buffer logic with a stand-in for the kernel call).
"""
import datetime

import torch
import torch.distributed as dist


class PeerLostError(RuntimeError):
    """A rank of the data-parallel group left, or did not reach the gradient exchange in time."""


def init_process_group(backend, timeout_s=600.0, **kw):
    """torch.distributed.init_process_group with a finite collective timeout: a gradient all-reduce that a peer never
    joins ends with an error after `timeout_s` instead of waiting for ever (the reference is single-process and has no
    counterpart; its only failure mode is std::exit, cpp/cuda_common.cuh:30-39)."""
    return dist.init_process_group(backend, timeout=datetime.timedelta(seconds=float(timeout_s)), **kw)


class PeerMonitor:
    """Host-side notice board on the process group's key-value store: a rank that leaves between steps says so, and the
    others find out BEFORE they launch the next step -- with no kernel or collective in flight on anybody's GPU.

        mon = PeerMonitor(rank, world)          # after init_process_group
        mon.check()                             # before every step: raises PeerLostError if somebody left
        mon.leave("out of data")                # on the way out, between steps
    """

    def __init__(self, rank, world, store=None, prefix="ringrnn/left/"):
        self.rank, self.world, self.prefix = rank, world, prefix
        self.store = store if store is not None else dist.distributed_c10d._get_default_store()

    def leave(self, reason=""):
        self.store.set(f"{self.prefix}{self.rank}", reason or "left")

    def check(self):
        for r in range(self.world):
            if r != self.rank and self.store.check([f"{self.prefix}{r}"]):
                why = self.store.get(f"{self.prefix}{r}").decode(errors="replace")
                raise PeerLostError(f"rank {r} left the data-parallel group ({why}); not launching the next step")


def shard_rows(t, rank, world):
    """Rows [rank*B/world, (rank+1)*B/world) of a batch-major tensor; B must divide evenly."""
    B = t.shape[0]
    if B % world != 0:
        raise ValueError(f"batch {B} does not divide over {world} ranks")
    per = B // world
    return t[rank * per:(rank + 1) * per].contiguous()


def grad_buffer_numel(N, a_dim):
    """[dWo (N*N) | dWa (a*N*N) | dJ0 dJ1 | loss_cos loss_amp]"""
    return (1 + a_dim) * N * N + 4


def split_grad_buffer(buf, N, a_dim):
    nn = N * N
    return {"dWo": buf[:nn].view(N, N), "dWa": buf[nn:(1 + a_dim) * nn].view(a_dim, N, N),
            "dJ": buf[(1 + a_dim) * nn:(1 + a_dim) * nn + 2], "loss_parts": buf[(1 + a_dim) * nn + 2:]}


def allreduce_grad_buffer(buf, group=None, timeout_s=None):
    """Sum over ranks, in place.  No-op without an initialised process group or with one rank.

    A peer that never arrives ends the call with PeerLostError: after `timeout_s` where the backend can wait with a
    limit on the host (gloo), else after the process group's own timeout (see init_process_group).  The buffer's
    contents are then undefined and the group should be torn down."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        try:
            if timeout_s is not None and dist.get_backend(group) == "gloo":
                work = dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group, async_op=True)
                work.wait(datetime.timedelta(seconds=float(timeout_s)))
            else:
                dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
        except RuntimeError as e:  # torch raises DistBackendError / RuntimeError on a timed-out or aborted collective
            raise PeerLostError(f"gradient all-reduce did not complete: {e}") from e
    return buf


def train_step(step_fn, local_inputs, N, a_dim, global_batch, T, buf=None, group=None, bump_weight=0.2,
               timeout_s=None):
    """Run one data-parallel fwd + loss + bwd.

    `step_fn(local_inputs, inv_count, grad_buffer) -> loss_parts[2]` runs the local shard and leaves
    [dWo | dWa | dJ0 dJ1] in `grad_buffer` (the fused operator does exactly this); the local losses are
    normalised by the GLOBAL count so that the summed buffer equals the single-process result.
    Returns (loss, views-of-buffer dict).
    """
    device = local_inputs[0].device
    if buf is None:
        buf = torch.empty(grad_buffer_numel(N, a_dim), dtype=torch.float32, device=device)
    parts = step_fn(local_inputs, 1.0 / (global_batch * T), buf)
    buf[-2:].copy_(parts)
    allreduce_grad_buffer(buf, group, timeout_s)
    out = split_grad_buffer(buf, N, a_dim)
    loss = out["loss_parts"][0] + bump_weight * out["loss_parts"][1]
    return loss, out


def fused_step_fn(Wa, J0, J1, Wo, alpha, activation, bump_weight=0.2, precision=None, ckpt_every=0):
    """step_fn for :func:`train_step` backed by the fused CUDA operator (`ckpt_every`: see ring_rnn_fused)."""
    from .fused import ring_rnn_fused

    def fn(local_inputs, inv_count, buf):
        A, r_init, target = local_inputs
        Wa_ = Wa.detach().requires_grad_(True)
        Wo_ = Wo.detach().requires_grad_(True)
        loss, parts, _, _ = ring_rnn_fused(A, Wa_, J0, J1, Wo_, r_init, alpha, activation, target, bump_weight,
                                           inv_count, precision, buf, ckpt_every)
        loss.backward()
        return parts

    return fn
