"""Data-parallel training step: the batch is sharded evenly over ranks, weights are replicated, and the only
exchange is one sum all-reduce per step of a contiguous fp32 buffer [dWo | dWa | dJ0 dJ1 | loss parts].

The reference is single-process; samples never interact in the recurrence and only the weight gradients
(legacy/bwd_fp32.py:104-107) and the mean-reduced losses sum over the batch, which is what makes this the
whole multi-GPU story.  Works on any torch.distributed backend (NCCL on GPUs; gloo in the CPU tests, which
exercise the sharding and buffer logic with a stand-in for the kernel call).
"""
import torch
import torch.distributed as dist


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


def allreduce_grad_buffer(buf, group=None):
    """Sum over ranks, in place.  No-op without an initialised process group or with one rank."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=group)
    return buf


def train_step(step_fn, local_inputs, N, a_dim, global_batch, T, buf=None, group=None, bump_weight=0.2):
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
    allreduce_grad_buffer(buf, group)
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
