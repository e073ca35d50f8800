"""Data-parallel host logic on CPU ranks (gloo, world_size 2): sharding, the contiguous gradient buffer and
its single all-reduce reproduce the single-process gradient.  The kernel call is replaced by the oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ring_oracle as orc
from rnn_train_ring_attractor_b200 import dp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_step_fn(case, N, a_dim):
    def fn(local_inputs, inv_count, buf):
        A, r_init, target = local_inputs
        Wa = case.Wa.clone().requires_grad_(True)
        Wo = case.Wo.clone().requires_grad_(True)
        hist = orc.ring_forward_lean(A, Wa, case.J0, case.J1, Wo, r_init, case.alpha, case.act)
        _, x, y, ta, _ = orc.fused_loss_terms(hist.detach(), target)
        bump = hist.permute(1, 0, 2)
        wave = orc.decode_normalised(bump)
        phi = orc.preferred_angles(N)
        th = torch.atan2((wave * torch.sin(phi)).sum(-1), (wave * torch.cos(phi)).sum(-1))
        l_cos = ((torch.cos(th) - torch.cos(target)) ** 2 + (torch.sin(th) - torch.sin(target)) ** 2).sum() * inv_count
        tav = bump.abs().sum(2)
        l_amp = ((tav - tav[:, 0:1]) ** 2).sum() * inv_count
        (l_cos + 0.2 * l_amp).backward()
        out = dp.split_grad_buffer(buf, N, a_dim)
        out["dWo"].copy_(Wo.grad)
        out["dWa"].copy_(Wa.grad)
        out["dJ"].zero_()
        return torch.stack([l_cos.detach(), l_amp.detach()])
    return fn


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    N, B, T = 16, 8, 12
    case = orc.make_case(N, B, T, "tanh", seed=3)
    local = tuple(dp.shard_rows(t, rank, world) for t in (case.A, case.r_init, case.target))
    loss, out = dp.train_step(_oracle_step_fn(case, N, 2), local, N, 2, B, T)
    if rank == 0:
        q.put((float(loss), out["dWo"].clone(), out["dWa"].clone()))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_gradient_equals_single_process():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    loss, dWo, dWa = q.get(timeout=120)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    case = orc.make_case(16, 8, 12, "tanh", seed=3)
    ref_loss, ref_dWo, ref_dWa, _ = orc.train_step_ref(case, lean=True)
    assert abs(loss - float(ref_loss)) < 1e-5
    assert orc.rel_err(dWo, ref_dWo) < 1e-5
    assert orc.rel_err(dWa, ref_dWa) < 1e-5


def test_shard_rows_and_buffer_views():
    t = torch.arange(24.).view(8, 3)
    assert torch.equal(dp.shard_rows(t, 1, 4), t[2:4])
    with pytest.raises(ValueError):
        dp.shard_rows(t, 0, 3)
    buf = torch.zeros(dp.grad_buffer_numel(4, 2))
    v = dp.split_grad_buffer(buf, 4, 2)
    assert v["dWo"].shape == (4, 4) and v["dWa"].shape == (2, 4, 4) and v["dJ"].numel() == 2
    v["dWa"][1, 3, 3] = 7.0
    assert buf[3 * 16 - 1] == 7.0
    assert dp.allreduce_grad_buffer(buf) is buf  # no process group: no-op


# ---- failure detection on the host: no GPU involved, nothing hangs ------------------------------------------------
def _report_and_exit(q, msg):
    """Flush the message to the parent, then leave without the collective teardown (the group is unusable after a
    timed-out collective, and a rank that has left has nobody to tear down with)."""
    q.put(msg)
    q.close()
    q.join_thread()
    os._exit(0)


def _absent_peer_worker(rank, world, port, q):
    """Rank 1 never joins the gradient exchange; rank 0's all-reduce must give up after its timeout and raise."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dp.init_process_group("gloo", timeout_s=30.0, rank=rank, world_size=world)
    torch.set_num_threads(1)
    if rank == 1:
        time.sleep(6.0)  # skips train_step altogether; long enough for rank 0 to time out
        _report_and_exit(q, ("rank1", "idle"))
    N, B, T = 8, 4, 5
    case = orc.make_case(N, B, T, "tanh", seed=1)
    local = tuple(dp.shard_rows(t, rank, world) for t in (case.A, case.r_init, case.target))
    t0 = time.time()
    try:
        dp.train_step(_oracle_step_fn(case, N, 2), local, N, 2, B, T, timeout_s=2.0)
        msg = ("rank0", "no error")
    except dp.PeerLostError as e:
        msg = ("rank0", f"PeerLostError after {time.time() - t0:.1f}s: {str(e)[:60]}")
    _report_and_exit(q, msg)


def test_allreduce_gives_up_when_a_peer_never_arrives():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_absent_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    assert got["rank0"].startswith("PeerLostError"), got
    assert float(got["rank0"].split()[2][:-2]) < 6.0, got  # gave up at its own 2 s limit, not at the group's 30 s


def _leaving_peer_worker(rank, world, port, q):
    """Rank 1 leaves between steps and says so on the store; rank 0 learns of it before launching its next step."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dp.init_process_group("gloo", timeout_s=30.0, rank=rank, world_size=world)
    torch.set_num_threads(1)
    mon = dp.PeerMonitor(rank, world)
    N, B, T = 8, 4, 5
    case = orc.make_case(N, B, T, "tanh", seed=1)
    local = tuple(dp.shard_rows(t, rank, world) for t in (case.A, case.r_init, case.target))
    mon.check()
    dp.train_step(_oracle_step_fn(case, N, 2), local, N, 2, B, T, timeout_s=20.0)  # step 1: both ranks
    if rank == 1:
        mon.leave("out of data")
        time.sleep(3.0)  # keep the store's client alive while rank 0 reads
        _report_and_exit(q, ("rank1", "left"))
    steps_launched = 1
    for _ in range(50):  # rank 0 polls before each would-be step
        try:
            mon.check()
        except dp.PeerLostError as e:
            _report_and_exit(q, ("rank0", f"PeerLostError: {e}", steps_launched))
        time.sleep(0.1)
    _report_and_exit(q, ("rank0", "never noticed", steps_launched))


def test_a_rank_that_leaves_between_steps_is_noticed_before_the_next_launch():
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_peer_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {m[0]: m for m in (q.get(timeout=120) for _ in range(2))}
    for p in procs:
        p.join(timeout=60)
    assert got["rank0"][1].startswith("PeerLostError: rank 1 left"), got
    assert "out of data" in got["rank0"][1] and got["rank0"][2] == 1
