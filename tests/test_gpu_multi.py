"""Data-parallel step on real GPUs over NCCL: G ranks, each with an even shard of ONE global batch, must reproduce the
single-GPU gradients of that batch (only the order of the fp32 sums over samples differs).  Needs at least two GPUs;
skipped otherwise.  The CPU twin of this test (gloo, the kernel replaced by the oracle) is tests/test_dp_cpu.py."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, q):
    import torch.distributed as dist
    from oracle import ring_oracle as orc
    from rnn_train_ring_attractor_b200 import dp
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dp.init_process_group("nccl", timeout_s=120.0, rank=rank, world_size=world, device_id=dev)
    out = {}
    for name, (N, B, T, act, prec) in {"bf16": (256, 1024, 24, "gelu", "bf16"), "fp32": (120, 256, 40, "tanh", "fp32")}.items():
        case = orc.make_case(N, B, T, act, seed=4)
        Wa, Wo = case.Wa.to(dev), case.Wo.to(dev)
        fn = dp.fused_step_fn(Wa, case.J0, case.J1, Wo, case.alpha, act, precision=prec)
        local = tuple(dp.shard_rows(t, rank, world).to(dev) for t in (case.A, case.r_init, case.target))
        loss, views = dp.train_step(fn, local, N, 2, B, T)
        if rank == 0:
            full = tuple(t.to(dev) for t in (case.A, case.r_init, case.target))
            buf1 = torch.empty(dp.grad_buffer_numel(N, 2), dtype=torch.float32, device=dev)
            parts = fn(full, 1.0 / (B * T), buf1)          # the whole batch on one GPU, no exchange
            one = dp.split_grad_buffer(buf1, N, 2)
            loss1 = parts[0] + 0.2 * parts[1]
            out[name] = dict(loss=abs(float(loss) - float(loss1)) / max(1.0, abs(float(loss1))),
                             dWo=orc.rel_err(views["dWo"], one["dWo"]), dWa=orc.rel_err(views["dWa"], one["dWa"]),
                             dJ0=abs(float(views["dJ"][0]) - float(one["dJ"][0])) / max(abs(float(one["dJ"][0])), 1e-30))
    dist.barrier()
    if rank == 0:
        q.put(out)
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_sharded_gradients_equal_single_gpu_gradients(world, achieved):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs, found {torch.cuda.device_count()}")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = q.get(timeout=600)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for name, e in out.items():
        achieved(f"{world} GPUs vs 1 GPU, same global batch, {name} mode", **e)
        assert e["loss"] < 1e-6 and e["dWo"] < 1e-5 and e["dWa"] < 1e-5, (name, e)
