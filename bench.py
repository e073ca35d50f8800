"""Benchmark of the ring-attractor training step (fused forward + loss + backward-through-time).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c3]

Metric: fwd+bwd sample-timesteps/s (= B*T / step time) at N=512, B=4096, T=512, GELU (workload "c3").
A step is one pass of the hot path over one synthetic batch: forward recurrence, decode + loss, reverse-time
recurrence, weight-gradient products and (N > 1) one all-reduce of the gradient buffer.  With N GPUs the ONE global
batch of the configuration (4096 samples for c3, generated from one seed) is sharded evenly by rows, rank r taking
rows [r*B/N, (r+1)*B/N) -- strong scaling, as the configuration is worded; --scaling weak gives every rank a full
per-GPU batch instead.  The line carries the loss and checksums of the all-reduced gradients, which are the same
numbers at every N up to fp32 summation order.

`value`  : inputs already resident in HBM, timed with CUDA events on the launching stream.
`e2e`    : the same step through the public Python API with inputs in pinned HOST memory (H2D copies and the
           D2H read of the loss inside the timed region).
`roofline`: dominant kernel class (per-kernel CUDA-event times recorded by the library inside the timed
           region) against the measured bf16 tensor peak of MEASURED_PEAKS.json.
`cpu_baseline` / --impl reference: the CPU oracle's reference-shaped PyTorch step (W_eff materialised per
           step, autograd) on the host cores, on a bounded slice of the same workload.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "c1": dict(N=120, B=128, T=120, act="tanh", max_av=0.1 * math.pi, cpu_slice=(128, 120)),
    "c2": dict(N=256, B=1024, T=256, act="relu", max_av=0.1 * math.pi, cpu_slice=(64, 32)),
    "c3": dict(N=512, B=4096, T=512, act="gelu", max_av=0.1 * math.pi, cpu_slice=(64, 16)),
    # defined on 8 GPUs (global batch 8192): B is the per-GPU shard, so --gpus 8 runs exactly the named configuration
    "c4": dict(N=1024, B=1024, T=2000, act="tanh", max_av=0.05 * math.pi, cpu_slice=(16, 8), defined_on=8),
    # forward-only rollout with the ideal cosine weights; decoded-angle error against the integrated target
    "c5": dict(N=120, B=65536, T=4000, act="tanh", max_av=0.1 * math.pi, cpu_slice=(1024, 200), rollout=True),
}
# DRAM bytes (read + write) per sample-timestep of each bf16-mode kernel, from the ncu captures summarised under
# profiles/ (N=512: T=64, B=4096; N=1024: T=32, B=1024, a case of about the size of L2, so its write figures are a
# lower bound; traffic is proportional to B*T).  None = no capture for that kernel/mode.
NCU_CAPTURE_SOURCE = {512: "ncu captures at T=64 summarised in profiles/{fwd,bwd}_tc_kernel_c3_T64.md, gemm_tc_kernel_dw_c3_T64.md",
                      1024: "ncu captures at T=32 summarised in profiles/{fwd,bwd}_tc_kernel_c4_T32.md (lower bound: part of the writes was still in L2)"}
NCU_DRAM_BYTES_PER_SAMPLE_STEP = {
    ("bf16", 512): {"fwd_recurrent": (16.50e6 + 545.05e6) / (4096 * 64), "bwd_recurrent": (309.09e6 + 751.43e6) / (4096 * 64),
                    "dw_product": (1073.80e6 + 4.66e6) / (4096 * 64)},
    ("bf16", 1024): {"fwd_recurrent": (13.56e6 + 96.37e6) / (1024 * 32), "bwd_recurrent": (83.09e6 + 147.29e6) / (1024 * 32)},
}
METRIC = "fwd+bwd sample-timesteps/s"
UNIT = "sample-timesteps/s"


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    # no driver-written file: an earlier measurement on the same pool (burst figure only)
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}, "fallback"


class ClockSampler:
    """nvidia-smi sampling (200 ms) of SM clock and throttle reasons while a timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, smax = [], set(), None
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1]))
                    smax = float(f[2])
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                     f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = sorted(sm)[len(sm) // 2:]  # upper half: samples under load
            out.update(sm_mhz=sorted(busy)[len(busy) // 2], sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm))
        return out


def cpu_reference_step_rate(wl, steps, warmup, threads=None):
    """Reference-shaped PyTorch step (oracle) on the host cores on a bounded slice; sample-timesteps/s."""
    from oracle import ring_oracle as orc
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    Bs, Ts = wl["cpu_slice"]
    Bs, Ts = min(Bs, wl["B"]), min(Ts, wl["T"])
    case = orc.make_case(wl["N"], Bs, Ts, wl["act"], seed=0, max_av=wl["max_av"])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        orc.train_step_ref(case, lean=False)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    per = sum(times) / len(times)
    sample = f"slice B={Bs}, T={Ts} of N={wl['N']}, B={wl['B']}, T={wl['T']} ({wl['act']}), fp32, torch {torch.__version__}"
    return Bs * Ts / per, per * 1e3, threads, sample


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rate, ms, threads, sample = cpu_reference_step_rate(wl, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": rate, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={wl['N']}, B={wl['B']}, T={wl['T']}, {wl['act']}, fwd+loss+bwd",
                   "sample": sample},
        "cpu_baseline": {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": rate, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def circular_error(a, b):
    d = torch.abs(a - b) % (2 * math.pi)
    return torch.minimum(d, 2 * math.pi - d)


def run_rollout(args, wl):
    """Forward-only workload: sample-timesteps/s of the rollout + decoded-angle error (mean and final step)."""
    from rnn_train_ring_attractor_b200 import _lib
    from rnn_train_ring_attractor_b200.build import build
    from rnn_train_ring_attractor_b200.fused import ring_rnn_rollout
    from rnn_train_ring_attractor_b200.inputs import benchmark_inputs
    from rnn_train_ring_attractor_b200.ring_rnn_cuda import choose_precision
    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise RuntimeError("the rollout workload is a single-GPU configuration")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    build()
    L = _lib.lib()
    N, B, T, act = wl["N"], wl["B"], wl["T"], wl["act"]
    prec = "bf16" if choose_precision(B, T, N, 2, _lib.ACT[act], 2, args.precision) == 1 else "fp32"
    host = benchmark_inputs(N, B, T, seed=1000, max_av=wl["max_av"], weights="ideal")
    pinned = {k: host[k].pin_memory() for k in ("A", "r_init")}
    Wa, Wo, target = host["Wa"].to(dev), host["Wo"].to(dev), host["target"].to(dev)
    resident = {k: pinned[k].to(dev) for k in pinned}

    def fwd(ins):
        return ring_rnn_rollout(ins["A"], Wa, host["J0"], host["J1"], Wo, ins["r_init"], 0.1, act, precision=prec)

    def timed(fn, steps):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / steps

    for _ in range(max(1, args.warmup)):
        decoded, _ = fwd(resident)
    err = circular_error(decoded, target)
    err_mean, err_final = float(err.mean()), float(err[:, -1].mean())
    L.ringrnn_timing_reset()
    L.ringrnn_timing_enable(1)
    sampler = ClockSampler(0)
    sampler.start()
    ms = timed(lambda: fwd(resident), args.steps)
    L.ringrnn_timing_enable(0)
    launches = int(L.ringrnn_launch_count())
    kern = _lib.timing_snapshot()

    def e2e_step():
        ins = {k: pinned[k].to(dev, non_blocking=True) for k in pinned}
        d, _ = fwd(ins)
        return float(circular_error(d[:, -1], target[:, -1]).mean())

    e2e_step()
    ms_e2e = timed(e2e_step, max(1, args.steps // 2))
    clocks = sampler.stop()
    peaks, peak_src = measured_peaks()
    ms_launch = kern["fwd_recurrent"][0] / max(1, kern["fwd_recurrent"][1])
    achieved = 6.0 * N * N * B * T / (ms_launch * 1e-3) / 1e12
    peak = float(peaks.get("bf16_tflops_sustained", peaks.get("bf16_tflops")))
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import ring_oracle as orc
        torch.set_num_threads(os.cpu_count() or 1)
        Bs, Ts = wl["cpu_slice"]
        c = {k: host[k][:Bs, :Ts].contiguous() if host[k].dim() > 1 and host[k].shape[0] == B else host[k]
             for k in ("A", "r_init", "target")}
        c["r_init"] = host["r_init"][:Bs].contiguous()
        t0 = time.perf_counter()
        with torch.no_grad():
            hist = orc.ring_forward_ref(c["A"], host["Wa"], host["J0"], host["J1"], host["Wo"], c["r_init"], 0.1, act)
        dt = time.perf_counter() - t0
        ref_dec = orc.decode_angle(hist)
        cpu = {"value": Bs * Ts / dt, "unit": UNIT, "cores": os.cpu_count(), "kind": "port",
               "sample": f"slice B={Bs}, T={Ts}, forward only, no_grad",
               "decoded_vs_oracle_mean_abs_err": float(circular_error(decoded[:Bs, :Ts].cpu(), ref_dec).mean())}
    line = {
        "metric": "forward sample-timesteps/s", "value": B * T / (ms * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16" if prec == "bf16" else "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={N}, B={B}, T={T}, {act}, alpha=0.1, ideal cosine weights, "
                               f"forward-only rollout with per-step population-vector decode, precision mode {prec}"},
        "decoded_angle_error": {"mean_rad": err_mean, "final_step_rad": err_final},
        "e2e": {"value": B * T / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": sum(v.numel() * 4 for v in pinned.values()), "d2h_bytes_per_step": 4},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "tensor", "kernel": "fwd_recurrent", "achieved": achieved, "peak": peak,
                     "unit": "TFLOP/s", "frac": achieved / peak, "traffic": None,
                     "peak_source": f"{peak_src} (sustained bf16 GEMM)", "ms_per_launch": ms_launch},
        "cpu_baseline": cpu,
    }
    print(json.dumps(line), flush=True)


# The reference's own published table (assets/REPORT.md, RTX PRO 6000 Blackwell, forward op latency at B=256, T=20):
# (N, a_dim, "CUDA" fp32 kernel ms, "CUDA WMMA" ms or None)
PUBLISHED_FORWARD_MS = [
    (128, 16, 0.372, 0.282), (256, 16, 0.897, 0.595), (384, 16, 1.755, 1.269), (512, 16, 2.795, 1.772),
    (1024, 16, 10.172, 6.163), (2048, 16, 46.110, 24.455), (2048, 32, 76.646, 36.741), (2048, 64, 139.247, 62.792),
    (1024, 2, 10.112, None), (1024, 3, 10.129, None), (1024, 6, 10.744, None), (1024, 12, 10.549, None),
]


def run_published_table(args):
    """Forward op latency on the shapes of the reference's published table, measured the way the reference measures
    (utils/benchmark.py:58-79: 2 warm-up calls, then 20 calls each bracketed by CUDA events and a synchronize), through
    the reference's own entry point ring_rnn_cuda_func.  Action signal as legacy/model_fp32.py:116-124
    (relu(av * linspace(-1, 1, a_dim))): every column is active somewhere in the batch.  One JSON line."""
    from rnn_train_ring_attractor_b200.build import build
    from rnn_train_ring_attractor_b200.inputs import generate_av, initial_bump_von_mises
    from rnn_train_ring_attractor_b200.ring_rnn_cuda import ring_rnn_cuda_func, set_precision
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    build()
    B, T = 256, 20
    rows = []
    for N, a_dim, ref_fp32_ms, ref_wmma_ms in PUBLISHED_FORWARD_MS:
        g = torch.Generator().manual_seed(N + a_dim)
        av, angle = generate_av(B, T, generator=g)
        A = torch.relu(av.unsqueeze(-1) * torch.linspace(-1, 1, a_dim)).contiguous().to(dev)
        Wa = (torch.randn(a_dim, N, N, generator=g) / math.sqrt(N)).to(dev)
        Wo = (torch.randn(N, N, generator=g) / math.sqrt(N)).to(dev)
        r0 = initial_bump_von_mises(angle[:, 0], N).to(dev)
        row = {"N": N, "a_dim": a_dim, "reference_fp32_ms": ref_fp32_ms, "reference_wmma_ms": ref_wmma_ms}
        # the fp32 parity mode is timed on the smaller shapes only (seconds per call at N = 2048)
        for mode in (("auto", "fp32") if N <= 512 else ("auto",)):
            set_precision(mode)
            with torch.no_grad():
                for _ in range(2):
                    ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.15, "tanh")
                torch.cuda.synchronize()
                times = []
                for _ in range(20):
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    ring_rnn_cuda_func(A, Wa, -0.1, 0.1, Wo, r0, 0.15, "tanh")
                    e1.record()
                    torch.cuda.synchronize()
                    times.append(e0.elapsed_time(e1))
            tt = torch.tensor(times)
            row["ms_" + mode] = float(tt.mean())
            row["std_" + mode] = float(tt.std(unbiased=False))
        set_precision("auto")
        rows.append(row)
    print(json.dumps({"metric": "forward op latency on the reference's published shapes", "unit": "ms", "B": B, "T": T,
                      "reference_hardware": "RTX PRO 6000 Blackwell (published, other hardware)", "rows": rows}),
          flush=True)


def run_timeline(args, wl):
    """In-kernel timeline of one CTA of the forward and of the reverse-time kernel (diagnostic; needs the library built by
    `python -m rnn_train_ring_attractor_b200.build --timeline`).  Prints, for a few steps in the steady state, the cycle
    at which each role passed each point of a step, relative to the step's first stamp:
      mma: pass start / first own chunk present / second half or pass start / accumulator 0, 1 committed
      epilogue (warp 4): accumulator 0, 1 seen complete / read out / arithmetic of sub-slice 1 done / peers' slots free /
      chunk published;  WAIT_W, WAIT_A: cycles the MMA-issuing thread spent waiting for weight stages and state chunks."""
    import ctypes as C
    from rnn_train_ring_attractor_b200 import _lib
    from rnn_train_ring_attractor_b200.build import TIMELINE_LIB
    if not os.path.exists(TIMELINE_LIB):
        raise RuntimeError("build the diagnostic library first: python -m rnn_train_ring_attractor_b200.build --timeline")
    _lib.LIB_PATH = TIMELINE_LIB
    from rnn_train_ring_attractor_b200.fused import ring_rnn_fused
    from rnn_train_ring_attractor_b200.inputs import benchmark_inputs
    torch.cuda.set_device(0)
    N, B, T, act = wl["N"], wl["B"], min(wl["T"], 64), wl["act"]
    d = benchmark_inputs(N, B, T, seed=0, max_av=wl["max_av"], device="cuda")
    for _ in range(2):
        Wa, Wo = d["Wa"].clone().requires_grad_(True), d["Wo"].clone().requires_grad_(True)
        loss, _, _, _ = ring_rnn_fused(d["A"], Wa, -0.1, 0.1, Wo, d["r_init"], 0.1, act, d["target"], precision="bf16")
        loss.backward()
    torch.cuda.synchronize()
    h = C.CDLL(TIMELINE_LIB)
    names = {"forward": ["mma:start", "mma:own_chunk", "mma:2nd_half", "mma:commit0", "mma:commit1", "epi:dfull0", "epi:read0",
                         "epi:dfull1", "epi:read1", "epi:math1_done", "epi:slots_free", "epi:published"],
             "reverse": ["mma:start", "mma:own_chunks", "mma:pass1", "mma:commit0", "mma:commit1", "epi:dfull0", "epi:read0",
                         "epi:dfull1", "epi:read1", "epi:carry_done", "epi:slots_free", "epi:DL_written", "epi:published"]}
    out = {"workload": f"{args.workload}: N={N}, B={B}, T={T}, {act}", "unit": "SM cycles relative to the step's first stamp"}
    for kernel, fn in (("forward", h.ringrnn_debug_timeline_read), ("reverse", h.ringrnn_debug_timeline_read_bwd)):
        buf = (C.c_longlong * (64 * 16))()
        if fn(buf) != 0:
            raise RuntimeError("reading the timeline failed")
        steps = []
        for g in (20, 21, 22, 40):
            base = buf[g * 16]
            # a point the kernel variant does not pass leaves its slot unstamped
            row = {n: (int(buf[g * 16 + i] - base) if 0 <= buf[g * 16 + i] - base < 10 ** 9 else None)
                   for i, n in enumerate(names[kernel])}
            row.update(step=g, next_step_start=int(buf[(g + 1) * 16] - base), WAIT_W=int(buf[g * 16 + 13]), WAIT_A=int(buf[g * 16 + 14]))
            steps.append(row)
        out[kernel] = steps
    print(json.dumps(out), flush=True)


def run_ours(args, wl):
    import torch.distributed as dist
    from rnn_train_ring_attractor_b200 import _lib, dp
    from rnn_train_ring_attractor_b200.build import build
    from rnn_train_ring_attractor_b200.inputs import benchmark_inputs
    from rnn_train_ring_attractor_b200.ring_rnn_cuda import choose_precision

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device; there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    if rank == 0:
        build()
    if world > 1:
        dist.barrier()
    L = _lib.lib()

    N, T, act = wl["N"], wl["T"], wl["act"]
    scaling = args.scaling or ("weak" if "defined_on" in wl else "strong")
    if scaling == "strong":
        if wl["B"] % world:
            raise RuntimeError(f"global batch {wl['B']} does not divide over {world} ranks")
        B_global, B_local = wl["B"], wl["B"] // world
    else:
        B_global, B_local = wl["B"] * world, wl["B"]
    prec_code = choose_precision(B_local, T, N, 2, _lib.ACT[act], 2, args.precision)
    prec = "bf16" if prec_code == 1 else "fp32"

    # one global batch and one set of weights from seed 0 on every rank; the rank keeps its rows
    host = benchmark_inputs(N, B_global, T, seed=0, max_av=wl["max_av"])
    for k in ("A", "r_init", "target"):
        host[k] = dp.shard_rows(host[k], rank, world)
    pinned = {k: host[k].pin_memory() for k in ("A", "r_init", "target")}
    Wa, Wo = host["Wa"].to(dev), host["Wo"].to(dev)
    resident = tuple(pinned[k].to(dev) for k in ("A", "r_init", "target"))
    buf = torch.empty(dp.grad_buffer_numel(N, 2), dtype=torch.float32, device=dev)
    step_fn = dp.fused_step_fn(Wa, host["J0"], host["J1"], Wo, 0.1, act, precision=prec, ckpt_every=args.ckpt_every)

    def step(inputs):
        return dp.train_step(step_fn, inputs, N, 2, B_global, T, buf=buf)

    def sync_all():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / steps

    # ---- device-resident value --------------------------------------------------------------------------
    for _ in range(max(1, args.warmup)):
        loss, grads = step(resident)
    torch.cuda.synchronize()
    # the all-reduced gradients of the one global batch: the same at every GPU count up to fp32 summation order
    checksum = {"dWo_norm": float(grads["dWo"].double().norm()), "dWa_norm": float(grads["dWa"].double().norm()),
                "dWo_sum": float(grads["dWo"].double().sum()), "dJ0": float(grads["dJ"][0]), "dJ1": float(grads["dJ"][1])}
    L.ringrnn_timing_reset()
    L.ringrnn_timing_enable(1)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms_step = timed(lambda: step(resident), args.steps)
    L.ringrnn_timing_enable(0)
    launches = int(L.ringrnn_launch_count())
    kern = _lib.timing_snapshot()
    loss_value = float(loss)

    # ---- end to end: pinned host inputs -> loss on the host ------------------------------------------
    h2d = sum(pinned[k].numel() * 4 for k in pinned)

    # Double-buffered: while step i computes, a copy stream brings step i+1's inputs from pinned host memory, as a
    # training loop would.  Every step still pays one H2D copy of (A, r_init, target) and one D2H read of the loss.
    keys = ("A", "r_init", "target")
    copy_stream = torch.cuda.Stream(device=dev)
    bufs = [{k: torch.empty_like(pinned[k], device=dev) for k in keys} for _ in range(2)]
    ready = [torch.cuda.Event(), torch.cuda.Event()]
    free = [torch.cuda.Event(), torch.cuda.Event()]
    for ev in free:
        ev.record()
    counter = {"i": 0}

    def issue_copy(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(free[slot])
            for k in keys:
                bufs[slot][k].copy_(pinned[k], non_blocking=True)
            ready[slot].record(copy_stream)

    issue_copy(0)

    def e2e_step():
        slot = counter["i"] & 1
        issue_copy(slot ^ 1)
        torch.cuda.current_stream().wait_event(ready[slot])
        l, _ = step(tuple(bufs[slot][k] for k in keys))
        free[slot].record()
        counter["i"] += 1
        return float(l)  # device -> host read of the step's result

    for _ in range(max(2, args.warmup // 2)):
        e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    clocks = sampler.stop()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    # ---- roofline of the dominant kernel class ----------------------------------------------------------
    peaks, peak_src = measured_peaks()
    # Algorithmic work of each kernel class per step: 6*N*N flop per sample-timestep for each of the forward
    # contraction, the delta propagation and the weight-gradient products.  With checkpoints a class runs in several
    # launches per step (one per stretch, plus the recompute in the forward class, whose work is not counted):
    # achieved = the class's algorithmic flops per step / the class's time per step.
    flops_per_class = 6.0 * N * N * B_local * T
    cand = {k: v for k, v in kern.items() if k in ("fwd_recurrent", "bwd_recurrent", "dw_product") and v[1] > 0}
    dom = max(cand, key=lambda k: cand[k][0]) if cand else None
    roof = None
    if dom:
        ms_class = cand[dom][0] / args.steps
        launches_per_step = cand[dom][1] / args.steps
        achieved = flops_per_class / (ms_class * 1e-3) / 1e12
        sustained = "bf16_tflops_sustained" in peaks
        peak = float(peaks["bf16_tflops_sustained"] if sustained else peaks["bf16_tflops"])
        cap = NCU_DRAM_BYTES_PER_SAMPLE_STEP.get((prec, N), {}).get(dom) if not args.ckpt_every else None
        traffic = cap * B_local * T / launches_per_step if cap is not None else None
        roof = {"bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                "frac": achieved / peak, "traffic": traffic,
                "traffic_source": NCU_CAPTURE_SOURCE.get(N) if traffic is not None else None,
                "peak_source": f"{peak_src} ({'sustained' if sustained else 'burst'} bf16 GEMM)",
                "ms_per_launch": ms_class / launches_per_step, "launches_per_step": launches_per_step,
                "kernels_ms_per_step": {k: v[0] / args.steps for k, v in kern.items() if v[1] > 0},
                # the recurrence is sequential: time per timestep of each recurrent kernel, the floor that batch
                # sharding cannot lower
                "us_per_timestep": {k: 1e3 * cand[k][0] / args.steps / T for k in ("fwd_recurrent", "bwd_recurrent")
                                    if k in cand}}

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        rate, _, threads, sample = cpu_reference_step_rate(wl, steps=3, warmup=1)
        cpu = {"value": rate, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample}

    value = B_global * T / (ms_step * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
        "dtype": "bf16" if prec == "bf16" else "f32", "data": "synthetic",
        "config": {"workload": f"{args.workload}: N={N}, B={B_local} per GPU, T={T}, {act}, alpha=0.1, "
                               f"fused fwd+loss+bwd, precision mode {prec}"
                               + (f", state checkpoints every {args.ckpt_every} steps + recompute in backward"
                                  if args.ckpt_every else "")
                               + (f" (the configuration is defined on {wl['defined_on']} GPUs, global batch "
                                  f"{wl['B'] * wl['defined_on']}; this run has {world})"
                                  if wl.get("defined_on", world) != world and scaling == "weak" else ""),
                   "global_batch": B_global, "parallelism": f"dp{world}",
                   "l2": "working set (saved states + delta, several GB) exceeds the 126 MB L2; no flush needed"},
        "e2e": {"value": B_global * T / (ms_e2e * 1e-3), "unit": UNIT, "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "how": "public API ring_rnn_fused via dp.train_step; inputs in pinned host memory, H2D double-buffered on a "
                       "copy stream, loss read back every step"},
        "gpu_launches": launches, "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "loss": loss_value,
        "grad_checksum": checksum,
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["published"])
    ap.add_argument("--precision", default="auto", choices=["auto", "bf16", "fp32"])
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="default: strong (the one global batch sharded over the GPUs); weak for the workload that is "
                         "defined by its per-GPU shard (c4)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--seq-len", type=int, default=0, help="override T (profiling on a smaller case of the same kernels)")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch (profiling)")
    ap.add_argument("--timeline", action="store_true",
                    help="diagnostic: print the in-kernel timeline of the recurrent kernels (needs the --timeline build)")
    ap.add_argument("--ckpt-every", type=int, default=0,
                    help="keep the state every K steps and recompute in backward (0 = keep every step)")
    args = ap.parse_args()
    if args.workload == "published":
        run_published_table(args)
        return
    wl = dict(WORKLOADS[args.workload])
    if args.seq_len:
        wl["T"] = args.seq_len
    if args.batch:
        wl["B"] = args.batch
    if args.timeline:
        run_timeline(args, wl)
    elif args.impl == "reference":
        run_reference(args, wl)
    elif wl.get("rollout"):
        run_rollout(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
