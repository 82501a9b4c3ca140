#!/usr/bin/env python
"""Headline benchmark: W8A8 per-channel linear at M=8192, [N=10240, K=2560].

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path (per-token quantise -> int8 tcgen05 GEMM
with the fused dequant epilogue) over one batch of 8192 synthetic tokens.
Prints ONE JSON line (rank 0).  Keys:

  value      whole-job int8 TOP/s (2*M*N*K per step per GPU), inputs resident in
             HBM, timed on the device with CUDA events, max over ranks
  e2e        the same metric through the public host-buffer op
             (cider_b200.ops.perchannel_linear_host) with pinned HOST buffers: H2D of x
             and D2H of y inside the timed region
  roofline   the dominant kernel (the GEMM) against the tensor roofline: achieved =
             2*M*N*K / its mean launch time (events around each launch, live);
             peak = 2 x the measured dense bf16 TF/s in MEASURED_PEAKS.json (int8
             dense is twice bf16 on this part; no int8 figure is measured)
  cpu_baseline  the CPU oracle (a port of the reference's semantics; the
             reference itself has no CPU path) on a bounded row sample
  clocks     SM clock / throttle reasons sampled through NVML while the step runs
             (a 0.25 s untimed pre-roll of the same step plus the timed region)

Multi-GPU (torchrun, one rank per GPU): tokens are the independent unit, so each
rank runs the full-size step on its own batch with no collective ("weak").
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N, K = 8192, 10240, 2560
WORKLOAD = "W8A8 per-channel linear, M=8192 tokens x [N=10240, K=2560], fp16 in/out"
OPS_PER_STEP = 2.0 * M * N * K
METRIC = "W8A8 GEMM int8 TOPS"
# dram__bytes_read.sum + dram__bytes_write.sum of one GEMM launch at this size,
# from the ncu capture summarised in profiles/gemm_tc_perchannel_M8192_N10240_K2560.md
GEMM_DRAM_TRAFFIC_BYTES = 175.0e6
CPU_SAMPLE_ROWS = 2048


def make_inputs(seed: int):
    """Seeded synthetic stand-ins for the reference's bench_full.py randn data:
    x ~ N(0,1) with 8 outlier channels x20 (fp16), W ~ N(0, 0.02) quantised per
    output channel to int8."""
    import numpy as np
    import torch
    from cider_b200 import ops
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:8]] *= 20
    x = x.to(torch.float16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.float16).float().numpy()
    wq, sw = ops.quantize_weight_int8(w)
    return x, torch.from_numpy(wq), torch.from_numpy(sw), np


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML (read only)."""

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksThrottleReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def measured_peaks(power_capped: bool):
    """int8 dense peak for the roofline: no int8 figure is measured on this pool,
    so it is 2 x the measured dense bf16 figure (int8 is twice bf16 on B200) - the
    sustained one when the run sat under the power cap, else the burst one."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        if power_capped and "bf16_tflops_sustained" in p:
            return 2.0 * float(p["bf16_tflops_sustained"]), \
                "2 x measured bf16 sustained (MEASURED_PEAKS.json; sw_power_cap was active)"
        return 2.0 * float(p["bf16_tflops"]), "2 x measured bf16 burst (MEASURED_PEAKS.json)"
    except Exception:
        return (2.0 * 1400.0, "2 x fallback bf16 sustained (1.4 PF)") if power_capped else \
            (2.0 * 1590.0, "2 x fallback bf16 burst (1.59 PF)")


def cpu_sample(x, wq, sw, rows: int, reps: int):
    """Time the CPU oracle (port of the reference semantics, all host threads)
    on the first `rows` tokens of the workload.  Returns (TOP/s, threads, s/rep)."""
    import oracle
    xs = x[:rows].numpy()
    wn, sn = wq.numpy(), sw.numpy()
    oracle.c_perchannel_linear(xs[:64], wn, sn)  # warm (page-in, thread pool)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        oracle.c_perchannel_linear(xs, wn, sn)
        times.append(time.perf_counter() - t0)
    best = min(times)
    return 2.0 * rows * N * K / best / 1e12, oracle.num_threads(), best


def run_reference(args, rank: int, world: int):
    """Reference arm: the reference has no CPU (or CUDA) implementation of this
    path - its primitives' eval_cpu throws and its kernels are Metal - so the arm
    times the CPU oracle, a port of its semantics, on the host cores."""
    if rank != 0:
        return
    x, wq, sw, _ = make_inputs(0)
    # one step ~1 s of wall time on 8 cores; shrink the sample for long runs
    rows = CPU_SAMPLE_ROWS if args.steps <= 100 else CPU_SAMPLE_ROWS // 4
    import oracle
    # all the host's cores, also under torchrun (which exports OMP_NUM_THREADS=1)
    oracle.set_num_threads(len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1))
    xs, wn, sn = x[:rows].numpy(), wq.numpy(), sw.numpy()
    for _ in range(max(args.warmup, 1)):
        oracle.c_perchannel_linear(xs[:256], wn, sn)
    steps = max(1, args.steps)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.c_perchannel_linear(xs, wn, sn)
    dt = (time.perf_counter() - t0) / steps
    tops = 2.0 * rows * N * K / dt / 1e12
    sample = f"first {rows} of {M} tokens per step, {steps} steps"
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": tops, "unit": "TOP/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    from cider_b200 import _lib, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not ops.is_available():
        raise RuntimeError("bench.py needs a B200 and the built cider_b200 CUDA library (no fallback)")
    lib = _lib.load()
    x, wq, sw, np = make_inputs(rank)
    xd = [x.to(dev), x.flip(0).contiguous().to(dev)]  # two activation buffers, alternated
    wd, sd = wq.to(dev), sw.to(dev)
    y = torch.empty((M, N), dtype=torch.float16, device=dev)
    a_q = torch.empty((M, K), dtype=torch.int8, device=dev)
    s_a = torch.empty((M,), dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream(dev)
    sp = int(stream.cuda_stream)

    def step(i, ev=None):
        xi = xd[i & 1]
        _lib.check(lib.cider_quantize_per_token(xi.data_ptr(), M, K, K, a_q.data_ptr(), s_a.data_ptr(), sp))
        if ev is not None:
            ev[0].record(stream)
        _lib.check(lib.cider_linear_prequantized(a_q.data_ptr(), s_a.data_ptr(), wd.data_ptr(), sd.data_ptr(),
                                                 _lib.F32, 0, None, y.data_ptr(), M, N, K, sp))
        if ev is not None:
            ev[1].record(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()

    # ---- device-timed region
    gemm_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
               for _ in range(args.steps)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank)
    sampler.start()
    # untimed pre-roll of the same step under the sampler: NVML answers in
    # milliseconds, the timed region alone is too short for more than a sample or two
    t_pre = time.perf_counter()
    i = 0
    while time.perf_counter() - t_pre < 0.25:
        step(i)
        i += 1
        if i % 50 == 0:
            torch.cuda.synchronize(dev)
    barrier()
    e0.record(stream)
    for i in range(args.steps):
        step(i, gemm_ev[i])
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    dev_ms = e0.elapsed_time(e1)
    gemm_ms = sum(a.elapsed_time(b) for a, b in gemm_ev) / args.steps

    # ---- end to end through the public op, host buffers in and out
    e2e_steps = max(1, min(args.steps, 20))
    xh = [x.pin_memory(), x.flip(0).contiguous().pin_memory()]
    yh = torch.empty((M, N), dtype=torch.float16).pin_memory()

    def e2e_step(i):
        # the public host-buffer op: chunked upload / quantise + GEMM / download, returns
        # when the result is in yh
        ops.perchannel_linear_host(xh[i & 1], wd, sd, out=yh)

    for i in range(2):
        e2e_step(i)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(stream)
    for i in range(e2e_steps):
        e2e_step(i)
    f1.record(stream)
    barrier()
    e2e_ms = f0.elapsed_time(f1)

    st = __import__("ctypes").c_uint(0)
    lib.cider_device_status(st)
    if st.value != 0:
        raise RuntimeError(f"a kernel recorded a bounded-wait time-out (status {st.value})")

    t = torch.tensor([dev_ms, e2e_ms, gemm_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, gemm_ms = t.tolist()
    if rank != 0:
        return
    value = OPS_PER_STEP * args.steps * world / (dev_ms * 1e-3) / 1e12
    e2e_val = OPS_PER_STEP * e2e_steps * world / (e2e_ms * 1e-3) / 1e12
    peak, peak_src = measured_peaks("sw_power_cap" in clocks.get("reasons", []))
    achieved = OPS_PER_STEP / (gemm_ms * 1e-3) / 1e12
    # CPU baseline on rank 0 at N=1 only (torchrun pins OMP threads; the reference arm covers N>1)
    cpu = None
    if world == 1:
        cpu_tops, cores, cpu_s = cpu_sample(x, wq, sw, CPU_SAMPLE_ROWS, 3)
        cpu = {"value": cpu_tops, "unit": "TOP/s", "cores": cores, "kind": "port",
               "sample": f"first {CPU_SAMPLE_ROWS} of {M} tokens, best of 3 ({cpu_s:.2f} s each)"}
    line = {
        "metric": METRIC, "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": {"workload": WORKLOAD, "parallelism": f"dp{world} (tokens sharded, no collective)",
                   "l2": "x + W + y = 236 MB per step exceed the 126 MB L2; x alternates between 2 buffers",
                   "ops": "2*M*N*K int8 multiply-adds per step per GPU"},
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "traffic": GEMM_DRAM_TRAFFIC_BYTES,
                     "kernel": "gemm_tc_pair_kernel<per-channel> (256x256 tile per CTA pair)", "peak_source": peak_src,
                     "gemm_ms": gemm_ms, "nominal_int8_dense_tops": 4500.0},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_val, "unit": "TOP/s", "h2d_bytes_per_step": M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    try:
        run_ours(args, rank, world, local_rank)
    finally:
        if world > 1:
            import torch.distributed as dist
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
