#!/usr/bin/env python
"""Headline benchmark: W8A8 per-channel linear at M=8192, [N=10240, K=2560], plus the
decoder throughput half of the metric as sub-records.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--decoder 0|1]

One "step" is one pass of the hot path (per-token quantise -> int8 tcgen05 GEMM with the
fused dequant epilogue) over one batch of 8192 synthetic tokens.  Prints ONE JSON line
(rank 0).  Keys:

  value      whole-job int8 TOP/s (2*M*N*K per step), inputs resident in HBM, timed on the
             device with CUDA events, max over ranks
  e2e        the same metric through the public host-buffer op
             (cider_b200.ops.perchannel_linear_host) with pinned HOST buffers: H2D of x and
             D2H of y inside the timed region
  roofline   the dominant kernel (the GEMM) against the tensor roofline: achieved =
             2*M*N*K / its mean launch time (events around each launch, live); peak = 2 x
             the measured dense bf16 TF/s in MEASURED_PEAKS.json (int8 dense is twice bf16
             on this part; no int8 figure is measured).  frac_burst and frac_sustained are
             both printed; frac is the burst one unless the timed region lasted a second or
             more.  yardstick = cuBLASLt's int8 GEMM (torch._int_mm) timed on the same
             operands with the same events: a measured int8 ceiling of this box, reported
             beside the kernel, not used by it
  cpu_baseline  the CPU oracle (a port of the reference's semantics; the reference itself
             has no CPU path) on a bounded row sample
  decoder_c3 (N=1)  Qwen3-VL-2B-architecture decoder, W8A8 per-channel against the same
             decoder with fp16 torch linears: prefill tok/s at 1334 / 2393 / 3455 prompt
             tokens, 256 greedy decode steps each, and the ratios
  decoder_c4_tp     Qwen3-8B-architecture decoder, W8A8 per-group gs=128, batch 8 x 2048 prompt
             tokens + 128 decode steps, tensor-parallel over the N GPUs of the run
  clocks     SM clock / throttle reasons sampled through NVML while the step runs

Multi-GPU (torchrun, one rank per GPU): the ONE linear is split over output channels -
rank r owns W[r*N/g:(r+1)*N/g], its scales and its slice of y; x is replicated; no data-path
collective.  The total work is fixed ("strong").
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
# dram__bytes_read.sum + dram__bytes_write.sum of one full-size GEMM launch (one ncu capture
# of this kernel at this size); a slice of the output channels moves its share of W and y
GEMM_DRAM_TRAFFIC_BYTES = 175.0e6
CPU_SAMPLE_ROWS = 2048
C3_PROMPTS = (1334, 2393, 3455)


def config_for(world: int) -> dict:
    par = "1 GPU" if world == 1 else f"output channels split over {world} GPUs (N/{world} each), x replicated, no collective"
    return {"workload": WORKLOAD, "parallelism": par,
            "l2": "x + W + y = 236 MB per step exceed the 126 MB L2; x alternates between 2 buffers",
            "ops": "2*M*N*K int8 multiply-adds per step"}


def make_inputs(seed: int, quantize_weight):
    """Seeded synthetic stand-ins for the reference's bench_full.py randn data:
    x ~ N(0,1) with 8 outlier channels x20 (fp16), W ~ N(0, 0.02) quantised per
    output channel to int8."""
    import torch
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:8]] *= 20
    x = x.to(torch.float16)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.float16).float().numpy()
    wq, sw = quantize_weight(w)
    return x, torch.from_numpy(wq), torch.from_numpy(sw)


class ClockSampler(threading.Thread):
    """Samples SM clock and clock-event reasons of one GPU through NVML (read only)."""

    def __init__(self, index: int, period_s: float = 0.002):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], {}, None
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
                        self.reasons[name] = self.reasons.get(name, 0) + 1
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        if self.is_alive():
            self.join(timeout=1.0)
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "reason_samples": dict(self.reasons)}


def measured_peaks():
    """int8 dense peak for the roofline: no int8 figure is measured on this pool, so it is
    2 x the measured dense bf16 figure (int8 is twice bf16 on B200).  Returns
    (burst, sustained, source)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return (2.0 * float(p["bf16_tflops"]), 2.0 * float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "2 x measured bf16 (MEASURED_PEAKS.json)")
    except Exception:
        return 2.0 * 1590.0, 2.0 * 1400.0, "2 x fallback bf16 (1.59 PF burst, 1.4 PF sustained)"


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
    times the CPU oracle, a port of its semantics, on the host cores.  Nothing of the
    cider_b200 package is imported here."""
    if rank != 0:
        return
    import oracle
    x, wq, sw = make_inputs(0, oracle.np_quantize_weight_int8)
    # one step ~1 s of wall time on 8 cores; shrink the sample for long runs
    rows = CPU_SAMPLE_ROWS if args.steps <= 100 else CPU_SAMPLE_ROWS // 4
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
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_for(world),
        "cpu_baseline": {"value": tops, "unit": "TOP/s", "cores": oracle.num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": tops, "unit": "TOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def decoder_c3(local_rank: int) -> dict:
    """Qwen3-VL-2B architecture, batch 1: W8A8 per-channel against fp16 torch linears."""
    import torch
    from cider_b200.decoder_bench import run_decoder
    out = {"model": "Qwen3-VL-2B architecture, random init, batch 1, 1024 vision positions + text, 256 greedy steps",
           "tok_s_definition": "prompt tokens / time to first token; generated tokens / time after it"}
    for mode in ("w8a8", "fp16"):
        dec = _c3_decoder(mode, local_rank)
        rec = {"prefill_tok_s": {}, "decode_tok_s": {}}
        for T in C3_PROMPTS:
            r, _ = run_decoder("qwen3vl2b", mode, prompt=T, decode=256, repeat=2, local=local_rank, dec=dec)
            rec["prefill_tok_s"][str(T)] = r["prefill_tok_s"]
            rec["decode_tok_s"][str(T)] = r["decode_tok_s"]
        out[mode] = rec
        del dec
        torch.cuda.empty_cache()
    out["prefill_ratio_vs_fp16"] = {k: out["w8a8"]["prefill_tok_s"][k] / out["fp16"]["prefill_tok_s"][k]
                                    for k in out["w8a8"]["prefill_tok_s"]}
    out["decode_ratio_vs_fp16"] = {k: out["w8a8"]["decode_tok_s"][k] / out["fp16"]["decode_tok_s"][k]
                                   for k in out["w8a8"]["decode_tok_s"]}
    return out


def _c3_decoder(mode: str, local_rank: int):
    from cider_b200.decoder import QWEN3_VL_2B, Decoder
    return Decoder(QWEN3_VL_2B, mode=mode, group_size=0, device=f"cuda:{local_rank}",
                   max_len=max(C3_PROMPTS) + 256 + 8, batch=1)


def decoder_c4(rank: int, world: int, local_rank: int) -> dict:
    """Qwen3-8B architecture, W8A8 gs=128, batch 8 x 2048 + 128 decode steps, tensor-parallel
    over the run's GPUs (column-parallel q/k/v and gate/up, row-parallel o/down + all-reduce:
    NCCL for the prefill messages, the library's peer-memory kernel inside the captured decode step)."""
    import torch
    from cider_b200.decoder_bench import run_decoder
    peer = None
    if world > 1:
        from cider_b200.peer import PeerGroup
        peer = PeerGroup(rank, world, device=torch.device("cuda", local_rank))
    try:
        r, dec = run_decoder("qwen3_8b", "w8a8", group_size=128, batch=8, prompt=2048, decode=128, repeat=1,
                             rank=rank, world=world, local=local_rank, peer=peer)
        del dec
    finally:
        if peer is not None:
            peer.close()
    torch.cuda.empty_cache()
    return {"model": "Qwen3-8B architecture, random init, W8A8 per-group gs=128, batch 8 x 2048 prompt + 128 steps",
            "tp": world, "prefill_tok_s": r["prefill_tok_s"], "decode_tok_s": r["decode_tok_s"],
            "decode_graph": r["graph"],
            "allreduce": "none" if world == 1 else "NCCL (prefill) + one-shot peer-memory kernel (decode)"}


def run_ours(args, rank: int, world: int, local_rank: int):
    import torch
    import torch.distributed as dist
    from cider_b200 import _lib, ops

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if not ops.is_available():
        raise RuntimeError("bench.py needs a B200 and the built cider_b200 CUDA library (no fallback)")
    if N % (world * 256) != 0:
        raise RuntimeError(f"N={N} does not split into {world} slices of whole 256-column tiles")
    lib = _lib.load()
    x, wq, sw = make_inputs(0, ops.quantize_weight_int8)
    Ns = N // world  # this rank's output channels
    sl = slice(rank * Ns, (rank + 1) * Ns)
    xd = [x.to(dev), x.flip(0).contiguous().to(dev)]  # two activation buffers, alternated
    wd, sd = wq[sl].contiguous().to(dev), sw[sl].contiguous().to(dev)
    y = torch.empty((M, Ns), dtype=torch.float16, device=dev)
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
                                                 _lib.F32, 0, None, y.data_ptr(), M, Ns, K, sp))
        if ev is not None:
            ev[1].record(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    warm = max(args.warmup, 3)
    for i in range(warm):
        step(i)
    barrier()
    kernel_name = lib.cider_testing_last_gemm_kernel().decode()

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

    # ---- yardstick: the vendor library's int8 GEMM on the same operands, same events
    yard = None
    try:
        wt = wd.t()  # [K, Ns] column-major view: the layout cuBLASLt's int8 GEMM takes
        c32 = torch.empty((a_q.shape[0], wt.shape[1]), dtype=torch.int32, device=dev)  # one result buffer: no allocator traffic inside the timed loop
        for _ in range(3):
            torch._int_mm(a_q, wt, out=c32)
        torch.cuda.synchronize(dev)
        y0, y1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = max(5, min(args.steps, 50))
        y0.record(stream)
        for _ in range(reps):
            torch._int_mm(a_q, wt, out=c32)
        y1.record(stream)
        torch.cuda.synchronize(dev)
        yard_ms = y0.elapsed_time(y1) / reps
        del c32
        yard = {"what": "torch._int_mm (cuBLASLt int8 -> int32, no dequant epilogue, int32 output)",
                "ms": yard_ms, "tops": 2.0 * M * Ns * K / (yard_ms * 1e-3) / 1e12}
    except Exception as exc:  # not a product path: report and go on
        yard = {"what": "torch._int_mm", "unavailable": str(exc)[:200]}

    # ---- end to end through the public op, host buffers in and out
    e2e_steps = max(1, min(args.steps, 20))
    xh = [x.pin_memory(), x.flip(0).contiguous().pin_memory()]
    yh = torch.empty((M, Ns), dtype=torch.float16).pin_memory()

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
    del xh, yh

    st = __import__("ctypes").c_uint(0)
    lib.cider_device_status(st)
    if st.value != 0:
        raise RuntimeError(f"a kernel recorded a time-out or an overflow (status {st.value})")

    t = torch.tensor([dev_ms, e2e_ms, gemm_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms, gemm_ms = t.tolist()

    # ---- the decoder half of the metric (sub-records; every rank takes part in the TP run)
    del xd, y, a_q, s_a
    torch.cuda.empty_cache()
    c3 = c4 = None
    if args.decoder:
        if world == 1:
            c3 = decoder_c3(local_rank)
        c4 = decoder_c4(rank, world, local_rank)
        lib.cider_device_status(st)
        if st.value != 0:
            raise RuntimeError(f"a decoder kernel recorded a time-out or an overflow (status {st.value})")
    if rank != 0:
        return
    value = OPS_PER_STEP * args.steps / (dev_ms * 1e-3) / 1e12
    e2e_val = OPS_PER_STEP * e2e_steps / (e2e_ms * 1e-3) / 1e12
    peak_burst, peak_sust, peak_src = measured_peaks()
    achieved = (OPS_PER_STEP / world) / (gemm_ms * 1e-3) / 1e12  # per GPU, against the per-GPU peak
    sustained_region = dev_ms >= 1000.0
    peak = peak_sust if sustained_region else peak_burst
    # CPU baseline on rank 0 at N=1 only (torchrun pins OMP threads; the reference arm covers N>1)
    cpu = None
    if world == 1:
        cpu_tops, cores, cpu_s = cpu_sample(x, wq, sw, CPU_SAMPLE_ROWS, 3)
        cpu = {"value": cpu_tops, "unit": "TOP/s", "cores": cores, "kind": "port",
               "sample": f"first {CPU_SAMPLE_ROWS} of {M} tokens, best of 3 ({cpu_s:.2f} s each)"}
    line = {
        "metric": METRIC, "value": value, "unit": "TOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warm, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "int8", "data": "synthetic",
        "config": config_for(world),
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                     "frac": achieved / peak, "frac_burst": achieved / peak_burst,
                     "frac_sustained": achieved / peak_sust, "peak_burst": peak_burst, "peak_sustained": peak_sust,
                     "peak_choice": ("sustained: the timed region lasted a second or more" if sustained_region else
                                     f"burst: the timed region lasted {dev_ms:.1f} ms"),
                     "traffic": GEMM_DRAM_TRAFFIC_BYTES * (26.2 / world + 21.0 + 168.0 / world) / 215.2,
                     "kernel": kernel_name, "peak_source": peak_src + ", of measured",
                     "gemm_ms": gemm_ms, "per_gpu": True, "nominal_int8_dense_tops": 4500.0,
                     "yardstick": yard},
        "cpu_baseline": cpu,
        "e2e": {"value": e2e_val, "unit": "TOP/s", "h2d_bytes_per_step": world * M * K * 2,
                "d2h_bytes_per_step": M * N * 2, "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                "note": "bytes are job totals: every rank uploads x, each downloads its slice of y"},
        "gpu_launches": 2 * args.steps,
        "clocks": clocks,
        "decoder_c3": c3,
        "decoder_c4_tp": c4,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--decoder", type=int, default=1, help="0: leave the decoder sub-records out (quick run)")
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
        # the exchange of the tensor-parallel decoder runs over plain NVLink peer traffic
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
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
