"""Operator latency sweep - the shapes of the reference's README table
(benchmarks/bench_full.py:17-27: M in {1,128,1024,4096,8192} x [N=10240,K=2560] and
[N=2560,K=10240]) for W8A8 per-channel, per-group gs=128 / gs=64 and W4A8.

    python -m cider_b200.sweep [--quick] [--json out.jsonl]

Each row is the whole linear (quantise + GEMM + dequant, or the matrix-vector
kernel for M == 1) through the public op, timed with CUDA events: 5 warm-ups, then
the median of 20 (the reference's protocol, bench_full.py:13-14,30-38), each sample
being a CUDA graph of 8 consecutive calls.  To keep
the numbers HBM-honest the op rotates over enough distinct weight copies that
their total exceeds the 126 MB L2 (an M == 1 call otherwise measures L2, not HBM).
Reports latency, int8 TOP/s (2*M*N*K), weight-stream GB/s for M == 1 and the
fraction of the matching roofline (2 x measured bf16 dense for compute rows, the
measured HBM copy rate for M == 1).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics

import numpy as np
import torch

from . import ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
L2_BYTES = 126 * 1024 * 1024


def _peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return 2.0 * p["bf16_tflops"], float(p["hbm_gbs"]), "measured"
    except Exception:
        return 2.0 * 1590.0, 6650.0, "fallback"


def _time(fn, warmup=5, repeat=20, calls=8, graph=True):
    """Median / min microseconds per call.  ``calls`` consecutive calls (rotating
    over the weight copies) are captured in one CUDA graph so that the Python and
    launch overhead of a ~5 us kernel does not end up in its number; the graph is
    replayed ``repeat`` times between CUDA events."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if not graph:  # plain launches between events (what a profiler capture wants: few launches)
        ts = []
        for r in range(repeat):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn(r)
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(ts), min(ts)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn(0)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(calls):
            fn(i)
    graph.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(repeat):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        ts.append(e0.elapsed_time(e1) * 1e3 / calls)
    del graph
    return statistics.median(ts), min(ts)


def make_case(mode: str, M: int, N: int, K: int, dev, seed=0):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(M, K, generator=g)
    x[:, torch.randperm(K, generator=g)[:8]] *= 20
    x = x.to(torch.float16).to(dev)
    w = (torch.randn(N, K, generator=g) * 0.02).to(torch.float16).float().to(dev)
    wbytes = N * K // 2 if mode.startswith("w4a8") else N * K
    copies = max(1, -(-2 * L2_BYTES // wbytes)) if M <= 128 else 1
    copies = (copies + 7) // 8 * 8 if copies > 1 else 1  # a multiple of the calls per graph
    from .decoder import quantize_weight_int8_torch, quantize_weight_pergroup_torch
    if mode == "pc":
        q, s = quantize_weight_int8_torch(w)
        ws = [(q.clone(), s) for _ in range(copies)]
        return lambda i: ops.perchannel_linear(x, ws[i % copies][0], ws[i % copies][1]), copies
    if mode.startswith("gs"):
        gs = int(mode[2:])
        q, s = quantize_weight_pergroup_torch(w, gs, torch.float16)
        ws = [(q.clone(), s) for _ in range(copies)]
        return lambda i: ops.pergroup_linear(x, ws[i % copies][0], ws[i % copies][1], gs), copies
    if mode in ("w4a8_rows", "w4a8_rows_gs64", "w4a8_rows_int8copy", "w4a8_rows_gs64_int8copy"):
        copy = mode.endswith("_int8copy")  # lend N*K bytes: int8 copy + int8 kernels beyond decode sizes
        wn = w.t().contiguous().cpu().numpy()
        if "gs64" not in mode:
            p, s = ops.pack_weight_int4(wn)
            gs = 0
        else:
            p, s = ops.pack_weight_int4_pergroup(wn, 64)
            gs = 64
        rows, s = ops.w4a8_repack(torch.from_numpy(p).to(dev)), torch.from_numpy(s).to(dev)
        ws = [rows.clone() for _ in range(copies)]
        return lambda i: ops.w4a8_linear_rows(x, ws[i % copies], s, group_size=gs, int8_scratch=copy), copies
    if mode in ("w4a8", "w4a8_gs64"):
        wn = w.t().contiguous().cpu().numpy()
        if mode == "w4a8":
            p, s = ops.pack_weight_int4(wn)
            gs = 0
        else:
            p, s = ops.pack_weight_int4_pergroup(wn, 64)
            gs = 64
        p, s = torch.from_numpy(p).to(dev), torch.from_numpy(s).to(dev)
        ws = [p.clone() for _ in range(copies)]
        return lambda i: ops.w4a8_linear(x, ws[i % copies], s, group_size=gs), copies
    raise ValueError(mode)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--quick", action="store_true", help="M in {1,128,8192} and the first shape only")
    ap.add_argument("--json", default=None)
    ap.add_argument("--modes", default="pc,gs128,gs64,w4a8,w4a8_gs64,w4a8_rows,w4a8_rows_gs64")
    ap.add_argument("--ms", default=None, help="comma-separated M values instead of the table's")
    ap.add_argument("--shape", default=None, help="N,K of the one shape to run instead of the table's two")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeat", type=int, default=20)
    ap.add_argument("--graph", type=int, default=1,
                    help="0: time single plain launches (short runs for a profiler capture; launch overhead included)")
    args = ap.parse_args()
    assert ops.is_available(), "needs a B200 and the built CUDA library"
    dev = torch.device("cuda", torch.cuda.current_device())
    tpeak, hbm, src = _peaks()
    shapes = [(10240, 2560), (2560, 10240)]
    Ms = [1, 128, 1024, 4096, 8192]
    if args.quick:
        shapes, Ms = shapes[:1], [1, 128, 8192]
    if args.ms:
        Ms = [int(v) for v in args.ms.split(",")]
    if args.shape:
        shapes = [tuple(int(v) for v in args.shape.split(","))]
    rows = []
    print(f"# peaks ({src}): int8 tensor {tpeak:.0f} TOP/s (2 x bf16), HBM {hbm:.0f} GB/s")
    print(f"{'mode':10s} {'N':>6s} {'K':>6s} {'M':>5s} {'median us':>10s} {'min us':>8s} {'TOP/s':>8s} {'GB/s':>8s} {'frac':>6s}")
    for mode in args.modes.split(","):
        for (N, K) in shapes:
            if mode.startswith("w4a8") and (N, K) != (10240, 2560):
                continue
            for M in Ms:
                fn, copies = make_case(mode, M, N, K, dev)
                med, mn = _time(fn, args.warmup, args.repeat, calls=max(8, copies), graph=bool(args.graph))
                tops = 2.0 * M * N * K / (med * 1e-6) / 1e12
                wbytes = N * K // 2 if mode.startswith("w4a8") else N * K
                gbs = (wbytes + 2 * M * K + 2 * M * N) / (med * 1e-6) / 1e9
                frac = gbs / hbm if M <= 128 else tops / tpeak
                row = {"mode": mode, "N": N, "K": K, "M": M, "median_us": med, "min_us": mn, "tops": tops,
                       "gbs": gbs, "frac": frac, "bound": "hbm" if M <= 128 else "tensor", "weight_copies": copies}
                rows.append(row)
                print(f"{mode:10s} {N:6d} {K:6d} {M:5d} {med:10.1f} {mn:8.1f} {tops:8.1f} {gbs:8.0f} {frac:6.2f}",
                      flush=True)
                del fn
                torch.cuda.empty_cache()
    if args.json:
        with open(args.json, "w") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
