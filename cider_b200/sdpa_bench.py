"""Decode-attention timing: python -m cider_b200.sdpa_bench [B Hq Hkv D T]

One launch of the split-K single-query attention over a random fp16 KV cache, timed
with CUDA events over a CUDA graph of 8 calls; prints microseconds and the cache
bytes per second (2 * T * Hkv * D * 2 bytes per sequence)."""
import statistics
import sys

import torch

from . import ops


def main():
    B, Hq, Hkv, D, T = (int(a) for a in sys.argv[1:6]) if len(sys.argv) >= 6 else (8, 32, 8, 128, 2054)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, Hq, D, device=dev, generator=g).half()
    kc = torch.randn(B, Hkv, T + 2, D, device=dev, generator=g).half()
    vc = torch.randn(B, Hkv, T + 2, D, device=dev, generator=g).half()
    tickets = torch.zeros(B * Hkv, dtype=torch.int32, device=dev)
    scale = D ** -0.5
    for use_tickets in (False, True):
        fn = lambda: ops.sdpa_decode(q, kc, vc, T, scale, tickets=tickets if use_tickets else None)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            fn()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(8):
                fn()
        ts = []
        for _ in range(15):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / 8)
        us = statistics.median(ts)
        nbytes = 2 * T * Hkv * D * 2 * B
        print(f"B={B} Hq={Hq} Hkv={Hkv} D={D} T={T} {'one launch (tickets)' if use_tickets else 'partial + combine'}: "
              f"{us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of cache")


if __name__ == "__main__":
    main()
