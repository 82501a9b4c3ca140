"""Decode-attention timing: python -m cider_b200.sdpa_bench [B Hq Hkv D T]

One launch of the split-K single-query attention over a random fp16 KV cache, timed
with CUDA events over a CUDA graph of 8 calls; prints microseconds and the cache
bytes per second (2 * T * Hkv * D * 2 bytes per sequence).  The calls rotate over
enough distinct caches that their total exceeds twice the 126 MB L2 (a decoder's
layers each have their own cache), and every kernel form is timed: the automatic
choice, the CUDA-core form and the tensor-core form (where the shape has one)."""
import statistics
import sys

import torch

from . import _lib, ops

L2_BYTES = 126 * 1024 * 1024


def main():
    B, Hq, Hkv, D, T = (int(a) for a in sys.argv[1:6]) if len(sys.argv) >= 6 else (8, 32, 8, 128, 2054)
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    q = torch.randn(B, Hq, D, device=dev, generator=g).half()
    nbytes = 2 * T * Hkv * D * 2 * B
    copies = max(1, -(-2 * L2_BYTES // nbytes))
    copies = (copies + 7) // 8 * 8 if copies > 1 else 1
    kcs = [torch.randn(B, Hkv, T + 2, D, device=dev, generator=g).half() for _ in range(copies)]
    vcs = [torch.randn(B, Hkv, T + 2, D, device=dev, generator=g).half() for _ in range(copies)]
    tickets = torch.zeros(B * Hkv, dtype=torch.int32, device=dev)
    scale = D ** -0.5
    lib = _lib.load()
    calls = max(8, copies)
    for mode, name in ((0, "automatic"), (1, "CUDA-core"), (2, "tensor-core")):
        lib.cider_testing_set_sdpa_kernel(mode)
        for use_tickets in (False, True):
            fn = lambda i: ops.sdpa_decode(q, kcs[i % copies], vcs[i % copies], T, scale,
                                           tickets=tickets if use_tickets else None)
            for i in range(3):
                fn(i)
            torch.cuda.synchronize()
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
            ts = []
            for _ in range(15):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                graph.replay()
                e1.record()
                e1.synchronize()
                ts.append(e0.elapsed_time(e1) * 1e3 / calls)
            us = statistics.median(ts)
            print(f"B={B} Hq={Hq} Hkv={Hkv} D={D} T={T} {name:11s} "
                  f"{'one launch (tickets)' if use_tickets else 'partial + combine  '}: "
                  f"{us:.1f} us, {nbytes / us / 1e3:.0f} GB/s of cache ({copies} caches in rotation)", flush=True)
    lib.cider_testing_set_sdpa_kernel(0)


if __name__ == "__main__":
    main()
