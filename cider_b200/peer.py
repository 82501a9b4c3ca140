"""Peer-memory group for the one-shot all-reduce of the tensor-parallel decode step.

One process per GPU.  Every rank allocates an inbox in its own device memory
(``cider_peer_alloc``), the 64-byte IPC handles are exchanged through
``torch.distributed`` (plumbing only), and every rank maps the inboxes of its peers
(``cider_peer_open``).  ``all_reduce`` then is one kernel of this library per call
(``cider_allreduce_f16``): peer stores over NVLink, a bounded wait on local flags, an
fp32 sum in rank order - no NCCL inside, so a decode step that uses it can be captured
and replayed as a CUDA graph.  The reference has no multi-device path; the loop this
serves is vlm_service/custom_qwen3vl.py:660-679.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib


class PeerGroup:
    def __init__(self, rank: int, world: int, device=None, group=None, inbox_bytes: int = 4 << 20,
                 wait_cycles: int = 0):
        import torch.distributed as dist
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.inbox_bytes, self.wait_cycles = int(inbox_bytes), int(wait_cycles)
        self.lib = _lib.load()
        self.max_bytes = int(self.lib.cider_peer_max_bytes(self.inbox_bytes))
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cider_peer_alloc(self.inbox_bytes, ctypes.byref(own), handle))
        self._own = own.value
        handles = [None] * world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self._mapped = []
        ptrs = []
        for q in range(world):
            if q == rank:
                ptrs.append(self._own)
                continue
            p = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[q])
            with torch.cuda.device(self.device):
                _lib.check(self.lib.cider_peer_open(buf, ctypes.byref(p)))
            self._mapped.append(p.value)
            ptrs.append(p.value)
        self._table = (ctypes.c_void_p * world)(*ptrs)
        dist.barrier(group=group)  # every inbox exists, is zero and is mapped everywhere

    def fits(self, t: torch.Tensor) -> bool:
        return (t.dtype == torch.float16 and t.is_contiguous() and t.numel() % 8 == 0
                and 0 < t.numel() * 2 <= self.max_bytes)

    def all_reduce(self, x: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Sum of ``x`` (fp16, contiguous, numel % 8 == 0, at most ``max_bytes``) over the ranks;
        every rank gets the same bits.  All ranks must make the same sequence of calls."""
        if not self.fits(x):
            raise ValueError("PeerGroup.all_reduce: need a contiguous fp16 tensor of a multiple of 8 elements "
                             f"and at most {self.max_bytes} bytes")
        if out is None:
            out = torch.empty_like(x)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cider_allreduce_f16(x.data_ptr(), out.data_ptr(), x.numel(), self.rank, self.world,
                                                    self._table, self.inbox_bytes, self.wait_cycles,
                                                    int(torch.cuda.current_stream(self.device).cuda_stream)))
        return out

    def fits_norm(self, partial: torch.Tensor) -> bool:
        """Shapes the fused all-reduce + residual add + RMSNorm (+ quantiser) kernel takes."""
        return (partial.dim() == 2 and self.fits(partial) and 1 <= partial.shape[0] <= 32
                and partial.shape[1] % 8 == 0 and partial.shape[1] <= 8192)

    def all_reduce_add_rmsnorm(self, partial: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
                               want_fp16: bool = True, want_int8: bool = False):
        """``delta = all_reduce(partial)``, ``x <- x + delta`` in place, RMSNorm of x - one kernel.
        Returns (y fp16 or None, q int8 or None, scale or None) like ``ops.add_rmsnorm``."""
        if not self.fits_norm(partial):
            raise ValueError("PeerGroup.all_reduce_add_rmsnorm: shape not supported")
        if x.dtype != torch.float16 or not x.is_contiguous() or x.shape != partial.shape:
            raise ValueError("PeerGroup.all_reduce_add_rmsnorm: x must be a contiguous fp16 tensor of the partial's shape")
        M, K = partial.shape
        wh = weight if (weight.dtype == torch.float16 and weight.is_contiguous()) else weight.to(torch.float16).contiguous()
        y = torch.empty_like(x) if want_fp16 else None
        q = torch.empty((M, K), dtype=torch.int8, device=x.device) if want_int8 else None
        s = torch.empty((M,), dtype=torch.float32, device=x.device) if want_int8 else None
        ptr = lambda t: None if t is None else t.data_ptr()  # noqa: E731
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cider_allreduce_add_rmsnorm_quant(
                partial.data_ptr(), x.data_ptr(), wh.data_ptr(), float(eps), M, K, ptr(y), ptr(q), ptr(s),
                self.rank, self.world, self._table, self.inbox_bytes, self.wait_cycles,
                int(torch.cuda.current_stream(self.device).cuda_stream)))
        return y, q, s

    def reset(self):
        """After a time-out: all ranks clear their flags and counters between two host barriers."""
        import torch.distributed as dist
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            _lib.check(self.lib.cider_peer_reset(self._own, None))
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)

    def close(self):
        """Unmap the peers' inboxes, then (after a barrier: nobody may still have it mapped or be
        writing to it) free the own one.  Call between steps, with no kernel in flight."""
        import torch.distributed as dist
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for p in self._mapped:
                self.lib.cider_peer_close(p)
            self._mapped = []
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
            self.lib.cider_peer_free(self._own)
        self._own = None
