"""The allocation-free entry point, cider_perchannel_linear_noalloc.

Some callers cannot allocate device memory at the point where they need a
linear layer - a plugin inside a host program that has already handed out all
of its memory, or a latency-critical path that must not run into cudaMalloc's
device-wide synchronisation - so they cannot give the regular entry point the
scratch buffer it asks for.  For them the library carries a fixed scratch array
of its own.  This test calls that entry point through the C ABI and requires
the same fp16 output as the regular entry point (the integer sums are exact and
the dequantising arithmetic is the same whichever kernel runs, so identical bits;
the suite's 2e-3 bar is asserted as well) and as the CPU oracle, several times in
a row with different shapes, so that every later call runs on an array still
holding the earlier calls' bytes.  The shapes cover the tensor-core tiles, a shape
for which the regular entry point splits K (the allocation-free one does not),
the weight-streaming kernel for a handful of rows (M = 8) and the M == 1
matrix-vector path.  It also checks the property in the entry point's name: the
device's free memory is the same before and after the calls.  It is collected
last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import numpy as np
import pytest
import torch

from conftest import make_activations, make_weight, rel_err

pytestmark = pytest.mark.gpu

TOL = 2e-3
DEV = "cuda:0"


def _regular(lib, _lib, x, w, sw, bias, M, N, K, stream):
    y = torch.empty((M, N), dtype=torch.float16, device=DEV)
    nbytes = lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, M, N, K)
    ws = torch.empty(max(nbytes, 1), dtype=torch.uint8, device=DEV)
    _lib.check(lib.cider_perchannel_linear(x.data_ptr(), w.data_ptr(), sw.data_ptr(),
                                           None if bias is None else bias.data_ptr(), y.data_ptr(),
                                           M, N, K, ws.data_ptr() if nbytes else None, nbytes, stream))
    return y


def _noalloc(lib, _lib, x, w, sw, bias, M, N, K, stream):
    y = torch.empty((M, N), dtype=torch.float16, device=DEV)
    _lib.check(lib.cider_perchannel_linear_noalloc(x.data_ptr(), w.data_ptr(), sw.data_ptr(),
                                                   None if bias is None else bias.data_ptr(),
                                                   y.data_ptr(), M, N, K, stream))
    return y


CASES = [(300, 1024, 2560, True), (37, 520, 1152, False), (8, 1032, 2560, True), (128, 256, 8192, False),
         (1, 256, 512, True)]


def test_noalloc_matches_regular_entry_point_twice(oracle):
    from cider_b200 import _lib, ops
    assert ops.is_available()
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = int(torch.cuda.current_stream().cuda_stream)
    # calls in a row; later ones are smaller, so most of the scratch they do not
    # overwrite still holds an earlier call's activations
    for call, (M, N, K, use_bias) in enumerate(CASES):
        xn = make_activations(M, K, seed=100 + call)
        x = torch.from_numpy(xn).to(DEV)
        wq, sw = ops.quantize_weight_int8(make_weight(N, K, seed=200 + call))
        w, s = torch.from_numpy(wq).to(DEV), torch.from_numpy(sw).to(DEV)
        bias = bn = None
        if use_bias:
            bn = (np.random.default_rng(call).standard_normal(N) * 0.05).astype(np.float16)
            bias = torch.from_numpy(bn).to(DEV)
        got = _noalloc(lib, _lib, x, w, s, bias, M, N, K, stream)
        want = _regular(lib, _lib, x, w, s, bias, M, N, K, stream)
        torch.cuda.synchronize()
        assert rel_err(got.cpu().numpy(), want.cpu().numpy()) <= TOL
        assert torch.equal(got, want), f"call {call}: outputs differ"
        ref = oracle.c_perchannel_linear(xn, wq, sw, bn)
        assert rel_err(got.cpu().numpy(), ref) <= TOL
        if M > 1:  # quantised path: the oracle's bits; M == 1 sums fp32 in a free order
            assert np.array_equal(got.cpu().numpy(), ref), f"call {call}: differs from the oracle"


def test_noalloc_leaves_free_device_memory_unchanged():
    """Free device memory (cudaMemGetInfo) is the same before and after the calls.  Inputs
    and outputs are allocated beforehand and one call per shape has already run, so that
    neither torch's allocator nor the CUDA runtime's lazy kernel loading moves the figure."""
    from cider_b200 import _lib, ops
    lib = _lib.load()
    torch.cuda.set_device(0)
    stream = int(torch.cuda.current_stream().cuda_stream)
    prepared = []
    for call, (M, N, K, _) in enumerate(CASES):
        x = torch.from_numpy(make_activations(M, K, seed=300 + call)).to(DEV)
        wq, sw = ops.quantize_weight_int8(make_weight(N, K, seed=400 + call))
        y = torch.empty((M, N), dtype=torch.float16, device=DEV)
        prepared.append((x, torch.from_numpy(wq).to(DEV), torch.from_numpy(sw).to(DEV), y, M, N, K))

    def run_all():
        for x, w, s, y, M, N, K in prepared:
            _lib.check(lib.cider_perchannel_linear_noalloc(x.data_ptr(), w.data_ptr(), s.data_ptr(), None,
                                                           y.data_ptr(), M, N, K, stream))
        torch.cuda.synchronize()

    run_all()  # loads every kernel involved, resolves the scratch address
    free_before, _ = torch.cuda.mem_get_info(0)
    run_all()
    run_all()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_before, f"free device memory moved by {free_before - free_after} bytes"


def test_noalloc_rejects_sizes_beyond_its_scratch():
    from cider_b200 import _lib
    lib = _lib.load()
    one = ctypes.c_void_p(256)  # never dereferenced: the size check comes first
    rc = lib.cider_perchannel_linear_noalloc(one, one, one, None, one, 4096, 64, 4096, None)
    assert rc == _lib.E_WORKSPACE
    msg = _lib.last_error()
    assert "built-in scratch" in msg and "8388608" in msg
    rc = lib.cider_perchannel_linear_noalloc(one, one, one, None, one, 20000, 64, 64, None)
    assert rc == _lib.E_WORKSPACE and "16384" in _lib.last_error()
    assert lib.cider_perchannel_linear_noalloc(one, one, one, None, one, 0, 64, 64, None) == 0
