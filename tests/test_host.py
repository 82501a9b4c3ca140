"""Host-side logic and the C-ABI boundary, without a GPU.

Covers: every symbol declared in include/cider_b200.h is exported by the built
library; argument validation returns error codes before anything is launched;
the numpy weight-quant helpers of cider_b200.ops reproduce the reference's
(golden fixtures); module constructors / convert_model behave like the
reference's off supported hardware.
"""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import cider_b200
from cider_b200 import _lib, nn as cnn, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _declared_symbols():
    names = set()
    for header in ("cider_b200.h", "cider_b200_testing.h"):
        text = open(os.path.join(ROOT, "include", header)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names |= set(re.findall(r"\b(cider_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/*.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes table and header disagree"
    assert lib.cider_version() >= 100


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setenv("CIDER_B200_LIB", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.load()
    monkeypatch.delenv("CIDER_B200_LIB")
    monkeypatch.setattr(_lib, "_lib", None)
    _lib.load()


def test_workspace_bytes():
    lib = _lib.load()
    assert lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, 1, 10240, 2560) == 0  # M == 1: no scratch
    assert lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, 128, 10240, 2560) == 128 * 2560 + 512
    # few output tiles and a long K: the per-channel linear also gets int32 split-K slabs
    # (20 tiles of 128 x 128 -> 7 splits of the 80 K blocks, rows padded to 128)
    assert lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, 128, 2560, 10240) == 128 * 10240 + 512 + 7 * 128 * 2560 * 4
    assert lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, 100, 2560, 10240) == 100 * 10240 + 512 + 7 * 128 * 2560 * 4
    # per-group split-K: 5 equal K pieces of fp32 slabs (the size does not depend on the group size)
    assert lib.cider_workspace_bytes(_lib.OP_PERGROUP, 128, 2560, 10240) == 128 * 10240 + 512 + 5 * 128 * 2560 * 4
    assert lib.cider_workspace_bytes(_lib.OP_PERGROUP, 128, 10240, 2560) == 128 * 2560 + 512
    assert lib.cider_workspace_bytes(_lib.OP_PERCHANNEL, 1024, 2560, 10240) == 1024 * 10240 + 4096  # M > 512
    # W4A8: the reference packing is transposed into rows (N*K/2); rows need no weight scratch,
    # except K the row kernels do not take (K < 128 or K % 32 != 0: an int8 copy)
    assert lib.cider_workspace_bytes(_lib.OP_W4A8, 1, 512, 256) == 256 + 256 + 512 * 128
    assert lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS, 1, 512, 256) == 256 + 256
    assert lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS, 8192, 10240, 2560) == 8192 * 2560 + 8192 * 4
    assert lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS_INT8COPY, 8192, 10240, 2560) == 8192 * 2560 + 8192 * 4 + 10240 * 2560
    assert lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS, 4, 512, 80) == 512 + 256 + 512 * 80
    assert lib.cider_workspace_bytes(_lib.OP_W4A8, 4, 512, 80) == 512 + 256
    assert lib.cider_workspace_bytes(99, 8, 8, 8) == 0
    assert lib.cider_sdpa_decode_workspace_bytes(1, 16, 8, 128, 4096) > 0


def test_validation_never_launches():
    """Bad arguments come back as status codes (no CUDA call is reached, so this
    runs on a machine without a GPU)."""
    lib = _lib.load()
    one = ctypes.c_void_p(16)  # any non-null, never dereferenced
    rc = lib.cider_pergroup_linear(one, one, one, _lib.F32, None, one, 4, 64, 128, 32, None, 0, None)
    assert rc == _lib.E_SHAPE and "group_size" in _lib.last_error()
    rc = lib.cider_pergroup_linear(one, one, one, _lib.F32, None, one, 4, 64, 192, 128, None, 0, None)
    assert rc == _lib.E_SHAPE and "multiple" in _lib.last_error()
    rc = lib.cider_perchannel_linear(None, one, one, None, one, 4, 64, 128, None, 0, None)
    assert rc == _lib.E_INVALID
    rc = lib.cider_perchannel_linear(one, one, one, None, one, 4, 0, 128, None, 0, None)
    assert rc == _lib.E_INVALID
    rc = lib.cider_perchannel_linear(one, one, one, None, one, 4, 64, 128, None, 0, None)
    assert rc == _lib.E_WORKSPACE and "workspace" in _lib.last_error()
    rc = lib.cider_perchannel_linear(one, one, one, None, one, 4, 64, 128, ctypes.c_void_p(8), 1 << 20, None)
    assert rc == _lib.E_ALIGNMENT
    rc = lib.cider_w4a8_linear(one, one, one, _lib.F32, 0, one, 4, 64, 127, None, 0, None)
    assert rc == _lib.E_SHAPE
    rc = lib.cider_w4a8_linear(one, one, one, 7, 0, one, 4, 64, 128, None, 0, None)
    assert rc == _lib.E_INVALID
    rc = lib.cider_quantize_per_token(one, 4, 64, 32, one, one, None)
    assert rc == _lib.E_INVALID  # ldx < K
    rc = lib.cider_sdpa_decode(one, one, one, one, 1, 6, 4, 128, 8, 8, 1.0, None, 0, None, None)
    assert rc == _lib.E_SHAPE
    rc = lib.cider_set_gemm_backend(5)
    assert rc == _lib.E_INVALID
    assert lib.cider_testing_set_tile(7, 0) == _lib.E_INVALID and lib.cider_testing_set_tile(0, 100) == _lib.E_INVALID
    assert lib.cider_testing_set_tile(0, 0) == 0
    # the exchange kernels: group shape, message size and alignment are refused before any launch
    tbl = (ctypes.c_void_p * 2)(256, 512)
    assert lib.cider_allreduce_f16(one, one, 64, 0, 1, tbl, 1 << 20, 0, None) == _lib.E_INVALID      # world < 2
    assert lib.cider_allreduce_f16(one, one, 63, 0, 2, tbl, 1 << 20, 0, None) == _lib.E_SHAPE        # count % 8
    assert lib.cider_allreduce_f16(one, one, 1 << 20, 0, 2, tbl, 1 << 20, 0, None) == _lib.E_WORKSPACE
    assert "inbox slot" in _lib.last_error()
    assert lib.cider_allreduce_f16(one, one, 64, 2, 2, tbl, 1 << 20, 0, None) == _lib.E_INVALID      # rank
    assert lib.cider_allreduce_f16(ctypes.c_void_p(24), one, 64, 0, 2, tbl, 1 << 20, 0, None) == _lib.E_ALIGNMENT
    assert lib.cider_peer_max_bytes(4 << 20) == (((4 << 20) - 4096) // 16) // 256 * 256
    assert lib.cider_peer_max_bytes(4096) == 0
    assert lib.cider_allreduce_add_rmsnorm_quant(one, one, one, 1e-6, 33, 4096, one, None, None, 0, 2, tbl, 4 << 20, 0,
                                                 None) == _lib.E_SHAPE                                # M > 32
    assert lib.cider_allreduce_add_rmsnorm_quant(one, one, one, 1e-6, 8, 4100, one, None, None, 0, 2, tbl, 4 << 20, 0,
                                                 None) == _lib.E_SHAPE                                # K % 8
    assert lib.cider_allreduce_add_rmsnorm_quant(one, one, one, 1e-6, 8, 4096, None, None, None, 0, 2, tbl, 4 << 20, 0,
                                                 None) == _lib.E_INVALID                              # no output
    assert lib.cider_sdpa_decode_fused(one, one, one, one, one, one, 1, 1e-6, one, one, one, 1, 16, 8, 64, 10, 16, 1.0,
                                       None, 0, None, None, None) == _lib.E_SHAPE                     # head_dim
    assert lib.cider_row_absmax(one, 4, 64, 32, one, None) == _lib.E_INVALID                          # ldx < K
    assert lib.cider_quantize_given_amax(one, 4, 64, 64, None, one, one, None) == _lib.E_INVALID
    assert lib.cider_testing_set_sdpa_kernel(3) == _lib.E_INVALID and lib.cider_testing_set_sdpa_kernel(0) == 0
    # empty batches are a successful no-op
    assert lib.cider_perchannel_linear(one, one, one, None, one, 0, 64, 128, None, 0, None) == 0
    assert lib.cider_int8_matmul_int32(one, one, one, 0, 8, 8, None) == 0
    with pytest.raises(ValueError):
        _lib.check(_lib.E_SHAPE)
    with pytest.raises(RuntimeError):
        _lib.check(_lib.E_CUDA)


def test_weight_helpers_match_reference_golden():
    g = np.load(os.path.join(GOLDEN, "weight_quant.npz"))
    for key in ("pc", "pc16"):
        q, s = ops.quantize_weight_int8(g[f"{key}_w"])
        assert np.array_equal(q, g[f"{key}_q"]) and np.array_equal(s, g[f"{key}_scale"])
        assert q.dtype == np.int8 and s.dtype == np.float32
    for gs in (64, 128, 256):
        q, s = cnn._symmetric_quantize_pergroup(g[f"pg{gs}_w"], gs)
        assert np.array_equal(q, g[f"pg{gs}_q"]) and np.array_equal(s, g[f"pg{gs}_scale"])
    p, s = ops.pack_weight_int4(g["w4_w"])
    assert np.array_equal(p, g["w4_packed"]) and np.array_equal(s, g["w4_scale"])
    with pytest.raises(AssertionError):
        ops.pack_weight_int4(np.zeros((3, 4), np.float32))


def test_pergroup_int4_helper_roundtrip():
    rng = np.random.default_rng(0)
    w = (rng.standard_normal((128, 24)) * 0.02).astype(np.float32)
    p, s = ops.pack_weight_int4_pergroup(w, 64)
    assert p.shape == (64, 24) and s.shape == (2, 24) and s.dtype == np.float16
    hi, lo = (p >> 4).astype(np.int32) - 8, (p & 15).astype(np.int32) - 8
    deq = np.empty_like(w)
    deq[0::2], deq[1::2] = hi, lo
    deq = deq.reshape(2, 64, 24) * s.astype(np.float32)[:, None, :]
    assert np.abs(deq.reshape(128, 24) - w).max() <= 0.5 * s.astype(np.float32).max() * 1.001 + 1e-9


def test_interleave_gate_up_layout():
    """Blocks of 32 gate rows followed by their 32 up rows; scales and bias follow; numpy and torch
    inputs give the same order; shapes that are not whole blocks are refused."""
    inter, K = 96, 5
    w = np.arange(2 * inter * K, dtype=np.int32).reshape(2 * inter, K)
    sw = np.arange(2 * inter, dtype=np.float32)
    wi, swi, bi = ops.interleave_gate_up(w, sw, None)
    assert bi is None and wi.shape == w.shape
    for b in range(inter // 32):
        assert np.array_equal(wi[64 * b:64 * b + 32], w[32 * b:32 * b + 32])                      # gate rows
        assert np.array_equal(wi[64 * b + 32:64 * b + 64], w[inter + 32 * b:inter + 32 * b + 32])  # their up rows
        assert np.array_equal(swi[64 * b:64 * b + 32], sw[32 * b:32 * b + 32])
        assert np.array_equal(swi[64 * b + 32:64 * b + 64], sw[inter + 32 * b:inter + 32 * b + 32])
    wt, swt, bt = ops.interleave_gate_up(torch.from_numpy(w), torch.from_numpy(sw), torch.from_numpy(sw).half())
    assert np.array_equal(wt.numpy(), wi) and np.array_equal(swt.numpy(), swi)
    assert np.array_equal(bt.float().numpy(), swi)
    assert sorted(swi.tolist()) == sw.tolist()  # a permutation
    with pytest.raises(ValueError):
        ops.interleave_gate_up(np.zeros((2 * 48, K), np.int8))


def test_swiglu_entry_points_validate_before_any_launch():
    lib = _lib.load()
    # N not a multiple of 64, null pointers, negative sizes: refused on the host
    assert lib.cider_swiglu_linear_prequantized(None, None, None, None, None, None, None, 128, 100, 64, None) == _lib.E_SHAPE
    assert lib.cider_swiglu_linear_prequantized(None, None, None, None, None, None, None, 128, 128, 64, None) == _lib.E_INVALID
    assert lib.cider_swiglu_linear_prequantized(None, None, None, None, None, None, None, -1, 128, 64, None) == _lib.E_INVALID
    assert lib.cider_swiglu_linear_prequantized(None, None, None, None, None, None, None, 0, 128, 64, None) == 0
    assert lib.cider_quantize_consume_amax(None, 0, 64, 64, None, None, None, None) == 0


def test_module_surface_without_gpu():
    assert cider_b200.get_mode() in ("auto", "unavailable")
    lin = torch.nn.Linear(128, 32, bias=True).half()
    m = cnn.CiderLinear.from_float(lin)
    assert m.input_dims == 128 and m.output_dims == 32 and m.group_size == 0
    assert m.w_int8.dtype == torch.int8 and m.scale_w.dtype == torch.float32 and m.bias.dtype == torch.float16
    assert tuple(m.scale_w.shape) == (32,)
    q, s = ops.quantize_weight_int8(lin.weight.detach().float().numpy())
    assert np.array_equal(m.w_int8.numpy(), q) and np.array_equal(m.scale_w.numpy(), s)
    mg = cnn.CiderLinear.from_float(lin, target_group_size=64)
    assert tuple(mg.scale_w.shape) == (2, 32) and mg.group_size == 64  # [K/gs, N], transposed
    with pytest.raises(ValueError, match="Unsupported group_size"):
        cnn.CiderLinear(m.w_int8, m.scale_w, 32, 128, 32)
    assert cnn.W8A8Linear is cnn.CiderLinear
    sd = m.state_dict()
    assert set(sd) == {"w_int8", "scale_w", "bias"}
    w4 = cnn.W4A8Linear.from_weights(np.random.default_rng(1).standard_normal((64, 16)).astype(np.float32),
                                     device="cpu")
    assert w4.input_dims == 64 and w4.output_dims == 16 and w4.packed_weight.dtype == torch.uint8
    with pytest.raises(TypeError):
        cnn.CiderLinear.from_float(torch.nn.ReLU())


def test_quantized_linear_requant():
    """from_float on an 8-bit group-quantised layer re-quantises per group (cider/nn.py:127-171)."""
    torch.manual_seed(0)
    w = torch.randn(16, 256) * 0.02
    ql = cnn.QuantizedLinear.quantize(w, group_size=64, bits=8)
    assert (ql.dequantize() - w).abs().max() < 1e-3
    m = cnn.CiderLinear.from_float(ql)
    assert m.group_size == 64 and tuple(m.scale_w.shape) == (4, 16)
    q4 = cnn.QuantizedLinear.quantize(w, group_size=64, bits=4)
    m4 = cnn.CiderLinear.from_float(q4)
    assert m4.group_size == 0  # non-8-bit source -> per-channel
    deq = m.w_int8.float().reshape(16, 4, 64) * m.scale_w.t().reshape(16, 4, 1)
    assert (deq.reshape(16, 256) - w).abs().max() < 2e-3


@pytest.mark.skipif(torch.cuda.is_available(), reason="degraded surface is what a machine without a GPU sees")
def test_unavailable_surface():
    import warnings
    from cider_b200 import convert as conv
    assert ops.is_available() is False
    with pytest.raises(RuntimeError, match="not available"):
        conv.convert_model(torch.nn.Linear(8, 8))
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        cider_b200.convert_model(torch.nn.Linear(8, 8))
    assert any("no-op" in str(x.message) for x in w)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.perchannel_linear(torch.zeros(2, 8, dtype=torch.float16), torch.zeros(4, 8, dtype=torch.int8),
                              torch.ones(4))


# ------------------------------------------------------------------ N > 1 on CPU
def test_bench_reference_arm_under_torchrun_two_ranks():
    """The launch contract of the reference arm at N=2: started by torchrun with two
    ranks (no GPU needed), rank 0 alone times the CPU oracle and prints ONE JSON line,
    the other rank exits 0 without work."""
    import json
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    port = 29000 + os.getpid() % 2000
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(root, "bench.py"),
           "--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "1"]
    out = subprocess.run(cmd, cwd=root, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["e2e"]["d2h_bytes_per_step"] == 0


def _split_worker(rank, world, port, ret):
    import numpy as np
    import torch
    import torch.distributed as dist
    import oracle
    from conftest import make_activations, make_weight
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    M, N, K = 9, 64, 128
    x = make_activations(M, K, seed=3)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=4))
    bias = (np.arange(N) % 7).astype(np.float16)
    lo, hi = rank * N // world, (rank + 1) * N // world
    # the path shards over output channels with no data-path collective: a rank owns a
    # slice of W, scale_w and bias; the activation quantiser sees the full K on every rank
    part = oracle.c_perchannel_linear(x, np.ascontiguousarray(wq[lo:hi]), np.ascontiguousarray(sw[lo:hi]),
                                      np.ascontiguousarray(bias[lo:hi]))
    parts = [torch.empty((M, N // world), dtype=torch.float16) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(part))  # test plumbing only
    if rank == 0:
        ret["y"] = torch.cat(parts, dim=1).numpy()
        ret["full"] = oracle.c_perchannel_linear(x, wq, sw, bias)
    dist.destroy_process_group()


def test_linear_split_over_output_channels_two_gloo_ranks():
    """N-split of one linear over two ranks (gloo, CPU, oracle arithmetic): concatenating
    the ranks' column slices reproduces the unsplit result bit for bit."""
    import numpy as np
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_split_worker, args=(2, 29000 + (os.getpid() + 7) % 2000, ret), nprocs=2, join=True)
    assert np.array_equal(ret["y"], ret["full"])


# ------------------------------------------------- already-quantised checkpoints
def _to_words(vals_u8, bits):
    """[N, K] unsigned field values -> int32 [N, ceil(K*bits/32)], little end first."""
    import numpy as np
    N, K = vals_u8.shape
    per = 32 // bits
    W = (K + per - 1) // per
    padded = np.zeros((N, W * per), dtype=np.uint32)
    padded[:, :K] = vals_u8
    words = np.zeros((N, W), dtype=np.uint32)
    for i in range(per):
        words |= padded[:, i::per] << np.uint32(i * bits)
    return words.view(np.int32)


def _offset8(q):
    """int8 weights -> the stored 8-bit fields: offset binary, field = weight + 128
    (tools/convert_compressed_tensors_to_mlx.py:51: offset = 1 << (num_bits - 1))."""
    import numpy as np
    return (q.astype(np.int16) + 128).astype(np.uint8)


def _reference_dequant(words_i32, scale, bits, K, group_size=None):
    """The reference's own read-back of a packed layer
    (tools/convert_compressed_tensors_to_mlx.py:236-249): ((word >> bits*i) & mask) - offset, times
    the channel or group scale."""
    import numpy as np
    packed = words_i32.view(np.uint32)
    per, offset = 32 // bits, 1 << (bits - 1)
    ref = np.zeros((packed.shape[0], K), dtype=np.float32)
    for i in range(per):
        vals = (packed >> np.uint32(bits * i)) & np.uint32((1 << bits) - 1)
        signed = vals.astype(np.int32) - offset
        cols = np.arange(packed.shape[1]) * per + i
        cols = cols[cols < K]
        if scale.shape[1] == 1:
            ref[:, cols] = signed[:, :len(cols)] * scale[:, 0:1]
        else:
            ref[:, cols] = signed[:, :len(cols)] * scale[:, cols // group_size]
    return ref


def test_compressed_tensors_int8_ingestion_is_exact():
    """Pack-quantised int8 layers (per-channel and per-group) and a raw-int8 layer
    become CiderLinear modules holding exactly the stored integers and scales."""
    import numpy as np
    import torch
    import oracle
    from conftest import make_weight
    from cider_b200 import checkpoint
    from cider_b200.nn import CiderLinear
    N, K = 24, 256
    w = make_weight(N, K, seed=11)
    q_pc, s_pc = oracle.np_quantize_weight_int8(w)
    q_pg, s_pg = oracle.np_quantize_weight_pergroup(w, 64)  # scales [N, K/64]
    state = {
        "a.weight_packed": torch.from_numpy(_to_words(_offset8(q_pc), 8)),
        "a.weight_scale": torch.from_numpy(s_pc[:, None].copy()),
        "a.weight_shape": torch.tensor([N, K]),
        "a.bias": torch.arange(N, dtype=torch.float16),
        "b.proj.weight_packed": torch.from_numpy(_to_words(_offset8(q_pg), 8)),
        "b.proj.weight_scale": torch.from_numpy(s_pg.astype(np.float16)),
        "b.proj.weight_shape": torch.tensor([N, K]),
        "c.weight": torch.from_numpy(q_pc.copy()),
        "c.weight_scale": torch.from_numpy(s_pc.copy()),
        "norm.weight": torch.ones(K),
    }
    mods, plain = checkpoint.modules_from_state_dict(state)
    assert set(mods) == {"a", "b.proj", "c"} and set(plain) == {"norm.weight"}
    a, b, c = mods["a"], mods["b.proj"], mods["c"]
    assert all(isinstance(m, CiderLinear) for m in (a, b, c))
    assert a.group_size == 0 and np.array_equal(a.w_int8.numpy(), q_pc) and np.array_equal(a.scale_w.numpy(), s_pc)
    assert np.array_equal(a.bias.numpy(), np.arange(N, dtype=np.float16))
    assert b.group_size == 64 and np.array_equal(b.w_int8.numpy(), q_pg)
    assert b.scale_w.dtype == torch.float16 and tuple(b.scale_w.shape) == (K // 64, N)
    assert np.array_equal(b.scale_w.numpy(), s_pg.astype(np.float16).T)
    assert c.group_size == 0 and np.array_equal(c.w_int8.numpy(), q_pc)
    # dequantised with the reference's own formula the packed words give the same weights as
    # the module's integers times its scales (a two's-complement reading would be off by 128)
    ref_a = _reference_dequant(state["a.weight_packed"].numpy(), s_pc[:, None], 8, K)
    assert np.array_equal(ref_a, a.w_int8.numpy().astype(np.float32) * a.scale_w.numpy()[:, None])
    s16 = s_pg.astype(np.float16).astype(np.float32)
    ref_b = _reference_dequant(state["b.proj.weight_packed"].numpy(), s16, 8, K, 64)
    got_b = b.w_int8.numpy().astype(np.float32) * np.repeat(b.scale_w.numpy().astype(np.float32).T, 64, axis=1)
    assert np.array_equal(ref_b, got_b)
    with pytest.raises(ValueError):  # group size outside 64 / 128 / 256
        checkpoint.linear_from_compressed(state["a.weight_packed"], torch.ones(N, K // 32), [N, K])
    with pytest.raises(ValueError):  # asymmetric
        checkpoint.linear_from_compressed(state["a.weight_packed"], state["a.weight_scale"], [N, K],
                                          zero_point=torch.ones(N, 1, dtype=torch.int8))


def test_compressed_tensors_int4_ingestion_matches_reference_packing():
    """A 4-bit pack-quantised layer lands in W4A8Linear's [K/2, N] packing (high nibble
    = even k) byte for byte equal to packing the same integers with the reference's helper."""
    import numpy as np
    import torch
    import oracle
    from conftest import make_weight
    from cider_b200 import checkpoint
    from cider_b200.nn import W4A8Linear
    N, K, gs = 16, 128, 64
    w_kn = np.ascontiguousarray(make_weight(N, K, seed=5).T)
    packed_ref, scale_ref = oracle.np_pack_weight_int4_pergroup(w_kn, gs)  # [K/2, N], [K/gs, N]
    # recover the stored nibbles (value + 8) per (n, k) from the reference packing
    nib = np.zeros((N, K), dtype=np.uint8)
    nib[:, 0::2] = (packed_ref >> 4).T
    nib[:, 1::2] = (packed_ref & 15).T
    mod = checkpoint.linear_from_compressed(torch.from_numpy(_to_words(nib, 4)),
                                            torch.from_numpy(np.ascontiguousarray(scale_ref.T)), [N, K], num_bits=4)
    assert isinstance(mod, W4A8Linear) and mod.group_size == gs and mod.input_dims == K and mod.output_dims == N
    assert np.array_equal(mod.packed_weight.numpy(), packed_ref)
    assert np.array_equal(mod.scale.numpy().astype(np.float32), scale_ref.astype(np.float32))


def test_load_compressed_checkpoint_swaps_modules_in_place():
    import numpy as np
    import torch
    from torch import nn
    import oracle
    from conftest import make_weight
    from cider_b200 import checkpoint
    from cider_b200.nn import CiderLinear

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.proj = nn.Linear(128, 8, bias=False)
            self.norm = nn.LayerNorm(128)

    model = nn.ModuleDict({"blk": Block()})
    q, s = oracle.np_quantize_weight_int8(make_weight(8, 128, seed=2))
    state = {"blk.proj.weight_packed": torch.from_numpy(_to_words(_offset8(q), 8)),
             "blk.proj.weight_scale": torch.from_numpy(s[:, None].copy()),
             "blk.proj.weight_shape": torch.tensor([8, 128]),
             "blk.norm.weight": torch.full((128,), 2.0), "blk.norm.bias": torch.zeros(128),
             "extra.tensor": torch.zeros(1)}
    res = checkpoint.load_compressed_checkpoint(model, state)
    assert res["n_quantized"] == 1 and res["unexpected_keys"] == ["extra.tensor"] and res["missing_keys"] == []
    assert isinstance(model["blk"].proj, CiderLinear)
    assert np.array_equal(model["blk"].proj.w_int8.numpy(), q)
    assert float(model["blk"].norm.weight[0]) == 2.0


def test_fuse_projections_structure_and_cache():
    """q/k/v and gate/up CiderLinear siblings become one layer each; the children keep
    their names; the fused GEMM runs once per input (checked with a stand-in forward)."""
    import numpy as np
    import torch
    from torch import nn
    from cider_b200.convert import FusedProjections, FusedSlice, fuse_projections
    from cider_b200.nn import CiderLinear

    def lin(n, k, seed, gs=0):
        g = torch.Generator().manual_seed(seed)
        w = torch.randint(-127, 128, (n, k), generator=g, dtype=torch.int8)
        s = torch.rand(n, generator=g) if gs == 0 else torch.rand(k // gs, n, generator=g).half()
        return CiderLinear(w, s, gs, k, n, torch.randn(n, generator=g).half())

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj, self.o_proj = lin(32, 64, 1), lin(16, 64, 2), lin(16, 64, 3), lin(64, 32, 4)

    class Mlp(nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj, self.up_proj, self.down_proj = lin(48, 64, 5, 64), lin(48, 64, 6, 64), lin(64, 48, 7)

    m = nn.ModuleDict({"attn": Attn(), "mlp": Mlp()})
    wq, wk, wv = (m["attn"].q_proj.w_int8.clone(), m["attn"].k_proj.w_int8.clone(), m["attn"].v_proj.w_int8.clone())
    sg, su = m["mlp"].gate_proj.scale_w.clone(), m["mlp"].up_proj.scale_w.clone()
    assert fuse_projections(m) == 2
    qkv, gu = m["attn"].fused_q_k_v, m["mlp"].fused_gate_up
    assert isinstance(qkv, FusedProjections) and isinstance(m["attn"].q_proj, FusedSlice)
    assert isinstance(m["attn"].o_proj, CiderLinear) and isinstance(m["mlp"].down_proj, CiderLinear)
    assert qkv.splits == [32, 16, 16] and qkv.linear.output_dims == 64
    assert torch.equal(qkv.linear.w_int8, torch.cat([wq, wk, wv]))
    assert gu.linear.group_size == 64 and torch.equal(gu.linear.scale_w, torch.cat([sg, su], dim=1))
    # the group is registered once (under the parent), not once per slice
    assert sum(1 for _ in m["attn"].modules() if isinstance(_, FusedProjections)) == 1
    # one GEMM per distinct input: count calls of a stand-in for the CUDA forward
    calls = []
    qkv.linear.forward = lambda x: (calls.append(1), torch.arange(64.0).repeat(x.shape[0], 1))[1]
    x = torch.zeros(3, 64)
    q, k, v = m["attn"].q_proj(x), m["attn"].k_proj(x), m["attn"].v_proj(x)
    assert len(calls) == 1 and q.shape == (3, 32) and k.shape == (3, 16)
    assert float(k[0, 0]) == 32.0 and float(v[0, 0]) == 48.0 and qkv._parts is None
    m["attn"].q_proj(torch.zeros(3, 64))
    assert len(calls) == 2
    # A model that calls only q_proj: the cache survives the call, but it holds the input
    # tensor, so a different activation cannot appear at the cached address; an in-place
    # change of the same tensor bumps its version and runs the GEMM again; and a forward
    # of the parent module starts and ends with an empty cache.
    x1 = torch.zeros(3, 64)
    m["attn"].q_proj(x1)
    assert len(calls) == 3 and qkv._x is x1
    x1.add_(1.0)
    m["attn"].q_proj(x1)
    assert len(calls) == 4
    m["attn"].forward = lambda x: m["attn"].q_proj(x)
    m["attn"](x1)
    assert qkv._parts is None and qkv._x is None
