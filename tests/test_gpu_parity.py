"""GPU parity: the CUDA path through the C ABI against the CPU oracle.

Bars (from the north star): int8 activations, fp32 scales and int32 accumulators
bit-exact; fp16 outputs within a relative error of 2e-3 (normalised max error,
``rel_err`` in conftest).  For M > 1 the CUDA epilogues use the same fp32
operation order as the oracle, so those outputs are additionally required to be
IDENTICAL; only the M == 1 matrix-vector path, whose fp32 summation order is
free, is held to the 2e-3 tolerance alone.
"""
import hashlib
import json
import os

import numpy as np
import pytest
import torch

from conftest import make_activations, make_weight, rel_err

pytestmark = pytest.mark.gpu

TOL = 2e-3  # relative error bar for fp16 outputs
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from cider_b200 import _lib, ops as o
    assert o.is_available(), "B200 + built CUDA library required"
    _lib.load().cider_clear_device_status()
    yield o
    st = __import__("ctypes").c_uint(0)
    assert _lib.load().cider_device_status(st) == 0
    assert st.value == 0, f"a kernel recorded a bounded-wait time-out (status {st.value})"


@pytest.fixture()
def backend():
    from cider_b200 import _lib

    def set_backend(b):
        assert _lib.load().cider_set_gemm_backend(b) == 0

    yield set_backend
    _lib.load().cider_set_gemm_backend(0)


def t(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def n(x):
    return x.detach().cpu().numpy()


# ---------------------------------------------------------------- S1 quantise
@pytest.mark.parametrize("M,K", [(1, 16), (2, 2560), (7, 513), (33, 4097), (128, 2560), (129, 10240),
                                 (64, 12288), (5, 40000), (300, 64), (3, 1)])
def test_quantize_bitexact(ops, oracle, M, K):
    x = make_activations(M, K, seed=M * 7 + K)
    if M > 2:
        x[1] = 0  # zero row -> scale 1
        x[2] = 0
        x[2, K // 2] = -3.0  # single max element
    q, s = ops.quantize_per_token(t(x))
    q_ref, s_ref = oracle.c_quantize_per_token(x)
    assert np.array_equal(n(s), s_ref)
    assert np.array_equal(n(q), q_ref)


def test_quantize_ties_and_stride(ops, oracle):
    rng = np.random.default_rng(0)
    x = (rng.integers(-254, 255, (64, 256)) * 0.5).astype(np.float16)  # halves: every other value a tie
    x[:, 0] = 127.0  # scale exactly 1
    q, s = ops.quantize_per_token(t(x))
    q_ref, s_ref = oracle.c_quantize_per_token(x)
    assert np.array_equal(n(q), q_ref) and np.array_equal(n(s), s_ref)
    assert (s_ref == 1.0).all()
    # strided rows (a column slice of a wider matrix)
    wide = t(make_activations(40, 512, seed=5))
    view = wide[:, 128:384]
    q, s = ops.quantize_per_token(view)
    q_ref, s_ref = oracle.c_quantize_per_token(n(view))
    assert np.array_equal(n(q), q_ref) and np.array_equal(n(s), s_ref)


def test_quantize_every_fp16_value(ops, oracle):
    """Rows holding every finite fp16 value not above the row's maximum, for maxima that make the
    scale a power of two, a value with a long reciprocal, the largest fp16 and a subnormal."""
    allv = np.arange(65536, dtype=np.uint16).view(np.float16)
    finite = allv[np.isfinite(allv)]
    rows = []
    for amax in (127.0, 1.0, 3.1416, 65504.0, 0.3333, 6.0e-8, 254.0, 17.0):
        a = np.float16(amax)
        v = finite[np.abs(finite.astype(np.float32)) <= np.float32(a)]
        row = np.zeros(65536, dtype=np.float16)  # K = 65536 takes the scalar kernel
        row[: v.size] = v
        row[-1] = a
        rows.append(row)
    x = np.stack(rows)
    for xs in (x, np.ascontiguousarray(x[:, :32768]), np.ascontiguousarray(x[:, 31744:31744 + 2560])):
        xs = xs.copy()
        xs[:, 0] = x[:, -1]  # keep the maximum in every slice
        q, s = ops.quantize_per_token(t(xs))
        q_ref, s_ref = oracle.c_quantize_per_token(xs)
        assert np.array_equal(n(s), s_ref)
        assert np.array_equal(n(q), q_ref)


# ------------------------------------------------------- S2 raw integer GEMM
with open(os.path.join(GOLDEN, "bitexact_int32.json")) as f:
    BITEXACT = json.load(f)["cases"]


def _bitexact_operands(M, K, N):
    np.random.seed(42)  # benchmarks/test_bitexact.py:45-47
    return (np.random.randint(-128, 128, (M, K), dtype=np.int8),
            np.random.randint(-128, 128, (N, K), dtype=np.int8))


@pytest.mark.parametrize("case", BITEXACT, ids=lambda c: f"{c['M']}x{c['K']}x{c['N']}")
@pytest.mark.parametrize("which", ["auto", "plain"])
def test_int8_matmul_reference_vectors(ops, backend, case, which):
    backend(0 if which == "auto" else 1)
    a, b = _bitexact_operands(case["M"], case["K"], case["N"])
    c = n(ops.int8_matmul_int32(t(a), t(b)))
    assert c.dtype == np.int32
    assert hashlib.sha256(c.tobytes()).hexdigest() == case["sha256"]


@pytest.mark.parametrize("M,N,K", [(128, 256, 128), (128, 256, 512), (256, 512, 2560), (129, 257, 144),
                                   (1000, 1000, 1008), (64, 10240, 2560), (130, 72, 4096), (8, 8, 128)])
def test_int8_matmul_tensor_core_vs_oracle(ops, oracle, backend, M, N, K):
    backend(2)  # must take the tcgen05 kernel
    rng = np.random.default_rng(M + N + K)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    c = n(ops.int8_matmul_int32(t(a), t(b)))
    assert np.array_equal(c, oracle.c_int8_matmul_int32(a, b))


@pytest.mark.parametrize("M,N,K", [(2, 2560, 10240), (8, 2560, 10240), (100, 264, 4096), (130, 2560, 10240),
                                   (300, 1000, 8192), (512, 256, 16400), (64, 1024, 1024)])
def test_int8_matmul_small_m_long_k(ops, oracle, M, N, K):
    """Few output tiles and a long K: the K pieces add their int32 partial tiles into the zeroed
    result (TMA reduce-add); integer sums are exact whatever the order."""
    from cider_b200 import _lib
    rng = np.random.default_rng(M * 7 + N + K)
    a = rng.integers(-128, 128, (M, K), dtype=np.int8)
    b = rng.integers(-128, 128, (N, K), dtype=np.int8)
    want = oracle.c_int8_matmul_int32(a, b)
    ta, tb = t(a), t(b)
    # twice: the second result usually lands on the memory of the first (the caching allocator
    # hands the block back), so values left there must not be added onto
    for _ in range(2):
        c = n(ops.int8_matmul_int32(ta, tb))
        kernel = _lib.load().cider_testing_last_gemm_kernel().decode()
        assert np.array_equal(c, want), kernel
    if (M, N, K) in ((8, 2560, 10240), (130, 2560, 10240)):
        assert "reduce-add" in kernel, kernel


def test_int8_matmul_extremes(ops, oracle):
    # all -128 x all -128 at K = 8192: 2^27 per element, no overflow
    a = np.full((130, 8192), -128, np.int8)
    b = np.full((70, 8192), -128, np.int8)
    c = n(ops.int8_matmul_int32(t(a), t(b)))
    assert (c == 8192 * 16384).all()
    b[:] = 127
    assert (n(ops.int8_matmul_int32(t(a), t(b))) == -128 * 127 * 8192).all()


# ----------------------------------------------------- S3..S7 fused linears
LINEAR_SHAPES = [(2, 256, 128), (7, 72, 512), (33, 1000, 1024), (64, 256, 2560), (65, 512, 640),
                 (128, 10240, 2560), (129, 2560, 10240), (300, 768, 1536),
                 # M <= 16 (per-group: <= 64): the streaming small-M kernel (K % 64 == 0), ragged N, long K
                 (3, 8, 64), (8, 6144, 4096), (8, 1032, 12288), (9, 264, 2560), (16, 1000, 2560), (5, 100, 192),
                 (12, 40, 12288), (40, 520, 5120)]


def pg_splitk_path(M, N, K):
    """Shapes whose per-group linear takes the split-K form (the workspace then holds fp32
    slabs): K pieces are summed after the groups of each piece, so the fp32 order differs
    from the oracle's ascending one (same bar as for the small-M kernel below)."""
    from cider_b200 import _lib
    base = ((M * K + 255) // 256 + (4 * M + 255) // 256) * 256
    return M > 1 and _lib.load().cider_workspace_bytes(_lib.OP_PERGROUP, M, N, K) > base


def close_bits(y, ref):
    return rel_err(y, ref) <= 1e-3 and (y != ref).mean() <= 0.05


def small_m_group_path(M, K, gs):
    """Shapes that the small-M per-group kernel takes: its fp32 group sums are added
    in a different order than the oracle's ascending one, so equality is not bit-wise
    there (the 2e-3 bar holds; observed differences are single fp16 ulps)."""
    return M <= 64 and gs > 0 and K % 64 == 0 and gs % 64 == 0


@pytest.mark.parametrize("M,N,K", LINEAR_SHAPES)
@pytest.mark.parametrize("use_bias", [False, True])
def test_perchannel_linear(ops, oracle, M, N, K, use_bias):
    x = make_activations(M, K, seed=M)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N))
    bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16) if use_bias else None
    y = n(ops.perchannel_linear(t(x), t(wq), t(sw), None if bias is None else t(bias)))
    ref = oracle.c_perchannel_linear(x, wq, sw, bias)
    assert rel_err(y, ref) <= TOL
    assert np.array_equal(y, ref), f"fp16 mismatch in {(y != ref).sum()} of {y.size}"


@pytest.mark.parametrize("M,N,K", [(128, 2560, 10240), (17, 8, 4096), (100, 136, 4112), (256, 2048, 6144),
                                   (257, 128, 16384), (200, 264, 8192), (129, 2560, 10240)])
def test_perchannel_linear_split_k(ops, oracle, M, N, K):
    """Small M, few output tiles, long K: the per-channel linear cuts K into pieces (int32 slabs in
    the workspace + a finishing kernel).  Integer partial sums: identical to the oracle."""
    from cider_b200 import _lib
    need = _lib.load().cider_workspace_bytes(_lib.OP_PERCHANNEL, M, N, K)
    assert need > ((M * K + 255) // 256 + (4 * M + 255) // 256) * 256, "this shape should take the split-K form"
    x = make_activations(M, K, seed=M + 3)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N + 1))
    bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16)
    for b in (None, bias):
        y = n(ops.perchannel_linear(t(x), t(wq), t(sw), None if b is None else t(b)))
        ref = oracle.c_perchannel_linear(x, wq, sw, b)
        assert np.array_equal(y, ref), f"fp16 mismatch in {(y != ref).sum()} of {y.size}"


@pytest.mark.parametrize("M,N,K", LINEAR_SHAPES)
@pytest.mark.parametrize("gs,sdt", [(64, np.float16), (128, np.float32), (128, np.float16), (256, np.float32)])
def test_pergroup_linear(ops, oracle, M, N, K, gs, sdt):
    if K % gs:
        pytest.skip("K not a multiple of the group size")
    x = make_activations(M, K, seed=M + 1)
    wq, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=N + 1), gs)
    sg_t = np.ascontiguousarray(sg.T).astype(sdt)  # [K/gs, N]
    bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16)
    y = n(ops.pergroup_linear(t(x), t(wq), t(sg_t), gs, t(bias)))
    ref = oracle.c_pergroup_linear(x, wq, sg_t, gs, bias)
    assert rel_err(y, ref) <= TOL
    if small_m_group_path(M, K, gs) or pg_splitk_path(M, N, K):
        assert close_bits(y, ref)
    else:
        assert np.array_equal(y, ref), f"fp16 mismatch in {(y != ref).sum()} of {y.size}"


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (2, 72, 512), (33, 1000, 1024), (128, 10240, 2560),
                                   (65, 512, 640)])
@pytest.mark.parametrize("gs", [0, 64])
def test_w4a8_linear(ops, oracle, M, N, K, gs):
    x = make_activations(M, K, seed=M + 2)
    w_kn = np.ascontiguousarray(make_weight(N, K, seed=N + 2).T)
    if gs == 0:
        packed, sw = oracle.np_pack_weight_int4(w_kn)
    else:
        packed, sw = oracle.np_pack_weight_int4_pergroup(w_kn, gs)
    y = n(ops.w4a8_linear(t(x), t(packed), t(sw), group_size=gs))
    ref = oracle.c_w4a8_linear(x, packed, sw, gs)
    assert rel_err(y, ref) <= TOL
    if small_m_group_path(M, K, gs):
        assert rel_err(y, ref) <= 1e-3 and (y != ref).mean() <= 0.05
    else:
        assert np.array_equal(y, ref)


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (2, 72, 512), (8, 6144, 4096), (16, 1000, 2560), (5, 264, 192),
                                   (8, 1032, 12288), (33, 1000, 1024), (130, 512, 640), (40, 520, 5120)])
@pytest.mark.parametrize("gs", [0, 64, 128])
def test_w4a8_linear_row_layout(ops, oracle, M, N, K, gs):
    """Weights repacked to rows ([N, K/2]): the repack is a byte transpose, and the
    linear gives what the reference layout gives - the streaming kernel (M <= 16, per
    group <= 64) expands nibbles in registers, larger M goes through the int8 copy."""
    if gs and K % gs:
        pytest.skip("K not a multiple of the group size")
    x = make_activations(M, K, seed=M + 3)
    w_kn = np.ascontiguousarray(make_weight(N, K, seed=N + 3).T)
    if gs == 0:
        packed, sw = oracle.np_pack_weight_int4(w_kn)
    else:
        packed, sw = oracle.np_pack_weight_int4_pergroup(w_kn, gs)
    rows = ops.w4a8_repack(t(packed))
    assert np.array_equal(n(rows), np.ascontiguousarray(packed.T))
    y = n(ops.w4a8_linear_rows(t(x), rows, t(sw), group_size=gs))
    ref = oracle.c_w4a8_linear(x, packed, sw, gs)
    assert rel_err(y, ref) <= TOL
    if small_m_group_path(M, K, gs):
        assert rel_err(y, ref) <= 1e-3 and (y != ref).mean() <= 0.05
    else:
        assert np.array_equal(y, ref)


def test_random_shapes_against_oracle(ops, oracle):
    """Seeded sweep over ragged shapes: every dispatch route (tcgen05 tiles, generic
    kernel, streaming small-M kernel, scalar fall-backs) must agree with the oracle."""
    rng = np.random.default_rng(1234)
    Ms = [1, 2, 3, 5, 8, 9, 15, 16, 17, 31, 33, 64, 65, 127, 129, 200]
    Ns = [1, 7, 8, 15, 16, 24, 40, 72, 136, 264, 1000]
    Ks = [16, 48, 64, 80, 128, 192, 320, 512, 1040, 2560]
    for case in range(48):
        M, N, K = int(rng.choice(Ms)), int(rng.choice(Ns)), int(rng.choice(Ks))
        x = make_activations(M, K, seed=case)
        w = make_weight(N, K, seed=100 + case)
        bias = (rng.standard_normal(N) * 0.05).astype(np.float16) if case % 2 else None
        wq, sw = oracle.np_quantize_weight_int8(w)
        y = n(ops.perchannel_linear(t(x), t(wq), t(sw), None if bias is None else t(bias)))
        ref = oracle.c_perchannel_linear(x, wq, sw, bias)
        if M == 1:
            assert rel_err(y, ref) <= TOL, (M, N, K)
        else:
            assert np.array_equal(y, ref), (M, N, K, "per-channel")
        for gs in (64, 128):
            if K % gs:
                continue
            wg, sg = oracle.np_quantize_weight_pergroup(w, gs)
            sg_t = np.ascontiguousarray(sg.T).astype(np.float16 if case % 3 else np.float32)
            yg = n(ops.pergroup_linear(t(x), t(wg), t(sg_t), gs, None if bias is None else t(bias)))
            refg = oracle.c_pergroup_linear(x, wg, sg_t, gs, bias)
            assert rel_err(yg, refg) <= TOL, (M, N, K, gs)
            # bit-identical wherever the large-M kernels run (the streaming kernel needs
            # K % 64 == 0, N % 8 == 0 and M <= 64; its fp32 order differs)
            if pg_splitk_path(M, N, K):
                assert close_bits(yg, refg), (M, N, K, gs)
            elif M > 64 or (M > 1 and (K % 64 or N % 8)):
                assert np.array_equal(yg, refg), (M, N, K, gs)
        if K % 2 == 0 and M > 1:
            packed, s4 = oracle.np_pack_weight_int4(np.ascontiguousarray(w.T))
            y4 = n(ops.w4a8_linear(t(x), t(packed), t(s4)))
            assert np.array_equal(y4, oracle.c_w4a8_linear(x, packed, s4, 0)), (M, N, K, "w4a8")
            if K % 16 == 0:
                y4r = n(ops.w4a8_linear_rows(t(x), ops.w4a8_repack(t(packed)), t(s4)))
                assert np.array_equal(y4r, y4), (M, N, K, "w4a8 rows")
    from cider_b200 import _lib
    import ctypes
    status = ctypes.c_uint(0)
    _lib.check(_lib.load().cider_device_status(status))
    assert status.value == 0


def test_empty_inputs_are_no_ops(ops):
    """M == 0 (an empty batch) succeeds and returns an empty result on every entry."""
    w = torch.zeros((8, 64), dtype=torch.int8, device=DEV)
    sw = torch.ones(8, device=DEV)
    x0 = torch.zeros((0, 64), dtype=torch.float16, device=DEV)
    assert ops.perchannel_linear(x0, w, sw).shape == (0, 8)
    assert ops.pergroup_linear(x0, w, torch.ones((1, 8), device=DEV), 64).shape == (0, 8)
    q0, s0 = ops.quantize_per_token(x0)
    assert q0.shape == (0, 64) and s0.shape == (0,)
    assert ops.linear_prequantized(q0, s0, w, sw).shape == (0, 8)
    packed = torch.full((32, 8), 0x88, dtype=torch.uint8, device=DEV)
    assert ops.w4a8_linear(x0, packed, sw).shape == (0, 8)
    assert ops.w4a8_linear_rows(x0, ops.w4a8_repack(packed), sw).shape == (0, 8)
    q1, s1 = ops.silu_mul_quant(torch.zeros((0, 128), dtype=torch.float16, device=DEV))
    assert q1.shape == (0, 64) and s1.shape == (0,)
    q2, s2 = ops.quantize_heads(torch.zeros((2, 4, 0, 16), dtype=torch.float16, device=DEV))
    assert q2.shape == (0, 64) and s2.shape == (0,)
    yh = ops.perchannel_linear_host(torch.zeros((0, 64), dtype=torch.float16), w, sw)
    assert tuple(yh.shape) == (0, 8)
    torch.cuda.synchronize()


@pytest.mark.parametrize("M,N,K,chunk", [(1, 256, 128, 0), (5, 72, 512, 0), (300, 768, 1536, 128),
                                         (257, 256, 128, 128), (2049, 1024, 640, 0), (4096, 2048, 256, 512)])
@pytest.mark.parametrize("pinned", [True, False])
def test_perchannel_linear_host_buffers(ops, oracle, M, N, K, chunk, pinned):
    """Host-buffer entry (chunked upload / kernels / download on three streams) must
    give the bytes of the device-buffer entry: same rows, same arithmetic; a last
    chunk of ONE row (257 = 2*128 + 1) must still be quantised."""
    x = make_activations(M, K, seed=M + 7)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N + 7))
    bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16)
    xh = torch.from_numpy(x)
    out = torch.empty((M, N), dtype=torch.float16)
    if pinned:
        xh, out = xh.pin_memory(), out.pin_memory()
    wd, sd, bd = t(wq), t(sw), t(bias)
    y_dev = n(ops.perchannel_linear(t(x), wd, sd, bd))
    for _ in range(2):  # the second call reuses the staging buffers of the first
        out.zero_()
        y_host = ops.perchannel_linear_host(xh, wd, sd, bd, out=out, chunk_rows=chunk)
        assert y_host.data_ptr() == out.data_ptr()
        assert np.array_equal(y_host.numpy(), y_dev)
    if M > 1:
        assert np.array_equal(y_dev, oracle.c_perchannel_linear(x, wq, sw, bias))


@pytest.mark.parametrize("N,K", [(256, 256), (10240, 2560), (2560, 10240), (1000, 4096), (7, 513),
                                 (6144, 2048), (151936, 2048), (33, 12288)])
def test_m1_matrix_vector(ops, oracle, N, K):
    """M == 1: activations are NOT quantised; fp32 summation order is free -> 2e-3."""
    x = make_activations(1, K, seed=K)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N + 3))
    bias = (np.random.default_rng(N).standard_normal(N) * 0.05).astype(np.float16)
    y = n(ops.perchannel_linear(t(x), t(wq), t(sw), t(bias)))
    ref = oracle.c_perchannel_linear(x, wq, sw, bias)
    assert y.shape == (1, N) and rel_err(y, ref) <= TOL
    for gs in (64, 128, 256):
        if K % gs:
            continue
        wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=N + 4), gs)
        sg_t = np.ascontiguousarray(sg.T)
        y = n(ops.pergroup_linear(t(x), t(wg), t(sg_t), gs, t(bias)))
        assert rel_err(y, oracle.c_pergroup_linear(x, wg, sg_t, gs, bias)) <= TOL
        y16 = n(ops.pergroup_linear(t(x), t(wg), t(sg_t.astype(np.float16)), gs, t(bias)))
        assert rel_err(y16, oracle.c_pergroup_linear(x, wg, sg_t.astype(np.float16), gs, bias)) <= TOL


def test_tensor_core_and_plain_kernels_agree(ops, oracle, backend):
    """Two independent kernels (tcgen05 vs dp4a), identical bits."""
    M, N, K = 200, 520, 1152
    x = make_activations(M, K, seed=11)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=12))
    wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=13), 128)
    sg_t = np.ascontiguousarray(sg.T)
    outs = []
    for b in (2, 1):
        backend(b)
        outs.append((n(ops.perchannel_linear(t(x), t(wq), t(sw))),
                     n(ops.pergroup_linear(t(x), t(wg), t(sg_t), 128))))
    assert np.array_equal(outs[0][0], outs[1][0])
    assert np.array_equal(outs[0][1], outs[1][1])


@pytest.mark.parametrize("tile,bn", [("128", ""), ("2", ""), ("128", "192"), ("128", "64")])
def test_forced_tile_kernels(tile, bn):
    """Both tensor-core kernel variants (single-CTA 128-row tiles with the N tile chosen by the
    heuristic or forced to 192 / 64, CTA pair) on ragged and small problems (subprocess: the
    override is process-wide)."""
    import subprocess
    import sys
    script = os.path.join(os.path.dirname(__file__), "tile_check.py")
    r = subprocess.run([sys.executable, script, tile] + ([bn] if bn else []), capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


def test_w4a8_module_uses_row_layout_and_tracks_weight_changes(ops, oracle):
    """W4A8Linear repacks its weights once into rows; replacing or overwriting the
    packed buffer must not leave a stale copy behind."""
    from cider_b200 import nn as cnn
    K, N = 256, 72
    w1 = np.ascontiguousarray(make_weight(N, K, seed=1).T)
    w2 = np.ascontiguousarray(make_weight(N, K, seed=2).T)
    lin = cnn.W4A8Linear.from_weights(w1, device=DEV)
    x = make_activations(5, K, seed=9)
    p1, s1 = oracle.np_pack_weight_int4(w1)
    p2, s2 = oracle.np_pack_weight_int4(w2)
    assert np.array_equal(n(lin(t(x))), oracle.c_w4a8_linear(x, p1, s1, 0))
    rows_before = lin._rows
    assert rows_before is not None and tuple(rows_before.shape) == (N, K // 2)
    lin.packed_weight.copy_(t(p2))  # in-place update (what load_state_dict does)
    lin.scale.copy_(t(s2))
    assert np.array_equal(n(lin(t(x))), oracle.c_w4a8_linear(x, p2, s2, 0))


def test_bf16_and_module_shapes(ops, oracle):
    """dtype rule: bf16 in -> computed in fp16 -> bf16 out; leading dims are flattened."""
    from cider_b200 import nn as cnn
    K, N = 256, 192
    lin = torch.nn.Linear(K, N, bias=True).to(DEV).half()
    m = cnn.CiderLinear.from_float(lin)
    x = t(make_activations(6 * 5, K, seed=21)).reshape(6, 5, K)
    y = m(x)
    assert y.shape == (6, 5, N) and y.dtype == torch.float16
    ref = oracle.c_perchannel_linear(n(x.reshape(-1, K)), n(m.w_int8), n(m.scale_w), n(m.bias))
    assert np.array_equal(n(y.reshape(-1, N)), ref)
    yb = m(x.to(torch.bfloat16))
    assert yb.dtype == torch.bfloat16
    xb16 = x.to(torch.bfloat16).to(torch.float16)
    refb = oracle.c_perchannel_linear(n(xb16.reshape(-1, K)), n(m.w_int8), n(m.scale_w), n(m.bias))
    assert torch.equal(yb.reshape(-1, N), torch.from_numpy(refb).to(DEV).to(torch.bfloat16))
    # decode-shaped call through the module: [1, 1, K]
    y1 = m(x[:1, :1])
    assert y1.shape == (1, 1, N)
    # M == 1 takes the matrix-vector path (no activation quantisation): compare with
    # the oracle's M == 1 branch, not with row 0 of the quantised GEMM
    ref1 = oracle.c_perchannel_linear(n(x[0, :1]), n(m.w_int8), n(m.scale_w), n(m.bias))
    assert rel_err(n(y1.reshape(1, N)), ref1) <= TOL


def test_convert_model_with_fused_projections_is_bit_identical(ops):
    """convert_model(fuse=True): q/k/v and gate/up run as one GEMM each and give the
    bytes of the unfused conversion (quantisation is per output channel)."""
    import copy
    import cider_b200 as cider
    from torch import nn

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj, self.k_proj, self.v_proj = nn.Linear(256, 256), nn.Linear(256, 64), nn.Linear(256, 64)
            self.gate_proj, self.up_proj = nn.Linear(256, 384, bias=False), nn.Linear(256, 384, bias=False)

        def forward(self, x):
            return torch.cat([self.q_proj(x), self.k_proj(x), self.v_proj(x), self.gate_proj(x) * self.up_proj(x)], -1)

    torch.manual_seed(3)
    a = Attn().half().to(DEV)
    b = copy.deepcopy(a)
    sa = cider.convert_model(a, verbose=False)
    sb = cider.convert_model(b, verbose=False, fuse=True)
    assert sa["n_converted"] == sb["n_converted"] == 5 and sb["n_fused_groups"] == 2
    for M in (1, 7, 200):
        x = torch.randn(M, 256, device=DEV).half()
        assert torch.equal(a(x), b(x))


def test_checkpoint_ingested_layers_run(ops, oracle):
    """Layers built from compressed-tensors words compute what the oracle computes from
    the same integers and scales (8-bit per-group, 4-bit per-group)."""
    from cider_b200 import checkpoint
    N, K = 72, 512
    x = make_activations(9, K, seed=21)
    w = make_weight(N, K, seed=22)
    qg, sg = oracle.np_quantize_weight_pergroup(w, 128)
    # 4 consecutive 8-bit fields per int32, little end first, each stored offset binary (+ 128)
    words = np.ascontiguousarray((qg.astype(np.int16) + 128).astype(np.uint8)).view(np.int32)
    lin = checkpoint.linear_from_compressed(torch.from_numpy(words.copy()), torch.from_numpy(sg.astype(np.float16)),
                                            [N, K]).to(DEV)
    sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
    ref = oracle.c_pergroup_linear(x, qg, sg_t, 128, None)
    y = n(lin(t(x)))
    assert rel_err(y, ref) <= 1e-3 and (y != ref).mean() <= 0.05  # M = 9: streaming kernel, fp32 order differs
    w_kn = np.ascontiguousarray(w.T)
    packed_ref, scale_ref = oracle.np_pack_weight_int4_pergroup(w_kn, 64)
    nib = np.zeros((N, K), dtype=np.uint32)
    nib[:, 0::2] = (packed_ref >> 4).T
    nib[:, 1::2] = (packed_ref & 15).T
    w4 = np.zeros((N, K // 8), dtype=np.uint32)
    for i in range(8):
        w4 |= nib[:, i::8] << np.uint32(4 * i)
    lin4 = checkpoint.linear_from_compressed(torch.from_numpy(w4.view(np.int32)),
                                             torch.from_numpy(np.ascontiguousarray(scale_ref.T)), [N, K],
                                             num_bits=4).to(DEV)
    x2 = make_activations(200, K, seed=23)
    assert np.array_equal(n(lin4(t(x2))), oracle.c_w4a8_linear(x2, packed_ref, scale_ref, 64))


def test_convert_model(ops):
    import cider_b200
    model = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.SiLU(),
                                torch.nn.ModuleList([torch.nn.Linear(256, 64), torch.nn.LayerNorm(64)])).to(DEV).half()
    x = t(make_activations(16, 128, seed=31))
    ref = model[2][0](model[1](model[0](x)))
    stats = cider_b200.convert_model(model, verbose=False)
    assert stats["n_converted"] == 2 and stats["elapsed_s"] >= 0
    assert isinstance(model[0], cider_b200.CiderLinear) and isinstance(model[2][0], cider_b200.CiderLinear)
    y = model[2][0](model[1](model[0](x)))
    cos = torch.nn.functional.cosine_similarity(y.float().flatten(), ref.float().flatten(), dim=0)
    assert cos > 0.999


def test_error_behaviour_on_gpu(ops):
    x = t(make_activations(4, 128, seed=1))
    w = torch.zeros(8, 128, dtype=torch.int8, device=DEV)
    with pytest.raises(ValueError):
        ops.pergroup_linear(x, w, torch.ones(4, 8, device=DEV), 32)
    with pytest.raises(ValueError):
        ops.perchannel_linear(x[0], w, torch.ones(8, device=DEV))
    with pytest.raises(ValueError):
        ops.perchannel_linear(x, w[:, :64], torch.ones(8, device=DEV))
    with pytest.raises(RuntimeError):
        ops.perchannel_linear(x.cpu(), w, torch.ones(8, device=DEV))
    assert ops.perchannel_linear(x[:0], w, torch.ones(8, device=DEV)).shape == (0, 8)


# ------------------------------------------- full-size, size-independent checks
def test_full_size_properties(ops, oracle):
    """BASELINE sizes (M = 8192, [10240, 2560]) where the CPU oracle would take
    minutes: (1) row sums of the int32 product equal A . colsum(B) (a checksum of
    checksums, exact in int64); (2) a sampled set of output rows equals the
    oracle run on just those rows (rows are independent in S1..S4)."""
    M, N, K = 8192, 10240, 2560
    g = torch.Generator(device="cpu").manual_seed(0)
    a = torch.randint(-128, 128, (M, K), generator=g, dtype=torch.int8).to(DEV)
    b = torch.randint(-128, 128, (N, K), generator=g, dtype=torch.int8).to(DEV)
    c = ops.int8_matmul_int32(a, b)
    lhs = c.to(torch.int64).sum(dim=1)
    colsum = b.to(torch.int64).sum(dim=0)  # [K]
    rhs = (a.to(torch.int64) * colsum[None, :]).sum(dim=1)
    assert torch.equal(lhs, rhs)
    lhs_t = c.to(torch.int64).sum(dim=0)
    rhs_t = (b.to(torch.int64) * a.to(torch.int64).sum(dim=0)[None, :]).sum(dim=1)
    assert torch.equal(lhs_t, rhs_t)
    del c

    x = make_activations(M, K, seed=0)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=1))
    y = ops.perchannel_linear(t(x), t(wq), t(sw))
    rows = np.array([0, 1, 127, 128, 4095, 4096, 8190, 8191])
    ref = oracle.c_perchannel_linear(x[rows], wq, sw)
    assert np.array_equal(n(y[torch.from_numpy(rows).to(DEV)]), ref)
    wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=2), 128)
    sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
    yg = ops.pergroup_linear(t(x), t(wg), t(sg_t), 128)
    refg = oracle.c_pergroup_linear(x[rows], wg, sg_t, 128)
    assert np.array_equal(n(yg[torch.from_numpy(rows).to(DEV)]), refg)


# ------------------------------------ BASELINE configs at their own sizes (sampled rows)
def _sample_rows(M, seed):
    """Rows on both sides of every 128- and 256-row tile boundary class plus seeded random ones."""
    fixed = [0, 1, 127, 128, 255, 256, M // 2 - 1, M // 2, M - 129, M - 2, M - 1]
    rnd = np.random.default_rng(seed).integers(0, M, 13).tolist()
    return np.array(sorted({r for r in fixed + rnd if 0 <= r < M}))


C1_SHAPES = [(10240, 2560), (2560, 10240)]


@pytest.mark.parametrize("N,K", C1_SHAPES)
@pytest.mark.parametrize("M", [1024, 4096, 8192])
def test_config1_sweep_perchannel(ops, oracle, M, N, K):
    """GEMM sweep of the baseline, per-channel: sampled rows against the oracle (rows are
    independent), and the whole output of the automatic kernel choice (CTA-pair 256 x 256
    tiles at these sizes) against the single-CTA 128-row kernel - two tilings, one result."""
    from cider_b200 import _lib
    x = make_activations(M, K, seed=M + K)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=N))
    bias = (np.random.default_rng(M).standard_normal(N) * 0.05).astype(np.float16)
    xd, wd, sd, bd = t(x), t(wq), t(sw), t(bias)
    y = ops.perchannel_linear(xd, wd, sd, bd)
    rows = _sample_rows(M, N)
    ref = oracle.c_perchannel_linear(x[rows], wq, sw, bias)
    assert np.array_equal(n(y[torch.from_numpy(rows).to(DEV)]), ref)
    lib = _lib.load()
    try:
        assert lib.cider_testing_set_tile(128, 0) == 0
        y128 = ops.perchannel_linear(xd, wd, sd, bd)
        assert lib.cider_testing_set_tile(2, 0) == 0
        ypair = ops.perchannel_linear(xd, wd, sd, bd)
    finally:
        lib.cider_testing_set_tile(0, 0)
    assert torch.equal(y, y128) and torch.equal(y, ypair)
    # the raw int32 product of the same quantised operands: row and column checksums (exact)
    q, _ = ops.quantize_per_token(xd)
    c = ops.int8_matmul_int32(q, wd)
    assert torch.equal(c.to(torch.int64).sum(dim=1), (q.to(torch.int64) * wd.to(torch.int64).sum(dim=0)[None, :]).sum(dim=1))
    assert torch.equal(c.to(torch.int64).sum(dim=0), (wd.to(torch.int64) * q.to(torch.int64).sum(dim=0)[None, :]).sum(dim=1))


@pytest.mark.parametrize("N,K", C1_SHAPES)
@pytest.mark.parametrize("M", [1024, 4096, 8192])
@pytest.mark.parametrize("gs", [128, 64])
def test_config1_sweep_pergroup(ops, oracle, M, N, K, gs):
    """GEMM sweep of the baseline, per-group gs = 128 / 64 with fp16 group scales: sampled
    rows against the oracle, identical bits."""
    x = make_activations(M, K, seed=M + K + gs)
    wq, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=N + gs), gs)
    sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
    y = ops.pergroup_linear(t(x), t(wq), t(sg_t), gs)
    rows = _sample_rows(M, N + gs)
    ref = oracle.c_pergroup_linear(x[rows], wq, sg_t, gs)
    got = n(y[torch.from_numpy(rows).to(DEV)])
    assert rel_err(got, ref) <= TOL
    assert np.array_equal(got, ref), f"fp16 mismatch in {(got != ref).sum()} of {got.size}"


@pytest.mark.parametrize("M,N,K,gs,sdt", [(300, 1000, 2624, 64, np.float32), (777, 520, 1024, 256, np.float32),
                                          (1334, 2048, 2048, 128, np.float16), (256, 128, 128, 128, np.float32),
                                          (513, 264, 192, 64, np.float16)])
def test_pergroup_linear_tall_tile(ops, oracle, M, N, K, gs, sdt):
    """The 128 x 256-tile per-group kernel (taken by itself for large weights), forced here on
    small ragged shapes: rows and columns past the last whole tile, a K that ends inside a
    128-wide block, every group size, both scale types, with a bias - identical bits with the
    oracle and with the 128 x 128 kernel."""
    from cider_b200 import _lib
    x = make_activations(M, K, seed=M + 7)
    wq, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=N + 7), gs)
    sg_t = np.ascontiguousarray(sg.T).astype(sdt)
    bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16)
    lib = _lib.load()
    try:
        assert lib.cider_testing_set_tile(0, 256) == 0
        y_tall = ops.pergroup_linear(t(x), t(wq), t(sg_t), gs, t(bias))
        assert b"gemm_tc_pg2_kernel" in lib.cider_testing_last_gemm_kernel()
        assert lib.cider_testing_set_tile(0, 128) == 0
        y_wide = ops.pergroup_linear(t(x), t(wq), t(sg_t), gs, t(bias))
        assert b"gemm_tc_pg_kernel" in lib.cider_testing_last_gemm_kernel()
    finally:
        lib.cider_testing_set_tile(0, 0)
    ref = oracle.c_pergroup_linear(x, wq, sg_t, gs, bias)
    assert np.array_equal(n(y_tall), ref), f"fp16 mismatch in {(n(y_tall) != ref).sum()} of {ref.size}"
    assert torch.equal(y_tall, y_wide)


@pytest.mark.parametrize("gs", [128, 64])
def test_pergroup_linear_large_weights(ops, oracle, gs):
    """Weights of 48 MB ([4096, 12288], the down projection of the 8B-shaped decoder) over 4096 rows:
    the dispatch takes the 128 x 256 tile; sampled rows against the oracle, identical bits, and the
    whole output against the 128 x 128 kernel."""
    from cider_b200 import _lib
    M, N, K = 4096, 4096, 12288
    x = make_activations(M, K, seed=gs + 11)
    wq, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=gs + 12), gs)
    sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
    xd, wd, sd = t(x), t(wq), t(sg_t)
    lib = _lib.load()
    y = ops.pergroup_linear(xd, wd, sd, gs)
    assert b"gemm_tc_pg2_kernel" in lib.cider_testing_last_gemm_kernel()
    rows = _sample_rows(M, N + gs)
    ref = oracle.c_pergroup_linear(x[rows], wq, sg_t, gs)
    got = n(y[torch.from_numpy(rows).to(DEV)])
    assert np.array_equal(got, ref), f"fp16 mismatch in {(got != ref).sum()} of {got.size}"
    try:
        assert lib.cider_testing_set_tile(0, 128) == 0
        y_wide = ops.pergroup_linear(xd, wd, sd, gs)
    finally:
        lib.cider_testing_set_tile(0, 0)
    assert torch.equal(y, y_wide)


@pytest.mark.parametrize("M", [1, 128, 1024, 8192])
@pytest.mark.parametrize("gs", [64, 0])
def test_config2_w4a8(ops, oracle, M, gs):
    """W4A8 of the baseline ([10240, 2560], int4 per group of 64 with fp16 scales; per-column
    fp32 scales as the reference has them for gs = 0), from the reference's [K/2, N] packing
    and from the row layout: sampled rows against the oracle.  The reference has no M == 1
    branch for W4A8: one row is quantised like any other."""
    N, K = 10240, 2560
    x = make_activations(M, K, seed=M + 4)
    w_kn = np.ascontiguousarray(make_weight(N, K, seed=N + 4).T)
    if gs == 0:
        packed, sw = oracle.np_pack_weight_int4(w_kn)
    else:
        packed, sw = oracle.np_pack_weight_int4_pergroup(w_kn, gs)
    rows = _sample_rows(M, 4 + gs) if M > 64 else np.arange(M)
    ref = oracle.c_w4a8_linear(x[rows], packed, sw, gs)
    pd, sd, xd = t(packed), t(sw), t(x)
    rows_d = torch.from_numpy(rows).to(DEV)
    rows_w = ops.w4a8_repack(pd)
    outs = [ops.w4a8_linear(xd, pd, sd, group_size=gs), ops.w4a8_linear_rows(xd, rows_w, sd, group_size=gs),
            ops.w4a8_linear_rows(xd, rows_w, sd, group_size=gs, int8_scratch=True)]
    for y in outs:
        got = n(y[rows_d])
        assert rel_err(got, ref) <= TOL
        if small_m_group_path(M, K, gs):
            assert rel_err(got, ref) <= 1e-3 and (got != ref).mean() <= 0.05
        else:
            assert np.array_equal(got, ref), f"fp16 mismatch in {(got != ref).sum()} of {got.size}"
    if M > 64:
        assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


@pytest.mark.parametrize("M", [2, 8, 16])
@pytest.mark.parametrize("N,K", [(4096, 12288), (264, 16384), (1024, 8192)])
def test_streaming_kernel_long_k_in_parts(ops, oracle, M, N, K):
    """Several activation rows and a long K: the streaming kernel walks K in parts (only one part of
    the rows staged in shared memory, partial sums per weight tile kept between the parts).
    Per-channel: integer sums, identical to the oracle; per-group: the small-M bar."""
    x = make_activations(M, K, seed=M + K)
    w = make_weight(N, K, seed=N + K)
    wq, sw = oracle.np_quantize_weight_int8(w)
    y = n(ops.perchannel_linear(t(x), t(wq), t(sw)))
    assert np.array_equal(y, oracle.c_perchannel_linear(x, wq, sw)), (M, N, K)
    wg, sg = oracle.np_quantize_weight_pergroup(w, 128)
    sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
    yg = n(ops.pergroup_linear(t(x), t(wg), t(sg_t), 128))
    assert close_bits(yg, oracle.c_pergroup_linear(x, wg, sg_t, 128, None)), (M, N, K)


def test_w4a8_rows_with_activations_off_the_16_byte_grid(ops, oracle):
    """The tensor-core W4A8 kernels want the quantised activations with every 8 k in the order
    k0 k2 k4 k6 k1 k3 k5 k7; the vectorised quantiser writes that order directly, and for an x
    pointer it cannot take (here 2 bytes past a 16-byte boundary) the scalar quantiser plus an
    in-place permutation does.  Same bits either way."""
    import ctypes
    from cider_b200 import _lib
    lib = _lib.load()
    M, N, K = 300, 520, 1152
    x = make_activations(M, K, seed=77)
    w_kn = np.ascontiguousarray(make_weight(N, K, seed=78).T)
    packed, sw = oracle.np_pack_weight_int4(w_kn)
    ref = oracle.c_w4a8_linear(x, packed, sw)
    rows = ops.w4a8_repack(t(packed))
    swd = t(sw)
    buf = torch.zeros(M * K + 8, dtype=torch.float16, device=DEV)
    for off in (0, 1):  # element offset: aligned, then 2 bytes off
        xv = buf[off:off + M * K].view(M, K)
        xv.copy_(t(x))
        assert (xv.data_ptr() % 16 == 0) == (off == 0)
        y = torch.empty((M, N), dtype=torch.float16, device=DEV)
        nbytes = lib.cider_workspace_bytes(_lib.OP_W4A8_ROWS, M, N, K)
        ws = torch.empty(nbytes + 256, dtype=torch.uint8, device=DEV)
        wp = (ws.data_ptr() + 255) // 256 * 256
        _lib.check(lib.cider_w4a8_linear_nk4(xv.data_ptr(), rows.data_ptr(), swd.data_ptr(), _lib.F32, 0, y.data_ptr(),
                                             M, N, K, ctypes.c_void_p(wp), nbytes, None))
        torch.cuda.synchronize()
        assert np.array_equal(n(y), ref), off


@pytest.mark.parametrize("M,N,K", [(128, 2560, 10240), (256, 2048, 6144), (100, 136, 4096), (200, 264, 8192)])
@pytest.mark.parametrize("gs", [0, 128, 64])
def test_small_m_long_k_every_form(ops, oracle, M, N, K, gs):
    """Few output tiles and a long K - the shapes a split-K plan exists for - in the raw int32,
    per-channel and per-group forms, whole outputs against the oracle."""
    x = make_activations(M, K, seed=M + 5)
    w = make_weight(N, K, seed=N + 5)
    if gs == 0:
        wq, sw = oracle.np_quantize_weight_int8(w)
        q, _ = ops.quantize_per_token(t(x))
        c = n(ops.int8_matmul_int32(q, t(wq)))
        assert np.array_equal(c, oracle.c_int8_matmul_int32(n(q), wq))
        y = n(ops.perchannel_linear(t(x), t(wq), t(sw)))
        assert np.array_equal(y, oracle.c_perchannel_linear(x, wq, sw))
    else:
        wq, sg = oracle.np_quantize_weight_pergroup(w, gs)
        sg_t = np.ascontiguousarray(sg.T).astype(np.float16)
        bias = (np.random.default_rng(K).standard_normal(N) * 0.05).astype(np.float16)
        y = n(ops.pergroup_linear(t(x), t(wq), t(sg_t), gs, t(bias)))
        ref = oracle.c_pergroup_linear(x, wq, sg_t, gs, bias)
        assert rel_err(y, ref) <= TOL
        if pg_splitk_path(M, N, K):
            assert close_bits(y, ref)
        else:
            assert np.array_equal(y, ref), f"fp16 mismatch in {(y != ref).sum()} of {y.size}"


def test_ops_on_a_side_stream(ops, oracle):
    """stream= other than the current stream: allocations, conversions and launches all run on
    that stream (a workspace allocated on the current stream could be handed out again while
    the side stream's kernels still use it)."""
    M, N, K = 300, 1024, 2560
    x = make_activations(M, K, seed=41)
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=42))
    wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=43), 128)
    sg_t = np.ascontiguousarray(sg.T)
    xd, wd, sd, wgd, sgd = t(x), t(wq), t(sw), t(wg), t(sg_t)
    side = torch.cuda.Stream(device=DEV)
    outs = []
    for _ in range(4):  # back to back: the allocator gets every chance to reuse a block
        y1 = ops.perchannel_linear(xd.to(torch.bfloat16).to(torch.float16), wd, sd, stream=side)
        y2 = ops.pergroup_linear(xd, wgd, sgd, 128, stream=side)
        junk = torch.empty(M * K + 4096, dtype=torch.uint8, device=DEV).fill_(0x7F)  # current stream
        outs.append((y1, y2, junk))
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    xb = n(xd.to(torch.bfloat16).to(torch.float16))
    ref1, ref2 = oracle.c_perchannel_linear(xb, wq, sw), oracle.c_pergroup_linear(x, wg, sg_t, 128)
    assert pg_splitk_path(M, N, K)  # the per-group call also has its fp32 slabs in the workspace
    for y1, y2, _ in outs:
        assert np.array_equal(n(y1), ref1) and close_bits(n(y2), ref2)
        assert np.array_equal(n(y2), n(outs[0][1]))  # same bits call after call


@pytest.mark.parametrize("M,K", [(1, 64), (37, 2048), (130, 4097), (5, 12288)])
def test_quantiser_in_two_halves(ops, oracle, M, K):
    """row_absmax + quantize_given_amax == quantize_per_token when given the row's own absmax,
    and with a larger absmax (the maximum over a wider row) the oracle's arithmetic on that scale."""
    from cider_b200.decoder import _quantize_with_amax
    x = make_activations(M, K, seed=M + K)
    xd = t(x)
    amax = ops.row_absmax(xd)
    assert np.array_equal(n(amax), np.abs(x.astype(np.float32)).max(axis=1))
    q, s = ops.quantize_given_amax(xd, amax)
    q_ref, s_ref = oracle.c_quantize_per_token(x)
    assert np.array_equal(n(q), q_ref) and np.array_equal(n(s), s_ref)
    wider = amax * 1.7 + 0.25
    q2, s2 = ops.quantize_given_amax(xd, wider)
    q2_ref, s2_ref = _quantize_with_amax(xd, wider)
    assert torch.equal(q2, q2_ref) and torch.equal(s2, s2_ref)


def test_kv_append_past_the_cache_is_skipped_and_reported(ops):
    """A device-side cache position that would fall outside the cache (one graph replay too
    many) writes nothing there and records the overflow bit in the status word."""
    import ctypes
    from cider_b200 import _lib
    lib = _lib.load()
    B, T, nq, nkv, D, Tcap = 1, 1, 4, 2, 128, 8
    qkv = torch.randn(B * T, (nq + 2 * nkv) * D, device=DEV).half()
    ones = torch.ones(D, device=DEV).half()
    inv_freq = torch.ones(D // 2, device=DEV)
    axis = torch.zeros(D // 2, dtype=torch.int8, device=DEV)
    pos = torch.zeros((3, 1), dtype=torch.int32, device=DEV)
    q_out = torch.empty((B, nq, T, D), dtype=torch.float16, device=DEV)
    # the caches sit in the middle of a guard region filled with a sentinel
    guard = torch.full((3, B, nkv, Tcap, D), 7.0, dtype=torch.float16, device=DEV)
    kc, vc = guard[1], guard[1].clone()
    st = ctypes.c_uint(0)
    lib.cider_clear_device_status()
    for base, ok in ((Tcap - 1, True), (Tcap, False), (-1, False), (1 << 20, False)):
        kc.fill_(7.0), vc.fill_(7.0)
        base_dev = torch.tensor([base], dtype=torch.int32, device=DEV)
        ops.qk_norm_rope_append(qkv, ones, ones, inv_freq, axis, pos, 0, 1e-6, q_out, kc, vc, B, T, nq, nkv,
                                base_dev=base_dev)
        assert lib.cider_device_status(st) == 0
        if ok:
            assert st.value == 0 and not (kc[:, :, Tcap - 1] == 7.0).all()
        else:
            assert st.value & 4, f"overflow at base {base} not reported"
            assert (kc == 7.0).all() and (vc == 7.0).all()
            lib.cider_clear_device_status()
        assert (guard[0] == 7.0).all() and (guard[2] == 7.0).all()
    # the host-side base is refused before any launch
    with pytest.raises(ValueError):
        ops.qk_norm_rope_append(qkv, ones, ones, inv_freq, axis, pos, Tcap, 1e-6, q_out, kc, vc, B, T, nq, nkv)


# --------------------------------------------------- decoder glue kernels
@pytest.mark.parametrize("M,K", [(1, 2048), (37, 2048), (130, 4096), (5, 520)])
def test_rmsnorm_quant(ops, oracle, M, K):
    x = make_activations(M, K, seed=M + K, outliers=0)
    w = (1.0 + 0.1 * np.random.default_rng(K).standard_normal(K)).astype(np.float16)
    y, q, s = ops.rmsnorm_quant(t(x), t(w), 1e-6)
    y_ref = oracle.c_rmsnorm(x, w, 1e-6)
    # the norm itself: within one fp16 ulp of the oracle (fp32 vs fp64 mean)
    assert rel_err(n(y), y_ref) <= TOL
    # the fused quantiser must be EXACTLY S1 applied to the fp16 norm output it wrote
    q_ref, s_ref = oracle.c_quantize_per_token(n(y))
    assert np.array_equal(n(q), q_ref) and np.array_equal(n(s), s_ref)
    _, q2, s2 = ops.rmsnorm_quant(t(x), t(w), 1e-6, want_fp16=False)
    assert torch.equal(q2, q) and torch.equal(s2, s)


@pytest.mark.parametrize("B,Hq,Hkv,D,T,Tcap", [(1, 16, 8, 128, 1334, 1600), (1, 16, 8, 128, 1, 64),
                                               (2, 32, 8, 128, 300, 300), (3, 8, 8, 64, 77, 128),
                                               (1, 16, 8, 128, 3711, 3712), (8, 4, 1, 128, 2049, 2176),
                                               (1, 8, 2, 128, 6000, 6144), (1, 4, 4, 64, 4097, 4100),
                                               (1, 8, 8, 128, 700, 704), (2, 16, 8, 128, 4096, 4096),
                                               # long splits: the shared-memory ring form, ragged last stage
                                               (8, 32, 8, 128, 2054, 2056), (8, 16, 8, 128, 1000, 1024),
                                               (4, 8, 8, 64, 5000, 5008), (2, 64, 8, 128, 3001, 3008)])
def test_sdpa_decode(ops, oracle, B, Hq, Hkv, D, T, Tcap):
    rng = np.random.default_rng(T)
    q = rng.standard_normal((B, Hq, D)).astype(np.float16)
    kc = rng.standard_normal((B, Hkv, Tcap, D)).astype(np.float16)
    vc = rng.standard_normal((B, Hkv, Tcap, D)).astype(np.float16)
    from cider_b200 import _lib
    lib = _lib.load()
    ref = oracle.c_sdpa_decode(q, kc, vc, T, 1.0 / np.sqrt(D))
    try:
        # automatic choice, the CUDA-core form, the tensor-core form (mma.sync; grouped queries
        # of 128 dims - other shapes keep the CUDA-core form under every setting)
        for mode in (0, 1, 2):
            assert lib.cider_testing_set_sdpa_kernel(mode) == 0
            out = n(ops.sdpa_decode(t(q), t(kc), t(vc), T, 1.0 / np.sqrt(D)))
            assert rel_err(out, ref) <= TOL, f"kernel mode {mode}"
            # one-launch form: same merge arithmetic, counters back at zero, reusable at once
            tickets = torch.zeros(B * Hkv, dtype=torch.int32, device=DEV)
            for _ in range(2):
                out1 = n(ops.sdpa_decode(t(q), t(kc), t(vc), T, 1.0 / np.sqrt(D), tickets=tickets))
                assert np.array_equal(out1, out)
                assert not tickets.any()
    finally:
        lib.cider_testing_set_sdpa_kernel(0)
