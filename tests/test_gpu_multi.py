"""Multi-GPU paths.

* A single linear split over output channels with no collective: every shard
  quantises the full activation itself (the per-token scale is a function of the
  whole row), so the concatenated result is bit-identical to the unsplit result.
  The shards run on two GPUs when the box has them, else one after the other on
  the same GPU (the arithmetic does not know the difference).
* The tensor-parallel decoder over two ranks (column-parallel q/k/v and gate/up,
  row-parallel o/down + all-reduce) against the one-GPU decoder: two NCCL ranks
  on two GPUs, and - also on a one-GPU box - two processes that share GPU 0 and
  exchange through gloo (host-mediated: no kernel of one rank ever waits for a
  kernel of the other, so sharing a GPU is safe).
* The one-shot peer-memory all-reduce: the ranks emulated as ONE cooperative
  launch on one GPU, its bounded wait, and two real ranks when there are two GPUs.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from conftest import make_activations, make_weight

pytestmark = pytest.mark.gpu

needs2 = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")


SPLIT_DEVS = (0, 1) if torch.cuda.device_count() >= 2 else (0, 0)


@pytest.mark.parametrize("M,N,K", [(300, 1024, 2560), (2048, 10240, 2560)])
def test_linear_split_over_output_channels_is_bit_identical(oracle, M, N, K):
    from cider_b200 import ops
    x = torch.from_numpy(make_activations(M, K, seed=1))
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=2))
    bias = torch.from_numpy((np.random.default_rng(3).standard_normal(N) * 0.05).astype(np.float16))
    wq, sw = torch.from_numpy(wq), torch.from_numpy(sw)
    full = ops.perchannel_linear(x.cuda(0), wq.cuda(0), sw.cuda(0), bias.cuda(0)).cpu()
    parts = []
    for dev, sl in ((SPLIT_DEVS[0], slice(0, N // 2)), (SPLIT_DEVS[1], slice(N // 2, N))):
        d = torch.device("cuda", dev)
        parts.append(ops.perchannel_linear(x.to(d), wq[sl].to(d), sw[sl].to(d), bias[sl].to(d)).cpu())
    assert torch.equal(torch.cat(parts, dim=1), full)
    wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=4), 128)
    wg, sg = torch.from_numpy(wg), torch.from_numpy(np.ascontiguousarray(sg.T))
    full = ops.pergroup_linear(x.cuda(0), wg.cuda(0), sg.cuda(0), 128).cpu()
    parts = []
    for dev, sl in ((SPLIT_DEVS[0], slice(0, N // 2)), (SPLIT_DEVS[1], slice(N // 2, N))):
        d = torch.device("cuda", dev)
        parts.append(ops.pergroup_linear(x.to(d), wg[sl].to(d), sg[:, sl].contiguous().to(d), 128).cpu())
    assert torch.equal(torch.cat(parts, dim=1), full)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, exact, backend, ret):
    import torch.distributed as dist
    from cider_b200.decoder import Decoder, mrope_position_ids
    from test_gpu_decoder import SMALL, _prompt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dev = rank if backend == "nccl" else 0  # gloo: both ranks share GPU 0
    torch.cuda.set_device(dev)
    if backend == "nccl":
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", dev))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    d = Decoder(SMALL, mode="w8a8", group_size=128, device=f"cuda:{dev}", max_len=256, seed=7,
                tp_rank=rank, tp_size=world, tp_exact_scales=exact)
    emb, pos = _prompt(d, 100, 64)
    logits = d.prefill(emb, pos)
    nxt = d.decode_step(logits.argmax(dim=-1))
    if rank == 0:
        ret["prefill"], ret["decode"] = logits.cpu(), nxt.cpu()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("backend", ["nccl", "gloo"])
@pytest.mark.parametrize("exact", [True, False])
def test_tensor_parallel_decoder_two_ranks(exact, backend):
    import torch.multiprocessing as mp
    if backend == "nccl" and torch.cuda.device_count() < 2:
        pytest.skip("two NCCL ranks need two GPUs")
    from cider_b200.decoder import Decoder
    from test_gpu_decoder import SMALL, _prompt
    ref = Decoder(SMALL, mode="w8a8", group_size=128, device="cuda:0", max_len=256, seed=7)
    emb, pos = _prompt(ref, 100, 64)
    want = ref.prefill(emb, pos)
    want2 = ref.decode_step(want.argmax(dim=-1))
    ret = mp.Manager().dict()
    mp.spawn(_tp_worker, args=(2, _free_port(), exact, backend, ret), nprocs=2, join=True)
    for got, w in ((ret["prefill"], want.cpu()), (ret["decode"], want2.cpu())):
        assert F.cosine_similarity(got.flatten(), w.flatten(), dim=0) >= 0.999


# ------------------------------------------------ one-shot peer-memory all-reduce
def _emulated(lib, _lib, ins, outs, inboxes, inbox_bytes, wait_cycles=0, absent=-1):
    import ctypes
    world = len(ins)
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])  # noqa: E731
    return lib.cider_testing_allreduce_emulated(arr(ins), arr(outs), ins[0].numel(), world, arr(inboxes),
                                                inbox_bytes, wait_cycles, absent,
                                                int(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("world,count", [(2, 8), (2, 4096), (4, 8 * 4096), (8, 8 * 4096), (3, 1000 * 8), (8, 2048)])
def test_peer_allreduce_ranks_emulated_in_one_launch(world, count):
    """All ranks of the one-shot all-reduce as ONE cooperative launch on one GPU (separate
    launches that wait for one another must not share a GPU): every rank's result equals the
    fp32 sum in rank order rounded once, bit for bit, over several calls in a row (sequence
    numbers, both parities) with fresh data each time."""
    import ctypes
    from cider_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    lib.cider_clear_device_status()
    inbox_bytes = 2 << 20
    assert count * 2 <= lib.cider_peer_max_bytes(inbox_bytes)
    inboxes = [torch.zeros(inbox_bytes, dtype=torch.uint8, device="cuda:0") for _ in range(world)]
    g = torch.Generator().manual_seed(world * 1000 + count)
    for call in range(5):
        ins = [(torch.randn(count, generator=g) * 3).half().cuda() for _ in range(world)]
        outs = [torch.full((count,), float("nan"), dtype=torch.float16, device="cuda:0") for _ in range(world)]
        _lib.check(_emulated(lib, _lib, ins, outs, inboxes, inbox_bytes))
        torch.cuda.synchronize()
        acc = torch.zeros(count, dtype=torch.float32, device="cuda:0")
        for x in ins:
            acc = acc + x.float()
        want = acc.half()
        for o in outs:
            assert torch.equal(o, want), f"call {call}"
    # in place
    ins = [(torch.randn(count, generator=g)).half().cuda() for _ in range(world)]
    want = sum(x.float() for x in ins).half()
    _lib.check(_emulated(lib, _lib, ins, ins, inboxes, inbox_bytes))
    torch.cuda.synchronize()
    assert all(torch.equal(x, want) for x in ins)
    st = ctypes.c_uint(0)
    assert lib.cider_device_status(st) == 0 and st.value == 0


@pytest.mark.parametrize("world,M,K", [(2, 8, 4096), (4, 1, 2048), (8, 8, 4096), (3, 5, 520), (2, 32, 8192)])
def test_peer_allreduce_fused_with_add_rmsnorm_quant(world, M, K):
    """The exchange fused with the residual add and the RMSNorm (+ quantiser) that follow it,
    ranks emulated in one cooperative launch: the updated residual equals half(x + all-reduce)
    bit for bit, the norm matches the stand-alone kernel within 2e-3, and the int8 output is
    EXACTLY the per-token quantiser applied to the fp16 norm output the kernel wrote."""
    import ctypes
    from cider_b200 import _lib, ops
    lib = _lib.load()
    torch.cuda.set_device(0)
    lib.cider_clear_device_status()
    inbox_bytes = 16 << 20
    assert M * K * 2 <= lib.cider_peer_max_bytes(inbox_bytes)
    inboxes = [torch.zeros(inbox_bytes, dtype=torch.uint8, device="cuda:0") for _ in range(world)]
    g = torch.Generator().manual_seed(world * 100 + M + K)
    w = (1 + 0.1 * torch.randn(K, generator=g)).half().cuda()
    arr = lambda ts: (ctypes.c_void_p * world)(*[t.data_ptr() for t in ts])  # noqa: E731
    for call in range(3):
        parts = [(torch.randn(M, K, generator=g) * 0.5).half().cuda() for _ in range(world)]
        x0 = torch.randn(M, K, generator=g).half().cuda()
        xs = [x0.clone() for _ in range(world)]
        ys = [torch.empty_like(x0) for _ in range(world)]
        qs = [torch.empty((M, K), dtype=torch.int8, device="cuda:0") for _ in range(world)]
        ss = [torch.empty(M, dtype=torch.float32, device="cuda:0") for _ in range(world)]
        _lib.check(lib.cider_testing_allreduce_norm_emulated(arr(parts), arr(xs), w.data_ptr(), 1e-6, M, K, arr(ys),
                                                             arr(qs), arr(ss), world, arr(inboxes), inbox_bytes,
                                                             int(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
        acc = torch.zeros(M, K, dtype=torch.float32, device="cuda:0")
        for pt in parts:
            acc = acc + pt.float()
        delta = acc.half()
        x_ref = x0.clone()
        y_ref, _, _ = ops.add_rmsnorm(x_ref, delta, w, 1e-6)
        for r in range(world):
            assert torch.equal(xs[r], x_ref), f"call {call} rank {r}: residual stream differs"
            assert (ys[r].float() - y_ref.float()).abs().max() <= 2e-3 * y_ref.float().abs().max()
            q2, s2 = ops.quantize_per_token(ys[r])
            assert torch.equal(qs[r], q2) and torch.equal(ss[r], s2)
            assert torch.equal(ys[r], ys[0]) and torch.equal(qs[r], qs[0])  # every rank: the same bits
    st = ctypes.c_uint(0)
    assert lib.cider_device_status(st) == 0 and st.value == 0


def test_peer_allreduce_wait_is_bounded():
    """A peer that never shows up: the wait on its flag runs out after the given number of
    clocks, the kernel records the time-out in the status word, writes no result and
    returns; the context stays usable and, after a reset of the inboxes, so does the group."""
    import ctypes
    from cider_b200 import _lib
    lib = _lib.load()
    torch.cuda.set_device(0)
    lib.cider_clear_device_status()
    world, count, inbox_bytes = 3, 4096, 1 << 20
    inboxes = [torch.zeros(inbox_bytes, dtype=torch.uint8, device="cuda:0") for _ in range(world)]
    ins = [torch.ones(count, dtype=torch.float16, device="cuda:0") * (q + 1) for q in range(world)]
    outs = [torch.full((count,), -7.0, dtype=torch.float16, device="cuda:0") for _ in range(world)]
    _lib.check(_emulated(lib, _lib, ins, outs, inboxes, inbox_bytes, wait_cycles=2_000_000, absent=1))  # ~1 ms
    st = ctypes.c_uint(0)
    assert lib.cider_device_status(st) == 0
    assert st.value & 8, "the time-out was not recorded"
    assert all((o == -7.0).all() for o in outs), "a result was written although a peer was missing"
    lib.cider_clear_device_status()
    for b in inboxes:  # what PeerGroup.reset does on every rank
        _lib.check(lib.cider_peer_reset(b.data_ptr(), None))
    _lib.check(_emulated(lib, _lib, ins, outs, inboxes, inbox_bytes))
    torch.cuda.synchronize()
    assert all((o == 6.0).all() for o in outs)
    assert lib.cider_device_status(st) == 0 and st.value == 0
    # argument checks come before any launch
    assert _emulated(lib, _lib, ins[:1], outs[:1], inboxes[:1], inbox_bytes) == _lib.E_INVALID
    big = [torch.zeros(1 << 20, dtype=torch.float16, device="cuda:0") for _ in range(2)]
    assert _emulated(lib, _lib, big, big, inboxes[:2], inbox_bytes) == _lib.E_WORKSPACE


def _peer_worker(rank, world, port, ret):
    import torch.distributed as dist
    from cider_b200.peer import PeerGroup
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pg = PeerGroup(rank, world, device=f"cuda:{rank}")
    ok = True
    for call in range(6):
        count = [8, 4096, 8 * 4096, 2048, 8 * 4096, 1000 * 8][call]
        g = torch.Generator().manual_seed(call)
        parts = [(torch.randn(count, generator=g) * 2).half() for _ in range(world)]
        want = sum(p.float() for p in parts).half()
        got = pg.all_reduce(parts[rank].cuda())
        ok = ok and torch.equal(got.cpu(), want)
    # replayed from a CUDA graph: the call counter lives in device memory
    x = torch.ones(4096, dtype=torch.float16, device=f"cuda:{rank}") * (rank + 1)
    y = torch.empty_like(x)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        pg.all_reduce(x, out=y)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        pg.all_reduce(x, out=y)
    for _ in range(5):
        y.zero_()
        gr.replay()
        torch.cuda.synchronize()
        ok = ok and bool((y == world * (world + 1) / 2).all())
    import ctypes
    from cider_b200 import _lib
    st = ctypes.c_uint(0)
    _lib.load().cider_device_status(st)
    ret[rank] = ok and st.value == 0
    pg.close()
    dist.destroy_process_group()


@needs2
def test_peer_allreduce_two_real_ranks():
    """Two processes, two GPUs: PeerGroup (IPC-mapped inboxes) against the fp32 sum in rank
    order, eager and replayed from a CUDA graph."""
    import torch.multiprocessing as mp
    ret = mp.Manager().dict()
    mp.spawn(_peer_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert ret[0] and ret[1]


def _tp_graph_worker(rank, world, port, fuse, ret):
    import torch.distributed as dist
    from cider_b200.decoder import Decoder
    from cider_b200.peer import PeerGroup
    from test_gpu_decoder import SMALL, _prompt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pg = PeerGroup(rank, world, device=f"cuda:{rank}")
    # two sequences with the fused exchange: a decode step of M = 2 rows takes the general path,
    # where the all-reduce, the residual add and the norm are one kernel (M = 1 folds the add and
    # the norm into the next matrix-vector kernel instead)
    B = 2 if fuse else 1
    d = Decoder(SMALL, mode="w8a8", group_size=128, device=f"cuda:{rank}", max_len=256, seed=7,
                tp_rank=rank, tp_size=world, peer=pg, batch=B)
    d.fuse_allreduce_norm = fuse
    emb, pos = _prompt(d, 100, 64)
    if B == 2:
        emb = torch.cat([emb, (emb.float() * 0.5).to(emb.dtype)], dim=0)
    eager, _ = d.generate(emb, pos, 24)
    graph, _ = d.generate(emb, pos, 24, use_graph=True)
    d.reset()
    logits = d.prefill(emb, pos)
    import ctypes
    from cider_b200 import _lib
    st = ctypes.c_uint(0)
    _lib.load().cider_device_status(st)
    if rank == 0:
        ret["eager"], ret["graph"], ret["logits"], ret["status"] = eager.cpu(), graph.cpu(), logits[:1].cpu(), st.value
    dist.barrier()
    pg.close()
    dist.destroy_process_group()


@needs2
@pytest.mark.parametrize("fuse", [False, True])
def test_tensor_parallel_decode_graph_with_peer_allreduce(fuse):
    """Tensor-parallel decode with the all-reduces done by the library's own kernel: the
    captured decode step (no NCCL inside) produces the tokens of the eager step, and the
    prefill logits match the one-GPU decoder (cosine >= 0.999)."""
    import torch.multiprocessing as mp
    from cider_b200.decoder import Decoder
    from test_gpu_decoder import SMALL, _prompt
    ref = Decoder(SMALL, mode="w8a8", group_size=128, device="cuda:0", max_len=256, seed=7)
    emb, pos = _prompt(ref, 100, 64)
    want = ref.prefill(emb, pos)
    ret = mp.Manager().dict()
    mp.spawn(_tp_graph_worker, args=(2, _free_port(), fuse, ret), nprocs=2, join=True)
    assert ret["status"] == 0
    assert torch.equal(ret["eager"], ret["graph"])
    assert F.cosine_similarity(ret["logits"].flatten(), want.cpu().flatten(), dim=0) >= 0.999
