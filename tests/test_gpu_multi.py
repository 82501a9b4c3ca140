"""Multi-GPU paths (need >= 2 GPUs; skipped otherwise).

* A single linear split over output channels across two GPUs with no collective:
  every GPU quantises the full activation itself (the per-token scale is a
  function of the whole row), so the concatenated result is bit-identical to the
  one-GPU result.
* The tensor-parallel decoder over two NCCL ranks (column-parallel q/k/v and
  gate/up, row-parallel o/down + all-reduce) against the one-GPU decoder.
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


@needs2
def test_linear_split_over_output_channels_is_bit_identical(oracle):
    from cider_b200 import ops
    M, N, K = 300, 1024, 2560
    x = torch.from_numpy(make_activations(M, K, seed=1))
    wq, sw = oracle.np_quantize_weight_int8(make_weight(N, K, seed=2))
    bias = torch.from_numpy((np.random.default_rng(3).standard_normal(N) * 0.05).astype(np.float16))
    wq, sw = torch.from_numpy(wq), torch.from_numpy(sw)
    full = ops.perchannel_linear(x.cuda(0), wq.cuda(0), sw.cuda(0), bias.cuda(0)).cpu()
    parts = []
    for dev, sl in ((0, slice(0, N // 2)), (1, slice(N // 2, N))):
        d = torch.device("cuda", dev)
        parts.append(ops.perchannel_linear(x.to(d), wq[sl].to(d), sw[sl].to(d), bias[sl].to(d)).cpu())
    assert torch.equal(torch.cat(parts, dim=1), full)
    wg, sg = oracle.np_quantize_weight_pergroup(make_weight(N, K, seed=4), 128)
    wg, sg = torch.from_numpy(wg), torch.from_numpy(np.ascontiguousarray(sg.T))
    full = ops.pergroup_linear(x.cuda(0), wg.cuda(0), sg.cuda(0), 128).cpu()
    parts = []
    for dev, sl in ((0, slice(0, N // 2)), (1, slice(N // 2, N))):
        d = torch.device("cuda", dev)
        parts.append(ops.pergroup_linear(x.to(d), wg[sl].to(d), sg[:, sl].contiguous().to(d), 128).cpu())
    assert torch.equal(torch.cat(parts, dim=1), full)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, exact, ret):
    import torch.distributed as dist
    from cider_b200.decoder import Decoder, mrope_position_ids
    from test_gpu_decoder import SMALL, _prompt
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    d = Decoder(SMALL, mode="w8a8", group_size=128, device=f"cuda:{rank}", max_len=256, seed=7,
                tp_rank=rank, tp_size=world, tp_exact_scales=exact)
    emb, pos = _prompt(d, 100, 64)
    logits = d.prefill(emb, pos)
    nxt = d.decode_step(logits.argmax(dim=-1))
    if rank == 0:
        ret["prefill"], ret["decode"] = logits.cpu(), nxt.cpu()
    dist.barrier()
    dist.destroy_process_group()


@needs2
@pytest.mark.parametrize("exact", [True, False])
def test_tensor_parallel_decoder_two_nccl_ranks(exact):
    import torch.multiprocessing as mp
    from cider_b200.decoder import Decoder
    from test_gpu_decoder import SMALL, _prompt
    ref = Decoder(SMALL, mode="w8a8", group_size=128, device="cuda:0", max_len=256, seed=7)
    emb, pos = _prompt(ref, 100, 64)
    want = ref.prefill(emb, pos)
    want2 = ref.decode_step(want.argmax(dim=-1))
    ret = mp.Manager().dict()
    mp.spawn(_tp_worker, args=(2, _free_port(), exact, ret), nprocs=2, join=True)
    for got, w in ((ret["prefill"], want.cpu()), (ret["decode"], want2.cpu())):
        assert F.cosine_similarity(got.flatten(), w.flatten(), dim=0) >= 0.999
