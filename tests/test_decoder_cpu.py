"""Decoder driver on CPU (float32 linears): architecture against transformers'
Qwen3VLTextModel, M-RoPE position ids against the reference's index arithmetic
(vlm_service/custom_qwen3vl.py:208-251), chunked prefill, the generation driver's
bookkeeping, and tensor-parallel sharding over 2 gloo ranks."""
import os
import socket

import numpy as np
import pytest
import torch

from cider_b200 import ops
from cider_b200.decoder import (Decoder, DecoderConfig, mrope_position_ids, quantize_weight_int8_torch,
                                quantize_weight_pergroup_torch, rope_cos_sin)

TINY = DecoderConfig(hidden=64, layers=2, n_q=4, n_kv=2, head_dim=16, inter=96, vocab=100,
                     mrope_section=(4, 2, 2), rope_theta=1e4)


def test_mrope_position_ids_follow_reference_arithmetic():
    # text(3) image(1x2x3) text(2) image(1x2x2) text(1)
    pos = mrope_position_ids([("text", 3), ("image", (1, 2, 3)), ("text", 2), ("image", (1, 2, 2)), ("text", 1)])
    # text 0,1,2 ; image starts at text_len + st_idx = 3: t=3, h=3..4, w=3..5 ; next text at max+1 = 6
    exp_t = [0, 1, 2, 3, 3, 3, 3, 3, 3, 6, 7, 8, 8, 8, 8, 10]
    exp_h = [0, 1, 2, 3, 3, 3, 4, 4, 4, 6, 7, 8, 8, 9, 9, 10]
    exp_w = [0, 1, 2, 3, 4, 5, 3, 4, 5, 6, 7, 8, 9, 8, 9, 10]
    assert pos.tolist() == [exp_t, exp_h, exp_w]
    # the bench prompt: a 32x32 grid first, then text starting at 32
    p = mrope_position_ids([("image", (1, 32, 32)), ("text", 310)])
    assert p.shape == (3, 1334) and p[:, 1024].tolist() == [32, 32, 32] and int(p.max()) == 32 + 309
    assert mrope_position_ids([]).shape == (3, 0)


def test_interleaved_mrope_slots():
    cfg = DecoderConfig(hidden=8, layers=1, n_q=1, n_kv=1, head_dim=128, inter=8, vocab=8,
                        mrope_section=(24, 20, 20), rope_theta=1e6)
    pos = torch.tensor([[5], [7], [11]])
    cos, _ = rope_cos_sin(cfg, pos)
    inv = 1.0 / (1e6 ** (torch.arange(0, 64, dtype=torch.float32) / 64))
    axis = [0] * 64
    for i in range(64):
        if i % 3 == 1 and i < 60:
            axis[i] = 1
        elif i % 3 == 2 and i < 60:
            axis[i] = 2
    want = torch.cos(torch.tensor([float(pos[a, 0]) for a in axis]) * inv)
    assert torch.allclose(cos[0, :64], want, atol=1e-6) and torch.allclose(cos[0, 64:], want, atol=1e-6)


def test_architecture_matches_transformers_qwen3vl_text_model():
    tf = pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLTextConfig
    hc = Qwen3VLTextConfig(vocab_size=100, hidden_size=64, intermediate_size=96, num_hidden_layers=2,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=16, rms_norm_eps=1e-6,
                           rope_parameters={"rope_type": "default", "rope_theta": 1e4, "mrope_section": [4, 2, 2],
                                            "mrope_interleaved": True},
                           attention_bias=False, tie_word_embeddings=True)
    hc._attn_implementation = "eager"
    m = tf.Qwen3VLTextModel(hc).eval().float()
    d = Decoder(TINY, mode="fp16", device="cpu", dtype=torch.float32, max_len=64)
    D = 16
    with torch.no_grad():
        for li, (hl, lw) in enumerate(zip(m.layers, d.layers)):
            q, k, v = lw.lin["qkv"].split([4 * D, 2 * D, 2 * D], 0)
            hl.self_attn.q_proj.weight.copy_(q)
            hl.self_attn.k_proj.weight.copy_(k)
            hl.self_attn.v_proj.weight.copy_(v)
            hl.self_attn.o_proj.weight.copy_(lw.lin["o"])
            g, u = lw.lin["gate_up"].split([96, 96], 0)
            hl.mlp.gate_proj.weight.copy_(g)
            hl.mlp.up_proj.weight.copy_(u)
            hl.mlp.down_proj.weight.copy_(lw.lin["down"])
            torch.manual_seed(li)
            for mine, theirs in ((("norm1", hl.input_layernorm)), ("norm2", hl.post_attention_layernorm),
                                 ("q_norm", hl.self_attn.q_norm), ("k_norm", hl.self_attn.k_norm)):
                w = 1 + 0.1 * torch.randn(theirs.weight.shape[0])
                setattr(lw, mine, w.clone())
                theirs.weight.copy_(w)
        m.norm.weight.fill_(1.0)
    pos = mrope_position_ids([("text", 3), ("image", (1, 4, 4)), ("text", 6)])
    emb = torch.randn(1, pos.shape[1], 64)
    with torch.no_grad():
        ref = m(inputs_embeds=emb, position_ids=pos[:, None, :]).last_hidden_state
        mine = d.forward(emb, pos)
    assert (ref - mine).abs().max() < 1e-5


def test_chunked_prefill_and_generation_driver():
    pos = mrope_position_ids([("image", (1, 4, 4)), ("text", 9)])
    emb = torch.randn(1, 25, 64, generator=torch.Generator().manual_seed(0))
    a = Decoder(TINY, mode="fp16", device="cpu", dtype=torch.float32, max_len=64)
    whole = a.prefill(emb, pos)
    a.reset()
    chunked = a.prefill(emb, pos, prefill_step_size=7)  # the image span straddles chunks
    assert torch.allclose(whole, chunked, atol=1e-5)
    toks, stats = a.generate(emb, pos, max_tokens=6, prefill_step_size=8)
    assert toks.shape == (1, 6) and a.cur_len == 25 + 5 and a.next_pos == int(pos.max()) + 1 + 5
    assert stats["prompt_tokens"] == 25 and stats["generation_tokens"] == 5
    assert stats["prompt_tps"] > 0 and stats["generation_tps"] > 0
    # greedy decode == re-running the whole sequence through prefill
    b = Decoder(TINY, mode="fp16", device="cpu", dtype=torch.float32, max_len=64)
    seq = torch.cat([emb, b.embed[toks[0, :3]][None]], dim=1)
    pos2 = torch.cat([pos, (int(pos.max()) + 1 + torch.arange(3)).expand(3, 3)], dim=1)
    assert int(b.prefill(seq, pos2).argmax()) == int(toks[0, 3])


def test_device_side_weight_quant_equals_host_helpers():
    torch.manual_seed(1)
    w = (torch.randn(48, 256) * 0.02).half()
    w[3] = 0
    q, s = quantize_weight_int8_torch(w)
    qn, sn = ops.quantize_weight_int8(w.float().numpy())
    assert np.array_equal(q.numpy(), qn) and np.array_equal(s.numpy(), sn)
    qg, sg = quantize_weight_pergroup_torch(w, 64, torch.float32)
    qgn, sgn = ops.quantize_weight_int8_pergroup(w.float().numpy(), 64)
    assert np.array_equal(qg.numpy(), qgn) and np.array_equal(sg.numpy(), sgn.T)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tp_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    d = Decoder(TINY, mode="fp16", device="cpu", dtype=torch.float32, max_len=64, tp_rank=rank, tp_size=world)
    pos = mrope_position_ids([("image", (1, 4, 4)), ("text", 5)])
    emb = torch.randn(1, 21, 64, generator=torch.Generator().manual_seed(3))
    logits = d.prefill(emb, pos)
    nxt = d.decode_step(logits.argmax(dim=-1))
    if rank == 0:
        ret["prefill"], ret["decode"] = logits, nxt
    dist.destroy_process_group()


def test_tensor_parallel_two_gloo_ranks_match_single_rank():
    import torch.multiprocessing as mp
    ref = Decoder(TINY, mode="fp16", device="cpu", dtype=torch.float32, max_len=64)
    pos = mrope_position_ids([("image", (1, 4, 4)), ("text", 5)])
    emb = torch.randn(1, 21, 64, generator=torch.Generator().manual_seed(3))
    want = ref.prefill(emb, pos)
    want2 = ref.decode_step(want.argmax(dim=-1))
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_tp_worker, args=(2, _free_port(), ret), nprocs=2, join=True)
    assert torch.allclose(ret["prefill"], want, atol=1e-4)
    assert torch.allclose(ret["decode"], want2, atol=1e-4)
