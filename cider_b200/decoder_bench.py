"""Prefill / decode throughput of the random-init decoders (configs 3 and 4).

    python -m cider_b200.decoder_bench --model qwen3vl2b --mode w8a8 --prompt 1334 --decode 256
    torchrun --nproc-per-node 4 -m cider_b200.decoder_bench --model qwen3_8b --group-size 128 \
        --batch 8 --prompt 2048 --decode 128

Prompts are synthetic stand-ins for the reference's recorded screenshot prompts
(benchmarks/bench_e2e_wxa16.py): for the VL model the first 1024 positions are
N(0,1) "vision" embeddings on a 32x32 M-RoPE grid, the rest uniform random token
ids.  tok/s follow vlm_service/custom_qwen3vl.py:798-803,825 (prompt tokens / time
to first token; generated tokens / time after it); the vision tower is not part
of the measurement.  Prints one JSON line per run (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from .decoder import QWEN3_8B, QWEN3_VL_2B, Decoder, mrope_position_ids


def build_prompt(dec: Decoder, batch: int, T: int, vision: int, seed: int = 0):
    g = torch.Generator().manual_seed(seed)
    cfg = dec.cfg
    ids = torch.randint(0, cfg.vocab, (batch, T - vision), generator=g).to(dec.device)
    text = dec.embed[ids]
    if vision:
        side = int(round(vision ** 0.5))
        assert side * side == vision
        vis = torch.randn(batch, vision, cfg.hidden, generator=g).to(dec.dtype).to(dec.device)
        emb = torch.cat([vis, text], dim=1)
        pos = mrope_position_ids([("image", (1, side, side)), ("text", T - vision)])
    else:
        emb = text
        pos = torch.arange(T).expand(3, T)
    return emb.contiguous(), pos


def run_decoder(model: str = "qwen3vl2b", mode: str = "w8a8", group_size: int = 0, batch: int = 1,
                prompt: int = 1334, vision: int = -1, decode: int = 256, layers=None, prefill_step: int = 8192,
                repeat: int = 2, graph: bool = True, int8_lm_head: bool = False, rank: int = 0, world: int = 1,
                local: int = 0, group=None, dec: Decoder = None, peer=None):
    """One configuration: a warm-up generation (lazy initialisation, graph capture: not
    counted) and then ``repeat`` timed generations; returns the best prefill and the best
    decode tok/s of the timed ones with the reference's definitions
    (vlm_service/custom_qwen3vl.py:798-803, :825).  ``dec`` reuses an already built decoder
    (a new prompt length on the same weights)."""
    cfg = QWEN3_VL_2B if model == "qwen3vl2b" else QWEN3_8B
    vision = vision if vision >= 0 else (1024 if model == "qwen3vl2b" else 0)
    if dec is None:
        dec = Decoder(cfg, mode=mode, group_size=group_size, device=f"cuda:{local}",
                      max_len=prompt + decode + 8, batch=batch, tp_rank=rank, tp_size=world,
                      group=group, layers=layers, int8_lm_head=int8_lm_head, peer=peer)
    assert prompt + decode <= dec.max_len
    emb, pos = build_prompt(dec, batch, prompt, vision)
    # a tensor-parallel prefill runs its NCCL all-reduces eagerly; its decode step, whose
    # all-reduces are this library's own kernel when a peer group is given, replays as a graph
    use_graph = bool(graph) and (world == 1 or dec.peer is not None)
    runs = []
    toks = None
    for i in range(repeat + 1):
        toks, stats = dec.generate(emb, pos, decode, prefill_step, use_graph=use_graph)
        if i > 0:  # the first run is the warm-up
            runs.append(stats)
    best_p = max(r["prompt_tps"] for r in runs)
    best_d = max(r["generation_tps"] for r in runs)
    out = {"model": model, "mode": mode, "group_size": group_size, "tp": world,
           "batch": batch, "prompt": prompt, "decode": decode,
           "layers": dec.n_layers, "graph": use_graph, "int8_lm_head": bool(int8_lm_head),
           "prefill_tok_s": best_p, "decode_tok_s": best_d,
           "ttft_ms": min(r["time_to_first_token_s"] for r in runs) * 1e3,
           "first_tokens": toks[0, :8].tolist()}
    return out, dec


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen3vl2b", choices=["qwen3vl2b", "qwen3_8b"])
    ap.add_argument("--mode", default="w8a8", choices=["w8a8", "fp16"])
    ap.add_argument("--group-size", type=int, default=0)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt", type=int, default=1334)
    ap.add_argument("--vision", type=int, default=-1, help="vision positions at the start (-1: 1024 for the VL model)")
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--prefill-step", type=int, default=8192)
    ap.add_argument("--repeat", type=int, default=2)
    ap.add_argument("--graph", type=int, default=1, help="capture the decode step in a CUDA graph")
    ap.add_argument("--int8-lm-head", type=int, default=0,
                    help="also quantise the output head (the reference leaves it in fp16)")
    ap.add_argument("--fuse-allreduce-norm", type=int, default=-1,
                    help="tensor parallel: all-reduce + residual add + RMSNorm as one kernel (1), separate (0), "
                         "or the decoder's default (-1)")
    ap.add_argument("--peer-allreduce", type=int, default=1,
                    help="tensor parallel: decode-step all-reduces by the one-shot peer-memory kernel (1) or NCCL (0)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = peer = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        if args.peer_allreduce:
            from .peer import PeerGroup
            peer = PeerGroup(rank, world, device=torch.device("cuda", local))
    dec = None
    if args.fuse_allreduce_norm >= 0:
        cfg = QWEN3_VL_2B if args.model == "qwen3vl2b" else QWEN3_8B
        dec = Decoder(cfg, mode=args.mode, group_size=args.group_size, device=f"cuda:{local}",
                      max_len=args.prompt + args.decode + 8, batch=args.batch, tp_rank=rank, tp_size=world,
                      group=group, layers=args.layers, int8_lm_head=bool(args.int8_lm_head), peer=peer)
        dec.fuse_allreduce_norm = bool(args.fuse_allreduce_norm)
    out, dec = run_decoder(args.model, args.mode, args.group_size, args.batch, args.prompt, args.vision, args.decode,
                           args.layers, args.prefill_step, args.repeat, bool(args.graph), bool(args.int8_lm_head),
                           rank, world, local, group, dec=dec, peer=peer)
    out["fuse_allreduce_norm"] = bool(dec.fuse_allreduce_norm)
    if rank == 0:
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        if peer is not None:
            peer.close()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
