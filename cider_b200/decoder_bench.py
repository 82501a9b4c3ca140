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
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = QWEN3_VL_2B if args.model == "qwen3vl2b" else QWEN3_8B
    vision = args.vision if args.vision >= 0 else (1024 if args.model == "qwen3vl2b" else 0)
    dec = Decoder(cfg, mode=args.mode, group_size=args.group_size, device=f"cuda:{local}",
                  max_len=args.prompt + args.decode + 8, batch=args.batch, tp_rank=rank, tp_size=world,
                  group=group, layers=args.layers, int8_lm_head=bool(args.int8_lm_head))
    emb, pos = build_prompt(dec, args.batch, args.prompt, vision)
    best = None
    for _ in range(args.repeat + 1):  # first run is the warm-up
        # CUDA-graph capture of steps that contain NCCL all-reduces is not used here: a
        # tensor-parallel run replays the eager launch sequence
        use_graph = bool(args.graph) and world == 1
        toks, stats = dec.generate(emb, pos, args.decode, args.prefill_step, use_graph=use_graph)
        if best is None or stats["generation_tps"] > best["generation_tps"]:
            prev = best
            best = stats
            if prev is not None:
                best["prompt_tps"] = max(best["prompt_tps"], prev["prompt_tps"])
    if rank == 0:
        out = {"model": args.model, "mode": args.mode, "group_size": args.group_size, "tp": world,
               "batch": args.batch, "prompt": args.prompt, "decode": args.decode,
               "layers": dec.n_layers, "graph": bool(args.graph) and world == 1,
               "int8_lm_head": bool(args.int8_lm_head),
               "prefill_tok_s": best["prompt_tps"], "decode_tok_s": best["generation_tps"],
               "ttft_ms": best["time_to_first_token_s"] * 1e3, "first_tokens": toks[0, :8].tolist()}
        print(json.dumps(out), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
