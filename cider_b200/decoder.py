"""Qwen3 / Qwen3-VL text decoder driver around the quantized linears.

The reference does not contain the decoder itself: attention, RMSNorm, M-RoPE and
the KV cache live in its un-vendored ``mlx_vlm`` dependency (its only in-tree
restatement is the stale cider/fused_hybrid.py:142-213).  What the reference does
own, and what is mirrored here, is the generation driver of
vlm_service/custom_qwen3vl.py: M-RoPE position ids pre-computed for the whole
prompt (:143-295), chunked prefill (:576-656), the greedy decode loop (:660-679)
and the tok/s accounting (:798-803, :825).

Architecture (checked on CPU against ``transformers``' Qwen3VLTextModel in
tests/test_decoder_cpu.py): pre-norm decoder, GQA attention with per-head RMSNorm
on q and k, rotary embedding (interleaved M-RoPE for the VL model), SwiGLU MLP,
tied or untied fp16 lm_head.  All seven projections of a layer run either as fp16
``torch`` linears (the cuBLAS baseline) or as W8A8 linears (per-channel or
per-group) through ``cider_b200.ops``; q/k/v and gate/up are fused along N, which
is exact for per-output-channel scales.
"""
from __future__ import annotations

import math
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F


@dataclass
class DecoderConfig:
    hidden: int
    layers: int
    n_q: int
    n_kv: int
    head_dim: int
    inter: int
    vocab: int
    rms_eps: float = 1e-6
    rope_theta: float = 1e6
    mrope_section: Optional[Tuple[int, int, int]] = None  # interleaved M-RoPE when set
    tie_embeddings: bool = True

    @property
    def qkv_out(self) -> int:
        return (self.n_q + 2 * self.n_kv) * self.head_dim


# Qwen3-VL-2B text decoder and Qwen3-8B, by architecture only (random init)
QWEN3_VL_2B = DecoderConfig(hidden=2048, layers=28, n_q=16, n_kv=8, head_dim=128, inter=6144,
                            vocab=151936, rope_theta=5e6, mrope_section=(24, 20, 20), tie_embeddings=True)
QWEN3_8B = DecoderConfig(hidden=4096, layers=36, n_q=32, n_kv=8, head_dim=128, inter=12288,
                         vocab=151936, rope_theta=1e6, mrope_section=None, tie_embeddings=False)


# ------------------------------------------------------------------ positions
def mrope_position_ids(segments: Sequence[Tuple[str, object]]) -> torch.Tensor:
    """[3, T] (t, h, w) position ids for a prompt made of text runs and image grids,
    the index arithmetic of vlm_service/custom_qwen3vl.py:208-251: a text run of n
    tokens gets n consecutive ids on all three axes starting at (previous max + 1);
    an image of (t, h, w) merged patches gets ids (ti, hi, wi) + that same start.

    ``segments``: ("text", n) or ("image", (t, h, w)) in LLM-grid units."""
    out: List[torch.Tensor] = []
    nxt = 0
    for kind, val in segments:
        if kind == "text":
            n = int(val)
            if n == 0:
                continue
            ids = torch.arange(n, dtype=torch.int64).expand(3, n) + nxt
        elif kind == "image":
            t, h, w = (int(v) for v in val)
            ti = torch.arange(t).view(t, 1, 1).expand(t, h, w).reshape(-1)
            hi = torch.arange(h).view(1, h, 1).expand(t, h, w).reshape(-1)
            wi = torch.arange(w).view(1, 1, w).expand(t, h, w).reshape(-1)
            ids = torch.stack([ti, hi, wi]).to(torch.int64) + nxt
        else:
            raise ValueError(f"unknown segment kind {kind!r}")
        out.append(ids)
        nxt = int(ids.max()) + 1
    if not out:
        return torch.zeros((3, 0), dtype=torch.int64)
    return torch.cat(out, dim=1)


def rope_cos_sin(cfg: DecoderConfig, pos3: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """cos/sin [T, head_dim] (fp32) for position ids [3, T] (text-only models pass the
    same ids on all three rows).  Interleaved M-RoPE: frequency slot i takes the h
    axis when i % 3 == 1 and i < 3*section[1], the w axis when i % 3 == 2 and
    i < 3*section[2], else the t axis."""
    half = cfg.head_dim // 2
    inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float32, device=pos3.device) / half))
    freqs = pos3.to(torch.float32)[:, :, None] * inv[None, None, :]  # [3, T, half]
    f = freqs[0].clone()
    if cfg.mrope_section is not None:
        for dim, off in ((1, 1), (2, 2)):
            length = cfg.mrope_section[dim] * 3
            f[:, off:length:3] = freqs[dim][:, off:length:3]
    emb = torch.cat([f, f], dim=-1)
    return emb.cos(), emb.sin()


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def _rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """fp32 throughout, one rounding to the input dtype at the end."""
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


# -------------------------------------------------------------------- weights
def quantize_weight_int8_torch(w: torch.Tensor):
    """Device-side twin of ops.quantize_weight_int8 (same fp32 arithmetic, round
    half to even), used to quantise whole models without a host round trip."""
    wf = w.float()
    scale = wf.abs().amax(dim=1) / 127.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round(wf / scale[:, None]), -128, 127).to(torch.int8)
    return q, scale


def quantize_weight_pergroup_torch(w: torch.Tensor, gs: int, scale_dtype=torch.float16):
    """Per-group twin (cider/nn.py:34-59); returns (int8 [N,K], scales [K/gs, N]).
    With fp16 scales the scale is rounded first and the weights divided by the
    rounded value, so that what is stored is what was used."""
    n, k = w.shape
    wf = w.float().reshape(n, k // gs, gs)
    scale = wf.abs().amax(dim=2) / 127.0
    scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    if scale_dtype != torch.float32:
        scale = scale.to(scale_dtype)
        scale = torch.where(scale == 0, torch.ones_like(scale), scale)
    q = torch.clamp(torch.round(wf / scale.float()[:, :, None]), -128, 127).to(torch.int8).reshape(n, k)
    return q, scale.t().contiguous()


@dataclass
class LayerWeights:
    norm1: torch.Tensor
    norm2: torch.Tensor
    q_norm: torch.Tensor
    k_norm: torch.Tensor
    lin: dict = field(default_factory=dict)  # name -> fp16 weight, or (int8, scale)


LINEARS = ("qkv", "o", "gate_up", "down")


def _lin_shapes(cfg: DecoderConfig):
    return {"qkv": (cfg.qkv_out, cfg.hidden), "o": (cfg.hidden, cfg.n_q * cfg.head_dim),
            "gate_up": (2 * cfg.inter, cfg.hidden), "down": (cfg.hidden, cfg.inter)}


class Decoder:
    """Random-init decoder of a given architecture with a static fp16 KV cache.

    mode: "fp16" - torch linears (cuBLAS), the baseline; "w8a8" - cider_b200 ops.
    group_size: 0 per-channel, 64/128/256 per-group (w8a8 only).
    Tensor parallelism (``tp_size`` > 1, one process per GPU): q/k/v and gate/up
    are column-parallel (heads / intermediate channels split), o_proj and
    down_proj row-parallel followed by an all-reduce over ``group`` (NCCL for the large
    prefill messages; with ``peer`` - a cider_b200.peer.PeerGroup - the small decode-step
    messages go through the library's one-shot peer-memory kernel, and the decode step
    replays as a CUDA graph); the KV cache and attention shard by head with no communication.  Per-token activation
    scales of the row-parallel linears are computed on the local K shard
    (``tp_exact_scales=False``) or from an all-reduced row absmax, which makes the
    int8 activations identical to the single-GPU ones (``True``).
    """

    def __init__(self, cfg: DecoderConfig, mode: str = "w8a8", group_size: int = 0, device="cuda",
                 dtype=torch.float16, seed: int = 0, max_len: int = 4096, batch: int = 1,
                 tp_rank: int = 0, tp_size: int = 1, group=None, tp_exact_scales: bool = False,
                 scale_dtype=torch.float16, layers: Optional[int] = None, int8_lm_head: bool = False,
                 peer=None):
        assert mode in ("fp16", "w8a8")
        assert cfg.n_kv % tp_size == 0 and cfg.inter % tp_size == 0
        self.cfg, self.mode, self.gs = cfg, mode, int(group_size)
        self.device, self.dtype = torch.device(device), dtype
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        self.tp_exact = tp_exact_scales
        # cider_b200.peer.PeerGroup: all-reduces of messages that fit its inbox run as this
        # library's one-shot peer-memory kernel (graph-capturable) instead of NCCL
        self.peer = peer
        # with a peer group: run the all-reduce of a row-parallel linear, the residual add and the
        # following RMSNorm (+ quantiser) as ONE kernel where the shape allows (decode-sized M)
        self.fuse_allreduce_norm = True
        # decode step: q/k norm + rope + KV append folded into the attention kernel (one launch
        # less per layer)
        self.fuse_rope_sdpa = True
        self.n_layers = cfg.layers if layers is None else layers
        self.nq, self.nkv = cfg.n_q // tp_size, cfg.n_kv // tp_size
        self.inter = cfg.inter // tp_size
        self.max_len, self.batch = max_len, batch
        # per-channel W8A8 on the GPU: prefill chunks run the gate/up projection with the SwiGLU in
        # the GEMM's epilogue (half the output bytes, and the quantiser behind it needs no reduction)
        self.fuse_swiglu = (mode == "w8a8" and self.gs == 0 and self.device.type == "cuda"
                            and not tp_exact_scales and self.inter % 32 == 0)
        self._rowmax = (torch.zeros(batch * max_len, dtype=torch.float32, device=self.device)
                        if self.fuse_swiglu else None)
        self.layers: List[LayerWeights] = []
        D = cfg.head_dim
        for li in range(self.n_layers):
            g = torch.Generator(device=self.device).manual_seed(seed * 1000 + li)

            def rnd(n, k):
                return (torch.randn(n, k, generator=g, device=self.device, dtype=torch.float32) * 0.02).to(dtype)

            full = {name: rnd(*shape) for name, shape in _lin_shapes(cfg).items()}
            ones = torch.ones(cfg.hidden, device=self.device, dtype=dtype)
            lw = LayerWeights(ones, ones.clone(), torch.ones(D, device=self.device, dtype=dtype),
                              torch.ones(D, device=self.device, dtype=dtype))
            for name, w in full.items():
                w = self._shard(name, w)
                if mode == "fp16":
                    lw.lin[name] = w
                elif self.gs == 0:
                    lw.lin[name] = quantize_weight_int8_torch(w)
                else:
                    lw.lin[name] = quantize_weight_pergroup_torch(w, self.gs, scale_dtype)
            if self.fuse_swiglu:
                # a second copy of the fused gate/up weights with the rows interleaved in blocks of 32:
                # what the GEMM with the SwiGLU in its epilogue takes (prefill chunks; the decode
                # kernels keep the [gate ; up] copy)
                from . import ops
                wq, sw = lw.lin["gate_up"]
                wi, swi, _ = ops.interleave_gate_up(wq, sw)
                lw.lin["gate_up_il"] = (wi, swi)
            self.layers.append(lw)
        g = torch.Generator(device=self.device).manual_seed(seed * 1000 + 999)
        self.embed = (torch.randn(cfg.vocab, cfg.hidden, generator=g, device=self.device,
                                  dtype=torch.float32) * 0.02).to(dtype)
        if cfg.tie_embeddings:
            self.lm_head = self.embed
        else:
            self.lm_head = (torch.randn(cfg.vocab, cfg.hidden, generator=g, device=self.device,
                                        dtype=torch.float32) * 0.02).to(dtype)
        # The reference's convert_model leaves the (tied) output head in fp16: it is not an
        # nn.Linear of the model.  Optionally quantise it too (per-channel W8A8): at batch
        # 1 the 151936 x hidden head is ~10 % of a decode step's bytes.
        self.lm_head_q = None
        if int8_lm_head and mode == "w8a8" and self.device.type == "cuda":
            self.lm_head_q = quantize_weight_int8_torch(self.lm_head)
        self.final_norm = torch.ones(cfg.hidden, device=self.device, dtype=dtype)
        self.kv = torch.zeros((self.n_layers, 2, batch, self.nkv, max_len, D), device=self.device, dtype=dtype)
        self.cur_len = 0
        self.next_pos = 0  # next rotary position (max position id so far + 1)
        self._graph = None
        self.use_pdl = True  # programmatic dependent launch inside the captured decode step
        if self.device.type == "cuda":
            half = D // 2
            self.inv_freq = (1.0 / (cfg.rope_theta ** (torch.arange(0, half, dtype=torch.float32) / half))).to(self.device)
            axis = torch.zeros(half, dtype=torch.int8)
            if cfg.mrope_section is not None:
                for dim, off in ((1, 1), (2, 2)):
                    axis[off:cfg.mrope_section[dim] * 3:3] = dim
            self.axis = axis.to(self.device)
            # [cache length before the step, after it]; the three position ids of the
            # next token; tokens generated so far; all advanced on the device
            # ticket counters of the one-launch decode attention (zero between calls).  Measured:
            # one launch wins at batch 8 (+4 % tok/s), the partial + combine pair at batch 1
            # (the last block's serial merge is a longer tail than a parallel combine kernel)
            self.sdpa_tickets = (torch.zeros(batch * self.nkv, dtype=torch.int32, device=self.device)
                                 if batch >= 4 else None)
            self.len_dev = torch.zeros(2, dtype=torch.int32, device=self.device)
            self.pos_dev = torch.zeros((3, 1), dtype=torch.int32, device=self.device)

    # ---- sharding -----------------------------------------------------------
    def _shard(self, name: str, w: torch.Tensor) -> torch.Tensor:
        if self.tp_size == 1:
            return w
        cfg, r, D = self.cfg, self.tp_rank, self.cfg.head_dim
        if name == "qkv":
            q, k, v = w.split([cfg.n_q * D, cfg.n_kv * D, cfg.n_kv * D], dim=0)
            return torch.cat([q[r * self.nq * D:(r + 1) * self.nq * D], k[r * self.nkv * D:(r + 1) * self.nkv * D],
                              v[r * self.nkv * D:(r + 1) * self.nkv * D]], dim=0).contiguous()
        if name == "gate_up":
            gate, up = w.split([cfg.inter, cfg.inter], dim=0)
            s = slice(r * self.inter, (r + 1) * self.inter)
            return torch.cat([gate[s], up[s]], dim=0).contiguous()
        if name == "o":
            return w[:, r * self.nq * D:(r + 1) * self.nq * D].contiguous()
        if name == "down":
            return w[:, r * self.inter:(r + 1) * self.inter].contiguous()
        raise KeyError(name)

    def _all_reduce(self, y: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            if self.peer is not None and self.peer.fits(y):
                return self.peer.all_reduce(y)
            if y.is_cuda and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("tensor-parallel step under CUDA-graph capture needs a PeerGroup whose inbox "
                                   "holds the message: a library collective is not captured")
            import torch.distributed as dist
            dist.all_reduce(y, group=self.group)
        return y

    def _reduce_add_norm(self, x: torch.Tensor, part: Optional[torch.Tensor], norm_w: torch.Tensor,
                         want_fp16: bool, want_int8: bool):
        """``x += all_reduce(part)`` (part: this rank's partial output of a row-parallel linear, or
        None) followed by the RMSNorm of x: (y fp16 | None, q int8 | None, scale | None).  With a
        peer group and a decode-sized message the exchange, the add and the norm are one kernel."""
        from . import ops
        if (part is not None and self.tp_size > 1 and self.fuse_allreduce_norm and self.peer is not None
                and self.peer.fits_norm(part)):
            return self.peer.all_reduce_add_rmsnorm(part, x, norm_w, self.cfg.rms_eps, want_fp16, want_int8)
        delta = None if part is None else self._all_reduce(part)
        return ops.add_rmsnorm(x, delta, norm_w, self.cfg.rms_eps, want_fp16=want_fp16, want_int8=want_int8)

    # ---- linears ------------------------------------------------------------
    def _linear(self, x: torch.Tensor, lw: LayerWeights, name: str, row_parallel: bool = False) -> torch.Tensor:
        """x [M, K] -> [M, N].  M == 1 takes the unquantised matrix-vector path."""
        if self.mode == "fp16":
            return F.linear(x, lw.lin[name])
        from . import ops
        wq, sw = lw.lin[name]
        M = x.shape[0]
        if row_parallel and self.tp_exact and self.tp_size > 1 and M > 1:
            import torch.distributed as dist
            # the quantiser in two halves: slice absmax, max over the ranks, quantise with
            # the full row's scale (kernels; the int8 activations equal the single-GPU ones)
            amax = ops.row_absmax(x)
            dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=self.group)
            q, s = ops.quantize_given_amax(x, amax)
            return ops.linear_prequantized(q, s, wq, sw, self.gs)
        if self.gs == 0:
            return ops.perchannel_linear(x, wq, sw)
        return ops.pergroup_linear(x, wq, sw, self.gs)

    def _norm_linear(self, x: torch.Tensor, norm_w: torch.Tensor, lw: LayerWeights, name: str) -> torch.Tensor:
        """RMSNorm followed by a linear; in w8a8 mode with M > 1 the norm and the
        per-token quantiser are one kernel and the GEMM reads int8 directly."""
        M = x.shape[0]
        if self.mode == "w8a8" and M > 1:
            from . import ops
            wq, sw = lw.lin[name]
            _, q, s = ops.rmsnorm_quant(x, norm_w, self.cfg.rms_eps, want_fp16=False)
            return ops.linear_prequantized(q, s, wq, sw, self.gs)
        return self._linear(_rmsnorm(x, norm_w, self.cfg.rms_eps), lw, name)

    # ---- forward ------------------------------------------------------------
    def reset(self):
        self.cur_len = 0
        self.next_pos = 0

    def forward(self, x: torch.Tensor, pos3: torch.Tensor) -> torch.Tensor:
        """x [B, T, hidden] embeddings of T new positions (appended to the cache),
        pos3 [3, T] their rotary position ids.  Returns hidden states [B, T, hidden]
        after the final norm."""
        if x.is_cuda:
            return self._forward_cuda(x, pos3)
        cfg, D = self.cfg, self.cfg.head_dim
        B, T, H = x.shape
        past = self.cur_len
        assert past + T <= self.max_len and B == self.batch
        cos, sin = rope_cos_sin(cfg, pos3.to(self.device))
        cos, sin = cos.to(x.dtype)[None, None], sin.to(x.dtype)[None, None]  # [1,1,T,D]
        x = x.reshape(B * T, H)
        scale = 1.0 / math.sqrt(D)
        for li, lw in enumerate(self.layers):
            qkv = self._norm_linear(x, lw.norm1, lw, "qkv").view(B, T, self.nq + 2 * self.nkv, D)
            q, k, v = qkv.split([self.nq, self.nkv, self.nkv], dim=2)
            q = _rmsnorm(q, lw.q_norm, cfg.rms_eps).transpose(1, 2)  # [B, nq, T, D]
            k = _rmsnorm(k, lw.k_norm, cfg.rms_eps).transpose(1, 2)
            q = q * cos + _rotate_half(q) * sin
            k = k * cos + _rotate_half(k) * sin
            self.kv[li, 0, :, :, past:past + T] = k
            self.kv[li, 1, :, :, past:past + T] = v.transpose(1, 2)
            if T == 1 and x.is_cuda:
                from . import ops
                attn = ops.sdpa_decode(q.reshape(B, self.nq, D).contiguous(), self.kv[li, 0], self.kv[li, 1],
                                       past + 1, scale).reshape(B, self.nq * D)
            else:
                kc, vc = self.kv[li, 0, :, :, :past + T], self.kv[li, 1, :, :, :past + T]
                if past == 0:
                    a = F.scaled_dot_product_attention(q, kc, vc, is_causal=True, enable_gqa=True, scale=scale)
                else:
                    mask = torch.ones(T, past + T, dtype=torch.bool, device=x.device).tril(diagonal=past)
                    a = F.scaled_dot_product_attention(q, kc, vc, attn_mask=mask, enable_gqa=True, scale=scale)
                attn = a.transpose(1, 2).reshape(B * T, self.nq * D)
            x = x + self._all_reduce(self._linear(attn, lw, "o", row_parallel=True))
            gu = self._norm_linear(x, lw.norm2, lw, "gate_up")
            act = F.silu(gu[:, :self.inter]) * gu[:, self.inter:]
            x = x + self._all_reduce(self._linear(act, lw, "down", row_parallel=True))
        self.cur_len = past + T
        return _rmsnorm(x, self.final_norm, cfg.rms_eps).view(B, T, H)

    def _forward_cuda(self, x: torch.Tensor, pos3: Optional[torch.Tensor], on_device_state: bool = False):
        """Same computation with the fused glue kernels (residual-add + RMSNorm
        (+ quantiser), q/k norm + rope + KV append, SwiGLU, split-K decode
        attention).  With ``on_device_state`` the cache offset, attended length and
        positions are read from device memory (self.len_dev / self.pos_dev), so the
        launch sequence is identical for every decode step (CUDA-graph replay)."""
        from . import ops
        cfg, D = self.cfg, self.cfg.head_dim
        B, T, H = x.shape
        past = self.cur_len
        assert B == self.batch and (on_device_state or past + T <= self.max_len)
        if on_device_state:
            pos_i32, base, base_dev, len_dev, att_len = self.pos_dev, 0, self.len_dev[0:1], self.len_dev[1:2], self.max_len
        else:
            pos_i32 = pos3.to(device=self.device, dtype=torch.int32).contiguous()
            base, base_dev, len_dev, att_len = past, None, None, past + T
        M = B * T
        if M == 1 and self.mode == "w8a8":
            return self._forward_cuda_m1(x, pos_i32, base, base_dev, len_dev, att_len, past, on_device_state)
        x = x.reshape(M, H).clone()  # residual stream, updated in place
        quant = self.mode == "w8a8" and M > 1
        scale = 1.0 / math.sqrt(D)
        delta = None
        q_out = torch.empty((B, self.nq, T, D), dtype=x.dtype, device=x.device)
        for li, lw in enumerate(self.layers):
            y, q8, s8 = self._reduce_add_norm(x, delta, lw.norm1, not quant, quant)
            if quant:
                qkv = ops.linear_prequantized(q8, s8, lw.lin["qkv"][0], lw.lin["qkv"][1], self.gs)
            else:
                qkv = self._linear(y, lw, "qkv")
            fused_attn = T == 1 and self.fuse_rope_sdpa and D == 128
            if not fused_attn:
                ops.qk_norm_rope_append(qkv, lw.q_norm, lw.k_norm, self.inv_freq, self.axis, pos_i32, base,
                                        cfg.rms_eps, q_out, self.kv[li, 0], self.kv[li, 1], B, T, self.nq, self.nkv,
                                        base_dev=base_dev)
            if fused_attn:
                attn = ops.sdpa_decode_fused(qkv, lw.q_norm, lw.k_norm, self.inv_freq, self.axis, pos_i32,
                                             cfg.rms_eps, self.kv[li, 0], self.kv[li, 1], att_len, scale, self.nq,
                                             self.nkv, length_dev=len_dev,
                                             tickets=self.sdpa_tickets).view(B, self.nq * D)
            elif T == 1:
                attn = ops.sdpa_decode(q_out.view(B, self.nq, D), self.kv[li, 0], self.kv[li, 1], att_len, scale,
                                       length_dev=len_dev, tickets=self.sdpa_tickets).view(B, self.nq * D)
            else:
                kc, vc = self.kv[li, 0, :, :, :past + T], self.kv[li, 1, :, :, :past + T]
                if past == 0:
                    a = F.scaled_dot_product_attention(q_out, kc, vc, is_causal=True, enable_gqa=True, scale=scale)
                else:
                    mask = torch.ones(T, past + T, dtype=torch.bool, device=x.device).tril(diagonal=past)
                    a = F.scaled_dot_product_attention(q_out, kc, vc, attn_mask=mask, enable_gqa=True, scale=scale)
                if quant and not (self.tp_exact and self.tp_size > 1):
                    # quantise the attention output where it lies ([B, heads, T, D]) - no
                    # transpose copy in front of the output projection
                    a8, as8 = ops.quantize_heads(a)
                    attn = None
                else:
                    attn = a.transpose(1, 2).reshape(M, self.nq * D)
            if attn is None:
                o_part = ops.linear_prequantized(a8, as8, lw.lin["o"][0], lw.lin["o"][1], self.gs)
            else:
                o_part = self._linear(attn, lw, "o", row_parallel=True)
            y, q8, s8 = self._reduce_add_norm(x, o_part, lw.norm2, not quant, quant)
            if quant and self.fuse_swiglu and M >= 128:
                # SwiGLU in the epilogue of the gate/up GEMM; its row maxima make the down
                # projection's quantiser a plain elementwise pass
                wi, swi = lw.lin["gate_up_il"]
                act, rowmax = ops.swiglu_linear_prequantized(q8, s8, wi, swi, rowmax=self._rowmax[:M])
                a8, as8 = ops.quantize_consume_amax(act, rowmax)
                delta = ops.linear_prequantized(a8, as8, lw.lin["down"][0], lw.lin["down"][1], self.gs)
                continue
            if quant:
                gu = ops.linear_prequantized(q8, s8, lw.lin["gate_up"][0], lw.lin["gate_up"][1], self.gs)
            else:
                gu = self._linear(y, lw, "gate_up")
            if quant and not (self.tp_exact and self.tp_size > 1):
                # SwiGLU and the down projection's quantiser in one pass (the activation
                # is never written as fp16)
                a8, as8 = ops.silu_mul_quant(gu)
                down = ops.linear_prequantized(a8, as8, lw.lin["down"][0], lw.lin["down"][1], self.gs)
            else:
                down = self._linear(ops.silu_mul(gu), lw, "down", row_parallel=True)
            delta = down  # this rank's partial sum; reduced together with the next norm
        h, _, _ = self._reduce_add_norm(x, delta, self.final_norm, True, False)
        if not on_device_state:
            self.cur_len = past + T
        return h.view(B, T, H)

    def _forward_cuda_m1(self, x, pos_i32, base, base_dev, len_dev, att_len, past, on_device_state):
        """Batch-1 decode step, W8A8: six kernels per layer.  The residual add +
        RMSNorm in front of the q/k/v and gate/up projections and the SwiGLU in front
        of the down projection are folded into the matrix-vector kernels' activation
        load (ops.linear_m1_fused); the residual stream ping-pongs between two
        buffers because the fused kernel may not update it in place."""
        from . import ops
        cfg, D = self.cfg, self.cfg.head_dim
        H = x.shape[-1]
        xa = x.reshape(1, H).clone()
        xb = torch.empty_like(xa)
        scale = 1.0 / math.sqrt(D)
        delta = None
        q_out = torch.empty((1, self.nq, 1, D), dtype=x.dtype, device=x.device)
        for li, lw in enumerate(self.layers):
            wq, sw = lw.lin["qkv"]
            qkv = ops.linear_m1_fused(xa, wq, sw, self.gs, prologue="add_norm", delta=delta,
                                      norm_weight=lw.norm1, eps=cfg.rms_eps, x_out=xb)
            xa, xb = xb, xa
            if self.fuse_rope_sdpa and D == 128:
                attn = ops.sdpa_decode_fused(qkv, lw.q_norm, lw.k_norm, self.inv_freq, self.axis, pos_i32,
                                             cfg.rms_eps, self.kv[li, 0], self.kv[li, 1], att_len, scale, self.nq,
                                             self.nkv, length_dev=len_dev,
                                             tickets=self.sdpa_tickets).view(1, self.nq * D)
            else:
                ops.qk_norm_rope_append(qkv, lw.q_norm, lw.k_norm, self.inv_freq, self.axis, pos_i32, base,
                                        cfg.rms_eps, q_out, self.kv[li, 0], self.kv[li, 1], 1, 1, self.nq, self.nkv,
                                        base_dev=base_dev)
                attn = ops.sdpa_decode(q_out.view(1, self.nq, D), self.kv[li, 0], self.kv[li, 1], att_len, scale,
                                       length_dev=len_dev, tickets=self.sdpa_tickets).view(1, self.nq * D)
            wq, sw = lw.lin["o"]
            o = self._all_reduce(ops.linear_m1_fused(attn, wq, sw, self.gs))
            wq, sw = lw.lin["gate_up"]
            gu = ops.linear_m1_fused(xa, wq, sw, self.gs, prologue="add_norm", delta=o, norm_weight=lw.norm2,
                                     eps=cfg.rms_eps, x_out=xb)
            xa, xb = xb, xa
            wq, sw = lw.lin["down"]
            delta = self._all_reduce(ops.linear_m1_fused(gu, wq, sw, self.gs, prologue="silu_mul"))
        h, _, _ = ops.add_rmsnorm(xa, delta, self.final_norm, cfg.rms_eps)
        if not on_device_state:
            self.cur_len = past + 1
        return h.view(1, 1, H)

    # ---- CUDA-graph decode loop ---------------------------------------------
    def _graph_step(self):
        """One decode step entirely on the device: embed the current token, run the
        layers, greedy-pick the next token, store it, advance length and positions."""
        x = self.embed[self._tok][:, None, :]
        h = self._forward_cuda(x, None, on_device_state=True)
        nxt = self.logits(h[:, -1]).argmax(dim=-1)
        self._tok.copy_(nxt)
        self._out.index_copy_(1, self._step, nxt[:, None])
        self._step += 1
        self.len_dev += 1
        self.pos_dev += 1

    def _sync_device_state(self, first_tok: torch.Tensor):
        self.len_dev.copy_(torch.tensor([self.cur_len, self.cur_len + 1], dtype=torch.int32))
        self.pos_dev.fill_(self.next_pos)
        self._tok.copy_(first_tok)
        self._step.zero_()

    def decode_graph(self, first_tok: torch.Tensor, n: int) -> torch.Tensor:
        """Greedy-decode ``n`` tokens after ``first_tok`` by replaying one captured
        decode step.  Returns [B, n]."""
        B = self.batch
        if self._graph is None:
            self._tok = torch.zeros(B, dtype=torch.int64, device=self.device)
            self._out = torch.zeros((B, self.max_len), dtype=torch.int64, device=self.device)
            self._step = torch.zeros(1, dtype=torch.int64, device=self.device)
            self._sync_device_state(first_tok)
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):  # warm-up outside capture (lazy inits, allocator)
                for _ in range(2):
                    self._graph_step()
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            from . import _lib
            self._graph = torch.cuda.CUDAGraph()
            lib = _lib.load()
            # the step's own kernels overlap their launch with the predecessor's tail
            lib.cider_set_programmatic_launch(1 if self.use_pdl else 0)
            try:
                with torch.cuda.graph(self._graph):
                    self._graph_step()
            finally:
                lib.cider_set_programmatic_launch(0)
        assert self.cur_len + n <= self.max_len
        self._sync_device_state(first_tok)
        if self.tp_size > 1:
            # the replayed step's peer all-reduce waits for the other ranks on the device with
            # a bounded wait: line the hosts up first (one rank may still have been capturing)
            import torch.distributed as dist
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)
        for _ in range(n):
            self._graph.replay()
        self.cur_len += n
        self.next_pos += n
        return self._out[:, :n].clone()

    def logits(self, h_last: torch.Tensor) -> torch.Tensor:
        """h_last [B, hidden] -> [B, vocab] (fp16 lm_head unless int8_lm_head, fp32 out)."""
        if self.lm_head_q is not None:
            from . import ops
            return ops.perchannel_linear(h_last.contiguous(), self.lm_head_q[0], self.lm_head_q[1]).float()
        return F.linear(h_last, self.lm_head).float()

    # ---- generation driver (vlm_service/custom_qwen3vl.py:576-679) -------------
    @torch.no_grad()
    def prefill(self, embeds: torch.Tensor, pos3: torch.Tensor, prefill_step_size: int = 8192,
                use_graph: bool = False) -> torch.Tensor:
        """Chunked prefill: position ids are computed for the whole prompt up front
        and sliced per chunk, so image spans may straddle chunks.  Returns the
        logits of the last prompt position, [B, vocab].  With ``use_graph`` (CUDA)
        each distinct (chunk length, cache offset) is captured once as a CUDA graph
        and replayed afterwards, which removes the per-kernel host overhead."""
        T = embeds.shape[1]
        h = None
        for st in range(0, T, prefill_step_size):
            ed = min(T, st + prefill_step_size)
            # a tensor-parallel prefill reduces its 100 MB-class partial sums with NCCL, launched
            # eagerly (a library collective is not captured into this library's graphs)
            if use_graph and embeds.is_cuda and self.tp_size == 1:
                h = self._forward_graph(embeds[:, st:ed], pos3[:, st:ed])
            else:
                h = self.forward(embeds[:, st:ed], pos3[:, st:ed])
        self.next_pos = int(pos3.max()) + 1 if T else 0
        return self.logits(h[:, -1])

    def _forward_graph(self, x: torch.Tensor, pos3: torch.Tensor) -> torch.Tensor:
        if not hasattr(self, "_fwd_graphs"):
            self._fwd_graphs = {}
        key = (x.shape[1], self.cur_len)
        past = self.cur_len
        ent = self._fwd_graphs.get(key)
        if ent is None:
            sx = x.clone()
            sp = pos3.to(device=self.device, dtype=torch.int32).contiguous()
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.forward(sx, sp)  # warm-up outside capture
            torch.cuda.current_stream(self.device).wait_stream(side)
            torch.cuda.synchronize(self.device)
            self.cur_len = past
            g = torch.cuda.CUDAGraph()
            from . import _lib
            lib = _lib.load()
            # this library's kernels overlap their launch and set-up with the predecessor's tail
            lib.cider_set_programmatic_launch(1 if self.use_pdl else 0)
            try:
                with torch.cuda.graph(g):
                    out = self.forward(sx, sp)
            finally:
                lib.cider_set_programmatic_launch(0)
            ent = (g, sx, sp, out)
            self._fwd_graphs[key] = ent
        g, sx, sp, out = ent
        sx.copy_(x)
        sp.copy_(pos3.to(device=self.device, dtype=torch.int32))
        self.cur_len = past
        g.replay()
        self.cur_len = past + x.shape[1]
        return out

    @torch.no_grad()
    def decode_step(self, tokens: torch.Tensor) -> torch.Tensor:
        """tokens [B] -> logits [B, vocab] for the next position."""
        x = self.embed[tokens][:, None, :]
        pos3 = torch.full((3, 1), self.next_pos, dtype=torch.int64)
        h = self.forward(x, pos3)
        self.next_pos += 1
        return self.logits(h[:, -1])

    @torch.no_grad()
    def generate(self, embeds: torch.Tensor, pos3: torch.Tensor, max_tokens: int,
                 prefill_step_size: int = 8192, use_graph: bool = False):
        """Greedy generation (argmax, ties -> lowest id).  Returns (tokens [B, n],
        stats) with the reference's definitions: prompt_tps = prompt tokens / time to
        the first token, generation_tps = generated tokens / time after it."""
        sync = torch.cuda.synchronize if embeds.is_cuda else (lambda: None)
        self.reset()
        sync()
        t0 = time.perf_counter()
        logits = self.prefill(embeds, pos3, prefill_step_size, use_graph=use_graph)
        tok = logits.argmax(dim=-1)
        sync()
        t1 = time.perf_counter()
        out = [tok]
        if use_graph and embeds.is_cuda and max_tokens > 1:
            rest = self.decode_graph(tok, max_tokens - 1)
            out.extend(rest.unbind(dim=1))
        else:
            for _ in range(max_tokens - 1):
                tok = self.decode_step(tok).argmax(dim=-1)
                out.append(tok)
        sync()
        t2 = time.perf_counter()
        n_prompt = embeds.shape[0] * embeds.shape[1]
        n_gen = embeds.shape[0] * (len(out) - 1)
        stats = {"prompt_tokens": n_prompt, "prompt_tps": n_prompt / (t1 - t0),
                 "generation_tokens": n_gen, "generation_tps": n_gen / max(t2 - t1, 1e-9),
                 "time_to_first_token_s": t1 - t0}
        return torch.stack(out, dim=1), stats


def _quantize_with_amax(x: torch.Tensor, amax: torch.Tensor):
    """Per-token int8 quantisation with a given row absmax (fp32), the same
    arithmetic as the quantiser kernel: s = amax/127 (0 -> 1), q = round-half-away
    (x * (1/s)).  Plain torch: the checker of ops.quantize_given_amax and the CPU
    stand-in of the quantiser in the tests; no product path calls it."""
    # tensor / tensor: a division by a Python scalar may be evaluated on the GPU as a
    # multiplication by its reciprocal, which is not the IEEE quotient the kernels compute
    s = amax / torch.full_like(amax, 127.0)
    s = torch.where(s == 0, torch.ones_like(s), s)
    v = x.float() * (torch.ones_like(s) / s)[:, None]
    a = v.abs()
    fl = a.floor()
    r = torch.sign(v) * (fl + ((a - fl) >= 0.5).float())
    return torch.clamp(r, -128, 127).to(torch.int8), s
