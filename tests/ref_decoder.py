"""Plain-torch reference of the quantized decoder (test infrastructure).

Same architecture and weights as cider_b200.decoder.Decoder, but every linear is
the reference's quantize -> int-matmul -> dequant semantics written with torch
ops in fp64/fp32 (no cider kernel), and the glue is the unfused torch path.  The
GPU decoder tests compare the kernel-backed decoder against it.
"""
import torch

from cider_b200.decoder import Decoder, _quantize_with_amax, _rmsnorm


class TorchQuantDecoder(Decoder):
    def forward(self, x, pos3):
        # route around the fused-kernel path: run the generic torch glue on a
        # CPU-flagged view of the call by temporarily hiding is_cuda
        return _torch_forward(self, x, pos3)

    def _linear(self, x, lw, name, row_parallel=False):
        if self.mode == "fp16":
            return torch.nn.functional.linear(x, lw.lin[name])
        wq, sw = lw.lin[name]
        M, K = x.shape
        wd = wq.double()
        if M == 1:  # matrix-vector path: activations are not quantised
            if self.gs == 0:
                y = (wd @ x[0].double()) * sw.double()
            else:
                G = K // self.gs
                part = (wd.view(-1, G, self.gs) * x[0].double().view(1, G, self.gs)).sum(-1)  # [N, G]
                y = (part * sw.double().t()).sum(-1)
            return y.to(torch.float16)[None, :]
        q, s = _quantize_with_amax(x, x.float().abs().amax(dim=1))
        if self.gs == 0:
            acc = (q.double() @ wd.t()).float()
            t = acc * s[:, None]
            return (t.double() * sw.double()[None, :]).float().to(torch.float16)
        G = K // self.gs
        accf = torch.zeros((M, wq.shape[0]), dtype=torch.float32, device=x.device)
        for g in range(G):
            sl = slice(g * self.gs, (g + 1) * self.gs)
            acc = q[:, sl].double() @ wd[:, sl].t()
            accf = (acc * sw[g].double()[None, :] + accf.double()).float()
        return (accf.double() * s.double()[:, None]).float().to(torch.float16)

    def _norm_linear(self, x, norm_w, lw, name):
        return self._linear(_rmsnorm(x, norm_w, self.cfg.rms_eps), lw, name)


def _torch_forward(self, x, pos3):
    import math
    import torch.nn.functional as F
    from cider_b200.decoder import _rotate_half, rope_cos_sin
    cfg, D = self.cfg, self.cfg.head_dim
    B, T, H = x.shape
    past = self.cur_len
    cos, sin = rope_cos_sin(cfg, pos3.to(self.device))
    cos, sin = cos[None, None], sin[None, None]
    x = x.reshape(B * T, H)
    scale = 1.0 / math.sqrt(D)
    for li, lw in enumerate(self.layers):
        qkv = self._norm_linear(x, lw.norm1, lw, "qkv").view(B, T, self.nq + 2 * self.nkv, D)
        q, k, v = qkv.split([self.nq, self.nkv, self.nkv], dim=2)
        q = _rmsnorm(q, lw.q_norm, cfg.rms_eps).transpose(1, 2).float()
        k = _rmsnorm(k, lw.k_norm, cfg.rms_eps).transpose(1, 2).float()
        q = (q * cos + _rotate_half(q) * sin).to(x.dtype)
        k = (k * cos + _rotate_half(k) * sin).to(x.dtype)
        self.kv[li, 0, :, :, past:past + T] = k
        self.kv[li, 1, :, :, past:past + T] = v.transpose(1, 2)
        kc, vc = self.kv[li, 0, :, :, :past + T], self.kv[li, 1, :, :, :past + T]
        mask = torch.ones(T, past + T, dtype=torch.bool, device=x.device).tril(diagonal=past)
        a = F.scaled_dot_product_attention(q.float(), kc.float(), vc.float(), attn_mask=mask, enable_gqa=True,
                                           scale=scale).to(x.dtype)
        attn = a.transpose(1, 2).reshape(B * T, self.nq * D)
        x = x + self._linear(attn, lw, "o", row_parallel=True)
        gu = self._norm_linear(x, lw.norm2, lw, "gate_up")
        act = F.silu(gu[:, :self.inter]) * gu[:, self.inter:]
        x = x + self._linear(act, lw, "down", row_parallel=True)
    self.cur_len = past + T
    return _rmsnorm(x, self.final_norm, cfg.rms_eps).view(B, T, H)
