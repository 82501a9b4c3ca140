// Small fused kernels of the decoder step around the quantized linears: per-head
// q/k RMSNorm + rotary embedding + KV-cache append, and SwiGLU.  The reference has
// none of these (they are MLX library ops inside its mlx_vlm dependency; the only
// in-tree trace is cider/fused_hybrid.py:177-213); they exist here so that a
// decode step is a fixed sequence of kernels with no host-side indexing and can
// be replayed as a CUDA graph: positions and the cache length are read from
// device memory.
#include "common.cuh"

namespace cider {

// Status word of this file's kernels (a __device__ variable is private to its
// translation unit); merged into cider_device_status() by read_device_status().
__device__ unsigned int g_glue_status = 0;

namespace {

// A block of 8 warps per token (times a few head groups when there are few tokens); a
// HALF-warp per head, every lane owning 8 consecutive elements (one 16-byte load / store):
// lanes 0..7 of the half hold d = 8l .. 8l+7 (first half of the head), lanes 8..15 the
// elements d + 64, so the rotary partner of a lane is 8 lanes away (one shuffle).  D == 128.
//   q / k heads: y = half(x * rsqrt(mean(x^2) + eps) * w)   (rounded to fp16, as an
//                unfused norm would), then rotate-half rope in fp32 from the
//                rounded values: o[d] = y[d]*cos - y[d+64]*sin, o[d+64] = y[d+64]*cos + y[d]*sin
//   v heads:     copied.
// Slot i's angle (i = d mod 64) is pos[axis[i]] * inv_freq[i] (interleaved M-RoPE picks the
// axis per slot; text-only models pass the same position on all three axes); it depends on
// the token only: 64 threads compute the token's sines and cosines once into shared memory
// (sincosf with its range reduction is most of this kernel's arithmetic).
// q goes to q_out [B, nq, T, D]; k, v to the caches [B, nkv, Tcap, D] at position
// base + t, base = *base_dev when given (graph replay) else base_host.  A slot outside
// [0, Tcap) - possible only with a device-side base, e.g. one graph replay too many -
// is not written: the K / V stores are skipped and kStatusKvOverflow is recorded.
constexpr int kRopeWarps = 8;
constexpr int kRopeHeadsPerPass = 2 * kRopeWarps;
__global__ void __launch_bounds__(kRopeWarps * 32)
qk_norm_rope_append_kernel(const __half *__restrict__ qkv, const __half *__restrict__ q_norm_w,
                           const __half *__restrict__ k_norm_w, const float *__restrict__ inv_freq,
                           const int8_t *__restrict__ axis, const int *__restrict__ pos3, int pos_stride,
                           const int *__restrict__ base_dev, int base_host, float eps,
                           __half *__restrict__ q_out, __half *__restrict__ k_cache,
                           __half *__restrict__ v_cache, int T, int nq, int nkv, int Tcap) {
  constexpr int D = 128, H = 64;
  __shared__ float2 cs_s[H];  // (cos, sin) per frequency slot of this token
  pdl_launch_dependents();
  pdl_wait();
  const int token = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int b = token / T, t = token % T;
  const int base = base_dev ? *base_dev : base_host;
  const bool slot_ok = base >= 0 && (int64_t)base + t < (int64_t)Tcap;
  if (!slot_ok && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(&g_glue_status, kStatusKvOverflow);
  if (threadIdx.x < H) {
    const int i = threadIdx.x;
    const float ang = __fmul_rn((float)pos3[axis[i] * pos_stride + t], inv_freq[i]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    cs_s[i] = make_float2(cs, sn);
  }
  __syncthreads();
  const int hl = lane & 15;             // lane within the half-warp
  const int d0 = 8 * hl;                // first element of this lane, 0 .. 127
  const int heads = nq + 2 * nkv;
  // the two halves of a warp work on different heads and may take different branches:
  // every shuffle names only the 16 lanes of its own half
  const unsigned hmask = lane < 16 ? 0x0000ffffu : 0xffff0000u;
  for (int hp = blockIdx.y * kRopeWarps + warp; 2 * hp < heads; hp += gridDim.y * kRopeWarps) {
    const int hd = 2 * hp + (lane >> 4);
    if (hd >= heads) continue;  // odd number of heads: the last pair has one
    const __half *src = qkv + ((int64_t)token * heads + hd) * D + d0;
    const uint4 raw = *reinterpret_cast<const uint4 *>(src);
    if (hd >= nq + nkv) {  // v: copy into the cache
      if (slot_ok)
        *reinterpret_cast<uint4 *>(v_cache + (((int64_t)b * nkv + (hd - nq - nkv)) * Tcap + base + t) * D + d0) = raw;
      continue;
    }
    const uint4 outv = norm_rope_head128(raw, hd < nq ? q_norm_w : k_norm_w, cs_s, eps, hl, hmask);
    if (hd < nq)
      *reinterpret_cast<uint4 *>(q_out + (((int64_t)b * nq + hd) * T + t) * D + d0) = outv;
    else if (slot_ok)
      *reinterpret_cast<uint4 *>(k_cache + (((int64_t)b * nkv + (hd - nq)) * Tcap + base + t) * D + d0) = outv;
  }
}

// act[m, i] = half(half(silu(g)) * u), g = gu[m, i], u = gu[m, inter + i]; the two
// roundings are those of an fp16 silu followed by an fp16 multiply.
__global__ void __launch_bounds__(256)
silu_mul_kernel(const __half *__restrict__ gu, __half *__restrict__ act, int64_t M, int inter) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t pairs = M * (inter / 2);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pairs;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / (inter / 2);
    const int c = (int)(i % (inter / 2)) * 2;
    const __half2 g = *reinterpret_cast<const __half2 *>(gu + m * 2 * inter + c);
    const __half2 u = *reinterpret_cast<const __half2 *>(gu + m * 2 * inter + inter + c);
    const float2 gf = __half22float2(g), uf = __half22float2(u);
    const float s0 = silu_to_half(gf.x);
    const float s1 = silu_to_half(gf.y);
    *reinterpret_cast<__half2 *>(act + m * inter + c) = __floats2half2_rn(s0 * uf.x, s1 * uf.y);
  }
}

}  // namespace

int launch_qk_norm_rope_append(const __half *qkv, const __half *qw, const __half *kw, const float *inv_freq,
                               const int8_t *axis, const int *pos3, int pos_stride, const int *base_dev,
                               int base_host, float eps, __half *q_out, __half *k_cache, __half *v_cache,
                               int64_t B, int64_t T, int nq, int nkv, int64_t Tcap, cudaStream_t st) {
  if (B * T == 0) return CIDER_OK;
  // few tokens (decode): a block per (token, 8 heads) so that more SMs take part; a prompt: a
  // block per token
  const int64_t groups = (nq + 2 * nkv + kRopeHeadsPerPass - 1) / kRopeHeadsPerPass;
  dim3 grid((unsigned)(B * T), (unsigned)(B * T >= 4 * sm_count(current_device()) ? 1 : groups));
  return check_cuda(launch_kernel(qk_norm_rope_append_kernel, grid, dim3(kRopeWarps * 32), 0, st, qkv, qw, kw, inv_freq, axis,
                                  pos3, pos_stride, base_dev, base_host, eps, q_out, k_cache, v_cache, (int)T,
                                  nq, nkv, (int)Tcap),
                    "qk_norm_rope_append launch");
}

int read_glue_status(unsigned int *out) {
  return check_cuda(cudaMemcpyFromSymbol(out, g_glue_status, sizeof(unsigned int)), "read glue status");
}
int clear_glue_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_glue_status, &z, sizeof(z)), "clear glue status");
}

int launch_silu_mul(const __half *gu, __half *act, int64_t M, int64_t inter, cudaStream_t st) {
  if (M * inter == 0) return CIDER_OK;
  const int64_t pairs = M * inter / 2;
  int64_t blocks = (pairs + 255) / 256;
  const int64_t cap = (int64_t)sm_count(current_device()) * 16;
  if (blocks > cap) blocks = cap;
  return check_cuda(launch_kernel(silu_mul_kernel, dim3((unsigned)blocks), dim3(256), 0, st, gu, act, M, (int)inter),
                    "silu_mul launch");
}

}  // namespace cider
