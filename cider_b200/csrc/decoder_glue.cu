// Small fused kernels of the decoder step around the quantized linears: per-head
// q/k RMSNorm + rotary embedding + KV-cache append, and SwiGLU.  The reference has
// none of these (they are MLX library ops inside its mlx_vlm dependency; the only
// in-tree trace is cider/fused_hybrid.py:177-213); they exist here so that a
// decode step is a fixed sequence of kernels with no host-side indexing and can
// be replayed as a CUDA graph: positions and the cache length are read from
// device memory.
#include "common.cuh"

namespace cider {
namespace {

// One block per (token, head); 64 threads, thread d owns the rotary pair
// (d, d + D/2).  D == 128.
//   q / k heads: y = half(x * rsqrt(mean(x^2) + eps) * w)   (rounded to fp16, as an
//                unfused norm would), then rotate-half rope in fp32 from the
//                rounded values: o[d] = y[d]*cos - y[d+64]*sin, o[d+64] = y[d+64]*cos + y[d]*sin
//   v heads:     copied.
// Slot d's angle is pos[axis[d]] * inv_freq[d] (interleaved M-RoPE picks the axis
// per slot; text-only models pass the same position on all three axes).
// q goes to q_out [B, nq, T, D]; k, v to the caches [B, nkv, Tcap, D] at position
// base + t, base = *base_dev when given (graph replay) else base_host.
__global__ void __launch_bounds__(64)
qk_norm_rope_append_kernel(const __half *__restrict__ qkv, const __half *__restrict__ q_norm_w,
                           const __half *__restrict__ k_norm_w, const float *__restrict__ inv_freq,
                           const int8_t *__restrict__ axis, const int *__restrict__ pos3, int pos_stride,
                           const int *__restrict__ base_dev, int base_host, float eps,
                           __half *__restrict__ q_out, __half *__restrict__ k_cache,
                           __half *__restrict__ v_cache, int T, int nq, int nkv, int Tcap) {
  constexpr int D = 128, H = 64;
  __shared__ float red[2];
  pdl_launch_dependents();
  pdl_wait();
  const int token = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
  const int b = token / T, t = token % T;
  const __half *src = qkv + ((int64_t)token * (nq + 2 * nkv) + head) * D;
  const float x1 = __half2float(src[d]), x2 = __half2float(src[d + H]);
  const int base = base_dev ? *base_dev : base_host;
  if (head >= nq + nkv) {  // v: copy into the cache
    __half *dst = v_cache + (((int64_t)b * nkv + (head - nq - nkv)) * Tcap + base + t) * D;
    dst[d] = src[d];
    dst[d + H] = src[d + H];
    return;
  }
  float ss = fmaf(x1, x1, x2 * x2);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((d & 31) == 0) red[d >> 5] = ss;
  __syncthreads();
  ss = red[0] + red[1];
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  const __half *w = head < nq ? q_norm_w : k_norm_w;
  const float y1 = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(x1, r), __half2float(w[d]))));
  const float y2 = __half2float(__float2half_rn(__fmul_rn(__fmul_rn(x2, r), __half2float(w[d + H]))));
  const float ang = __fmul_rn((float)pos3[axis[d] * pos_stride + t], inv_freq[d]);
  float sn, cs;
  sincosf(ang, &sn, &cs);
  const float o1 = __fsub_rn(__fmul_rn(y1, cs), __fmul_rn(y2, sn));
  const float o2 = __fadd_rn(__fmul_rn(y2, cs), __fmul_rn(y1, sn));
  __half *dst;
  if (head < nq)
    dst = q_out + (((int64_t)b * nq + head) * T + t) * D;
  else
    dst = k_cache + (((int64_t)b * nkv + (head - nq)) * Tcap + base + t) * D;
  dst[d] = __float2half_rn(o1);
  dst[d + H] = __float2half_rn(o2);
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
    const float s0 = __half2float(__float2half_rn(gf.x / (1.0f + expf(-gf.x))));
    const float s1 = __half2float(__float2half_rn(gf.y / (1.0f + expf(-gf.y))));
    *reinterpret_cast<__half2 *>(act + m * inter + c) = __floats2half2_rn(s0 * uf.x, s1 * uf.y);
  }
}

}  // namespace

int launch_qk_norm_rope_append(const __half *qkv, const __half *qw, const __half *kw, const float *inv_freq,
                               const int8_t *axis, const int *pos3, int pos_stride, const int *base_dev,
                               int base_host, float eps, __half *q_out, __half *k_cache, __half *v_cache,
                               int64_t B, int64_t T, int nq, int nkv, int64_t Tcap, cudaStream_t st) {
  if (B * T == 0) return CIDER_OK;
  dim3 grid((unsigned)(B * T), (unsigned)(nq + 2 * nkv));
  return check_cuda(launch_kernel(qk_norm_rope_append_kernel, grid, dim3(64), 0, st, qkv, qw, kw, inv_freq, axis,
                                  pos3, pos_stride, base_dev, base_host, eps, q_out, k_cache, v_cache, (int)T,
                                  nq, nkv, (int)Tcap),
                    "qk_norm_rope_append launch");
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
