// Per-token activation quantiser (fp16 -> int8 + fp32 row scale), optionally
// fused behind an RMSNorm.  Semantics of cider/kernels/w8a8_quantize.metal:17-87:
//   amax = max_k |x|;  s = amax/127 (0 -> 1);  inv = 1/s;
//   q = int8(clamp(round_half_away(float(x)*inv), -128, 127))
//
// HBM-bound: each row is read once (kept in registers between the absmax pass
// and the quantise pass) with 128-bit loads, and written with 128-bit stores.
// A row is owned by TPR threads (32..256, a power of two) so that K up to
// 16*8*256 = 32768 stays in registers; other shapes take the scalar kernel.
#include "common.cuh"

namespace cider {
namespace {

constexpr int kBlock = 256;
constexpr int kMaxChunks = 8;  // most 16-half chunks cached per thread (template NC <= this)

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Reduce over the TPR threads that own one row.  `red` has one float per warp
// of the block; rows never share a warp when TPR >= 32.
template <int TPR, bool kMax>
__device__ __forceinline__ float row_reduce(float v, float *red, int tid) {
  v = kMax ? warp_max(v) : warp_sum(v);
  if constexpr (TPR > 32) {
    constexpr int kWarpsPerRow = TPR / 32;
    const int warp = tid >> 5;
    __syncthreads();  // protect `red` from the previous use
    if ((tid & 31) == 0) red[warp] = v;
    __syncthreads();
    const int first = (warp / kWarpsPerRow) * kWarpsPerRow;
    float r = red[first];
#pragma unroll
    for (int i = 1; i < kWarpsPerRow; ++i) r = kMax ? fmaxf(r, red[first + i]) : r + red[first + i];
    v = r;
  }
  return v;
}

// Vector kernel.  Requirements (checked by the launcher): K % 16 == 0,
// ldx % 8 == 0, x / q / y 16-byte aligned, K/16 <= TPR*kMaxChunks.
// kNorm: apply RMSNorm with weight w first; the normalised value is rounded to
// fp16 before it is quantised (and optionally stored to y).
template <int TPR, int NC, bool kNorm>
__global__ void __launch_bounds__(kBlock, NC <= 2 ? 4 : (NC <= 4 ? 2 : (NC <= 6 && !kNorm ? 3 : 1)))
quantize_rows_kernel(const __half *x, int64_t ldx, const __half *__restrict__ w,
                     float eps, __half *__restrict__ y, int8_t *__restrict__ q,
                     float *__restrict__ scale, int M, int K, const __half *__restrict__ delta,
                     __half *x_out,  // x_out may alias x (in-place residual update)
                     int gT, int gD,   // gT > 0: x is [B, K/gD, gT, gD] and row (b, t) gathers its heads
                     int perm8) {      // every 8 values stored as k0 k2 k4 k6 k1 k3 k5 k7 (W4A8 tensor-core path)
  __shared__ float red[kBlock / 32];
  constexpr int kRows = kBlock / TPR;
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int t = tid % TPR;
  int row = blockIdx.x * kRows + tid / TPR;
  const bool live = row < M;
  if (!live) row = M - 1;  // keep every thread in the barriers; stores are masked
  const int chunks = K >> 4;
  const uint4 *xr = reinterpret_cast<const uint4 *>(x + (int64_t)row * ldx);

  uint4 v[NC][2];
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = i * TPR + t;
    if (c < chunks) {
      if (!kNorm && gT > 0) {
        // attention output as the attention kernel leaves it, [B, heads, T, D]: row
        // (b, t) of the linear is the concatenation of its heads' D-vectors
        const int bb = row / gT, tt = row - bb * gT;
        const int head = (16 * c) / gD, off = (16 * c) - head * gD;
        const uint4 *hp = reinterpret_cast<const uint4 *>(
            x + (((int64_t)bb * (K / gD) + head) * gT + tt) * gD + off);
        v[i][0] = __ldg(hp);
        v[i][1] = __ldg(hp + 1);
      } else {
        v[i][0] = __ldg(xr + 2 * c);
        v[i][1] = __ldg(xr + 2 * c + 1);
      }
    } else {
      v[i][0] = make_uint4(0, 0, 0, 0);
      v[i][1] = make_uint4(0, 0, 0, 0);
    }
  }

  if constexpr (!kNorm) {
    if (delta != nullptr) {
      // SwiGLU input: x points at the gate half of fused [gate | up] rows (row pitch
      // ldx), delta at the up half; the row to quantise is half(half(silu(g)) * u),
      // the two roundings of an fp16 silu followed by an fp16 multiply
      const uint4 *ur = reinterpret_cast<const uint4 *>(delta + (int64_t)row * ldx);
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = i * TPR + t;
        if (c < chunks) {
          uint4 uv[2] = {__ldg(ur + 2 * c), __ldg(ur + 2 * c + 1)};
          uint32_t *u = reinterpret_cast<uint32_t *>(&v[i][0]);
          const uint32_t *uu = reinterpret_cast<const uint32_t *>(&uv[0]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(&u[j]));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&uu[j]));
            const float s0 = silu_to_half(g.x);
            const float s1 = silu_to_half(g.y);
            __half2 h = __floats2half2_rn(s0 * b.x, s1 * b.y);
            u[j] = *reinterpret_cast<uint32_t *>(&h);
          }
        }
      }
    }
  }
  if constexpr (kNorm) {
    if (delta != nullptr) {
      // residual update: x <- half(x + delta), written back, then normalised
      const uint4 *dr = reinterpret_cast<const uint4 *>(delta + (int64_t)row * K);
      uint4 *xo = reinterpret_cast<uint4 *>(x_out + (int64_t)row * ldx);
#pragma unroll
      for (int i = 0; i < NC; ++i) {
        const int c = i * TPR + t;
        if (c < chunks) {
          uint4 dv[2] = {__ldg(dr + 2 * c), __ldg(dr + 2 * c + 1)};
          uint32_t *u = reinterpret_cast<uint32_t *>(&v[i][0]);
          const uint32_t *ud = reinterpret_cast<const uint32_t *>(&dv[0]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&u[j]));
            float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&ud[j]));
            __half2 h = __floats2half2_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
            u[j] = *reinterpret_cast<uint32_t *>(&h);
          }
          if (live) {
            xo[2 * c] = v[i][0];
            xo[2 * c + 1] = v[i][1];
          }
        }
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const uint32_t *u = reinterpret_cast<const uint32_t *>(&v[i][0]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[j]));
        ss = fmaf(f.x, f.x, ss);
        ss = fmaf(f.y, f.y, ss);
      }
    }
    ss = row_reduce<TPR, false>(ss, red, tid);
    const float r = 1.0f / sqrtf(ss / (float)K + eps);
    const uint4 *wr = reinterpret_cast<const uint4 *>(w);
    uint4 *yr = y ? reinterpret_cast<uint4 *>(y + (int64_t)row * K) : nullptr;
#pragma unroll
    for (int i = 0; i < NC; ++i) {
      const int c = i * TPR + t;
      if (c < chunks) {
        uint4 wv[2] = {__ldg(wr + 2 * c), __ldg(wr + 2 * c + 1)};
        uint32_t *u = reinterpret_cast<uint32_t *>(&v[i][0]);
        const uint32_t *uw = reinterpret_cast<const uint32_t *>(&wv[0]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&u[j]));
          float2 g = __half22float2(*reinterpret_cast<const __half2 *>(&uw[j]));
          __half2 h = __floats2half2_rn(__fmul_rn(__fmul_rn(f.x, r), g.x),
                                        __fmul_rn(__fmul_rn(f.y, r), g.y));
          u[j] = *reinterpret_cast<uint32_t *>(&h);
        }
        if (yr && live) {
          yr[2 * c] = v[i][0];
          yr[2 * c + 1] = v[i][1];
        }
      }
    }
  }

  if (kNorm && q == nullptr) return;  // norm only (all threads of the block agree)

  // absmax in fp16 (exact: |.| and max commute with the widening conversion)
  __half2 hm = __float2half2_rn(0.0f);
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const uint32_t *u = reinterpret_cast<const uint32_t *>(&v[i][0]);
#pragma unroll
    for (int j = 0; j < 8; ++j) hm = __hmax2(hm, __habs2(*reinterpret_cast<const __half2 *>(&u[j])));
  }
  float amax = fmaxf(__low2float(hm), __high2float(hm));
  amax = row_reduce<TPR, true>(amax, red, tid);

  float s = __fdiv_rn(amax, 127.0f);
  if (s == 0.0f) s = 1.0f;
  const float inv = __fdiv_rn(1.0f, s);
  if (t == 0 && live) scale[row] = s;

  uint4 *qr = reinterpret_cast<uint4 *>(q + (int64_t)row * K);
#pragma unroll
  for (int i = 0; i < NC; ++i) {
    const int c = i * TPR + t;
    if (c < chunks && live) {
      const uint32_t *u = reinterpret_cast<const uint32_t *>(&v[i][0]);
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&u[2 * j]));
        float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&u[2 * j + 1]));
        o[j] = pack4(quant_one(f0.x, inv), quant_one(f0.y, inv), quant_one(f1.x, inv),
                     quant_one(f1.y, inv));
      }
      if (perm8) {
        // the order in which the W4A8 converters produce the weights of 8 k: even k, then odd k
        // (a dot product does not care, as long as both operands agree)
        const uint32_t a0 = __byte_perm(o[0], o[1], 0x6420), a1 = __byte_perm(o[0], o[1], 0x7531);
        const uint32_t a2 = __byte_perm(o[2], o[3], 0x6420), a3 = __byte_perm(o[2], o[3], 0x7531);
        o[0] = a0; o[1] = a1; o[2] = a2; o[3] = a3;
      }
      qr[c] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// Scalar kernel for any K / stride / alignment: one block per row, the row is
// read twice (three times with the norm).
template <bool kNorm>
__global__ void __launch_bounds__(kBlock)
quantize_rows_scalar_kernel(const __half *x, int64_t ldx,
                            const __half *__restrict__ w, float eps, __half *__restrict__ y,
                            int8_t *__restrict__ q, float *__restrict__ scale, int M, int K,
                            const __half *__restrict__ delta, __half *x_out) {
  __shared__ float red[kBlock / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  const int row = blockIdx.x;
  const __half *xr = x + (int64_t)row * ldx;
  float r = 1.0f;
  if constexpr (kNorm) {
    if (delta != nullptr) {
      __half *xo = x_out + (int64_t)row * ldx;
      for (int k = tid; k < K; k += kBlock)
        xo[k] = __float2half_rn(__fadd_rn(__half2float(xr[k]), __half2float(delta[(int64_t)row * K + k])));
      __syncthreads();
      xr = xo;
    }
    float ss = 0.0f;
    for (int k = tid; k < K; k += kBlock) {
      float f = __half2float(xr[k]);
      ss = fmaf(f, f, ss);
    }
    ss = row_reduce<kBlock, false>(ss, red, tid);
    r = 1.0f / sqrtf(ss / (float)K + eps);
  }
  auto value = [&](int k) -> __half {
    if constexpr (kNorm) {
      return __float2half_rn(__fmul_rn(__fmul_rn(__half2float(xr[k]), r), __half2float(w[k])));
    } else {
      if (delta != nullptr) {  // SwiGLU input, see the vector kernel
        const float g = __half2float(xr[k]), u = __half2float(delta[(int64_t)row * ldx + k]);
        const float sl = silu_to_half(g);
        return __float2half_rn(sl * u);
      }
      return xr[k];
    }
  };
  if (kNorm && q == nullptr) {
    for (int k = tid; k < K; k += kBlock) y[(int64_t)row * K + k] = value(k);
    return;
  }
  float amax = 0.0f;
  for (int k = tid; k < K; k += kBlock) amax = fmaxf(amax, fabsf(__half2float(value(k))));
  amax = row_reduce<kBlock, true>(amax, red, tid);
  float s = __fdiv_rn(amax, 127.0f);
  if (s == 0.0f) s = 1.0f;
  const float inv = __fdiv_rn(1.0f, s);
  if (tid == 0) scale[row] = s;
  for (int k = tid; k < K; k += kBlock) {
    __half h = value(k);
    if (kNorm && y) y[(int64_t)row * K + k] = h;
    q[(int64_t)row * K + k] = (int8_t)quant_one(__half2float(h), inv);
  }
}

// The quantiser in two halves, for a row whose absmax is not known from the row alone
// (a tensor-parallel rank holding a K-slice of the activation: the ranks exchange
// their slice maxima and every rank quantises with the full row's scale):
//   kGiven == false: amax[row] = max_k |x[row, k]|                       (fp32)
//   kGiven == true : s = amax[row] / 127 (0 -> 1), q = round_half_away(x * (1/s)),
//                    scale[row] = s - the arithmetic of the one-pass kernel.
// One block per row; 16-byte loads when the row allows them.
template <bool kGiven>
__global__ void __launch_bounds__(kBlock)
quantize_amax_kernel(const __half *__restrict__ x, int64_t ldx, float *amax, int8_t *__restrict__ q,
                     float *__restrict__ scale, int K, int vec, int reset) {
  __shared__ float red[kBlock / 32];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, row = blockIdx.x;
  const __half *xr = x + (int64_t)row * ldx;
  if constexpr (!kGiven) {
    float m = 0.0f;
    if (vec) {
      const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
      __half2 hm = __float2half2_rn(0.0f);
      for (int c = tid; c < K / 8; c += kBlock) {
        const uint4 v = __ldg(xv + c);
        const uint32_t *u = reinterpret_cast<const uint32_t *>(&v);
#pragma unroll
        for (int j = 0; j < 4; ++j) hm = __hmax2(hm, __habs2(*reinterpret_cast<const __half2 *>(&u[j])));
      }
      m = fmaxf(__low2float(hm), __high2float(hm));
    } else {
      for (int k = tid; k < K; k += kBlock) m = fmaxf(m, fabsf(__half2float(xr[k])));
    }
    m = row_reduce<kBlock, true>(m, red, tid);
    if (tid == 0) amax[row] = m;
  } else {
    float s = __fdiv_rn(amax[row], 127.0f);
    if (reset) {  // the maxima are an accumulator of the kernel before this one: leave it zeroed for its next run
      __syncthreads();
      if (tid == 0) amax[row] = 0.0f;
    }
    if (s == 0.0f) s = 1.0f;
    const float inv = __fdiv_rn(1.0f, s);
    if (tid == 0) scale[row] = s;
    int8_t *qr = q + (int64_t)row * K;
    if (vec) {
      const uint4 *xv = reinterpret_cast<const uint4 *>(xr);
      uint2 *qv = reinterpret_cast<uint2 *>(qr);
      // four 16-byte loads per thread in flight before the first is used (a row of 6144 values is
      // three of them; one load per loop pass would be three latencies in a row)
      const int n8 = K / 8;
      for (int c0 = tid; c0 < n8; c0 += 4 * kBlock) {
        uint4 v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (c0 + i * kBlock < n8) v[i] = __ldg(xv + c0 + i * kBlock);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          if (c0 + i * kBlock < n8) {
            const uint32_t *u = reinterpret_cast<const uint32_t *>(&v[i]);
            uint32_t o[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const float2 f0 = __half22float2(*reinterpret_cast<const __half2 *>(&u[2 * j]));
              const float2 f1 = __half22float2(*reinterpret_cast<const __half2 *>(&u[2 * j + 1]));
              o[j] = pack4(quant_one(f0.x, inv), quant_one(f0.y, inv), quant_one(f1.x, inv), quant_one(f1.y, inv));
            }
            qv[c0 + i * kBlock] = make_uint2(o[0], o[1]);
          }
        }
      }
    } else {
      for (int k = tid; k < K; k += kBlock) qr[k] = (int8_t)quant_one(__half2float(xr[k]), inv);
    }
  }
}

template <bool kNorm>
int launch_impl(const __half *x, int64_t ldx, const __half *w, float eps, __half *y, int8_t *q,
                float *scale, int64_t M, int64_t K, cudaStream_t st, const __half *delta = nullptr,
                __half *x_out = nullptr, int gT = 0, int gD = 0, int perm8 = 0) {
  if (M == 0 || K == 0) {
    // nothing to read: an empty row has amax 0 -> scale 1 (zero guard)
    if (M > 0) {
      quantize_rows_scalar_kernel<kNorm><<<(unsigned)M, kBlock, 0, st>>>(x, ldx, w, eps, y, q, scale,
                                                                        (int)M, 0, delta, x_out);
      return check_cuda(cudaGetLastError(), "quantize launch");
    }
    return CIDER_OK;
  }
  auto aligned16 = [](const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  const int64_t chunks = K / 16;
  bool vec = (K % 16 == 0) && (ldx % 8 == 0) && aligned16(x) && (q == nullptr || aligned16(q)) &&
             chunks <= (int64_t)kMaxChunks * 256;
  if (kNorm) vec = vec && aligned16(w) && (y == nullptr || aligned16(y)) &&
                   (delta == nullptr || (aligned16(delta) && aligned16(x_out)));
  else vec = vec && (delta == nullptr || aligned16(delta));
  if (gT > 0) vec = vec && (gD % 16 == 0) && (K % gD == 0);
  if (!vec) {
    if (perm8) return fail(CIDER_E_ALIGNMENT, "quantize (permuted): needs K % 16 == 0 and 16-byte aligned buffers");
    if (gT > 0) return fail(CIDER_E_SHAPE, "quantize_heads: needs head_dim % 16 == 0 and 16-byte aligned buffers");
    quantize_rows_scalar_kernel<kNorm><<<(unsigned)M, kBlock, 0, st>>>(x, ldx, w, eps, y, q, scale,
                                                                      (int)M, (int)K, delta, x_out);
    return check_cuda(cudaGetLastError(), "quantize launch");
  }
  // fewest threads per row that keep the row in registers; at least 5 chunks
  // per thread keeps enough loads in flight per thread.
  int tpr = 32;
  while ((int64_t)tpr * kMaxChunks < chunks) tpr <<= 1;
  // small M: spread each row over more threads so that more SMs get work
  while (tpr < 256 && (M * tpr) / kBlock < 2 * sm_count(current_device()) && chunks >= 2 * tpr) tpr <<= 1;
  // with a norm or a SwiGLU in front (more registers, more arithmetic per element) the
  // 8-chunk instantiation and its one block per SM lose 15-25 %: spread the row over
  // more threads instead.  The plain quantiser is faster as it is.
  if (kNorm || delta != nullptr)
    while (tpr < 256 && (chunks + tpr - 1) / tpr > 4) tpr <<= 1;
  const unsigned grid = (unsigned)((M + (kBlock / tpr) - 1) / (kBlock / tpr));
  // chunks cached per thread: the smallest of 2 / 4 / 6 / 8 that holds the row (fewer
  // registers -> more resident warps -> more loads in flight)
  const int per_thread = (int)((chunks + tpr - 1) / tpr);
  const int nc = per_thread <= 2 ? 2 : (per_thread <= 4 ? 4 : (per_thread <= 6 ? 6 : 8));
#define CIDER_Q_LAUNCH(T, C) \
  launch_kernel(quantize_rows_kernel<T, C, kNorm>, dim3(grid), dim3(kBlock), 0, st, x, ldx, w, eps, y, q, scale, \
                (int)M, (int)K, delta, x_out, gT, gD, perm8)
#define CIDER_Q_CASE(T)                      \
  case T:                                    \
    if (nc == 2) CIDER_Q_LAUNCH(T, 2);       \
    else if (nc == 4) CIDER_Q_LAUNCH(T, 4);  \
    else if (nc == 6) CIDER_Q_LAUNCH(T, 6);  \
    else CIDER_Q_LAUNCH(T, 8);               \
    break;
  switch (tpr) {
    CIDER_Q_CASE(32)
    CIDER_Q_CASE(64)
    CIDER_Q_CASE(128)
    default:
      if (nc == 2) CIDER_Q_LAUNCH(256, 2);
      else if (nc == 4) CIDER_Q_LAUNCH(256, 4);
      else if (nc == 6) CIDER_Q_LAUNCH(256, 6);
      else CIDER_Q_LAUNCH(256, 8);
      break;
  }
#undef CIDER_Q_CASE
#undef CIDER_Q_LAUNCH
  return check_cuda(cudaGetLastError(), "quantize launch");
}

}  // namespace

int launch_quantize_per_token(const __half *x, int64_t M, int64_t K, int64_t ldx, int8_t *q,
                              float *scale, cudaStream_t st) {
  return launch_impl<false>(x, ldx, nullptr, 0.0f, nullptr, q, scale, M, K, st);
}

// The same with every aligned run of 8 quantised values stored as k0 k2 k4 k6 k1 k3 k5 k7.
bool quantize_perm8_ok(const __half *x, int64_t K, int64_t ldx, const int8_t *q) {
  return K % 16 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
         (reinterpret_cast<uintptr_t>(q) & 15u) == 0 && K / 16 <= (int64_t)kMaxChunks * 256;
}
int launch_quantize_per_token_perm8(const __half *x, int64_t M, int64_t K, int64_t ldx, int8_t *q,
                                    float *scale, cudaStream_t st) {
  return launch_impl<false>(x, ldx, nullptr, 0.0f, nullptr, q, scale, M, K, st, nullptr, nullptr, 0, 0, 1);
}

// In-place form of the same permutation for quantised rows that already exist (only taken when
// the input of the quantiser was not aligned for its vectorised form): 8 bytes per thread.
__global__ void __launch_bounds__(256) permute8_kernel(uint2 *q, int64_t n8) {
  pdl_launch_dependents();
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (int64_t)gridDim.x * blockDim.x) {
    const uint2 v = q[i];
    q[i] = make_uint2(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531));
  }
}
int launch_permute8(int8_t *q, int64_t bytes, cudaStream_t st) {
  if (bytes % 8 != 0 || (reinterpret_cast<uintptr_t>(q) & 7u)) return fail(CIDER_E_ALIGNMENT, "permute8: needs 8-byte units");
  const int64_t n8 = bytes / 8;
  if (n8 == 0) return CIDER_OK;
  int64_t blocks = (n8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  return check_cuda(launch_kernel(permute8_kernel, dim3((unsigned)blocks), dim3(256), 0, st,
                                  reinterpret_cast<uint2 *>(q), n8),
                    "permute8 launch");
}

int launch_rmsnorm_quant(const __half *x, const __half *w, float eps, int64_t M, int64_t K,
                         __half *y, int8_t *q, float *scale, cudaStream_t st) {
  return launch_impl<true>(x, K, w, eps, y, q, scale, M, K, st);
}

int launch_row_absmax(const __half *x, int64_t M, int64_t K, int64_t ldx, float *amax, cudaStream_t st) {
  if (M == 0) return CIDER_OK;
  const int vec = K % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0;
  return check_cuda(launch_kernel(quantize_amax_kernel<false>, dim3((unsigned)M), dim3(kBlock), 0, st, x, ldx, amax,
                                  static_cast<int8_t *>(nullptr), static_cast<float *>(nullptr), (int)K, vec, 0),
                    "row_absmax launch");
}

int launch_quantize_given_amax(const __half *x, int64_t M, int64_t K, int64_t ldx, const float *amax, int8_t *q,
                               float *scale, cudaStream_t st, bool reset_amax) {
  if (M == 0) return CIDER_OK;
  const int vec = K % 8 == 0 && ldx % 8 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
                  (reinterpret_cast<uintptr_t>(q) & 7u) == 0;
  return check_cuda(launch_kernel(quantize_amax_kernel<true>, dim3((unsigned)M), dim3(kBlock), 0, st, x, ldx,
                                  const_cast<float *>(amax), q, scale, (int)K, vec, reset_amax ? 1 : 0),
                    "quantize_given_amax launch");
}

// Per-token quantiser of an attention output in [B, heads, T, D] layout: row (b, t) of
// the result is the concatenation of the heads (what a transpose + reshape would
// have produced, without the copy).
int launch_quantize_heads(const __half *a, int64_t B, int64_t heads, int64_t T, int64_t D, int8_t *q,
                          float *scale, cudaStream_t st) {
  return launch_impl<false>(a, heads * D, nullptr, 0.0f, nullptr, q, scale, B * T, heads * D, st, nullptr, nullptr,
                            (int)T, (int)D);
}

// Per-token quantiser of SwiGLU(gate_up): rows of gate_up are [gate | up], 2*inter wide.
int launch_silu_mul_quant(const __half *gate_up, int64_t M, int64_t inter, int8_t *q, float *scale,
                          cudaStream_t st) {
  return launch_impl<false>(gate_up, 2 * inter, nullptr, 0.0f, nullptr, q, scale, M, inter, st, gate_up + inter,
                            nullptr);
}

// x <- half(x + delta) in place, then the RMSNorm (+ optional quantiser) of the sum.
int launch_add_rmsnorm_quant(__half *x, const __half *delta, const __half *w, float eps, int64_t M,
                             int64_t K, __half *y, int8_t *q, float *scale, cudaStream_t st) {
  return launch_impl<true>(x, K, w, eps, y, q, scale, M, K, st, delta, x);
}

}  // namespace cider
