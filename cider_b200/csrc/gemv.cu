// M == 1 decode path: y[n] = sum_k W[n,k] * x[k] with int8 weights and an fp16
// activation that is NOT quantised (csrc/src/w8a8_primitive.mm:157-178).
//   per-channel: half(fma(sw[n], dot, bias[n]))            (w8a8_int8_mv.metal:34-69)
//   per-group  : half(sum over 16-wide chunks sw[g,n]*dot16 + bias[n])
//                (pergroup_int8_mv.metal:50-103 applies the group scale per
//                 8-element chunk before the lane reduction; 16 here)
// Pure weight streaming (N*K bytes), so the kernel is shaped for HBM: 128-bit
// streaming weight loads, every byte touched once, one resident block per SM
// with ten 16-byte loads in flight per lane.  Sums are fp32; the order differs
// from the reference's SIMD-group order, which the 2e-3 tolerance of the M == 1
// path covers.
#include <mutex>

#include "common.cuh"

namespace cider {
namespace {

constexpr int kWarps = 8;
constexpr int kMaxSteps = 5;  // 16-byte chunks of x held per lane (80 fp32 registers)

// What the compute warps do to the activation while they load it (the weights are
// already streaming): nothing, SwiGLU of a fused [gate | up] vector, or residual
// add + RMSNorm.  Folding these into the matrix-vector kernel removes three small
// kernels per decoder layer from a batch-1 decode step, where launch latency and
// not HBM is what a 2B model is bound by.
constexpr int kProloguePlain = 0, kPrologueSiluMul = 1, kPrologueAddNorm = 2;
struct GemvPrologue {
  int mode = kProloguePlain;
  const __half *delta = nullptr;   // add+norm: optional residual delta [K]
  const __half *norm_w = nullptr;  // add+norm: RMSNorm weight [K]
  __half *x_out = nullptr;         // add+norm: x + delta is written here (must not alias x)
  float eps = 0.0f;
};

__device__ __forceinline__ float sw_at(const void *sw, int is_half, int64_t idx) {
  return is_half ? __half2float(reinterpret_cast<const __half *>(sw)[idx])
                 : __ldg(reinterpret_cast<const float *>(sw) + idx);
}

// Dot product of 16 int8 weights with 16 fp32 activations held as 8 packed pairs.
// int8 -> fp32 without the conversion unit (16 lanes per clock, it would bound the
// kernel below HBM speed): w ^ 0x80 is the byte w + 128 as unsigned; a byte
// permute drops it into the low mantissa byte of 0x4B000000 (= 8388608.0f), which
// reads as 8388608 + 128 + w, and subtracting 8388736 is exact.  The subtract and
// the multiply-add are the packed two-lane fp32 instructions.
__device__ __forceinline__ float dot16(const uint4 &w, const uint64_t *xp) {
  const uint32_t u[4] = {w.x ^ 0x80808080u, w.y ^ 0x80808080u, w.z ^ 0x80808080u, w.w ^ 0x80808080u};
  const float2 negc = make_float2(-8388736.0f, -8388736.0f);
  const uint64_t neg = *reinterpret_cast<const uint64_t *>(&negc);
  uint64_t acc = 0ull;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint2 a = make_uint2(__byte_perm(u[i], 0x4B000000u, 0x7540), __byte_perm(u[i], 0x4B000000u, 0x7541));
    uint2 b = make_uint2(__byte_perm(u[i], 0x4B000000u, 0x7542), __byte_perm(u[i], 0x4B000000u, 0x7543));
    uint64_t fa, fb;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(fa) : "l"(*reinterpret_cast<uint64_t *>(&a)), "l"(neg));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(fb) : "l"(*reinterpret_cast<uint64_t *>(&b)), "l"(neg));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(acc) : "l"(fa), "l"(xp[2 * i]), "l"(acc));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(acc) : "l"(fb), "l"(xp[2 * i + 1]), "l"(acc));
  }
  const float2 r = *reinterpret_cast<const float2 *>(&acc);
  return r.x + r.y;
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---- bounded shared-memory barrier waits (same policy as the GEMM kernels: a
// wait that runs out records a status bit and the kernel winds down)
__device__ unsigned int g_gemv_status = 0;
constexpr long long kWaitCycles = 4000000000ll;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > kWaitCycles) {
      *abort_flag = 1;
      atomicOr(&g_gemv_status, kStatusWaitTimeout);
      return false;
    }
  }
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// Streaming kernel: K % 16 == 0, w and x 16-byte aligned, K <= 16*32*kMaxSteps*kWarps.
// One CTA per SM owns a contiguous range of rows.  A producer thread streams the
// weights of WR consecutive rows at a time (WR*K contiguous bytes, one bulk
// asynchronous copy) into a ring of shared-memory stages, so the bytes in flight
// per SM are set by the ring (~150 KB) and not by how many loads the compute warps
// can hold in registers - that is what it takes to keep HBM3e busy from 148 SMs.
// The 8 compute warps form WR row-groups of WK warps; warp (wr, wk) takes row wr
// of the stage and chunks [wk*S*32, (wk+1)*S*32) of K, whose activations it holds
// in registers for the whole kernel; it copies its piece of the row to registers,
// releases the stage, and only then does the arithmetic.
template <int S, bool kGroup>
__global__ void __launch_bounds__((kWarps + 1) * 32, 1)
gemv_kernel(const __half *__restrict__ x, const int8_t *__restrict__ w, const void *__restrict__ sw,
            int sw_half, int gs, const __half *__restrict__ bias, __half *__restrict__ y, int N,
            int K, int WK, int stages, int rows_cap, const GemvPrologue pro) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full_bar[16], empty_bar[16];
  __shared__ float part[2][kWarps];
  __shared__ int abort_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int WR = kWarps / WK;
  const int chunks = K >> 4;
  const uint32_t stage_bytes = (uint32_t)WR * (uint32_t)K;

  // rows of this CTA: as even a split of N as possible
  const int lo = N / gridDim.x, extra = N % gridDim.x;
  const int begin = blockIdx.x * lo + min((int)blockIdx.x, extra);
  const int count = lo + ((int)blockIdx.x < extra ? 1 : 0);
  const int iters = (count + WR - 1) / WR;

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), kWarps);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  float *row_sw = reinterpret_cast<float *>(ring + (size_t)stages * stage_bytes);
  float *row_bias = row_sw + rows_cap;

  if (warp == kWarps) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int issued = 0;
      for (int it = 0; it < iters; ++it) {
        if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &abort_s)) break;
        const int rows = min(WR, count - it * WR);
        const uint32_t bytes = (uint32_t)rows * (uint32_t)K;
        const uint32_t fb = smem_u32(&full_bar[stage]);
        mbar_expect_tx(fb, bytes);
        bulk_load(smem_u32(ring + (size_t)stage * stage_bytes), w + (int64_t)(begin + it * WR) * K, bytes, fb);
        ++issued;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (abort_s) {  // gave up: let the copies already issued land before the CTA exits
        const int last = issued < stages ? issued : stages;
        for (int i = 0; i < last; ++i) {
          const int f = issued - 1 - i;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&full_bar[f % stages]), (uint32_t)(f / stages) & 1u) &&
                 clock64() - t0 < kWaitCycles) {
          }
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- compute warps
  // (the producer is already streaming weights while these set up)
  // per-row epilogue constants of this CTA's rows, fetched once: a global load per
  // row inside the loop would put an L2 / DRAM round trip on every iteration
  for (int i = threadIdx.x; i < count; i += kWarps * 32) {
    row_sw[i] = kGroup ? 0.0f : sw_at(sw, sw_half, begin + i);
    row_bias[i] = bias ? __half2float(bias[begin + i]) : 0.0f;
  }
  const int wr = warp / WK, wk = warp % WK;
  // Everything above reads weights only.  The activation (and, further down, every
  // write) waits for the kernels this one depends on.
  pdl_wait();
  uint64_t xr[S][8];  // 16 fp32 activations per step as packed pairs
  int goff[S];
  float ss = 0.0f;  // sum of squares of this warp's slice (norm prologue)
#pragma unroll
  for (int s = 0; s < S; ++s) {
    const int c = (wk * S + s) * 32 + lane;
    goff[s] = 0;
    if (c < chunks) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(x + 16 * c);
      uint4 h[2] = {__ldg(xp), __ldg(xp + 1)};
      __half2 *h2 = reinterpret_cast<__half2 *>(h);
      if (pro.mode == kPrologueSiluMul) {
        // x = [gate | up] of length 2K: activation = half(half(silu(g)) * u)
        const uint4 *up = reinterpret_cast<const uint4 *>(x + K + 16 * c);
        uint4 u[2] = {__ldg(up), __ldg(up + 1)};
        const __half2 *u2 = reinterpret_cast<const __half2 *>(u);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 g = __half22float2(h2[j]), uu = __half22float2(u2[j]);
          const float s0 = __half2float(__float2half_rn(g.x / (1.0f + expf(-g.x))));
          const float s1 = __half2float(__float2half_rn(g.y / (1.0f + expf(-g.y))));
          h2[j] = __floats2half2_rn(s0 * uu.x, s1 * uu.y);
        }
      } else if (pro.mode == kPrologueAddNorm) {
        if (pro.delta != nullptr) {
          const uint4 *dp = reinterpret_cast<const uint4 *>(pro.delta + 16 * c);
          uint4 d[2] = {__ldg(dp), __ldg(dp + 1)};
          const __half2 *d2 = reinterpret_cast<const __half2 *>(d);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float2 a = __half22float2(h2[j]), b = __half22float2(d2[j]);
            h2[j] = __floats2half2_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
          }
        }
        if (blockIdx.x == 0 && wr == 0 && pro.x_out != nullptr) {  // one row-group publishes the new residual
          uint4 *op = reinterpret_cast<uint4 *>(pro.x_out + 16 * c);
          op[0] = h[0];
          op[1] = h[1];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 f = __half22float2(h2[j]);
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float2 f = __half22float2(h2[j]);
        xr[s][j] = *reinterpret_cast<const uint64_t *>(&f);
      }
      if constexpr (kGroup) goff[s] = ((16 * c) / gs) * N;
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) xr[s][j] = 0ull;
    }
  }
  if (pro.mode == kPrologueAddNorm) {
    // RMSNorm of the full activation: reduce over the lanes and the WK warps that
    // together hold one copy of it, then n = half(v * r * w) like the stand-alone kernel
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (WK > 1) {
      if (lane == 0) part[0][warp] = ss;
      group_barrier(1 + wr, WK * 32);
      ss = 0.0f;
      for (int k = 0; k < WK; ++k) ss += part[0][wr * WK + k];
      group_barrier(1 + wr, WK * 32);  // part[] is reused by the row loop
    }
    const float r = 1.0f / sqrtf(ss / (float)K + pro.eps);
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int c = (wk * S + s) * 32 + lane;
      if (c < chunks) {
        const uint4 *wp = reinterpret_cast<const uint4 *>(pro.norm_w + 16 * c);
        uint4 nw[2] = {__ldg(wp), __ldg(wp + 1)};
        const __half2 *w2 = reinterpret_cast<const __half2 *>(nw);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 v = *reinterpret_cast<const float2 *>(&xr[s][j]);
          const float2 g = __half22float2(w2[j]);
          const float2 n = __half22float2(__floats2half2_rn(__fmul_rn(__fmul_rn(v.x, r), g.x),
                                                            __fmul_rn(__fmul_rn(v.y, r), g.y)));
          xr[s][j] = *reinterpret_cast<const uint64_t *>(&n);
        }
      }
    }
  }

  group_barrier(15, kWarps * 32);  // row_sw / row_bias visible to all compute warps
  int stage = 0;
  uint32_t phase = 0;
  // per-group: this lane's group scales of the NEXT row are requested one iteration
  // ahead (they depend on the row, unlike the activations)
  float gsc[S], gsn[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    gsc[s] = 0.0f;
    gsn[s] = 0.0f;
    if constexpr (kGroup) {
      if (wr < count) gsc[s] = sw_at(sw, sw_half, goff[s] + begin + wr);
    }
  }
  for (int it = 0; it < iters; ++it) {
    if constexpr (kGroup) {
      const int nn = (it + 1) * WR + wr;
#pragma unroll
      for (int s = 0; s < S; ++s) gsn[s] = nn < count ? sw_at(sw, sw_half, goff[s] + begin + nn) : 0.0f;
    }
    uint32_t got = 0;
    if (lane == 0) got = mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_s);
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) break;
    const int n = begin + it * WR + wr;
    const bool live = it * WR + wr < count;
    const uint4 *row = reinterpret_cast<const uint4 *>(ring + (size_t)stage * stage_bytes + (size_t)wr * K);
    uint4 wv[S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int c = (wk * S + s) * 32 + lane;
      wv[s] = (live && c < chunks) ? row[c] : make_uint4(0, 0, 0, 0);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));  // stage may be refilled now
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
    float a = 0.0f;
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float d = dot16(wv[s], xr[s]);
      if constexpr (kGroup) a = fmaf(gsc[s], d, a);
      else a += d;
    }
    if constexpr (kGroup) {
#pragma unroll
      for (int s = 0; s < S; ++s) gsc[s] = gsn[s];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
    if (WK > 1) {
      if (lane == 0) part[it & 1][warp] = a;
      group_barrier(1 + wr, WK * 32);
      if (wk == 0 && lane == 0) {
        float sum = 0.0f;
        for (int k = 0; k < WK; ++k) sum += part[it & 1][wr * WK + k];
        a = sum;
      }
    }
    if (wk == 0 && lane == 0 && live) {
      const float b = row_bias[it * WR + wr];
      float v;
      if constexpr (kGroup) v = a + b;
      else v = fmaf(row_sw[it * WR + wr], a, b);
      y[n] = __float2half_rn(v);
    }
  }
}

// Scalar kernel for any K / alignment: one warp per row.
__global__ void __launch_bounds__(128)
gemv_scalar_kernel(const __half *__restrict__ x, const int8_t *__restrict__ w,
                   const void *__restrict__ sw, int sw_half, int gs,
                   const __half *__restrict__ bias, __half *__restrict__ y, int N, int K) {
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (n >= N) return;
  float acc = 0.0f;
  for (int k = lane; k < K; k += 32) {
    float t = (float)w[(int64_t)n * K + k] * __half2float(x[k]);
    if (gs > 0) t *= sw_at(sw, sw_half, (int64_t)(k / gs) * N + n);
    acc += t;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) {
    const float b = bias ? __half2float(bias[n]) : 0.0f;
    y[n] = __float2half_rn(gs > 0 ? acc + b : fmaf(sw_at(sw, sw_half, n), acc, b));
  }
}

// [K/2, N] packed int4 (high nibble = even k) -> [N, K] int8.  One thread
// expands 8 packed rows x 1 column into 16 consecutive bytes of one output row;
// a warp reads 32 consecutive bytes of each packed row.
__global__ void __launch_bounds__(256)
unpack_w4_kernel(const uint8_t *__restrict__ packed, int8_t *__restrict__ w, int N, int K) {
  const int n = blockIdx.x * 32 + (threadIdx.x & 31);
  const int kp0 = (blockIdx.y * 8 + (threadIdx.x >> 5)) * 8;  // first k-pair of this thread
  if (n >= N || 2 * kp0 >= K) return;
  uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (2 * (kp0 + i) < K) {
      const uint32_t byte = packed[(int64_t)(kp0 + i) * N + n];
      const uint32_t even = (uint32_t)(uint8_t)(int8_t)((int)(byte >> 4) - 8);
      const uint32_t odd = (uint32_t)(uint8_t)(int8_t)((int)(byte & 15u) - 8);
      v[i >> 1] |= (even | (odd << 8)) << (16 * (i & 1));
    }
  }
  int8_t *dst = w + (int64_t)n * K + 2 * kp0;
  if (2 * kp0 + 16 <= K && (K % 16) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0) {
    *reinterpret_cast<uint4 *>(dst) = make_uint4(v[0], v[1], v[2], v[3]);
  } else {
    for (int i = 0; i < 16 && 2 * kp0 + i < K; ++i) dst[i] = (int8_t)(v[i >> 2] >> (8 * (i & 3)));
  }
}

}  // namespace

static int launch_gemv_impl(const __half *x, const int8_t *w, const void *sw, int sw_is_half, int gs,
                            const __half *bias, __half *y, int64_t N, int64_t K, const GemvPrologue &pro,
                            cudaStream_t st) {
  if (N == 0) return CIDER_OK;
  const int64_t steps = (K / 16 + 31) / 32;  // 512-byte steps per row
  const bool vec = K > 0 && (K % 16 == 0) && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && steps <= kMaxSteps * kWarps &&
                   N < (1 << 30);
  if (!vec) {
    if (pro.mode != kProloguePlain)
      return fail(CIDER_E_SHAPE, "fused matrix-vector prologue needs K % 16 == 0 and 16-byte aligned operands");
    gemv_scalar_kernel<<<(unsigned)((N + 3) / 4), 128, 0, st>>>(x, w, sw, sw_is_half, gs, bias, y,
                                                               (int)N, (int)K);
    return check_cuda(cudaGetLastError(), "gemv launch");
  }
  int wk = 1;
  while ((steps + wk - 1) / wk > kMaxSteps) wk <<= 1;
  const int S = (int)((steps + wk - 1) / wk);
  const int wr = kWarps / wk;
  const size_t stage_bytes = (size_t)wr * (size_t)K;
  int stages = (int)((160 * 1024) / stage_bytes);
  if (stages > 16) stages = 16;
  if (stages < 2) stages = 2;
  // one CTA per SM, fewer when there are not `wr` rows for each
  int64_t grid = sm_count(current_device());
  if (grid * wr > N) grid = (N + wr - 1) / wr;
  const int rows_cap = (int)((N + grid - 1) / grid);
  if ((size_t)rows_cap * 8 > 32 * 1024) {  // keep the per-row constants within 32 KB
    stages = (int)((128 * 1024) / stage_bytes);
    if (stages < 2) stages = 2;
  }
  const size_t smem = stage_bytes * stages + (size_t)rows_cap * 8;
  if (smem > 200 * 1024 && pro.mode != kProloguePlain)
    return fail(CIDER_E_SHAPE, "fused matrix-vector prologue: problem too large");
  if (smem > 200 * 1024) {
    gemv_scalar_kernel<<<(unsigned)((N + 3) / 4), 128, 0, st>>>(x, w, sw, sw_is_half, gs, bias, y,
                                                               (int)N, (int)K);
    return check_cuda(cudaGetLastError(), "gemv launch");
  }
#define CIDER_GEMV_CASE(SV)                                                                         \
  case SV: {                                                                                        \
    auto kg = gemv_kernel<SV, true>;                                                                \
    auto kc = gemv_kernel<SV, false>;                                                               \
    static std::atomic<unsigned long long> done_g{0}, done_c{0};                                    \
    int arc = ensure_dynamic_smem(kg, 200 * 1024, done_g, "gemv shared-memory attribute");          \
    if (arc) return arc;                                                                            \
    if ((arc = ensure_dynamic_smem(kc, 200 * 1024, done_c, "gemv shared-memory attribute"))) return arc; \
    cudaError_t le;                                                                                 \
    if (gs > 0)                                                                                     \
      le = launch_kernel(kg, dim3((unsigned)grid), dim3((kWarps + 1) * 32), smem, st, x, w, sw,     \
                         sw_is_half, gs, bias, y, (int)N, (int)K, wk, stages, rows_cap, pro);       \
    else                                                                                            \
      le = launch_kernel(kc, dim3((unsigned)grid), dim3((kWarps + 1) * 32), smem, st, x, w, sw,     \
                         sw_is_half, gs, bias, y, (int)N, (int)K, wk, stages, rows_cap, pro);       \
    if (le != cudaSuccess) return check_cuda(le, "gemv launch");                                    \
  } break;
  switch (S) {
    CIDER_GEMV_CASE(1)
    CIDER_GEMV_CASE(2)
    CIDER_GEMV_CASE(3)
    CIDER_GEMV_CASE(4)
    CIDER_GEMV_CASE(5)
    default:
      return fail(CIDER_E_SHAPE, "gemv: internal step count out of range");
  }
#undef CIDER_GEMV_CASE
  return check_cuda(cudaGetLastError(), "gemv launch");
}

int launch_gemv(const __half *x, const int8_t *w, const void *sw, int sw_is_half, int gs,
                const __half *bias, __half *y, int64_t N, int64_t K, cudaStream_t st) {
  return launch_gemv_impl(x, w, sw, sw_is_half, gs, bias, y, N, K, GemvPrologue{}, st);
}

int launch_gemv_fused(const __half *x, int mode, const __half *delta, const __half *norm_w, float eps,
                      __half *x_out, const int8_t *w, const void *sw, int sw_is_half, int gs,
                      const __half *bias, __half *y, int64_t N, int64_t K, cudaStream_t st) {
  GemvPrologue pro;
  pro.mode = mode;
  pro.delta = delta;
  pro.norm_w = norm_w;
  pro.x_out = x_out;
  pro.eps = eps;
  return launch_gemv_impl(x, w, sw, sw_is_half, gs, bias, y, N, K, pro, st);
}

// Status word of the matrix-vector kernels (bounded waits), OR-ed into
// cider_device_status().
int read_gemv_status(unsigned int *out) {
  return check_cuda(cudaMemcpyFromSymbol(out, g_gemv_status, sizeof(unsigned int)), "read gemv status");
}
int clear_gemv_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_gemv_status, &z, sizeof(z)), "clear gemv status");
}

int launch_unpack_w4(const uint8_t *packed, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st) {
  if (N == 0 || K == 0) return CIDER_OK;
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K / 2 + 63) / 64));
  if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "unpack_w4: K too large");
  unpack_w4_kernel<<<grid, 256, 0, st>>>(packed, w_nk, (int)N, (int)K);
  return check_cuda(cudaGetLastError(), "unpack_w4 launch");
}

}  // namespace cider
