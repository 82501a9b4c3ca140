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
#include "common.cuh"

namespace cider {
namespace {

constexpr int kWarps = 8;
constexpr int kMaxSteps = 5;  // 16-byte chunks of x held per lane (80 fp32 registers)

__device__ __forceinline__ float sw_at(const void *sw, int is_half, int64_t idx) {
  return is_half ? __half2float(reinterpret_cast<const __half *>(sw)[idx])
                 : __ldg(reinterpret_cast<const float *>(sw) + idx);
}

__device__ __forceinline__ float dot16(const uint4 &w, const float *xr) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
  float acc = 0.0f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    acc = fmaf((float)(int8_t)(u[i]), xr[4 * i + 0], acc);
    acc = fmaf((float)(int8_t)(u[i] >> 8), xr[4 * i + 1], acc);
    acc = fmaf((float)(int8_t)(u[i] >> 16), xr[4 * i + 2], acc);
    acc = fmaf((float)(int8_t)(u[i] >> 24), xr[4 * i + 3], acc);
  }
  return acc;
}

__device__ __forceinline__ void group_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Vector kernel: K % 16 == 0, w 16-byte aligned, K <= 16*32*kMaxSteps*kWarps.
// The 8 warps of a block form WR row-groups of WK warps; warp `wk` of a group
// owns chunks [wk*S*32, (wk+1)*S*32) of K and keeps its slice of x in registers
// for every row it visits, so the inner loop is weight loads, conversions and
// FMAs only.  Rows are dealt out to the row-groups of the whole grid as evenly
// as possible (they differ by at most one row) and visited two at a time.
template <int S, bool kGroup>
__global__ void __launch_bounds__(kWarps * 32)
gemv_kernel(const __half *__restrict__ x, const int8_t *__restrict__ w, const void *__restrict__ sw,
            int sw_half, int gs, const __half *__restrict__ bias, __half *__restrict__ y, int N,
            int K, int WK) {
  __shared__ float part[2][kWarps][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int WR = kWarps / WK;
  const int wr = warp / WK, wk = warp % WK;
  const int chunks = K >> 4;

  float xr[S][16];
  int goff[S];
#pragma unroll
  for (int s = 0; s < S; ++s) {
    const int c = (wk * S + s) * 32 + lane;
    goff[s] = 0;
    if (c < chunks) {
      const uint4 *xp = reinterpret_cast<const uint4 *>(x + 16 * c);
      uint4 h[2] = {__ldg(xp), __ldg(xp + 1)};
      const __half2 *h2 = reinterpret_cast<const __half2 *>(h);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float2 f = __half22float2(h2[j]);
        xr[s][2 * j] = f.x;
        xr[s][2 * j + 1] = f.y;
      }
      if constexpr (kGroup) goff[s] = ((16 * c) / gs) * N;
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) xr[s][j] = 0.0f;
    }
  }

  // rows of this row-group
  const int groups = gridDim.x * WR;
  const int gidx = blockIdx.x * WR + wr;
  const int lo = N / groups, extra = N % groups;
  const int begin = gidx * lo + min(gidx, extra);
  const int count = lo + (gidx < extra ? 1 : 0);
  const int iters = (lo + (extra ? 1 : 0) + 1) / 2;  // same for every group of the grid

  for (int it = 0; it < iters; ++it) {
    const int r0 = begin + 2 * it;
    const bool live0 = 2 * it < count, live1 = 2 * it + 1 < count;
    const int n0 = live0 ? r0 : 0, n1 = live1 ? r0 + 1 : n0;
    const uint4 *w0 = reinterpret_cast<const uint4 *>(w + (int64_t)n0 * K);
    const uint4 *w1 = reinterpret_cast<const uint4 *>(w + (int64_t)n1 * K);
    uint4 wv[2][S];
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const int c = (wk * S + s) * 32 + lane;
      const bool in = c < chunks;
      wv[0][s] = (in && live0) ? __ldcs(w0 + c) : make_uint4(0, 0, 0, 0);
      wv[1][s] = (in && live1) ? __ldcs(w1 + c) : make_uint4(0, 0, 0, 0);
    }
    float a0 = 0.0f, a1 = 0.0f;
#pragma unroll
    for (int s = 0; s < S; ++s) {
      const float d0 = dot16(wv[0][s], xr[s]);
      const float d1 = dot16(wv[1][s], xr[s]);
      if constexpr (kGroup) {
        a0 = fmaf(sw_at(sw, sw_half, goff[s] + n0), d0, a0);
        a1 = fmaf(sw_at(sw, sw_half, goff[s] + n1), d1, a1);
      } else {
        a0 += d0;
        a1 += d1;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      a0 += __shfl_xor_sync(0xffffffffu, a0, o);
      a1 += __shfl_xor_sync(0xffffffffu, a1, o);
    }
    if (WK > 1) {
      if (lane == 0) {
        part[it & 1][warp][0] = a0;
        part[it & 1][warp][1] = a1;
      }
      group_barrier(1 + wr, WK * 32);
      if (wk == 0 && lane < 2) {
        float s = 0.0f;
        for (int k = 0; k < WK; ++k) s += part[it & 1][wr * WK + k][lane];
        a0 = s;  // lane 0 -> row 0, lane 1 -> row 1
      }
    } else {
      if (lane == 1) a0 = a1;
    }
    if (wk == 0 && lane < 2) {
      const bool live = lane == 0 ? live0 : live1;
      const int n = lane == 0 ? n0 : n1;
      if (live) {
        const float b = bias ? __half2float(bias[n]) : 0.0f;
        float v;
        if constexpr (kGroup) v = a0 + b;
        else v = fmaf(sw_at(sw, sw_half, n), a0, b);
        y[n] = __float2half_rn(v);
      }
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

int launch_gemv(const __half *x, const int8_t *w, const void *sw, int sw_is_half, int gs,
                const __half *bias, __half *y, int64_t N, int64_t K, cudaStream_t st) {
  if (N == 0) return CIDER_OK;
  const int64_t steps = (K / 16 + 31) / 32;  // 512-byte steps per row
  const bool vec = K > 0 && (K % 16 == 0) && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 &&
                   (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && steps <= kMaxSteps * kWarps &&
                   N < (1 << 30);
  if (!vec) {
    gemv_scalar_kernel<<<(unsigned)((N + 3) / 4), 128, 0, st>>>(x, w, sw, sw_is_half, gs, bias, y,
                                                               (int)N, (int)K);
    return check_cuda(cudaGetLastError(), "gemv launch");
  }
  int wk = 1;
  while ((steps + wk - 1) / wk > kMaxSteps) wk <<= 1;
  const int S = (int)((steps + wk - 1) / wk);
  const int wr = kWarps / wk;
  // one block per SM, fewer when there are not two rows per row-group
  int64_t grid = sm_count(current_device());
  if (grid * wr * 2 > N) grid = (N + wr * 2 - 1) / (wr * 2);
#define CIDER_GEMV_CASE(SV)                                                                        \
  case SV:                                                                                         \
    if (gs > 0)                                                                                    \
      gemv_kernel<SV, true><<<(unsigned)grid, kWarps * 32, 0, st>>>(x, w, sw, sw_is_half, gs, bias, \
                                                                   y, (int)N, (int)K, wk);         \
    else                                                                                           \
      gemv_kernel<SV, false><<<(unsigned)grid, kWarps * 32, 0, st>>>(x, w, sw, sw_is_half, gs,     \
                                                                    bias, y, (int)N, (int)K, wk);  \
    break;
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

int launch_unpack_w4(const uint8_t *packed, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st) {
  if (N == 0 || K == 0) return CIDER_OK;
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K / 2 + 63) / 64));
  if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "unpack_w4: K too large");
  unpack_w4_kernel<<<grid, 256, 0, st>>>(packed, w_nk, (int)N, (int)K);
  return check_cuda(cudaGetLastError(), "unpack_w4 launch");
}

}  // namespace cider
