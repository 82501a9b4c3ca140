// Plain CUDA-core integer GEMM (dp4a) with the same epilogues as the tensor-core
// kernel.  It exists for the shapes the TMA-fed kernel cannot take (K not a
// multiple of 16, unaligned pointers, packed-int4 weights read in place) and as
// an independent second implementation the tests compare the tensor-core kernel
// against.  Any M, N, K >= 0; every access is bounds-checked.
//
//   raw       : C[m,n] = sum_k A[m,k]*B[n,k]                         (w8a8_matmul.metal:301-453)
//   perchannel: half(fma(float(acc)*sa[m], sw[n], bias[n]))          (w8a8_matmul.metal:63-81)
//   pergroup  : accf = fma(float(acc_g), sw[g,n], accf) per group,
//               half(fma(accf, sa[m], bias[n]))                      (pergroup_int8_gemm.metal:99-191)
//   packed4   : B[n,k] = nibble(packed[k/2, n]) - 8, high nibble = even k
//               (w4a8_matmul.metal:47-70)
#include "common.cuh"

namespace cider {
namespace {

constexpr int BM = 64, BN = 64, BK = 64;
constexpr int kThreads = 256;
constexpr int LDW = BK / 4 + 1;  // words per smem row (+1 pad)

struct Params {
  const int8_t *a;
  const int8_t *b;
  const uint8_t *p4;
  void *out;
  const float *sa;
  const void *sw;
  const __half *bias;
  int64_t M, N, K;
  int gs;
  int epi;
  int sw_half;
  int vec_a, vec_b;  // 16-byte loads allowed
};

__device__ __forceinline__ float load_sw(const void *sw, int is_half, int64_t idx) {
  return is_half ? __half2float(reinterpret_cast<const __half *>(sw)[idx])
                 : reinterpret_cast<const float *>(sw)[idx];
}

__global__ void __launch_bounds__(kThreads) gemm_generic_kernel(Params p) {
  __shared__ uint32_t As[BM][LDW];
  __shared__ uint32_t Bs[BN][LDW];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int64_t m0 = (int64_t)blockIdx.y * BM, n0 = (int64_t)blockIdx.x * BN;

  int acc[4][4];
  float accf[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0;
      accf[i][j] = 0.0f;
    }

  const int lrow = tid >> 2;        // 0..63
  const int lseg = (tid & 3) * 16;  // byte offset in the 64-byte k slab

  for (int64_t k0 = 0; k0 < p.K; k0 += BK) {
    // ---- A tile: 64 rows x 64 bytes, 16 bytes per thread
    {
      const int64_t m = m0 + lrow;
      uint32_t v[4] = {0, 0, 0, 0};
      if (m < p.M) {
        const int8_t *src = p.a + m * p.K + k0 + lseg;
        if (p.vec_a && k0 + lseg + 16 <= p.K) {
          uint4 u = *reinterpret_cast<const uint4 *>(src);
          v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (k0 + lseg + i < p.K) v[i >> 2] |= (uint32_t)(uint8_t)src[i] << (8 * (i & 3));
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) As[lrow][lseg / 4 + i] = v[i];
    }
    // ---- B tile
    if (p.p4 == nullptr) {
      const int64_t n = n0 + lrow;
      uint32_t v[4] = {0, 0, 0, 0};
      if (n < p.N) {
        const int8_t *src = p.b + n * p.K + k0 + lseg;
        if (p.vec_b && k0 + lseg + 16 <= p.K) {
          uint4 u = *reinterpret_cast<const uint4 *>(src);
          v[0] = u.x; v[1] = u.y; v[2] = u.z; v[3] = u.w;
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (k0 + lseg + i < p.K) v[i >> 2] |= (uint32_t)(uint8_t)src[i] << (8 * (i & 3));
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) Bs[lrow][lseg / 4 + i] = v[i];
    } else {
      // packed int4: 32 k-pair rows x 64 columns of bytes; thread -> column
      // (tid & 63), k-pair rows (tid >> 6) * 8 .. +7; consecutive threads read
      // consecutive bytes of one packed row.
      const int nn = tid & 63;
      const int64_t n = n0 + nn;
      const int i0 = (tid >> 6) * 8;
      uint32_t v[4] = {0, 0, 0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t kp = k0 / 2 + i0 + i;
        if (n < p.N && 2 * kp < p.K) {
          const uint32_t byte = p.p4[kp * p.N + n];
          const uint32_t even = (uint32_t)(uint8_t)(int8_t)((int)(byte >> 4) - 8);
          const uint32_t odd = (uint32_t)(uint8_t)(int8_t)((int)(byte & 15u) - 8);
          // k = 2*(i0+i) and +1 -> bytes (2i, 2i+1) of this thread's 16-byte span
          v[i >> 1] |= (even | (odd << 8)) << (16 * (i & 1));
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) Bs[nn][i0 / 2 + i] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int kw = 0; kw < BK / 4; ++kw) {
      int av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = (int)As[ty * 4 + i][kw];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = (int)Bs[tx * 4 + j][kw];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
    if (p.epi == (int)Epi::kPerGroup && ((k0 + BK) % p.gs) == 0) {
      const int64_t g = k0 / p.gs;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int64_t n = n0 + tx * 4 + j;
        const float s = n < p.N ? load_sw(p.sw, p.sw_half, g * p.N + n) : 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          accf[i][j] = __fmaf_rn(__int2float_rn(acc[i][j]), s, accf[i][j]);
          acc[i][j] = 0;
        }
      }
    }
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    const float sam = p.epi == (int)Epi::kRawInt32 ? 0.0f : p.sa[m];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      if (p.epi == (int)Epi::kRawInt32) {
        reinterpret_cast<int32_t *>(p.out)[m * p.N + n] = acc[i][j];
      } else {
        const float b = p.bias ? __half2float(p.bias[n]) : 0.0f;
        float r;
        if (p.epi == (int)Epi::kPerChannel) {
          const float t = __fmul_rn(__int2float_rn(acc[i][j]), sam);
          r = __fmaf_rn(t, load_sw(p.sw, p.sw_half, n), b);
        } else {
          r = __fmaf_rn(accf[i][j], sam, b);
        }
        reinterpret_cast<__half *>(p.out)[m * p.N + n] = __float2half_rn(r);
      }
    }
  }
}

}  // namespace

int launch_gemm_generic(const GemmArgs &g, cudaStream_t st) {
  if (g.M == 0 || g.N == 0) return CIDER_OK;
  Params p;
  p.a = g.a; p.b = g.b; p.p4 = g.packed4; p.out = g.out; p.sa = g.sa; p.sw = g.sw;
  p.bias = g.bias; p.M = g.M; p.N = g.N; p.K = g.K; p.gs = g.gs > 0 ? g.gs : 1;
  p.epi = (int)g.epi; p.sw_half = g.sw_is_half;
  auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  p.vec_a = (g.K % 16 == 0) && a16(g.a);
  p.vec_b = g.b != nullptr && (g.K % 16 == 0) && a16(g.b);
  dim3 grid((unsigned)((g.N + BN - 1) / BN), (unsigned)((g.M + BM - 1) / BM));
  if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "gemm_generic: M too large for the plain kernel");
  gemm_generic_kernel<<<grid, kThreads, 0, st>>>(p);
  return check_cuda(cudaGetLastError(), "gemm_generic launch");
}

}  // namespace cider
