// Weight-streaming matrix products for a handful of activation rows: the M == 1
// decode path and the 2 <= M <= 16 (batched decode) path of the quantised linears.
//
//   M == 1: y[n] = sum_k W[n,k] * x[k] with int8 weights and an fp16 activation that
//   the reference does NOT quantise (csrc/src/w8a8_primitive.mm:157-178):
//     per-channel: half(fma(sw[n], dot, bias[n]))            (w8a8_int8_mv.metal:34-69)
//     per-group  : half(sum_g sw[g,n] * dot_g + bias[n])     (pergroup_int8_mv.metal:50-103)
//   2 <= M <= 16: int8 activations from the per-token quantiser, the epilogues of
//   the large-M kernels.
//
// Both are pure weight streaming (N*K bytes, every byte touched once), so one kernel
// shaped for HBM serves both: one CTA per SM, a producer warp that keeps a ring of
// ~40 KB shared-memory stages filled with bulk asynchronous copies, and eight
// compute warps that run the warp-level int8 tensor instruction on the stages.
// The fp16 activation of the M == 1 case reaches the integer instruction through an
// error-free style split into three int8 vectors (x = s1*q1 + s2*q2 + s3*q3 + r,
// |r| <= amax * 6.1e-8, s2 = s1/254, s3 = s2/254): the three are rows of the
// activation operand, their integer dot products are exact, and the epilogue
// recombines them in fp32.  The result differs from an fp32 dot product of the
// unquantised activation by less than fp32 summation-order noise; converting the
// int8 weights to floating point instead costs two instructions per weight byte
// and held the kernel at a third of the HBM rate.
#include <mutex>

#include "common.cuh"

namespace cider {
namespace {

constexpr int kWarps = 8;

// What the compute warps do to the M == 1 activation while they load it (the weights
// are already streaming): nothing, SwiGLU of a fused [gate | up] vector, or residual
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

// Where the activation rows come from: int8 rows + scales (already quantised), or
// one fp16 vector that the kernel splits itself.
struct StreamX {
  const int8_t *xq = nullptr;  // [M, K]
  const float *sa = nullptr;   // [M]
  const __half *x = nullptr;   // split mode: [K] ([2K] for the SwiGLU prologue)
  int split = 0;
  GemvPrologue pro;
};

__device__ __forceinline__ float sw_at(const void *sw, int is_half, int64_t idx) {
  return is_half ? __half2float(reinterpret_cast<const __half *>(sw)[idx])
                 : __ldg(reinterpret_cast<const float *>(sw) + idx);
}

// Two adjacent scales (even index) as raw bits - no conversion, so that nothing
// waits on the load where it is issued - and the conversion for the point of use.
__device__ __forceinline__ uint2 sw_raw2(const void *sw, int is_half, uint32_t idx) {
  if (is_half) return make_uint2(__ldg(reinterpret_cast<const uint32_t *>(sw) + (idx >> 1)), 0u);
  return __ldg(reinterpret_cast<const uint2 *>(sw) + (idx >> 1));
}
__device__ __forceinline__ float2 sw_cvt2(uint2 raw, int is_half) {
  if (is_half) return __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
  return make_float2(__uint_as_float(raw.x), __uint_as_float(raw.y));
}
// int32 -> fp32 for |v| < 2^22 without the conversion unit (a quarter-rate pipe):
// v + 0x4B400000 is the bit pattern of 12582912.0f + v.
__device__ __forceinline__ float small_int_to_float(int v) {
  return __int_as_float(v + 0x4B400000) - 12582912.0f;
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

// D(16x8, int32) += A(16x32, int8, row) * B(32x8, int8, col)
__device__ __forceinline__ void mma_s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kStageRows = 16;   // weight rows per stage: two 8-row tiles
constexpr int kMaxBlocks = 5;    // 64-byte blocks per warp and slice (slices are <= 2560 bytes)
constexpr int kMaxSlice = 2560;

// Row strides in shared memory are 64 mod 128 bytes: lane (g, t) of a warp reads 16
// bytes at t*16 of row g, and the eight lanes of a quarter warp (two rows) then
// cover all 32 banks.
__host__ __device__ inline int pad_stride(int bytes) { return bytes + ((bytes % 128) == 0 ? 64 : 0); }
// Packed int4 weight rows (two weights per byte) are read 8 bytes per lane, a half
// warp covering four rows of 32 bytes: their stride is 32 mod 64 bytes.
__host__ __device__ inline int pad_stride_w4(int bytes) { return bytes + ((bytes % 64) == 32 ? 0 : 32); }

// Eight packed bytes (high nibble = even k, value + 8, as the reference packs them)
// -> four words of signed int8: even and odd k of the first and of the second
// four bytes.  t = n ^ 8 is the 4-bit two's complement of n - 8; its sign bit times
// 0x1E fills the high nibble (0x08 * 0x1E = 0xF0 stays inside the byte).
__device__ __forceinline__ uint32_t nibbles_to_s8(uint32_t n) {
  const uint32_t t = (n & 0x0F0F0F0Fu) ^ 0x08080808u;
  return t | ((t & 0x08080808u) * 0x1Eu);
}
__device__ __forceinline__ uint4 unpack_w4_words(uint2 p) {
  return make_uint4(nibbles_to_s8(p.x >> 4), nibbles_to_s8(p.x), nibbles_to_s8(p.y >> 4), nibbles_to_s8(p.y));
}

// sum (or max) over the 256 compute threads; every thread gets the result
__device__ __forceinline__ float compute_warps_reduce(float v, bool is_max, float *sred, int warp, int lane) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float u = __shfl_xor_sync(0xffffffffu, v, o);
    v = is_max ? fmaxf(v, u) : v + u;
  }
  if (lane == 0) sred[warp] = v;
  group_barrier(15, kWarps * 32);
  float r = sred[0];
#pragma unroll
  for (int i = 1; i < kWarps; ++i) r = is_max ? fmaxf(r, sred[i]) : r + sred[i];
  group_barrier(15, kWarps * 32);  // sred may be written again
  return r;
}

// One kernel for both cases.  Work split:
//   CTA    = a contiguous range of 8-row weight tiles (N/8 tiles over the grid, so
//            the CTAs differ by at most one tile);
//   stage  = two consecutive tiles (16 weight rows) x one K-slice of KS <= 2560
//            bytes: one bulk copy per row (issued by 16 lanes of the producer warp
//            at once), rows padded to a conflict-free stride;
//   warp w = a contiguous range of the slice's 64-byte blocks, for both tiles.
// For a block, lane (g = lane/4, t = lane%4) loads 16 bytes at t*16 of weight row g
// of each tile and of activation row g (and g+8 when MR == 16): the four words are
// the k-quarters of two m16n8k32 instructions whose 16-row operand holds the
// ACTIVATION rows and whose 8-column operand the weight rows.  The instruction's own
// k order is permuted by this, identically for both operands, which a dot product
// does not see.
//   per-channel: int32 accumulators over the whole K, summed across the eight warps
//            in shared memory, then half(fma(float(acc)*sa[m], sw[n], bias[n])) -
//            bit-identical to the tensor-core path;
//   per-group:   a block lies in one K-group (gs % 64 == 0): its int32 result is
//            converted and scaled at once, accf += float(part) * sw[g,n]; the fp32
//            partials of the eight warps are then added.  The fp32 summation order
//            therefore differs from the ascending-group order of the large-M kernels
//            (~1e-6 relative, far inside the 2e-3 bar of the fp16 output);
//   split (M == 1): activation rows 0..2 are the three int8 terms of the fp16
//            vector; out = s1*R0 + s2*R1 + s3*R2 replaces float(acc)*sa.
//   kW4:    the weight rows are packed int4, [N, K/2] bytes.  A lane loads 8 bytes (16
//            weights) per row and block and expands them in registers into the
//            even-k and odd-k words; the activation rows are staged with the same
//            even / odd split inside every 8 bytes, so the operands still agree.
// kGroup: 0 per-channel scales; 1 per-group, every 64-wide block of K promoted by itself; 2 per-group with
// gs >= 128 and every warp's block range made of whole pairs: the int32 sums of the two blocks of a pair
// (one group) are promoted together.  kMulti: K walked in parts (kparts > 1)
template <int MR, int kGroup, bool kW4, bool kMulti = false>
__global__ void __launch_bounds__((kWarps + 1) * 32, 1)
stream_mm_kernel(const StreamX xa, const int8_t *__restrict__ w, const void *__restrict__ sw, int sw_half, int gs,
                 const __half *__restrict__ bias, __half *__restrict__ y, int M, int N, int K, int KS,
                 int stages, int kparts_arg) {
  const int kparts = kMulti ? kparts_arg : 1;
  constexpr int NT = MR / 8;  // halves (rows g / g+8) of the activation operand in use
  constexpr int CT = 2 * NT;  // results per lane and tile
  constexpr int CP = 2 * CT;  // ... and stage
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full_bar[16], empty_bar[16];
  __shared__ float sred[kWarps];
  __shared__ int abort_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int xrows = xa.split ? 3 : M;
  // kparts > 1 (several activation rows and a long K): K is walked in kparts equal parts, the
  // CTA's weight tiles once per part, with only that part of the activations staged - the
  // ring then gets the shared memory the full rows would take; partial sums per tile wait in
  // shared memory between the parts
  const int KP = K / kparts;
  const int KSP = kW4 ? pad_stride_w4(KS >> 1) : pad_stride(KS), XP = pad_stride(KP);
  const int wshift = kW4 ? 1 : 0;  // weight bytes per k: 1 >> wshift
  const uint32_t stage_bytes = (uint32_t)kStageRows * (uint32_t)KSP;
  const int tiles = (N + 7) / 8;
  const int t_begin = (int)((int64_t)blockIdx.x * tiles / gridDim.x);
  const int t_end = (int)((int64_t)(blockIdx.x + 1) * tiles / gridDim.x);
  const int row_end = min(t_end * 8, N);
  const int pairs = (t_end - t_begin + 1) / 2;
  const int ns = (KP + KS - 1) / KS;  // slices per pair of tiles (and part of K)
  const int iters = kparts * pairs * ns;

  pdl_launch_dependents();
  if (threadIdx.x < stages) {
    mbar_init(smem_u32(&full_bar[threadIdx.x]), 1);
    mbar_init(smem_u32(&empty_bar[threadIdx.x]), kWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 32) abort_s = 0;
  __syncthreads();
  uint8_t *x_s = ring + (size_t)stages * stage_bytes;             // [xrows][XP] int8
  int *red = reinterpret_cast<int *>(x_s + (size_t)xrows * XP);  // [2][kWarps][32 * CP]
  int *part_s = red + 2 * kWarps * 32 * CP;                       // kparts > 1: [pairs][kStageRows * MR]

  if (warp == kWarps) {  // ---------------------------- producer warp: lane r copies row r
    int stage = 0, issued = 0, p = 0, sl = 0, kpart = 0;
    uint32_t phase = 0;
    for (int it = 0; it < iters; ++it) {
      uint32_t got = 0;
      if (lane == 0) got = mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, &abort_s);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      const int n0 = (t_begin + 2 * p) * 8, k0 = kpart * KP + sl * KS;
      const int len = min(KS, KP - sl * KS), rows = min(kStageRows, row_end - n0);
      if (++sl == ns) {
        sl = 0;
        if (++p == pairs && kMulti) {
          p = 0;
          ++kpart;
        }
      }
      const uint32_t fb = smem_u32(&full_bar[stage]);
      if (lane == 0) mbar_expect_tx(fb, (uint32_t)rows * (uint32_t)(len >> wshift));
      __syncwarp();
      if (lane < rows)
        bulk_load(smem_u32(ring + (size_t)stage * stage_bytes + (size_t)lane * KSP),
                  w + (((int64_t)(n0 + lane) * K + k0) >> wshift), (uint32_t)(len >> wshift), fb);
      ++issued;
      if (++stage == stages) {
        stage = 0;
        phase ^= 1u;
      }
    }
    if (lane == 0 && abort_s) {  // copies in flight must land before the CTA's shared memory goes away
      const int last = issued < stages ? issued : stages;
      for (int i = 0; i < last; ++i) {
        const int f = issued - 1 - i;
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(&full_bar[f % stages]), (uint32_t)(f / stages) & 1u) &&
               clock64() - t0 < kWaitCycles) {
        }
      }
    }
    return;
  }

  // ------------------------------------------------------------ compute warps
  // Everything above reads weights only.  The activation (and every write) waits
  // for the kernels this one depends on - but the RMSNorm weight of the add+norm
  // prologue is static too: this thread's first two chunks of it are requested
  // before the wait, which takes one global-memory round trip off the prologue.
  uint4 nw_pre[2] = {make_uint4(0, 0, 0, 0), make_uint4(0, 0, 0, 0)};
  if (xa.split && xa.pro.mode == kPrologueAddNorm) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + i * kWarps * 32;
      if (c < (K >> 3)) nw_pre[i] = __ldg(reinterpret_cast<const uint4 *>(xa.pro.norm_w) + c);
    }
  }
  pdl_wait();
  float s_split[3] = {0.0f, 0.0f, 0.0f};
  if (xa.split) {
    // fp16 activation -> prologue -> three int8 terms.  Each thread keeps its 8-element
    // chunks in a shared-memory scratch row between the passes (it only ever reads
    // back what it wrote itself).
    uint4 *tmp = reinterpret_cast<uint4 *>(red + 2 * kWarps * 32 * CP);
    const GemvPrologue &pro = xa.pro;
    const int chunks = K >> 3;
    float amax = 0.0f, ss = 0.0f;
    for (int c = threadIdx.x; c < chunks; c += kWarps * 32) {
      uint4 h = __ldg(reinterpret_cast<const uint4 *>(xa.x) + c);
      __half2 *h2 = reinterpret_cast<__half2 *>(&h);
      if (pro.mode == kPrologueSiluMul) {
        // x = [gate | up] of length 2K: activation = half(half(silu(g)) * u)
        const uint4 u = __ldg(reinterpret_cast<const uint4 *>(xa.x + K) + c);
        const __half2 *u2 = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 gt = __half22float2(h2[j]), uu = __half22float2(u2[j]);
          const float s0 = silu_to_half(gt.x);
          const float s1 = silu_to_half(gt.y);
          h2[j] = __floats2half2_rn(s0 * uu.x, s1 * uu.y);
        }
      } else if (pro.mode == kPrologueAddNorm) {
        if (pro.delta != nullptr) {
          const uint4 d = __ldg(reinterpret_cast<const uint4 *>(pro.delta) + c);
          const __half2 *d2 = reinterpret_cast<const __half2 *>(&d);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 a = __half22float2(h2[j]), b = __half22float2(d2[j]);
            h2[j] = __floats2half2_rn(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y));
          }
        }
        if (blockIdx.x == 0 && pro.x_out != nullptr)  // one CTA publishes the new residual
          reinterpret_cast<uint4 *>(pro.x_out)[c] = h;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h2[j]);
          ss = fmaf(f.x, f.x, ss);
          ss = fmaf(f.y, f.y, ss);
        }
      }
      if (pro.mode != kPrologueAddNorm) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h2[j]);
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
      tmp[c] = h;
    }
    if (pro.mode == kPrologueAddNorm) {
      // RMSNorm of the full activation, n = half(v * r * w) like the stand-alone kernel
      ss = compute_warps_reduce(ss, false, sred, warp, lane);
      const float r = 1.0f / sqrtf(ss / (float)K + pro.eps);
      for (int c = threadIdx.x, ci = 0; c < chunks; c += kWarps * 32, ++ci) {
        uint4 h = tmp[c];
        __half2 *h2 = reinterpret_cast<__half2 *>(&h);
        const uint4 nw = ci == 0 ? nw_pre[0]
                                 : (ci == 1 ? nw_pre[1] : __ldg(reinterpret_cast<const uint4 *>(pro.norm_w) + c));
        const __half2 *w2 = reinterpret_cast<const __half2 *>(&nw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 v = __half22float2(h2[j]), gw = __half22float2(w2[j]);
          h2[j] = __floats2half2_rn(__fmul_rn(__fmul_rn(v.x, r), gw.x), __fmul_rn(__fmul_rn(v.y, r), gw.y));
          const float2 f = __half22float2(h2[j]);
          amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
        tmp[c] = h;
      }
    }
    amax = compute_warps_reduce(amax, true, sred, warp, lane);
    const float s1 = amax > 0.0f ? amax / 127.0f : 1.0f;
    const float s2 = s1 / 254.0f, s3 = s2 / 254.0f;
    const float i1 = 1.0f / s1, i2 = 1.0f / s2, i3 = 1.0f / s3;
    s_split[0] = s1;
    s_split[1] = s2;
    s_split[2] = s3;
    for (int c = threadIdx.x; c < chunks; c += kWarps * 32) {
      const uint4 h = tmp[c];
      const __half *hv = reinterpret_cast<const __half *>(&h);
      // round-to-nearest through the fp32 magic number 1.5 * 2^23: the sum's low
      // mantissa byte is the two's-complement int8, and sum - magic the rounded value.
      // |v| <= amax and |residual| <= (previous scale) / 2 keep every term within
      // +-127 (a half-ulp excess rounds to +-127 as well), so nothing needs clamping.
      const float magic = 12582912.0f;
      uint32_t q[3][2] = {{0, 0}, {0, 0}, {0, 0}};
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float v = __half2float(hv[j]);
        const float t1 = fmaf(v, i1, magic);
        const float r1 = fmaf(-(t1 - magic), s1, v);
        const float t2 = fmaf(r1, i2, magic);
        const float r2 = fmaf(-(t2 - magic), s2, r1);
        const float t3 = fmaf(r2, i3, magic);
        q[0][j >> 2] |= (__float_as_uint(t1) & 0xffu) << (8 * (j & 3));
        q[1][j >> 2] |= (__float_as_uint(t2) & 0xffu) << (8 * (j & 3));
        q[2][j >> 2] |= (__float_as_uint(t3) & 0xffu) << (8 * (j & 3));
      }
#pragma unroll
      for (int r = 0; r < 3; ++r)
        *reinterpret_cast<uint2 *>(x_s + (size_t)r * XP + (size_t)c * 8) = make_uint2(q[r][0], q[r][1]);
    }
  }
  // the quantised activation rows of one part of K into shared memory
  auto stage_x = [&](int kpart) {
    const int chunks = KP >> 4;
    for (int i = threadIdx.x; i < xrows * chunks; i += kWarps * 32) {
      const int m = i / chunks, c = i % chunks;
      uint4 v = __ldg(reinterpret_cast<const uint4 *>(xa.xq + (int64_t)m * K + (int64_t)kpart * KP) + c);
      if constexpr (kW4)  // every 8 bytes: even k first, then odd k
        v = make_uint4(__byte_perm(v.x, v.y, 0x6420), __byte_perm(v.x, v.y, 0x7531),
                       __byte_perm(v.z, v.w, 0x6420), __byte_perm(v.z, v.w, 0x7531));
      *reinterpret_cast<uint4 *>(x_s + (size_t)m * XP + (size_t)c * 16) = v;
    }
  };
  if (!xa.split) stage_x(0);
  group_barrier(15, kWarps * 32);

  const int g = lane >> 2, t = lane & 3;
  // the output element this thread finishes after the cross-warp sum: activation row
  // em, weight row enl of the stage (tile enl/8, column enl%8 of that tile)
  const int em = threadIdx.x / kStageRows, enl = threadIdx.x % kStageRows;
  const int etile = enl >> 3, enn = enl & 7;
  const bool e_live = xa.split ? threadIdx.x < kStageRows : (threadIdx.x < kStageRows * MR && em < M);
  const float e_sa = (!xa.split && e_live) ? __ldg(xa.sa + em) : 0.0f;
  float e_sw = 0.0f, e_bias = 0.0f;

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  int acc[2][4], acc2[2][4];  // two accumulator sets (even / odd blocks): shorter dependency chains
  float accf[2][4];
  // group scales of one iteration's blocks of this warp, as raw bits: sc[j][tile] holds
  // those of block j for weight rows 2t, 2t+1 of the tile (N % 8 == 0, so the pair is
  // aligned and inside the matrix whenever its tile is).  Requested one iteration
  // ahead.  gs / 64 is a power of two: the group of a block is a shift.
  uint2 sc[kMaxBlocks][2], sc_next[kMaxBlocks][2];
  const int gshift = 31 - __clz(gs > 0 ? gs >> 6 : 1);
  auto load_scales = [&](uint2(&dst)[kMaxBlocks][2], int kp, int pp, int ss) {
    const int n0 = (t_begin + 2 * pp) * 8, k0 = kp * KP + ss * KS;
    const int nb = min(KS, KP - ss * KS) >> 6;
    const int b0 = warp * nb / kWarps;
    const uint32_t c0 = (uint32_t)(n0 + 2 * t);
    const uint32_t c1 = n0 + 8 < N ? c0 + 8u : c0;  // a tile past the matrix: any valid address
#pragma unroll
    for (int j = 0; j < kMaxBlocks; ++j) {
      const uint32_t row = (uint32_t)(((k0 >> 6) + min(b0 + j, nb - 1)) >> gshift) * (uint32_t)N;
      dst[j][0] = sw_raw2(sw, sw_half, row + c0);
      dst[j][1] = sw_raw2(sw, sw_half, row + c1);
    }
  };
  if constexpr (kGroup) {
    if (iters > 0) load_scales(sc_next, 0, 0, 0);
  }
  int p = 0, sl = 0, kpart = 0, done = 0;  // done: finished (pair, part) units - alternates the reduction buffer
  for (int it = 0; it < iters; ++it) {
    if (it > 0) {  // advance (part, pair, slice), the slice running fastest
      if (++sl == ns) {
        sl = 0;
        if constexpr (kMulti) {
          if (++p == pairs) {
            p = 0;
            ++kpart;
            // the next part of K: every warp has finished reading the previous one
            group_barrier(15, kWarps * 32);
            stage_x(kpart);
            group_barrier(15, kWarps * 32);
          }
        } else {
          ++p;
        }
      }
    }
    const int n0 = (t_begin + 2 * p) * 8, kx = sl * KS, k0 = kpart * KP + kx;
    const int len = min(KS, KP - kx), nb = len >> 6;
    const int b0 = warp * nb / kWarps, b1 = (warp + 1) * nb / kWarps;
    if (sl == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        acc[i >> 2][i & 3] = 0;
        acc2[i >> 2][i & 3] = 0;
        accf[i >> 2][i & 3] = 0.0f;
      }
      if (e_live) {  // row constants of this stage's epilogue, in flight while it streams
        const int n = min(n0 + enl, N - 1);
        e_sw = kGroup ? 0.0f : sw_at(sw, sw_half, n);
        e_bias = bias ? __half2float(bias[n]) : 0.0f;
      }
    }
    if constexpr (kGroup) {
#pragma unroll
      for (int j = 0; j < kMaxBlocks; ++j) {
        sc[j][0] = sc_next[j][0];
        sc[j][1] = sc_next[j][1];
      }
      if (it + 1 < iters) {
        const bool wrap = sl + 1 == ns, pwrap = wrap && p + 1 == pairs;
        load_scales(sc_next, pwrap ? kpart + 1 : kpart, pwrap ? 0 : (wrap ? p + 1 : p), wrap ? 0 : sl + 1);
      }
    }
    if (ok) {
      uint32_t got = 0;
      if (lane == 0) got = mbar_wait(smem_u32(&full_bar[stage]), phase, &abort_s);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) ok = false;  // no early exit: the other warps still meet this one at the barrier below
    }
    if (ok) {
      const uint8_t *wa = ring + (size_t)stage * stage_bytes + (size_t)g * KSP + t * (kW4 ? 8 : 16);
      const uint8_t *xp = x_s + (size_t)g * XP + kx + t * 16;
      // all of this warp's fragments first (a block past the warp's range re-reads the
      // first one with a zero activation), then the arithmetic
      uint4 w0[kMaxBlocks], w1[kMaxBlocks], x0[kMaxBlocks], x1[kMaxBlocks];
#pragma unroll
      for (int j = 0; j < kMaxBlocks; ++j) {
        const bool live = b0 + j < b1;
        const int off = (live ? b0 + j : b0) * 64;
        if constexpr (kW4) {
          w0[j] = unpack_w4_words(*reinterpret_cast<const uint2 *>(wa + (off >> 1)));
          w1[j] = unpack_w4_words(*reinterpret_cast<const uint2 *>(wa + 8 * KSP + (off >> 1)));
        } else {
          w0[j] = *reinterpret_cast<const uint4 *>(wa + off);
          w1[j] = *reinterpret_cast<const uint4 *>(wa + 8 * KSP + off);
        }
        x0[j] = make_uint4(0, 0, 0, 0);
        x1[j] = make_uint4(0, 0, 0, 0);
        if (live && g < xrows) x0[j] = *reinterpret_cast<const uint4 *>(xp + off);
        if (MR == 16 && live && g + 8 < xrows) x1[j] = *reinterpret_cast<const uint4 *>(xp + (size_t)8 * XP + off);
      }
      int c0[4], c1[4];  // per-group: the int32 sums of the block (or pair of blocks) being worked on
#pragma unroll
      for (int j = 0; j < kMaxBlocks; ++j) {
        if constexpr (kGroup != 0) {
          if (kGroup == 1 || (j & 1) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              c0[i] = 0;
              c1[i] = 0;
            }
          }
          mma_s8(c0, x0[j].x, x1[j].x, x0[j].y, x1[j].y, w0[j].x, w0[j].y);
          mma_s8(c1, x0[j].x, x1[j].x, x0[j].y, x1[j].y, w1[j].x, w1[j].y);
          mma_s8(c0, x0[j].z, x1[j].z, x0[j].w, x1[j].w, w0[j].z, w0[j].w);
          mma_s8(c1, x0[j].z, x1[j].z, x0[j].w, x1[j].w, w1[j].z, w1[j].w);
          if (kGroup == 1 || (j & 1) == 1 || j == kMaxBlocks - 1) {  // resolved at compile time
            const float2 s0 = sw_cvt2(sc[j][0], sw_half), s1 = sw_cvt2(sc[j][1], sw_half);
#pragma unroll
            for (int i = 0; i < CT; ++i) {
              accf[0][i] = fmaf(small_int_to_float(c0[i]), (i & 1) ? s0.y : s0.x, accf[0][i]);
              accf[1][i] = fmaf(small_int_to_float(c1[i]), (i & 1) ? s1.y : s1.x, accf[1][i]);
            }
          }
        } else {
          int(&a0)[4] = (j & 1) ? acc2[0] : acc[0];
          int(&a1)[4] = (j & 1) ? acc2[1] : acc[1];
          mma_s8(a0, x0[j].x, x1[j].x, x0[j].y, x1[j].y, w0[j].x, w0[j].y);
          mma_s8(a1, x0[j].x, x1[j].x, x0[j].y, x1[j].y, w1[j].x, w1[j].y);
          mma_s8(a0, x0[j].z, x1[j].z, x0[j].w, x1[j].w, w0[j].z, w0[j].w);
          mma_s8(a1, x0[j].z, x1[j].z, x0[j].w, x1[j].w, w1[j].z, w1[j].w);
        }
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&empty_bar[stage]));
    if (++stage == stages) {
      stage = 0;
      phase ^= 1u;
    }
    if (sl == ns - 1) {  // both tiles done: add the eight warps' partial results and store
      int *mine = red + (((size_t)(done & 1) * kWarps + warp) * 32 + lane) * CP;
#pragma unroll
      for (int i = 0; i < CT; ++i) {
        mine[i] = kGroup ? __float_as_int(accf[0][i]) : acc[0][i] + acc2[0][i];
        mine[CT + i] = kGroup ? __float_as_int(accf[1][i]) : acc[1][i] + acc2[1][i];
      }
      group_barrier(15, kWarps * 32);
      if (e_live) {
        const int *base = red + (size_t)(done & 1) * kWarps * 32 * CP;
        const int n = n0 + enl;
        float v;
        if (xa.split) {
          float r[3];
#pragma unroll
          for (int mm = 0; mm < 3; ++mm) {
            const int *src = base + (mm * 4 + (enn >> 1)) * CP + etile * CT + (enn & 1);
            int si = 0;
            float sf = 0.0f;
#pragma unroll
            for (int ww = 0; ww < kWarps; ++ww) {
              if constexpr (kGroup) sf += __int_as_float(src[ww * 32 * CP]);
              else si += src[ww * 32 * CP];
            }
            r[mm] = kGroup ? sf : __int2float_rn(si);
          }
          const float dot = fmaf(s_split[2], r[2], fmaf(s_split[1], r[1], __fmul_rn(s_split[0], r[0])));
          v = kGroup ? __fadd_rn(dot, e_bias) : __fmaf_rn(e_sw, dot, e_bias);
        } else {
          const int *src = base + ((em & 7) * 4 + (enn >> 1)) * CP + etile * CT + (em >> 3) * 2 + (enn & 1);
          int si = 0;
          float sf = 0.0f;
#pragma unroll
          for (int ww = 0; ww < kWarps; ++ww) {
            if constexpr (kGroup) sf += __int_as_float(src[ww * 32 * CP]);
            else si += src[ww * 32 * CP];
          }
          if constexpr (kMulti) {  // sums of the parts of K meet here (this thread owns the slot)
            int *slot = part_s + (size_t)p * (kStageRows * MR) + threadIdx.x;
            if (kpart > 0) {
              if constexpr (kGroup) sf += __int_as_float(*slot);
              else si += *slot;
            }
            *slot = kGroup ? __float_as_int(sf) : si;
          }
          v = kGroup ? __fmaf_rn(sf, e_sa, e_bias) : __fmaf_rn(__fmul_rn(__int2float_rn(si), e_sa), e_sw, e_bias);
        }
        if (ok && n < row_end && kpart == kparts - 1) y[(int64_t)em * N + n] = __float2half_rn(v);
      }
      ++done;
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

// Byte transpose [K/2, N] -> [N, K/2]: the reference's packed int4 layout (N
// contiguous) into weight rows that can be streamed (K contiguous).  128 x 128 byte
// tiles through shared memory: 16-byte loads along N (a row of the tile is one 128-byte
// line), then every group of 8 lanes writes one 128-byte line of an output row, each lane 16
// bytes gathered down a column of the tile.  Needs N % 16 == 0, (K/2) % 16 == 0 and 16-byte
// aligned buffers; repack_w4_small_kernel takes the other shapes.
// (16-byte chunks of a tile row are XOR-swizzled by row / 16, so that the 8 lanes that gather one
// output line - rows 16 apart, the same column - read 8 different banks)
constexpr int kRepackTile = 128;
__global__ void __launch_bounds__(256)
repack_w4_kernel(const uint8_t *__restrict__ packed, uint8_t *__restrict__ out, int N, int KP) {
  __shared__ __align__(16) uint8_t tile[kRepackTile][kRepackTile];
  pdl_launch_dependents();
  pdl_wait();
  const int n0 = blockIdx.x * kRepackTile, k0 = blockIdx.y * kRepackTile;
  const int tid = threadIdx.x;
  {
    const int c = (tid & 7) * 16, r0 = tid >> 3;  // 8 threads per tile row, 32 rows per pass
#pragma unroll
    for (int pass = 0; pass < kRepackTile / 32; ++pass) {
      const int r = r0 + pass * 32;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (k0 + r < KP && n0 + c < N) v = __ldg(reinterpret_cast<const uint4 *>(packed + (int64_t)(k0 + r) * N + n0 + c));
      *reinterpret_cast<uint4 *>(&tile[r][(((c >> 4) ^ ((r >> 4) & 7)) << 4)]) = v;
    }
  }
  __syncthreads();
  {
    const int seg = (tid & 7) * 16, nr0 = tid >> 3;  // 8 threads per output row, 32 output rows per pass
#pragma unroll
    for (int pass = 0; pass < kRepackTile / 32; ++pass) {
      const int nr = nr0 + pass * 32;
      if (n0 + nr >= N || k0 + seg >= KP) continue;
      uint32_t w[4];
      const int col = ((((nr >> 4) ^ ((seg >> 4) & 7)) << 4)) + (nr & 15);  // rows seg .. seg + 15 share row / 16
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        w[j] = (uint32_t)tile[seg + 4 * j][col] | ((uint32_t)tile[seg + 4 * j + 1][col] << 8) |
               ((uint32_t)tile[seg + 4 * j + 2][col] << 16) | ((uint32_t)tile[seg + 4 * j + 3][col] << 24);
      }
      *reinterpret_cast<uint4 *>(out + (int64_t)(n0 + nr) * KP + k0 + seg) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// the same for any N and K/2: 32 x 32 byte tiles, one byte per access
__global__ void __launch_bounds__(256)
repack_w4_small_kernel(const uint8_t *__restrict__ packed, uint8_t *__restrict__ out, int N, int KP) {
  __shared__ uint8_t tile[32][33];
  const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
#pragma unroll
  for (int r = ty; r < 32; r += 8)
    if (k0 + r < KP && n0 + tx < N) tile[r][tx] = packed[(int64_t)(k0 + r) * N + n0 + tx];
  __syncthreads();
#pragma unroll
  for (int r = ty; r < 32; r += 8)
    if (n0 + r < N && k0 + tx < KP) out[(int64_t)(n0 + r) * KP + k0 + tx] = tile[tx][r];
}

// [N, K/2] packed int4 -> [N, K] int8: a thread expands 8 bytes into 16.
__global__ void __launch_bounds__(256)
unpack_w4_nk_kernel(const uint8_t *__restrict__ w4, int8_t *__restrict__ w, int64_t total8) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8;
       i += (int64_t)gridDim.x * blockDim.x) {
    const uint2 p = __ldg(reinterpret_cast<const uint2 *>(w4) + i);
    const uint4 e = unpack_w4_words(p);  // (even, odd) k of bytes 0-3, then of bytes 4-7
    // interleave back to ascending k
    reinterpret_cast<uint4 *>(w)[i] =
        make_uint4(__byte_perm(e.x, e.y, 0x5140), __byte_perm(e.x, e.y, 0x7362), __byte_perm(e.z, e.w, 0x5140),
                   __byte_perm(e.z, e.w, 0x7362));
  }
}

}  // namespace

// Shared-memory plan of the streaming kernel for `xrows` activation rows of length
// K: the K-slice, the ring depth and the grid.  ok == false when even two stages of
// the smallest slice do not fit.
namespace {
struct StreamPlan {
  bool ok = false;
  int ks = 0, stages = 0, grid = 0, kparts = 1;
  size_t smem = 0;
};
constexpr size_t kStreamSmem = 200 * 1024;

StreamPlan plan_stream(int xrows, int mr, int64_t N, int64_t K, bool split, bool w4 = false) {
  constexpr size_t smem_cap = kStreamSmem;
  StreamPlan p;
  const int cp = 4 * (mr / 8);
  const int64_t tiles = (N + 7) / 8;
  int64_t grid = sm_count(current_device());
  if (grid > (tiles + 1) / 2) grid = (tiles + 1) / 2;
  // Several activation rows and a long K: the staged rows would take the shared memory the ring
  // needs (8 x 12288 bytes: half of it, and the kernel streamed at 2.1 TB/s where shorter rows reach
  // 4.3).  K is then walked in equal parts with only one part of the rows staged; the partial sums
  // of a CTA's tile pairs wait in shared memory between the parts, so only when those are few.
  const int64_t pairs_per_cta = ((tiles + grid - 1) / grid + 1) / 2 + 1;
  int kparts = 1;
  if (!split)
    while (kparts < 8 && (size_t)xrows * pad_stride((int)(K / kparts)) > 64 * 1024 && pairs_per_cta <= 16 &&
           K % (2 * kparts * 64) == 0)
      kparts *= 2;
  const int64_t KP = K / kparts;
  const size_t fixed = (size_t)xrows * pad_stride((int)KP) + (size_t)2 * kWarps * 32 * cp * sizeof(int) +
                       (split ? (size_t)2 * K : 0) +
                       (kparts > 1 ? (size_t)pairs_per_cta * kStageRows * mr * sizeof(int) : 0);
  const int64_t ns = (KP + kMaxSlice - 1) / kMaxSlice;
  int ks = (int)(((KP + ns - 1) / ns + 63) / 64 * 64);
  auto stage = [w4](int s) { return (size_t)kStageRows * (w4 ? pad_stride_w4(s >> 1) : pad_stride(s)); };
  // (asking for four stages of shorter slices instead of three was measured: M = 1 over
  // [2560, 10240] went from 10.9 to 15.2 us - more, shorter row copies cost more than the deeper
  // ring gains)
  while (fixed + 3 * stage(ks) > smem_cap && ks > 512) ks = (ks / 2 + 63) / 64 * 64;
  if (fixed + 2 * stage(ks) > smem_cap) return p;
  p.ok = true;
  p.ks = ks;
  p.kparts = kparts;
  p.stages = (int)((smem_cap - fixed) / stage(ks));
  if (p.stages > 16) p.stages = 16;
  p.smem = fixed + (size_t)p.stages * stage(ks);
  p.grid = (int)grid;
  return p;
}

bool stream_shape_ok(int64_t N, int64_t K, int gs, const void *w, const void *sw) {
  if (N < 1 || N >= (1 << 27) || K < 64 || (K % 64) != 0 || K >= (1 << 24)) return false;
  if (reinterpret_cast<uintptr_t>(w) & 15u) return false;
  if (gs == 0) return true;
  // per-group: groups of 64 * 2^i, scale pairs aligned and indexable in 32 bits
  return gs >= 64 && (gs & (gs - 1)) == 0 && (N % 8) == 0 && (K / gs) * N < (int64_t(1) << 31) &&
         (reinterpret_cast<uintptr_t>(sw) & 7u) == 0;
}

int launch_stream(const StreamX &xa, int mr, const StreamPlan &p, const int8_t *w, const void *sw, int sw_is_half,
                  int gs, const __half *bias, __half *y, int M, int64_t N, int64_t K, cudaStream_t st,
                  bool w4 = false) {
#define CIDER_STREAM_LAUNCH(MRV, G)                                                                        \
  do {                                                                                                     \
    if (w4) CIDER_STREAM_LAUNCH_W(MRV, G, true);                                                           \
    else CIDER_STREAM_LAUNCH_W(MRV, G, false);                                                             \
  } while (0)
#define CIDER_STREAM_LAUNCH_W(MRV, G, W4)                                                                  \
  do {                                                                                                     \
    if (p.kparts > 1) CIDER_STREAM_LAUNCH_K(MRV, G, W4, true);                                             \
    else CIDER_STREAM_LAUNCH_K(MRV, G, W4, false);                                                         \
  } while (0)
#define CIDER_STREAM_LAUNCH_K(MRV, G, W4, KM)                                                              \
  do {                                                                                                     \
    auto kern = stream_mm_kernel<MRV, G, W4, KM>;                                                          \
    static std::atomic<unsigned long long> done{0};                                                        \
    int arc = ensure_dynamic_smem(kern, (int)kStreamSmem, done, "streaming GEMM shared-memory attribute"); \
    if (arc) return arc;                                                                                   \
    cudaError_t le = launch_kernel(kern, dim3((unsigned)p.grid), dim3((kWarps + 1) * 32), p.smem, st, xa,  \
                                   w, sw, sw_is_half, gs, bias, y, M, (int)N, (int)K, p.ks, p.stages,      \
                                   p.kparts);                                                              \
    if (le != cudaSuccess) return check_cuda(le, "streaming GEMM launch");                                 \
  } while (0)
  // pairs of blocks promoted together: groups of 128 and more, slices of whole 1024s (every warp's
  // range then is an even number of blocks starting at an even block) and no short last slice
  const bool paired = gs >= 128 && p.ks % 1024 == 0 && (K / p.kparts) % p.ks == 0;
  if (mr == 8) {
    if (gs > 0 && paired) CIDER_STREAM_LAUNCH(8, 2);
    else if (gs > 0) CIDER_STREAM_LAUNCH(8, 1);
    else CIDER_STREAM_LAUNCH(8, 0);
  } else {
    if (gs > 0 && paired) CIDER_STREAM_LAUNCH(16, 2);
    else if (gs > 0) CIDER_STREAM_LAUNCH(16, 1);
    else CIDER_STREAM_LAUNCH(16, 0);
  }
#undef CIDER_STREAM_LAUNCH
#undef CIDER_STREAM_LAUNCH_W
#undef CIDER_STREAM_LAUNCH_K
  return check_cuda(cudaGetLastError(), "streaming GEMM launch");
}
}  // namespace

static int launch_gemv_impl(const __half *x, const int8_t *w, const void *sw, int sw_is_half, int gs,
                            const __half *bias, __half *y, int64_t N, int64_t K, const GemvPrologue &pro,
                            cudaStream_t st) {
  if (N == 0) return CIDER_OK;
  StreamPlan p;
  if (stream_shape_ok(N, K, gs, w, sw) && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 &&
      (pro.delta == nullptr || (reinterpret_cast<uintptr_t>(pro.delta) & 15u) == 0) &&
      (pro.norm_w == nullptr || (reinterpret_cast<uintptr_t>(pro.norm_w) & 15u) == 0) &&
      (pro.x_out == nullptr || (reinterpret_cast<uintptr_t>(pro.x_out) & 15u) == 0))
    p = plan_stream(3, 8, N, K, true);
  if (!p.ok) {
    if (pro.mode != kProloguePlain)
      return fail(CIDER_E_SHAPE,
                  "fused matrix-vector prologue needs K % 64 == 0, 16-byte aligned operands and K <= ~24K");
    gemv_scalar_kernel<<<(unsigned)((N + 3) / 4), 128, 0, st>>>(x, w, sw, sw_is_half, gs, bias, y, (int)N,
                                                               (int)K);
    return check_cuda(cudaGetLastError(), "gemv launch");
  }
  StreamX xa;
  xa.x = x;
  xa.split = 1;
  xa.pro = pro;
  return launch_stream(xa, 8, p, w, sw, sw_is_half, gs, bias, y, 1, N, K, st);
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

// Status word of the streaming kernels (bounded waits), OR-ed into
// cider_device_status().
int read_gemv_status(unsigned int *out) {
  return check_cuda(cudaMemcpyFromSymbol(out, g_gemv_status, sizeof(unsigned int)), "read gemv status");
}
int clear_gemv_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_gemv_status, &z, sizeof(z)), "clear gemv status");
}

// Small-M route of cider_linear_prequantized: up to 16 already-quantised rows
// (per-group weights: up to 64, taken 16 at a time - re-reading the weights four
// times is still several times faster than a 128-row tensor-core tile whose
// epilogue rescales every K-group).  Returns false when the shape does not fit
// (the caller then uses the tensor-core kernel).
bool smallm_eligible(int64_t M, int64_t N, int64_t K, int gs, const void *xq, const void *w, const void *sw,
                     bool w4) {
  if (M < 1 || M > (gs > 0 ? 64 : 16) || !stream_shape_ok(N, K, gs, w, sw)) return false;
  if (reinterpret_cast<uintptr_t>(xq) & 15u) return false;
  return plan_stream((int)(M < 8 ? M : 8), 8, N, K, false, w4).ok;
}

int launch_smallm(const int8_t *xq, const float *sa, const int8_t *w, const void *sw, int sw_is_half, int gs,
                  const __half *bias, __half *y, int64_t M, int64_t N, int64_t K, cudaStream_t st, bool w4) {
  for (int64_t m0 = 0; m0 < M;) {
    const int64_t left = M - m0;
    int rows = (int)(left < 16 ? left : 16), mr = rows > 8 ? 16 : 8;
    StreamPlan p = plan_stream(rows, mr, N, K, false, w4);
    // sixteen activation rows that leave the ring less than ~96 KB to keep in flight
    // (long K) cost more than streaming the weights twice: eight at a time
    if (rows > 8 && (!p.ok || (size_t)p.stages * kStageRows * pad_stride(p.ks) < (w4 ? 48 : 96) * 1024)) {
      rows = 8;
      mr = 8;
      p = plan_stream(rows, mr, N, K, false, w4);
    }
    if (!p.ok) return fail(CIDER_E_SHAPE, "small-M GEMM: problem too large");
    StreamX xa;
    xa.xq = xq + m0 * K;
    xa.sa = sa + m0;
    int rc = launch_stream(xa, mr, p, w, sw, sw_is_half, gs, bias, y + m0 * N, rows, N, K, st, w4);
    if (rc) return rc;
    m0 += rows;
  }
  return CIDER_OK;
}

int launch_repack_w4(const uint8_t *packed_kn, uint8_t *w_nk4, int64_t N, int64_t K, cudaStream_t st) {
  if (N == 0 || K == 0) return CIDER_OK;
  const int64_t kp = K / 2;
  const bool wide = N % 16 == 0 && kp % 16 == 0 && (reinterpret_cast<uintptr_t>(packed_kn) & 15u) == 0 &&
                    (reinterpret_cast<uintptr_t>(w_nk4) & 15u) == 0;
  if (wide) {
    dim3 grid((unsigned)((N + kRepackTile - 1) / kRepackTile), (unsigned)((kp + kRepackTile - 1) / kRepackTile));
    if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "w4a8_repack: K too large");
    return check_cuda(launch_kernel(repack_w4_kernel, grid, dim3(256), (size_t)0, st, packed_kn, w_nk4, (int)N, (int)kp),
                      "w4a8_repack launch");
  }
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((kp + 31) / 32));
  if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "w4a8_repack: K too large");
  repack_w4_small_kernel<<<grid, 256, 0, st>>>(packed_kn, w_nk4, (int)N, (int)kp);
  return check_cuda(cudaGetLastError(), "w4a8_repack launch");
}

// K % 16 == 0 and 16-byte aligned buffers (the caller checks).
int launch_unpack_w4_nk(const uint8_t *w_nk4, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st) {
  const int64_t total8 = N * K / 16;
  if (total8 == 0) return CIDER_OK;
  int64_t blocks = (total8 + 255) / 256;
  const int64_t cap = (int64_t)sm_count(current_device()) * 16;
  if (blocks > cap) blocks = cap;
  unpack_w4_nk_kernel<<<(unsigned)blocks, 256, 0, st>>>(w_nk4, w_nk, total8);
  return check_cuda(cudaGetLastError(), "w4a8 unpack launch");
}

int launch_unpack_w4(const uint8_t *packed, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st) {
  if (N == 0 || K == 0) return CIDER_OK;
  dim3 grid((unsigned)((N + 31) / 32), (unsigned)((K / 2 + 63) / 64));
  if (grid.y > 65535u) return fail(CIDER_E_SHAPE, "unpack_w4: K too large");
  unpack_w4_kernel<<<grid, 256, 0, st>>>(packed, w_nk, (int)N, (int)K);
  return check_cuda(cudaGetLastError(), "unpack_w4 launch");
}

}  // namespace cider
