// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05, sm_100a)
// with the dequantising epilogues of the reference fused behind it.
//
//   C[m,n] = sum_k A[m,k] * B[n,k]        A [M,K] int8, B [N,K] int8, both K-major
//   raw       : int32 out                                  (w8a8_matmul.metal:301-453)
//   perchannel: half(fma(float(acc)*sa[m], sw[n], bias[n]))  (w8a8_matmul.metal:63-81)
//   pergroup  : accf = fma(float(acc_g), sw[g,n], accf) per K-group,
//               half(fma(accf, sa[m], bias[n]))            (pergroup_int8_gemm.metal:99-191)
//
// Structure (one persistent CTA per SM, 192 threads, warp-specialised):
//   warp 0      TMA producer: 128-byte-swizzled [128 x 128B] A tile and
//               [BN x 128B] B tile per stage into a shared-memory ring
//   warp 1      MMA issuer: one lane issues tcgen05.mma.kind::i8 (M128 x N(BN) x K32),
//               4 per stage, accumulating int32 in tensor memory; owns TMEM alloc
//   warps 2..5  epilogue: tcgen05.ld their 32-lane quarter of the accumulator,
//               dequantise in registers, store fp16 / int32 to global
// Tensor memory holds two accumulators so the epilogue of one tile (or K-group)
// overlaps the MMAs of the next.  Out-of-range rows / columns / K are zero-filled
// by TMA on load and masked on store, so M, N need no alignment; K % 16 == 0 and
// 16-byte aligned A / B are required by TMA (other shapes use the plain kernel).
//
// Every wait on a shared-memory barrier is bounded: when it runs out the kernel
// records kStatusWaitTimeout in a device status word, every role leaves its
// loop, in-flight copies and MMAs are drained (bounded), TMEM is released and
// the kernel returns.
#include <mutex>

#include "common.cuh"

namespace cider {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes (= int8 elements) of K per stage: one 128B swizzle row
constexpr int UMMA_K = 32;
constexpr int kThreads = 192;
constexpr int kEpiThreads = 128;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s at boost clock

template <int BN>
struct Cfg {
  static constexpr int kStages = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
  static constexpr int kEpiBytes = 4 * BN * 8;  // per epilogue warp: BN fp32 scales + BN fp32 bias
  static constexpr int kBarBytes = (2 * kStages + 5) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kEpiBytes + kBarBytes + 1024;
};

struct TcParams {
  void *out;
  const float *sa;
  const void *sw;
  const __half *bias;
  int M, N, K;
  int gs;
  int sw_half;
  int vec_store;  // 16-byte stores allowed (row pitch and base aligned)
};

// ---------------------------------------------------------------- PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
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
// Bounded wait.  Returns false when the wait ran out or another role gave up.
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
      atomicOr(&g_device_status, kStatusWaitTimeout);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes,
// stored as 8-row x 128-byte atoms with the 128B swizzle (what TMA writes with
// CU_TENSOR_MAP_SWIZZLE_128B): start address, leading byte offset 1 (unused for
// swizzled K-major), stride byte offset 1024 (one 8-row atom), descriptor
// version 1, layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
  uint64_t d = (uint64_t)((smem_addr >> 4) & 0x3FFFu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::i8: D = s32 (2 at bit 4), A = B = signed 8-bit
// (1 at bits 7 and 10), both K-major (bits 15, 16 clear), N >> 3 at bit 17,
// M >> 4 at bit 24, no saturation.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ float sw_load(const void *sw, int is_half, int64_t idx) {
  return is_half ? __half2float(reinterpret_cast<const __half *>(sw)[idx])
                 : __ldg(reinterpret_cast<const float *>(sw) + idx);
}

// ------------------------------------------------------------------ kernel
template <int BN, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const TcParams p) {
  using C = Cfg<BN>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint8_t *smem_a = smem;                                 // kStages x [128 x 128B]
  uint8_t *smem_b = smem + kStages * C::kABytes;          // kStages x [BN x 128B]
  float *epi_s = reinterpret_cast<float *>(smem + kStages * C::kStageBytes);  // [4 warps][2][BN]
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(epi_s) + C::kEpiBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kStages;
  uint64_t *tmem_full_bar = bars + 2 * kStages;       // [2]
  uint64_t *tmem_empty_bar = bars + 2 * kStages + 2;  // [2]
  uint64_t *drain_bar = bars + 2 * kStages + 4;
  uint32_t *tmem_ptr_s = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 5);
  volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_ptr_s + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  // per-group: accumulator hand-over every `gs` of K (gs is a multiple of 64)
  const int mma_per_group = EPI == (int)Epi::kPerGroup ? p.gs / UMMA_K : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 4);  // one arrival per epilogue warp
    }
    mbar_init(smem_u32(drain_bar), 1);
    *abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_ptr_s)),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      int stage = 0;
      uint32_t phase = 0;
      uint32_t fills = 0;  // total fills issued
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t / num_n) * BM, n0 = (t % num_n) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_s)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, C::kStageBytes);
          tma_load_2d(smem_u32(smem_a + stage * C::kABytes), &tma_a, fb, kb * BK, m0);
          tma_load_2d(smem_u32(smem_b + stage * C::kBBytes), &tma_b, fb, kb * BK, n0);
          ++fills;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (!ok || *abort_s) {
        // drain: wait (bounded) until every copy that was issued has landed
        const uint32_t last = fills < (uint32_t)kStages ? fills : (uint32_t)kStages;
        for (uint32_t i = 0; i < last; ++i) {
          const uint32_t f = fills - 1 - i;  // fill index, newest first
          const uint32_t s = f % kStages, par = (f / kStages) & 1u;
          const long long t0 = clock64();
          while (!mbar_try_wait(smem_u32(&full_bar[s]), par) && clock64() - t0 < kWaitCycles) {
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t handover = 0;  // accumulator hand-overs so far (tile, or K-group)
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        uint32_t buf = handover & 1u;
        uint32_t in_group = 0;
        bool fresh = true;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[buf]), ((handover >> 1) & 1u) ^ 1u, abort_s)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb && ok; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_desc = make_smem_desc(smem_u32(smem_a + stage * C::kABytes));
          const uint64_t b_desc = make_smem_desc(smem_u32(smem_b + stage * C::kBBytes));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            if (EPI == (int)Epi::kPerGroup && kb * BK + k * UMMA_K >= p.K) break;
            const uint32_t d_tmem = tmem_base + buf * BN;
            // advance 32 bytes of K inside the swizzle atom: +2 in 16-byte units
            tc_mma_i8(d_tmem, a_desc + (uint64_t)(k * (UMMA_K >> 4)),
                      b_desc + (uint64_t)(k * (UMMA_K >> 4)), idesc, fresh ? 0u : 1u);
            fresh = false;
            if (EPI == (int)Epi::kPerGroup && ++in_group == (uint32_t)mma_per_group) {
              // group complete: hand this accumulator to the epilogue, move on
              tc_commit(smem_u32(&tmem_full_bar[buf]));
              ++handover;
              in_group = 0;
              fresh = true;
              const bool last = (kb * BK + (k + 1) * UMMA_K >= p.K);
              if (!last) {
                buf = handover & 1u;
                if (!mbar_wait(smem_u32(&tmem_empty_bar[buf]), ((handover >> 1) & 1u) ^ 1u,
                               abort_s)) {
                  ok = false;
                  break;
                }
                tc_fence_after();
              }
            }
          }
          tc_commit(smem_u32(&empty_bar[stage]));  // stage reusable once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (EPI != (int)Epi::kPerGroup && ok) {
          tc_commit(smem_u32(&tmem_full_bar[buf]));
          ++handover;
        }
      }
      // drain: every MMA issued by this thread has retired once this commit lands
      tc_commit(smem_u32(drain_bar));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(drain_bar), 0) && clock64() - t0 < kWaitCycles) {
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    float *sw_s = epi_s + ew * 2 * BN;
    float *bias_s = sw_s + BN;
    uint32_t handover = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int m0 = (t / num_n) * BM, n0 = (t % num_n) * BN;
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < p.M;
      float sa_m = 0.0f;
      if (EPI != (int)Epi::kRawInt32) {
        sa_m = row_ok ? __ldg(p.sa + m) : 0.0f;
        __syncwarp();
        for (int j = lane; j < BN; j += 32) {
          const int n = n0 + j;
          if (EPI == (int)Epi::kPerChannel)
            sw_s[j] = n < p.N ? sw_load(p.sw, p.sw_half, n) : 0.0f;
          bias_s[j] = (p.bias != nullptr && n < p.N) ? __half2float(p.bias[n]) : 0.0f;
        }
        __syncwarp();
      }

      if (EPI == (int)Epi::kPerGroup) {
        // ---- fp32 accumulation across K-groups, BN columns per thread
        float accf[BN];
#pragma unroll
        for (int j = 0; j < BN; ++j) accf[j] = 0.0f;
        const int groups = p.K / p.gs;
        for (int g = 0; g < groups && ok; ++g) {
          const uint32_t buf = handover & 1u;
          uint32_t got = 0;
          if (lane == 0) got = mbar_wait(smem_u32(&tmem_full_bar[buf]), (handover >> 1) & 1u, abort_s);
          got = __shfl_sync(0xffffffffu, got, 0);
          if (!got) {
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c * 32, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int n = n0 + c * 32 + j;
              const float s = n < p.N ? sw_load(p.sw, p.sw_half, (int64_t)g * p.N + n) : 0.0f;
              accf[c * 32 + j] = __fmaf_rn(__int2float_rn((int)r[j]), s, accf[c * 32 + j]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
          ++handover;
        }
        if (ok && row_ok) {
          __half *orow = reinterpret_cast<__half *>(p.out) + (int64_t)m * p.N + n0;
#pragma unroll
          for (int c = 0; c < BN / 8; ++c) {
            __half2 h[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = c * 8 + 2 * j;
              h[j] = __floats2half2_rn(__fmaf_rn(accf[col], sa_m, bias_s[col]),
                                       __fmaf_rn(accf[col + 1], sa_m, bias_s[col + 1]));
            }
            if (p.vec_store && n0 + c * 8 + 8 <= p.N) {
              *reinterpret_cast<uint4 *>(orow + c * 8) = *reinterpret_cast<const uint4 *>(h);
            } else {
              const __half *hs = reinterpret_cast<const __half *>(h);
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (n0 + c * 8 + j < p.N) orow[c * 8 + j] = hs[j];
            }
          }
        }
        continue;
      }

      // ---- raw / per-channel: one accumulator per tile
      const uint32_t buf = handover & 1u;
      uint32_t got = 0;
      if (lane == 0) got = mbar_wait(smem_u32(&tmem_full_bar[buf]), (handover >> 1) & 1u, abort_s);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) {
        ok = false;
        break;
      }
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tc_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + c * 32, r);
        tc_wait_ld();
        const int nc = n0 + c * 32;
        if (EPI == (int)Epi::kRawInt32) {
          if (row_ok) {
            int32_t *orow = reinterpret_cast<int32_t *>(p.out) + (int64_t)m * p.N + nc;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              if (p.vec_store && nc + 4 * j + 4 <= p.N) {
                *reinterpret_cast<uint4 *>(orow + 4 * j) =
                    make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i)
                  if (nc + 4 * j + i < p.N) orow[4 * j + i] = (int32_t)r[4 * j + i];
              }
            }
          }
        } else {
          uint32_t h[16];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float4 s4 = *reinterpret_cast<const float4 *>(sw_s + c * 32 + 4 * j);
            const float4 b4 = *reinterpret_cast<const float4 *>(bias_s + c * 32 + 4 * j);
            const float v0 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 0]), sa_m), s4.x, b4.x);
            const float v1 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 1]), sa_m), s4.y, b4.y);
            const float v2 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 2]), sa_m), s4.z, b4.z);
            const float v3 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 3]), sa_m), s4.w, b4.w);
            __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
            h[2 * j] = *reinterpret_cast<uint32_t *>(&h01);
            h[2 * j + 1] = *reinterpret_cast<uint32_t *>(&h23);
          }
          if (row_ok) {
            __half *orow = reinterpret_cast<__half *>(p.out) + (int64_t)m * p.N + nc;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (p.vec_store && nc + 8 * j + 8 <= p.N) {
                *reinterpret_cast<uint4 *>(orow + 8 * j) =
                    make_uint4(h[4 * j], h[4 * j + 1], h[4 * j + 2], h[4 * j + 3]);
              } else {
                const __half *hs = reinterpret_cast<const __half *>(&h[4 * j]);
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  if (nc + 8 * j + i < p.N) orow[8 * j + i] = hs[i];
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
      ++handover;
    }
  }

  // ---- teardown (every path reaches this: all waits above are bounded)
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void *f = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(f);
  });
  return fn;
}

// 2-D int8 tensor map over a row-major [rows, K] matrix, box [box_rows x 128 bytes],
// 128-byte swizzle, zero fill outside the matrix.
int make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t K, int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)K};
  cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r));
  return CIDER_OK;
}

template <int BN, int EPI>
int launch_cfg(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_tc_kernel<BN, EPI>;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [&] {
    attr_err = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  });
  if (attr_err != cudaSuccess) return check_cuda(attr_err, "gemm_tc shared-memory attribute");
  CUtensorMap ma, mb;
  int rc = make_map(&ma, g.a, g.M, g.K, BM);
  if (rc) return rc;
  rc = make_map(&mb, g.b, g.N, g.K, BN);
  if (rc) return rc;
  const int64_t tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  kern<<<grid, kThreads, C::kSmemBytes, st>>>(ma, mb, p);
  return check_cuda(cudaGetLastError(), "gemm_tc launch");
}

template <int EPI>
int launch_epi(const GemmArgs &g, const TcParams &p, int bn, cudaStream_t st) {
  switch (bn) {
    case 256: return launch_cfg<256, EPI>(g, p, st);
    case 128: return launch_cfg<128, EPI>(g, p, st);
    default: return launch_cfg<64, EPI>(g, p, st);
  }
}

}  // namespace

bool gemm_tc_eligible(const GemmArgs &g) {
  auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (g.packed4 != nullptr || g.a == nullptr || g.b == nullptr) return false;
  if (g.M < 1 || g.N < 1 || g.K < BK || (g.K % 16) != 0) return false;
  if (g.M > (1 << 30) || g.N > (1 << 30) || g.K > (1 << 30)) return false;
  if (((g.M + BM - 1) / BM) * ((g.N + 63) / 64) > (int64_t)(1u << 30)) return false;
  if (!a16(g.a) || !a16(g.b)) return false;
  if (g.epi == Epi::kPerGroup && (g.gs % 64 != 0 || g.K % g.gs != 0)) return false;
  return true;
}

int launch_gemm_tc(const GemmArgs &g, cudaStream_t st) {
  if (!gemm_tc_eligible(g)) return fail(CIDER_E_SHAPE, "gemm_tc: shape or alignment not supported");
  TcParams p;
  p.out = g.out; p.sa = g.sa; p.sw = g.sw; p.bias = g.bias;
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.gs = g.gs; p.sw_half = g.sw_is_half;
  const bool o16 = (reinterpret_cast<uintptr_t>(g.out) & 15u) == 0;
  p.vec_store = g.epi == Epi::kRawInt32 ? (o16 && g.N % 4 == 0) : (o16 && g.N % 8 == 0);
  // widest N tile that still gives every SM a tile
  const int sms = sm_count(current_device());
  const int64_t num_m = (g.M + BM - 1) / BM;
  int bn = 256;
  while (bn > 64 && num_m * ((g.N + bn - 1) / bn) < sms) bn >>= 1;
  switch (g.epi) {
    case Epi::kRawInt32: return launch_epi<(int)Epi::kRawInt32>(g, p, bn, st);
    case Epi::kPerChannel: return launch_epi<(int)Epi::kPerChannel>(g, p, bn, st);
    default:
      // per-group keeps BN fp32 partial sums per thread: 64 columns at most
      return launch_cfg<64, (int)Epi::kPerGroup>(g, p, st);
  }
}

int read_device_status(unsigned int *out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return check_cuda(e, "device synchronize");
  return check_cuda(cudaMemcpyFromSymbol(out, g_device_status, sizeof(unsigned int)), "read status");
}

int clear_device_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_device_status, &z, sizeof(z)), "clear status");
}

}  // namespace cider
