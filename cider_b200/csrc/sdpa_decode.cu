// Split-K single-query attention for the decode step (one new token per
// sequence) over an fp16 KV cache: out[b,h,:] = softmax(q[b,h,:].K^T * scale) V.
//
// The reference has no kernel of its own here: its model code calls MLX's
// scaled_dot_product_attention (visible at cider/fused_hybrid.py:192).  On B200
// the step is pure KV streaming (2*T*Hkv*D*2 bytes per layer and sequence), so:
//   - the T cached positions are split over `S` blocks per (batch, KV head) so
//     that all SMs stream (flash-decoding), each block keeping online-softmax
//     state (m, l, o) in registers;
//   - the Hq/Hkv query heads that share a KV head are processed together, so a
//     K/V row is read from HBM once per group, in 16-byte loads;
//   - the S partial states are merged by a second small kernel, or - when the
//     caller lends a zeroed ticket counter per (batch, KV head) - by whichever
//     block of that head finishes last (it finds the others' states in global
//     memory, merges them and puts the counter back to zero): one launch instead
//     of two, which is what a decode step at short context is bound by.
// Layouts: q, out [B,Hq,D]; k_cache, v_cache [B,Hkv,Tcap,D]; fp32 workspace
// [B,Hq,S,D] partial outputs followed by [B,Hq,S,2] (m, l).
#include <atomic>

#include "common.cuh"

namespace cider {

// status word of this file's kernels (the fused append's bound check); merged into
// cider_device_status() by read_device_status()
__device__ unsigned int g_sdpa_status = 0;

namespace {

// The decode step's attention prologue folded into the attention kernel (D == 128): the raw
// fused projection output of the new token, per-head q / k RMSNorm weights, rotary tables
// and the caches to append to - what qk_norm_rope_append_kernel would have done in a launch
// of its own (same arithmetic, same roundings).
struct RopeArgs {
  const __half *qkv;       // [B, (Hq + 2 Hkv) * D], null: q is given already normalised and rotated
  const __half *q_norm_w, *k_norm_w;
  const float *inv_freq;   // [D/2]
  const int8_t *axis;      // [D/2]
  const int *pos3;         // [3, pos_stride], column 0 = the new token
  int pos_stride;
  float eps;
  __half *k_cache, *v_cache;  // writable views of kc / vc
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr float kNegBig = -1.0e30f;

// kernel choice for the tests: 0 automatic, 1 CUDA-core form, 2 tensor-core form (where it exists)
std::atomic<int> g_sdpa_kernel{0};

int pick_splits(int64_t B, int64_t Hkv, int64_t T, int blocks_per_sm = 2) {
  if (T <= 0) return 1;
  int64_t s = (blocks_per_sm * 148) / (B * Hkv);  // rounded down: a few blocks more than fit at once would run alone at the end
  const int64_t max_by_len = (T + 63) / 64;
  if (s > max_by_len) s = max_by_len;
  if (s > 128) s = 128;
  if (s < 1) s = 1;
  return (int)s;
}

// Fused prologue of a decode step's attention (D == 128): per-head RMSNorm + rope of this
// block's REP query heads into q_s (fp32 copies of the fp16-rounded values; every block of
// the KV head repeats this: REP heads of 128 values), and - in the one block whose split
// holds the newest position T - 1 - of the new key, which is appended to the cache together
// with the new value before the positions are walked.  A half-warp per head of
// [q heads of the group | the k head | the v head] (norm_rope_head128).  Ends with a block
// barrier: q_s is complete and the appended row is visible to this block's loads.
template <int REP>
__device__ __forceinline__ void fused_prologue(const RopeArgs &ra, float (*q_s)[128], int b, int kvh, int split,
                                               int Hq, int Hkv, int T, int Tcap, int t_begin, int t_end,
                                               const int *length_dev, int nwarps) {
  __shared__ float2 cs_s[64];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x < 64) {
    const int i = threadIdx.x;
    const float ang = __fmul_rn((float)ra.pos3[ra.axis[i] * ra.pos_stride], ra.inv_freq[i]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    cs_s[i] = make_float2(cs, sn);
  }
  __syncthreads();
  // a length beyond the cache (one graph replay too many): nothing is appended, the
  // overflow is recorded
  const bool overflow = length_dev != nullptr && *length_dev > Tcap;
  if (overflow && threadIdx.x == 0 && split == 0) atomicOr(&g_sdpa_status, kStatusKvOverflow);
  const bool newest_here = !overflow && T > 0 && t_begin <= T - 1 && T - 1 < t_end;
  const int heads = Hq + 2 * Hkv;
  const int hl = lane & 15, d0 = 8 * hl;
  const unsigned hmask = lane < 16 ? 0x0000ffffu : 0xffff0000u;
  // jobs: the REP query heads of the group, then the new key head and the new value head
  for (int job = 2 * warp + (lane >> 4); job < REP + 2; job += 2 * nwarps) {
    const bool is_q = job < REP, is_k = job == REP;
    if (!is_q && !newest_here) continue;
    const int head = is_q ? kvh * REP + job : (is_k ? Hq + kvh : Hq + Hkv + kvh);
    const uint4 raw = *reinterpret_cast<const uint4 *>(ra.qkv + ((int64_t)b * heads + head) * 128 + d0);
    const int64_t slot = (((int64_t)b * Hkv + kvh) * (int64_t)Tcap + (T - 1)) * 128 + d0;
    if (!is_q && !is_k) {  // v: copy
      *reinterpret_cast<uint4 *>(ra.v_cache + slot) = raw;
      continue;
    }
    const uint4 outv = norm_rope_head128(raw, is_q ? ra.q_norm_w : ra.k_norm_w, cs_s, ra.eps, hl, hmask);
    if (is_q) {
      const __half2 *oh = reinterpret_cast<const __half2 *>(&outv);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(oh[j]);
        q_s[job][d0 + 2 * j] = f.x;
        q_s[job][d0 + 2 * j + 1] = f.y;
      }
    } else {
      *reinterpret_cast<uint4 *>(ra.k_cache + slot) = outv;
    }
  }
  __syncthreads();
}

// One block: (split, kv head, batch).  A warp covers 32 / LPP positions per step, LPP
// lanes per position, each lane DL = D / LPP consecutive head dims.  LPP = 8 for up to
// two query heads per KV head.  With four or more, a lane's q and o state for 16 dims of
// every head is 194 registers: one block of 8 warps per SM, and the kernel waits on its
// loads (ncu at 8 sequences x 2 K context: 1.4 TB/s, issue slots 39 % busy, stall reason
// long_scoreboard).  LPP = 16 halves that state so that two blocks fit.
template <int D, int REP, int LPP>
__global__ void __launch_bounds__(kThreads, (LPP == 16 && REP <= 4) ? 2 : 1)
sdpa_decode_partial_kernel(const __half *__restrict__ q, const __half *__restrict__ kc,
                           const __half *__restrict__ vc, float *part_o, float *part_ml, int Hq, int Hkv,
                           int T_host, int Tcap, int S, float scale_log2e, const int *__restrict__ length_dev,
                           unsigned int *tickets, __half *__restrict__ out_final, const RopeArgs ra) {
  constexpr int DL = D / LPP;
  constexpr int PPW = 32 / LPP;  // positions per warp and step
  __shared__ float sm_o[kWarps][REP][D];
  __shared__ float sm_ml[kWarps][REP][2];
  __shared__ unsigned int last_s;
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPP, l8 = lane % LPP;

  // the attended length may live in device memory (CUDA-graph replay); the split
  // count was sized on the host from an upper bound of it
  const int T = length_dev ? min(*length_dev, Tcap) : T_host;
  // positions of this split: [t_begin, t_end), chunk rounded to 32 positions
  int chunk = (T + S - 1) / S;
  chunk = (chunk + 31) / 32 * 32;
  const int t_begin = split * chunk;
  const int t_end = min(T, t_begin + chunk);

  float qf[REP][DL];
  __shared__ float q_s[D == 128 ? REP : 1][128];
  if constexpr (D == 128) {
    if (ra.qkv != nullptr) {
      fused_prologue<REP>(ra, q_s, b, kvh, split, Hq, Hkv, T, Tcap, t_begin, t_end, length_dev, kWarps);
#pragma unroll
      for (int r = 0; r < REP; ++r)
#pragma unroll
        for (int d = 0; d < DL; ++d) qf[r][d] = q_s[r][l8 * DL + d] * scale_log2e;
    }
  }
  if (D != 128 || ra.qkv == nullptr) {
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      const __half *qp = q + ((int64_t)b * Hq + kvh * REP + r) * D + l8 * DL;
#pragma unroll
      for (int d = 0; d < DL; ++d) qf[r][d] = __half2float(qp[d]) * scale_log2e;
    }
  }
  float m[REP], l[REP], o[REP][DL];
#pragma unroll
  for (int r = 0; r < REP; ++r) {
    m[r] = kNegBig;
    l[r] = 0.0f;
#pragma unroll
    for (int d = 0; d < DL; ++d) o[r][d] = 0.0f;
  }

  const __half *kbase = kc + ((int64_t)b * Hkv + kvh) * (int64_t)Tcap * D + l8 * DL;
  const __half *vbase = vc + ((int64_t)b * Hkv + kvh) * (int64_t)Tcap * D + l8 * DL;

  for (int t0 = t_begin + warp * PPW; t0 < t_end; t0 += kWarps * PPW) {
    const int t = t0 + sub;
    const bool live = t < t_end;
    const int tt = live ? t : t_begin;  // any valid row; its weight is forced to zero
    uint4 kv[DL / 8], vv[DL / 8];
#pragma unroll
    for (int i = 0; i < DL / 8; ++i) {
      kv[i] = __ldcs(reinterpret_cast<const uint4 *>(kbase + (int64_t)tt * D) + i);
      vv[i] = __ldcs(reinterpret_cast<const uint4 *>(vbase + (int64_t)tt * D) + i);
    }
    float kf[DL], vf[DL];
    {
      const __half2 *k2 = reinterpret_cast<const __half2 *>(kv);
      const __half2 *v2 = reinterpret_cast<const __half2 *>(vv);
#pragma unroll
      for (int i = 0; i < DL / 2; ++i) {
        float2 a = __half22float2(k2[i]);
        float2 c = __half22float2(v2[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y;
        vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
      }
    }
#pragma unroll
    for (int r = 0; r < REP; ++r) {
      float s = 0.0f;
#pragma unroll
      for (int d = 0; d < DL; ++d) s = fmaf(qf[r][d], kf[d], s);
#pragma unroll
      for (int off = 1; off < LPP; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (!live) s = kNegBig;
      const float mn = fmaxf(m[r], s);
      const float alpha = exp2f(m[r] - mn);
      const float pw = live ? exp2f(s - mn) : 0.0f;
      m[r] = mn;
      l[r] = fmaf(l[r], alpha, pw);
#pragma unroll
      for (int d = 0; d < DL; ++d) o[r][d] = fmaf(pw, vf[d], o[r][d] * alpha);
    }
  }

  // merge the position sub-groups of the warp (lanes differing in the bits above LPP)
#pragma unroll
  for (int r = 0; r < REP; ++r) {
#pragma unroll
    for (int off = LPP; off <= 16; off <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[r], off);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[r], off);
      const float mn = fmaxf(m[r], m2);
      const float a1 = exp2f(m[r] - mn), a2 = exp2f(m2 - mn);
      l[r] = l[r] * a1 + l2 * a2;
#pragma unroll
      for (int d = 0; d < DL; ++d) {
        const float o2 = __shfl_xor_sync(0xffffffffu, o[r][d], off);
        o[r][d] = o[r][d] * a1 + o2 * a2;
      }
      m[r] = mn;
    }
    if (sub == 0) {
#pragma unroll
      for (int d = 0; d < DL; ++d) sm_o[warp][r][l8 * DL + d] = o[r][d];
      if (l8 == 0) {
        sm_ml[warp][r][0] = m[r];
        sm_ml[warp][r][1] = l[r];
      }
    }
  }
  __syncthreads();
  // merge the warps; thread -> (head r, dim d)
  for (int idx = threadIdx.x; idx < REP * D; idx += kThreads) {
    const int r = idx / D, d = idx % D;
    float mm = kNegBig;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) mm = fmaxf(mm, sm_ml[w][r][0]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float a = exp2f(sm_ml[w][r][0] - mm);
      ll = fmaf(sm_ml[w][r][1], a, ll);
      oo = fmaf(sm_o[w][r][d], a, oo);
    }
    const int64_t row = ((int64_t)b * Hq + kvh * REP + r) * S + split;
    part_o[row * D + d] = oo;
    if (d == 0) {
      part_ml[row * 2] = mm;
      part_ml[row * 2 + 1] = ll;
    }
  }
  if (tickets == nullptr) return;
  // ---- one-kernel form: the block that takes the last ticket of its (batch, KV
  // head) merges all S states.  Writers fence before the ticket, the merger reads
  // around L1 (the other blocks' stores are in L2).
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = atomicAdd(&tickets[b * Hkv + kvh], 1u) == (unsigned)(S - 1) ? 1u : 0u;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < REP * D; idx += kThreads) {
    const int r = idx / D, d = idx % D;
    const int64_t bh = (int64_t)b * Hq + kvh * REP + r;
    float mm = kNegBig;
    for (int s2 = 0; s2 < S; ++s2) mm = fmaxf(mm, __ldcg(part_ml + (bh * S + s2) * 2));
    float ll = 0.0f, oo = 0.0f;
    for (int s2 = 0; s2 < S; ++s2) {
      const float a = exp2f(__ldcg(part_ml + (bh * S + s2) * 2) - mm);
      ll = fmaf(__ldcg(part_ml + (bh * S + s2) * 2 + 1), a, ll);
      oo = fmaf(__ldcg(part_o + (bh * S + s2) * D + d), a, oo);
    }
    out_final[bh * D + d] = __float2half_rn(ll > 0.0f ? oo / ll : 0.0f);
  }
  if (threadIdx.x == 0) tickets[b * Hkv + kvh] = 0u;  // as found: the next launch starts from zero
}

// ---------------------------------------------------------------- tensor-core form
// The same split-K decode attention for grouped queries (D == 128, 2 .. 8 query heads per KV
// head) with Q K^T and P V on the warp-level fp16 tensor instruction (mma.sync m16n8k16,
// fp32 accumulation): the group's query heads are the rows of a 16-row operand (rows past
// REP are zero), so a K / V row read once from HBM serves all of them without the per-position
// shuffle reductions of the CUDA-core form (which is bound by issue slots and registers at
// 8 sequences x 2 K context, not by HBM).  The legacy instruction on purpose: a decode step has
// 2 .. 8 query rows per KV head, a 128-row tcgen05 tile would be 94 % padding, and the kernel
// is bound by KV bytes.
//   block = (split, KV head, batch), 4 warps; warp w walks the split's positions in tiles of
//   16 (tiles w, w + 4, ...), each tile's K and V rows (4 KB + 4 KB) copied into the warp's
//   own 4-deep shared-memory ring with cp.async (16-byte chunks XOR-swizzled by the row so
//   that ldmatrix is conflict-free), three tiles in flight per warp;
//   S = Q K^T: 8 k-steps x 2 position tiles; online softmax on the accumulator fragments (a
//   row's 16 scores sit in the 4 lanes of a quad); P goes straight from the score fragments
//   to the A operand of P V (16 dim tiles, V fragments by ldmatrix.trans); 64 fp32 output
//   accumulators per lane.  P is rounded to fp16 (relative 2^-11, inside the 2e-3 bar).
//   The warps' states merge through shared memory as in the CUDA-core form, and the partial
//   states have the same layout, so the combine kernel / ticket merge is shared.
constexpr int kMmaWarps = 4, kMmaThreads = kMmaWarps * 32, kMmaTile = 16, kMmaStages = 3;
constexpr int kMmaTileBytes = kMmaTile * 128 * 2;                        // K (or V) rows of one tile
constexpr int kMmaSmemBytes = kMmaWarps * kMmaStages * 2 * kMmaTileBytes;  // 96 KB: two blocks per SM

__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// D(16x8, fp32) += A(16x16, fp16, row) * B(16x8, fp16, col); rows 8..15 of A are zero here
__device__ __forceinline__ void mma_f16(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
  const uint32_t z = 0u;
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(z), "r"(a2), "r"(z), "r"(b0), "r"(b1));
}

template <int REP>
__global__ void __launch_bounds__(kMmaThreads, 2)
sdpa_decode_mma_kernel(const __half *__restrict__ q, const __half *__restrict__ kc, const __half *__restrict__ vc,
                       float *part_o, float *part_ml, int Hq, int Hkv, int T_host, int Tcap, int S,
                       float scale_log2e, const int *__restrict__ length_dev, unsigned int *tickets,
                       __half *__restrict__ out_final, const RopeArgs ra) {
  constexpr int D = 128;
  extern __shared__ __align__(128) uint8_t ring_raw[];
  __shared__ float q_s[REP][128];
  __shared__ float sm_o[kMmaWarps][REP][D];
  __shared__ float sm_ml[kMmaWarps][REP][2];
  __shared__ unsigned int last_s;
  pdl_launch_dependents();
  pdl_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t4 = lane & 3;  // fragment row (query head) and column pair

  const int T = length_dev ? min(*length_dev, Tcap) : T_host;
  int chunk = (T + S - 1) / S;
  chunk = (chunk + 31) / 32 * 32;
  const int t_begin = split * chunk;
  const int t_end = min(T, t_begin + chunk);

  if (ra.qkv != nullptr) {
    fused_prologue<REP>(ra, q_s, b, kvh, split, Hq, Hkv, T, Tcap, t_begin, t_end, length_dev, kMmaWarps);
  } else {
    for (int idx = threadIdx.x; idx < REP * D; idx += kMmaThreads)
      q_s[idx / D][idx % D] = __half2float(q[((int64_t)b * Hq + kvh * REP + idx / D) * D + idx % D]);
    __syncthreads();
  }
  // A fragments of Q for the 8 k-steps: a0 = (row g, dims 16 ks + 2 t4, +1), a2 = (row g, + 8)
  uint32_t qa0[8], qa2[8];
#pragma unroll
  for (int ks = 0; ks < 8; ++ks) {
    __half2 lo = __floats2half2_rn(0.0f, 0.0f), hi = lo;
    if (g < REP) {
      lo = __floats2half2_rn(q_s[g][16 * ks + 2 * t4], q_s[g][16 * ks + 2 * t4 + 1]);  // exact: fp16 values
      hi = __floats2half2_rn(q_s[g][16 * ks + 2 * t4 + 8], q_s[g][16 * ks + 2 * t4 + 9]);
    }
    qa0[ks] = *reinterpret_cast<const uint32_t *>(&lo);
    qa2[ks] = *reinterpret_cast<const uint32_t *>(&hi);
  }

  // this warp's ring: kMmaStages x [K tile | V tile]
  const uint32_t ring = smem_addr(ring_raw) + warp * kMmaStages * 2 * kMmaTileBytes;
  const __half *kbase = kc + ((int64_t)b * Hkv + kvh) * (int64_t)Tcap * D;
  const __half *vbase = vc + ((int64_t)b * Hkv + kvh) * (int64_t)Tcap * D;
  const int tiles_total = (t_end - t_begin + kMmaTile - 1) / kMmaTile;  // <= 0: nothing to do
  const int my_tiles = tiles_total > warp ? (tiles_total - warp + kMmaWarps - 1) / kMmaWarps : 0;

  auto issue = [&](int i) {  // copy tile i of this warp into stage i % kMmaStages
    if (i < my_tiles) {
      const int t0 = t_begin + (warp + i * kMmaWarps) * kMmaTile;
      const uint32_t st = ring + (i % kMmaStages) * 2 * kMmaTileBytes;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        const int c = c8 * 32 + lane;      // 16-byte chunk of the tile: 16 per row
        const int row = c >> 4, col = c & 15;
        const int tpos = min(t0 + row, t_end - 1);  // rows past the end repeat the last one (masked below)
        const uint32_t off = row * 256 + ((col ^ (row & 7)) << 4);
        cp_async16(st + off, kbase + (int64_t)tpos * D + col * 8);
        cp_async16(st + kMmaTileBytes + off, vbase + (int64_t)tpos * D + col * 8);
      }
    }
    cp_async_commit();  // (an empty group keeps the group count uniform)
  };

  float o[16][4];
#pragma unroll
  for (int nt = 0; nt < 16; ++nt)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[nt][j] = 0.0f;
  float m_run = kNegBig, l_run = 0.0f;  // row g; l_run is this lane's share of the row sum

#pragma unroll
  for (int i = 0; i < kMmaStages - 1; ++i) issue(i);
  for (int i = 0; i < my_tiles; ++i) {
    cp_async_wait<kMmaStages - 2>();  // this lane's copies of tile i have landed
    __syncwarp();                     // ... and every lane's; all lanes are done with tile i - 1
    issue(i + kMmaStages - 1);        // refill the stage tile i - 1 used
    const uint32_t st = ring + (i % kMmaStages) * 2 * kMmaTileBytes;
    const int t0 = t_begin + (warp + i * kMmaWarps) * kMmaTile;

    // ---- S = Q K^T for 16 positions: two 8-position tiles
    float sc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    {
      const int mtx = lane >> 3;                     // which 8x8 matrix this lane addresses
      const int pos = (mtx >> 1) * 8 + (lane & 7);   // its row (position)
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int col = 2 * ks + (mtx & 1);
        uint32_t bk[4];
        ldmatrix_x4(st + pos * 256 + ((col ^ (pos & 7)) << 4), bk);
        mma_f16(sc[0], qa0[ks], qa2[ks], bk[0], bk[1]);
        mma_f16(sc[1], qa0[ks], qa2[ks], bk[2], bk[3]);
      }
    }
    // ---- online softmax of row g: this lane holds positions t0 + {2 t4, 2 t4 + 1, 8 + 2 t4, 9 + 2 t4}
    float sv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tpos = t0 + (j >> 1) * 8 + 2 * t4 + (j & 1);
      sv[j] = tpos < t_end ? sc[j >> 1][j & 1] * scale_log2e : kNegBig;
    }
    float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float mn = fmaxf(m_run, mx);
    const float alpha = exp2f(m_run - mn);
    float pv[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int tpos = t0 + (j >> 1) * 8 + 2 * t4 + (j & 1);
      pv[j] = tpos < t_end ? exp2f(sv[j] - mn) : 0.0f;
    }
    m_run = mn;
    const __half2 p01 = __floats2half2_rn(pv[0], pv[1]), p23 = __floats2half2_rn(pv[2], pv[3]);
    // the sum uses the rounded weights, the ones the output is built from
    const float2 r01 = __half22float2(p01), r23 = __half22float2(p23);
    l_run = fmaf(l_run, alpha, (r01.x + r01.y) + (r23.x + r23.y));
    const uint32_t pa0 = *reinterpret_cast<const uint32_t *>(&p01), pa2 = *reinterpret_cast<const uint32_t *>(&p23);
    // ---- O = O * alpha + P V
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      o[nt][0] *= alpha;
      o[nt][1] *= alpha;
    }
    {
      const int mtx = lane >> 3;
      const int pos = (mtx & 1) * 8 + (lane & 7);
#pragma unroll
      for (int nt = 0; nt < 16; nt += 2) {
        const int col = nt + (mtx >> 1);
        uint32_t bv[4];
        ldmatrix_x4_trans(st + kMmaTileBytes + pos * 256 + ((col ^ (pos & 7)) << 4), bv);
        mma_f16(o[nt], pa0, pa2, bv[0], bv[1]);
        mma_f16(o[nt + 1], pa0, pa2, bv[2], bv[3]);
      }
    }
  }
  cp_async_wait<0>();
  // row sum over the quad
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
  l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
  if (g < REP) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      sm_o[warp][g][8 * nt + 2 * t4] = o[nt][0];
      sm_o[warp][g][8 * nt + 2 * t4 + 1] = o[nt][1];
    }
    if (t4 == 0) {
      sm_ml[warp][g][0] = m_run;
      sm_ml[warp][g][1] = l_run;
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < REP * D; idx += kMmaThreads) {
    const int r = idx / D, d = idx % D;
    float mm = kNegBig;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) mm = fmaxf(mm, sm_ml[w][r][0]);
    float ll = 0.0f, oo = 0.0f;
#pragma unroll
    for (int w = 0; w < kMmaWarps; ++w) {
      const float a = exp2f(sm_ml[w][r][0] - mm);
      ll = fmaf(sm_ml[w][r][1], a, ll);
      oo = fmaf(sm_o[w][r][d], a, oo);
    }
    const int64_t row = ((int64_t)b * Hq + kvh * REP + r) * S + split;
    part_o[row * D + d] = oo;
    if (d == 0) {
      part_ml[row * 2] = mm;
      part_ml[row * 2 + 1] = ll;
    }
  }
  if (tickets == nullptr) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) last_s = atomicAdd(&tickets[b * Hkv + kvh], 1u) == (unsigned)(S - 1) ? 1u : 0u;
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < REP * D; idx += kMmaThreads) {
    const int r = idx / D, d = idx % D;
    const int64_t bh = (int64_t)b * Hq + kvh * REP + r;
    float mm = kNegBig;
    for (int s2 = 0; s2 < S; ++s2) mm = fmaxf(mm, __ldcg(part_ml + (bh * S + s2) * 2));
    float ll = 0.0f, oo = 0.0f;
    for (int s2 = 0; s2 < S; ++s2) {
      const float a = exp2f(__ldcg(part_ml + (bh * S + s2) * 2) - mm);
      ll = fmaf(__ldcg(part_ml + (bh * S + s2) * 2 + 1), a, ll);
      oo = fmaf(__ldcg(part_o + (bh * S + s2) * D + d), a, oo);
    }
    out_final[bh * D + d] = __float2half_rn(ll > 0.0f ? oo / ll : 0.0f);
  }
  if (threadIdx.x == 0) tickets[b * Hkv + kvh] = 0u;
}

// One block per (batch, q head): merge S partial states, normalise, write fp16.
template <int D>
__global__ void __launch_bounds__(D)
sdpa_decode_combine_kernel(const float *__restrict__ part_o, const float *__restrict__ part_ml,
                           __half *__restrict__ out, int S) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t bh = blockIdx.x;
  const int d = threadIdx.x;
  float mm = kNegBig;
  for (int s = 0; s < S; ++s) mm = fmaxf(mm, part_ml[(bh * S + s) * 2]);
  float ll = 0.0f, oo = 0.0f;
  for (int s = 0; s < S; ++s) {
    const float a = exp2f(part_ml[(bh * S + s) * 2] - mm);
    ll = fmaf(part_ml[(bh * S + s) * 2 + 1], a, ll);
    oo = fmaf(part_o[(bh * S + s) * D + d], a, oo);
  }
  out[bh * D + d] = __float2half_rn(ll > 0.0f ? oo / ll : 0.0f);
}

template <int D, int REP>
int launch_t(const __half *q, const __half *kc, const __half *vc, __half *out, int64_t B, int64_t Hq,
             int64_t Hkv, int64_t T, int64_t Tcap, float scale, float *po, float *pml, int S,
             const int *length_dev, unsigned int *tickets, const RopeArgs &ra, cudaStream_t st) {
  dim3 grid((unsigned)S, (unsigned)Hkv, (unsigned)B);
  constexpr int LPP = (D == 128 && REP >= 4) ? 16 : 8;
  auto kern = sdpa_decode_partial_kernel<D, REP, LPP>;
  // 16-33 KB of static shared memory per block: without the large carve-out the driver sizes
  // shared memory for one block and the second block of an SM does not fit
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, 0, attr_done, "sdpa_decode shared-memory attribute");
  if (rc) return rc;
  rc = check_cuda(launch_kernel(kern, grid, dim3(kThreads), (size_t)0, st, q, kc, vc, po,
                                    pml, (int)Hq, (int)Hkv, (int)T, (int)Tcap, S,
                                    scale * 1.4426950408889634f, length_dev, tickets, out, ra),
                      "sdpa_decode launch");
  if (rc || tickets != nullptr) return rc;
  return check_cuda(launch_kernel(sdpa_decode_combine_kernel<D>, dim3((unsigned)(B * Hq)), dim3(D), 0, st,
                                  (const float *)po, (const float *)pml, out, S),
                    "sdpa_decode combine launch");
}

template <int REP>
int launch_mma(const __half *q, const __half *kc, const __half *vc, __half *out, int64_t B, int64_t Hq, int64_t Hkv,
               int64_t T, int64_t Tcap, float scale, float *po, float *pml, int S, const int *length_dev,
               unsigned int *tickets, const RopeArgs &ra, cudaStream_t st) {
  auto kern = sdpa_decode_mma_kernel<REP>;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, kMmaSmemBytes, attr_done, "sdpa_decode (tensor-core) shared-memory attribute");
  if (rc) return rc;
  dim3 grid((unsigned)S, (unsigned)Hkv, (unsigned)B);
  rc = check_cuda(launch_kernel(kern, grid, dim3(kMmaThreads), (size_t)kMmaSmemBytes, st, q, kc, vc, po, pml,
                                (int)Hq, (int)Hkv, (int)T, (int)Tcap, S, scale * 1.4426950408889634f, length_dev,
                                tickets, out, ra),
                  "sdpa_decode (tensor-core) launch");
  if (rc || tickets != nullptr) return rc;
  return check_cuda(launch_kernel(sdpa_decode_combine_kernel<128>, dim3((unsigned)(B * Hq)), dim3(128), 0, st,
                                  (const float *)po, (const float *)pml, out, S),
                    "sdpa_decode combine launch");
}

}  // namespace

int set_sdpa_kernel(int mode) {
  if (mode < 0 || mode > 2) return fail(CIDER_E_INVALID, "set_sdpa_kernel: 0, 1 or 2");
  g_sdpa_kernel.store(mode);
  return CIDER_OK;
}

size_t sdpa_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || D <= 0) return 0;
  const int S = pick_splits(B, Hkv, T);
  return (size_t)B * Hq * S * (D + 2) * sizeof(float);
}

int read_sdpa_status(unsigned int *out) {
  return check_cuda(cudaMemcpyFromSymbol(out, g_sdpa_status, sizeof(unsigned int)), "read sdpa status");
}
int clear_sdpa_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_sdpa_status, &z, sizeof(z)), "clear sdpa status");
}

static int launch_sdpa_impl(const __half *q, const __half *kc, const __half *vc, __half *out, int64_t B, int64_t Hq,
                            int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale, void *workspace,
                            size_t ws_bytes, const int *length_dev, unsigned int *tickets, const RopeArgs &ra,
                            cudaStream_t st);

int launch_sdpa_decode(const __half *q, const __half *kc, const __half *vc, __half *out, int64_t B,
                       int64_t Hq, int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale,
                       void *workspace, size_t ws_bytes, const int *length_dev, unsigned int *tickets,
                       cudaStream_t st) {
  RopeArgs ra = {};
  return launch_sdpa_impl(q, kc, vc, out, B, Hq, Hkv, D, T, Tcap, scale, workspace, ws_bytes, length_dev, tickets, ra,
                          st);
}

int launch_sdpa_decode_fused(const __half *qkv, const __half *q_norm_w, const __half *k_norm_w, const float *inv_freq,
                             const int8_t *axis, const int *pos3, int pos_stride, float eps, __half *kc, __half *vc,
                             __half *out, int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Tcap, float scale,
                             void *workspace, size_t ws_bytes, const int *length_dev, unsigned int *tickets,
                             cudaStream_t st) {
  RopeArgs ra = {qkv, q_norm_w, k_norm_w, inv_freq, axis, pos3, pos_stride, eps, kc, vc};
  return launch_sdpa_impl(nullptr, kc, vc, out, B, Hq, Hkv, 128, T, Tcap, scale, workspace, ws_bytes, length_dev,
                          tickets, ra, st);
}

static int launch_sdpa_impl(const __half *q, const __half *kc, const __half *vc, __half *out, int64_t B, int64_t Hq,
                            int64_t Hkv, int64_t D, int64_t T, int64_t Tcap, float scale, void *workspace,
                            size_t ws_bytes, const int *length_dev, unsigned int *tickets, const RopeArgs &ra,
                            cudaStream_t st) {
  const size_t need = sdpa_decode_workspace_bytes(B, Hq, Hkv, D, T);
  if (workspace == nullptr || ws_bytes < need)
    return fail(CIDER_E_WORKSPACE, "sdpa_decode: workspace too small: need " + std::to_string(need));
  if ((reinterpret_cast<uintptr_t>(workspace) & 15u) || (reinterpret_cast<uintptr_t>(kc) & 15u) ||
      (reinterpret_cast<uintptr_t>(vc) & 15u))
    return fail(CIDER_E_ALIGNMENT, "sdpa_decode: workspace and caches must be 16-byte aligned");
  if (B > 65535 || Hkv > 65535) return fail(CIDER_E_SHAPE, "sdpa_decode: B and Hkv must be <= 65535");
  const int rep = (int)(Hq / Hkv);
  // Tensor-core form: grouped queries of 128 dims (one block of 4 warps per SM).
  const int mode = g_sdpa_kernel.load();
  const bool mma_ok = D == 128 && (rep == 2 || rep == 4 || rep == 8);
  const int S_mma = pick_splits(B, Hkv, T, 2);
  // measured (8 sequences x 2 K context, 4 query heads per KV head): 17.8 us against 35.7 us for
  // the CUDA-core form; also ahead at batch 1 in the two-launch form, so it is the default
  // wherever it exists
  const bool use_mma = mma_ok && mode != 1;
  const int S = use_mma ? S_mma : pick_splits(B, Hkv, T);
  float *po = static_cast<float *>(workspace);
  float *pml = po + (size_t)B * Hq * S * D;
  if (use_mma) {
    if (rep == 2) return launch_mma<2>(q, kc, vc, out, B, Hq, Hkv, T, Tcap, scale, po, pml, S, length_dev, tickets, ra, st);
    if (rep == 4) return launch_mma<4>(q, kc, vc, out, B, Hq, Hkv, T, Tcap, scale, po, pml, S, length_dev, tickets, ra, st);
    return launch_mma<8>(q, kc, vc, out, B, Hq, Hkv, T, Tcap, scale, po, pml, S, length_dev, tickets, ra, st);
  }
#define CIDER_SDPA_CASE(DV, RV)                                                                   \
  if (D == DV && rep == RV)                                                                       \
    return launch_t<DV, RV>(q, kc, vc, out, B, Hq, Hkv, T, Tcap, scale, po, pml, S, length_dev, tickets, ra, st);
  CIDER_SDPA_CASE(128, 1)
  CIDER_SDPA_CASE(128, 2)
  CIDER_SDPA_CASE(128, 4)
  CIDER_SDPA_CASE(128, 8)
  CIDER_SDPA_CASE(64, 1)
  CIDER_SDPA_CASE(64, 2)
  CIDER_SDPA_CASE(64, 4)
  CIDER_SDPA_CASE(64, 8)
#undef CIDER_SDPA_CASE
  return fail(CIDER_E_SHAPE, "sdpa_decode: Hq/Hkv must be 1, 2, 4 or 8");
}

}  // namespace cider
