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
#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.cuh"

namespace cider {

__device__ unsigned int g_device_status = 0;

namespace {

constexpr int BM = 128;
constexpr int BK = 128;  // bytes (= int8 elements) of K per stage: one 128B swizzle row
constexpr int UMMA_K = 32;
constexpr int kThreads = 192;
constexpr long long kWaitCycles = 4000000000ll;  // ~2 s at boost clock

// W4: the weight operand arrives as packed int4 rows.  TMA puts the BN x 64 packed bytes of
// a stage into the UPPER HALF of the stage's own B tile (kPOff); the converter warps read
// them into registers, meet at a named barrier, and then overwrite the whole tile with the
// int8 expansion - no shared memory beyond the int8 kernels' and the same number of
// stages; one more barrier per stage ("packed bytes have landed").
template <int BN, bool W4 = false>
struct Cfg {
  static constexpr int kStages = BN == 256 ? 4 : (BN == 192 ? 5 : (BN == 128 ? 6 : 8));
  static constexpr int kABytes = BM * BK;
  static constexpr int kBBytes = BN * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kPBytes = BN * (BK / 2);       // packed int4 rows of a stage
  static constexpr int kPOff = kBBytes - kPBytes;      // where they land inside the B tile
  static constexpr int kTmemCols = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);  // a power of two
  static constexpr int kEpiBytes = 4 * BN * 8;  // per epilogue warp: BN fp32 scales + BN fp32 bias
  static constexpr int kBarBytes = (2 * kStages + 5 + (W4 ? kStages : 0)) * 8 + 16;
  static constexpr int kStoreBytes = 4 * 4096;  // per epilogue warp: one [32 x 128 B] output box
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kEpiBytes + kBarBytes + 1024;
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
  int tma_store;  // output goes through shared memory + TMA (needs 16-byte aligned rows)
  // split-K (single-CTA kernel, raw int32 output only): when split_mtiles > 0 the output is
  // [splits * split_mtiles * 128, N], M counts those rows, and M tile mt covers rows
  // (mt % split_mtiles) * 128 of A over K blocks [s * kb_per_split, ...), s = mt / split_mtiles
  int split_mtiles, kb_per_split;
  // split-K of the raw int32 product WITHOUT slabs: every (tile, piece) adds its int32 partial
  // tile into the zeroed [M_real, N] result with TMA reduce-adds (integer adds commute: exact
  // and deterministic); the rows of tile mt are then (mt % split_mtiles) * 128 of the result
  int reduce_out, M_real;
  // W4A8: the weight operand as packed int4 rows [N, K/2] (byte j of row n holds k = 2j in its
  // high and k = 2j + 1 in its low nibble, value + 8); expanded to int8 inside the kernel
  const uint8_t *w4;
  // SwiGLU epilogue of the per-channel kernels (see GemmArgs::rowmax): out_cols is the width of
  // the output matrix (N, or N / 2 with the SwiGLU epilogue)
  float *rowmax;
  int out_cols;
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
// Arrive without release semantics, for hand-overs whose payload is ordered by other
// means (tcgen05.wait::ld + tcgen05.fence for TMEM reads): a release arrive may wait
// for every memory operation of the thread still in flight, and the per-group
// epilogue always has a scale row in flight.
__device__ __forceinline__ void mbar_arrive_relaxed(uint32_t bar) {
  asm volatile("mbarrier.arrive.relaxed.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// (A suspend-time hint on the poll - the thread stays suspended until the phase completes - was
// measured 2-4 % slower in every kernel of this file than the plain poll.)
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
// One lane of the (converged) warp: the whole warp runs an issue loop so that its control flow,
// barrier addresses and descriptors are warp-uniform (the tensor-core instructions take their
// operands from the uniform register file: computed by one lane of a divergent branch they
// would be moved there one by one, with the latency of each move in the issue path), and
// this lane alone executes the single-thread instructions.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
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
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_ldn(uint32_t taddr, uint32_t (&r)[32]) { tc_ld32(taddr, r); }
__device__ __forceinline__ void tc_ldn(uint32_t taddr, uint32_t (&r)[16]) { tc_ld16(taddr, r); }
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

// ------------------------------------------------- W4A8: int4 -> int8 in shared memory
// The weight operand of a W4A8 GEMM never exists as int8 in global memory: TMA brings the
// packed rows of a stage (half the bytes of int8) into the upper half of the stage's B tile,
// converter warps expand the nibbles with a few logic operations and write the int8 tile
// over it in exactly the layout TMA would have produced for int8 weights (8-row
// x 128-byte atoms, 16-byte chunks XOR-swizzled by the row), make it visible to the tensor
// core's reads (fence.proxy.async) and arrive on the stage's "full" barrier beside the TMA
// bytes of the activation tile.  The reference unpacks in its fragment load the same way
// (cider/kernels/w4a8_matmul.metal:47-70).  (Reading the packed rows from global memory
// into registers several stages ahead instead - no packed slot - was tried first: 3.5x
// slower, the loads of different stages did not stay in flight together.)
//
// 16 packed bytes = 32 weights.  Byte b = (w_even + 8) << 4 | (w_odd + 8).  The tile the
// tensor core reads holds 16 * w, and the 8 weights of every packed word in the order
// k0 k2 k4 k6 k1 k3 k5 k7:
//   * a nibble n = w + 8 in the HIGH half of a byte is the byte 16 n, and 16 n XOR 0x80 is
//     16 n - 128 = 16 w as a two's complement int8 - so the high nibbles of a word (its
//     even k) become four finished int8 values with one AND-XOR, the low nibbles (odd k) with
//     a shift and the same AND-XOR: three instructions per eight weights and no byte permutes;
//   * the activation tile must then have the same k order - the quantiser in front of these
//     kernels writes it (launch_quantize_per_token_perm8) - and the integer sums come out 16 times
//     too large, exactly (|16 acc| < 2^31 for K up to 2^17): the epilogues fold the factor 1/16,
//     a power of two, into the row scale (per-channel) or the group scale (per-group), which
//     changes no rounding.
__device__ __forceinline__ void w4_expand(const uint4 v, uint32_t (&o)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = (w[i] & 0xF0F0F0F0u) ^ 0x80808080u;             // k0 k2 k4 k6
    o[2 * i + 1] = ((w[i] << 4) & 0xF0F0F0F0u) ^ 0x80808080u;  // k1 k3 k5 k7
  }
}
constexpr float kW4Unscale = 0.0625f;  // the factor 16 of the expanded weights, taken out again
__device__ __forceinline__ void group_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Arrival of a converter warp on the stage's "full" barrier (possibly in the other CTA of
// the pair).  Relaxed: the payload - the warp's shared-memory writes - is ordered for the
// tensor core by the fence.proxy.async in front of it; a release at cluster scope costs a
// full memory fence per stage (measured: it made every stage wait ~1 us).
__device__ __forceinline__ void mbar_arrive_conv(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// Converter role: CT threads expand BROWS packed weight rows x 64 bytes (128 k) per stage.
// TMA has put the packed rows of stage s into the upper half of the stage's own B tile
// (`smem_b + s * b_stage_bytes + p_off`, row pitch 64 bytes, no swizzle) and completed
// pfull_bar[s]; the producer issued that copy only after the MMAs that read the tile's
// previous contents had retired.  The expansion is in place: every converter thread first
// takes its packed pieces into registers, all of them meet at named barrier `bar_id`, and
// only then is the tile overwritten with int8.  Thread ctid owns 16-byte chunk (ctid & 3) of
// rows (ctid >> 2) + pass * CT/4: a quarter warp reads 128 contiguous packed bytes and writes
// 8 different 16-byte bank groups.  `total` = stages this CTA goes through (its tiles x K blocks).
// `first` / `step`: a group of CT converter threads takes the fills first, first + step, ...
// (two groups taking alternate stages keep two stages in flight: the proxy fence and the barrier of
// one stage then overlap the loads and the arithmetic of the next; needs kStages % step == 0)
template <int BROWS, int CT, int kStages>
__device__ __forceinline__ void w4_converter(int total, uint8_t *smem_b, int b_stage_bytes, int p_off,
                                             uint64_t *pfull_bar, uint32_t full_bar0_cluster, volatile int *abort_s,
                                             int ctid, int bar_id, int first = 0, int step = 1) {
  constexpr int RPP = CT / 4;      // rows per pass
  constexpr int P = BROWS / RPP;   // 16-byte pieces per thread and stage
  static_assert(BROWS % RPP == 0, "converter threads must tile the weight rows");
  const int row0 = ctid >> 2, chunk = ctid & 3, lane = ctid & 31;
  int stage = first;
  uint32_t phase = 0;
  for (int it = first; it < total; it += step) {
    // (a wait that ran out: every converter thread sees the abort flag and leaves here, so
    // nobody is left alone at the named barrier below for longer than its own wait)
    const bool ok = mbar_wait(smem_u32(&pfull_bar[stage]), phase, abort_s);
    uint8_t *bs = smem_b + stage * b_stage_bytes;
    const uint8_t *ps_base = bs + p_off + row0 * (BK / 2) + chunk * 16;
    uint4 v[P];
#pragma unroll
    for (int ps = 0; ps < P; ++ps)
      v[ps] = ok ? *reinterpret_cast<const uint4 *>(ps_base + ps * RPP * (BK / 2)) : make_uint4(0, 0, 0, 0);
    // all packed bytes of the tile are in registers
    group_bar_sync(bar_id, CT);
    if (!ok) return;
#pragma unroll
    for (int ps = 0; ps < P; ++ps) {
      const int r = ps * RPP + row0;
      uint32_t o[8];
      w4_expand(v[ps], o);
      uint8_t *rowp = bs + (r >> 3) * 1024 + (r & 7) * 128;
      *reinterpret_cast<uint4 *>(rowp + (((2 * chunk) ^ (r & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
      *reinterpret_cast<uint4 *>(rowp + (((2 * chunk + 1) ^ (r & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
    }
    // generic-proxy accesses of the tile, before the tensor core's (and, a ring turn later,
    // TMA's) async-proxy accesses
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0) mbar_arrive_conv(full_bar0_cluster + 8u * stage);
    stage += step;
    if (stage >= kStages) {
      stage -= kStages;
      phase ^= 1u;
    }
  }
}

// ------------------------------------------------------ shared tile epilogue
// Output store through shared memory + TMA.  A thread owns one accumulator row,
// so direct stores from registers make every warp-wide store touch 32 different
// rows (32 half-filled sectors); measured on the headline shape that costs ~45 us
// of a 185 us GEMM.  Instead each epilogue warp assembles a [32 rows x 128 bytes]
// box (64 fp16 or 32 int32 columns) in a 4 KB staging buffer, written with the
// 128-byte swizzle so the 16-byte pieces of the eight rows of a quarter-warp fall
// into different banks, and one lane hands the box to TMA, which writes whole
// 128-byte lines and clips rows / columns outside the matrix.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Store one [32 rows x 128 bytes] unit held as out[32] per thread (row m = m_box +
// lane, first column nu): through the staging buffer and TMA when the output
// allows it, else straight from registers with bounds checks.
template <int EPI>
__device__ __forceinline__ void store_unit(const TcParams &p, const CUtensorMap *tma_c, const uint32_t (&out)[32],
                                           int m, int m_box, int nu, uint8_t *stage_buf, int lane) {
  const int m_lim = p.reduce_out ? p.M_real : p.M;
  const bool row_ok = m < m_lim;
  if (p.tma_store) {
    // the previous box must have been read out of the staging buffer
    if (lane == 0) tma_store_wait_read();
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 8; ++j)
      *reinterpret_cast<uint4 *>(stage_buf + lane * 128 + ((j ^ (lane & 7)) << 4)) =
          make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    if (lane == 0 && nu < p.out_cols && m_box < m_lim) {
      if (p.reduce_out) tma_reduce_add_2d(tma_c, smem_u32(stage_buf), nu, m_box);
      else tma_store_2d(tma_c, smem_u32(stage_buf), nu, m_box);
      tma_store_commit();
    }
  } else if (row_ok) {
    if (EPI == (int)Epi::kRawInt32) {
      int32_t *orow = reinterpret_cast<int32_t *>(p.out) + (int64_t)m * p.out_cols + nu;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (p.vec_store && nu + 4 * j + 4 <= p.out_cols) {
          *reinterpret_cast<uint4 *>(orow + 4 * j) =
              make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (nu + 4 * j + i < p.out_cols) orow[4 * j + i] = (int32_t)out[4 * j + i];
        }
      }
    } else {
      __half *orow = reinterpret_cast<__half *>(p.out) + (int64_t)m * p.out_cols + nu;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (p.vec_store && nu + 8 * j + 8 <= p.out_cols) {
          *reinterpret_cast<uint4 *>(orow + 8 * j) =
              make_uint4(out[4 * j], out[4 * j + 1], out[4 * j + 2], out[4 * j + 3]);
        } else {
          const __half *hs = reinterpret_cast<const __half *>(&out[4 * j]);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (nu + 8 * j + i < p.out_cols) orow[8 * j + i] = hs[i];
        }
      }
    }
  }
}

// Drains NCOLS accumulator columns of this warp's 32 TMEM lanes starting at
// `taddr`, applies the epilogue and stores rows [m_box, m_box+32) x columns
// [n0, n0+NCOLS).  `m` = m_box + lane is this thread's row.
template <int EPI, int NCOLS>
__device__ __forceinline__ void epilogue_tile(const TcParams &p, const CUtensorMap *tma_c, uint32_t taddr,
                                              int m, int m_box, int n0, float sa_m, const float *sw_s,
                                              const float *bias_s, uint8_t *stage_buf, int lane) {
  constexpr int kUnitCols = EPI == (int)Epi::kRawInt32 ? 32 : 64;  // 128 bytes of output per row
  if constexpr (EPI == (int)Epi::kPerChannel && NCOLS % 128 == 0) {
    if (p.rowmax != nullptr) {
      // SwiGLU: 64 accumulator columns are 32 gate columns and their 32 up columns; two such
      // units give the 64 outputs of one 128-byte box row
      __half2 hmax = __float2half2_rn(0.0f);
#pragma unroll 1
      for (int v = 0; v < NCOLS / 128; ++v) {
        uint32_t res[32];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          uint32_t gu[32];  // 16 words of gate halves, 16 words of up halves
#pragma unroll
          for (int hf = 0; hf < 2; ++hf) {
            uint32_t r[32];
            const int c0 = v * 128 + w * 64 + hf * 32;
            tc_ld32(taddr + c0, r);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float4 s4 = *reinterpret_cast<const float4 *>(sw_s + c0 + 4 * j);
              const float4 b4 = *reinterpret_cast<const float4 *>(bias_s + c0 + 4 * j);
              const float v0 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 0]), sa_m), s4.x, b4.x);
              const float v1 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 1]), sa_m), s4.y, b4.y);
              const float v2 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 2]), sa_m), s4.z, b4.z);
              const float v3 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 3]), sa_m), s4.w, b4.w);
              __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
              gu[hf * 16 + 2 * j] = *reinterpret_cast<uint32_t *>(&h01);
              gu[hf * 16 + 2 * j + 1] = *reinterpret_cast<uint32_t *>(&h23);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // the roundings of an fp16 linear output, an fp16 silu and an fp16 multiply
            const float2 g = __half22float2(*reinterpret_cast<const __half2 *>(&gu[i]));
            const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&gu[16 + i]));
            __half2 h = __floats2half2_rn(silu_to_half(g.x) * b.x, silu_to_half(g.y) * b.y);
            res[w * 16 + i] = *reinterpret_cast<uint32_t *>(&h);
            hmax = __hmax2(hmax, __habs2(h));  // exact: |.| and max commute with the widening conversion
          }
        }
        store_unit<EPI>(p, tma_c, res, m, m_box, (n0 + v * 128) >> 1, stage_buf, lane);
      }
      // columns past N contribute zeros (their scales and biases are zero); rows past M are not counted
      const float amax = fmaxf(__low2float(hmax), __high2float(hmax));
      if (m < p.M && amax > 0.0f) atomicMax(reinterpret_cast<unsigned int *>(p.rowmax + m), __float_as_uint(amax));
      return;
    }
  }
#pragma unroll 1
  for (int u = 0; u < NCOLS / kUnitCols; ++u) {
    uint32_t out[32];
    if (EPI == (int)Epi::kRawInt32) {
      tc_ld32(taddr + u * 32, out);
      tc_wait_ld();
    } else {
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t r[32];
        const int c0 = u * 64 + hf * 32;
        tc_ld32(taddr + c0, r);
        tc_wait_ld();
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float4 s4 = *reinterpret_cast<const float4 *>(sw_s + c0 + 4 * j);
          const float4 b4 = *reinterpret_cast<const float4 *>(bias_s + c0 + 4 * j);
          const float v0 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 0]), sa_m), s4.x, b4.x);
          const float v1 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 1]), sa_m), s4.y, b4.y);
          const float v2 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 2]), sa_m), s4.z, b4.z);
          const float v3 = __fmaf_rn(__fmul_rn(__int2float_rn((int)r[4 * j + 3]), sa_m), s4.w, b4.w);
          __half2 h01 = __floats2half2_rn(v0, v1), h23 = __floats2half2_rn(v2, v3);
          out[hf * 16 + 2 * j] = *reinterpret_cast<uint32_t *>(&h01);
          out[hf * 16 + 2 * j + 1] = *reinterpret_cast<uint32_t *>(&h23);
        }
      }
    }
    store_unit<EPI>(p, tma_c, out, m, m_box, n0 + u * kUnitCols, stage_buf, lane);
  }
}

// ------------------------------------------------------------------ kernel
// W4: packed int4 weight rows, expanded into the B half of every stage by converter warps
// (warps 6 and up: 128 threads, 256 for the 256-column tile) - see w4_converter.
template <int BN>
__host__ __device__ constexpr int conv_threads() { return BN == 256 ? 256 : 128; }
template <int BN, int EPI, bool W4 = false>
__global__ void __launch_bounds__(W4 ? kThreads + conv_threads<BN>() : kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
               const __grid_constant__ CUtensorMap tma_c, const TcParams p) {
  using C = Cfg<BN, W4>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint8_t *smem_a = smem;                                 // kStages x [128 x 128B]
  uint8_t *smem_b = smem + kStages * C::kABytes;          // kStages x [BN x 128B]
  uint8_t *store_s = smem + kStages * C::kStageBytes;     // [4 warps][4 KB], 1024-byte aligned
  float *epi_s = reinterpret_cast<float *>(store_s + C::kStoreBytes);  // [4 warps][2][BN]
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(epi_s) + C::kEpiBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kStages;
  uint64_t *tmem_full_bar = bars + 2 * kStages;       // [2]
  uint64_t *tmem_empty_bar = bars + 2 * kStages + 2;  // [2]
  uint64_t *drain_bar = bars + 2 * kStages + 4;
  uint64_t *pfull_bar = bars + 2 * kStages + 5;       // W4: [kStages]
  uint32_t *tmem_ptr_s = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 5 + (W4 ? kStages : 0));
  volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_ptr_s + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (p.M + BM - 1) / BM, num_n = (p.N + BN - 1) / BN;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  // per-group: accumulator hand-over every `gs` of K (gs is a multiple of 64)
  const int mma_per_group = EPI == (int)Epi::kPerGroup ? p.gs / UMMA_K : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), W4 ? 1 + 2 : 1);  // TMA + the two warps of one converter group
      mbar_init(smem_u32(&empty_bar[s]), 1);
      if (W4) mbar_init(smem_u32(&pfull_bar[s]), 1);
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
  // Programmatic dependent launch: the next kernel of the stream may start its own
  // set-up now; it waits (as the roles below do) before touching dependent data.
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      pdl_wait();  // the operands may come from the kernel before this one
      int stage = 0;
      uint32_t phase = 0;
      uint32_t fills = 0;  // total fills issued
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mt = t / num_n, kb_begin = 0, kb_end = num_kb;
        const int n0 = (t % num_n) * BN;
        if (p.split_mtiles > 0) {
          kb_begin = (mt / p.split_mtiles) * p.kb_per_split;
          kb_end = min(num_kb, kb_begin + p.kb_per_split);
          mt %= p.split_mtiles;
        }
        const int m0 = mt * BM;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_s)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, W4 ? C::kABytes : C::kStageBytes);
          tma_load_2d(smem_u32(smem_a + stage * C::kABytes), &tma_a, fb, kb * BK, m0);
          if (W4) {  // packed int4 rows: their own slot and barrier; the converters take it from there
            const uint32_t pb = smem_u32(&pfull_bar[stage]);
            mbar_expect_tx(pb, C::kPBytes);
            tma_load_2d(smem_u32(smem_b + stage * C::kBBytes + C::kPOff), &tma_b, pb, kb * (BK / 2), n0);
          } else {
            tma_load_2d(smem_u32(smem_b + stage * C::kBBytes), &tma_b, fb, kb * BK, n0);
          }
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
          if (W4) {  // the packed rows of the same fill
            while (!mbar_try_wait(smem_u32(&pfull_bar[s]), par) && clock64() - t0 < kWaitCycles) {
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    // (the whole warp walks the loop, one elected lane issues: see elect_one)
    {
      const uint32_t issuer = elect_one();
      const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
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
        int kb_count = num_kb;
        if (p.split_mtiles > 0) {
          const int kb_begin = ((t / num_n) / p.split_mtiles) * p.kb_per_split;
          kb_count = min(num_kb, kb_begin + p.kb_per_split) - kb_begin;
        }
        for (int kb = 0; kb < kb_count && ok; ++kb) {
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
            const uint32_t d_tmem = tmem_base_u + buf * BN;
            // advance 32 bytes of K inside the swizzle atom: +2 in 16-byte units
            if (issuer)
              tc_mma_i8(d_tmem, a_desc + (uint64_t)(k * (UMMA_K >> 4)),
                        b_desc + (uint64_t)(k * (UMMA_K >> 4)), idesc, fresh ? 0u : 1u);
            fresh = false;
            if (EPI == (int)Epi::kPerGroup && ++in_group == (uint32_t)mma_per_group) {
              // group complete: hand this accumulator to the epilogue, move on
              if (issuer) tc_commit(smem_u32(&tmem_full_bar[buf]));
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
          if (issuer) tc_commit(smem_u32(&empty_bar[stage]));  // stage reusable once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (EPI != (int)Epi::kPerGroup && ok) {
          if (issuer) tc_commit(smem_u32(&tmem_full_bar[buf]));
          ++handover;
        }
      }
      // drain: every MMA issued by this thread has retired once this commit lands
      if (issuer) tc_commit(smem_u32(drain_bar));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(drain_bar), 0) && clock64() - t0 < kWaitCycles) {
        }
      }
    }
  } else if (warp >= 6) {
    // ------------------------------------------- int4 -> int8 converters (W4 only)
    if constexpr (W4) {
      pdl_wait();
      const int first = (int)blockIdx.x, stride = (int)gridDim.x;
      const int my_tiles = first < num_tiles ? (num_tiles - first + stride - 1) / stride : 0;
      // groups of two warps take the stages in turn (see w4_converter)
      constexpr int kGroups = conv_threads<BN>() / 64;
      static_assert(kStages % kGroups == 0, "the converter groups must divide the stage count");
      const int ctid = (int)threadIdx.x - kThreads, grp = ctid >> 6;
      w4_converter<BN, 64, kStages>(my_tiles * num_kb, smem_b, C::kBBytes, C::kPOff, pfull_bar,
                                    smem_u32(&full_bar[0]), abort_s, ctid & 63, 15 - grp, grp, kGroups);
    }
  } else {
    // ------------------------------------------------------------ epilogue
    pdl_wait();  // scales may come from, and the output may still be read by, earlier kernels
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int ew = warp - 2;
    float *sw_s = epi_s + ew * 2 * BN;
    float *bias_s = sw_s + BN;
    uint32_t handover = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
      const int mt_all = t / num_n;
      const int m0 = (p.reduce_out ? mt_all % p.split_mtiles : mt_all) * BM, n0 = (t % num_n) * BN;
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < (p.reduce_out ? p.M_real : p.M);
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
      epilogue_tile<EPI, BN>(p, &tma_c, tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN, m, m0 + q * 32, n0,
                             W4 ? sa_m * kW4Unscale : sa_m, sw_s, bias_s, store_s + (warp - 2) * 4096, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&tmem_empty_bar[buf]));
      ++handover;
    }
  }

  // output boxes still being read out of the staging buffers
  if (warp >= 2 && warp < 6 && lane == 0) tma_store_wait_read();

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

// --------------------------------------------------- CTA-pair (cta_group::2) variant
// Two CTAs of a cluster (two SMs) own one 256 x 256 tile: CTA r loads rows
// [m0 + 128 r, +128) of A and rows [n0 + 128 r, +128) of B into its own shared
// memory; the pair's leader (rank 0) issues tcgen05.mma.cta_group::2 (M256 x N256 x K32),
// for which each SM's tensor core reads its own A half plus both B halves and
// accumulates its 128 rows in its own tensor memory.  Per SM and per MAC that is
// two thirds of the operand bytes of the single-CTA 128 x 256 tile (32 KB instead
// of 48 KB per 128 bytes of K), so six stages fit and more MMA time is covered by
// the copies in flight.  Both accumulator buffers are kept, so the epilogue still
// overlaps the next tile.
//
// Barriers (same layout in both CTAs):
//   full[s]        leader only: 1 arrival (its expect_tx of both CTAs' bytes) + the
//                  bytes of both producers' TMA copies (the peer's copies signal the
//                  leader's barrier through its cluster address)
//   empty[s]       per CTA: the leader's tcgen05.commit arrives on its own and,
//                  with a second commit, on the peer's barrier
//   tmem_full[b]   per CTA, same two commits
//   tmem_empty[b]  leader only: 8 arrivals (4 epilogue warps of each CTA; the
//                  peer's arrive remotely)
// No load in this kernel carries a multicast qualifier.
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Arrival on a (possibly remote) barrier of the CTA pair.  Relaxed: the only thing
// the waiter (the MMA issuer) learns is that this warp's tcgen05.ld of the
// accumulator has completed, which tcgen05.wait::ld + tcgen05.fence already
// order; a release at cluster scope would add a memory fence per hand-over (it
// showed up as the top stall of the per-group kernel).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar_cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tc_mma_i8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

template <bool W4 = false>
struct CfgPairT {
  static constexpr int BMP = 256, BNP = 256;  // tile of the CTA pair
  static constexpr int kStages = 6;
  static constexpr int kABytes = 128 * BK;  // per CTA: its 128 rows of A
  static constexpr int kBBytes = 128 * BK;  // per CTA: its 128 rows of B
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kPBytes = 128 * (BK / 2);      // W4, per CTA: its 128 packed int4 rows of a stage
  static constexpr int kPOff = kBBytes - kPBytes;     // ... landing in the upper half of its B tile
  static constexpr int kTmemCols = 512;
  static constexpr int kEpiBytes = 4 * BNP * 8;
  static constexpr int kStoreBytes = 4 * 4096;
  static constexpr int kBarBytes = (2 * kStages + 5 + (W4 ? kStages : 0)) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreBytes + kEpiBytes + kBarBytes + 1024;
};
using CfgPair = CfgPairT<false>;

// W4: the weight operand comes as packed int4 rows; six more warps per CTA (warps 6..11, three
// groups of two that take the stages in turn) expand this CTA's 128 weight rows of every stage
// into the B half of the stage (see w4_converter); the producer then only loads A, and a stage is "full" when the A bytes of
// both CTAs have landed and the four converter warps that own the stage (two per CTA) have arrived.
constexpr int kConvThreadsPair = 192;  // three groups of two warps
template <int EPI, bool W4>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(W4 ? kThreads + kConvThreadsPair : kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                    const __grid_constant__ CUtensorMap tma_c, const TcParams p) {
  using C = CfgPairT<W4>;
  constexpr int kStages = C::kStages;
  constexpr int BNP = C::BNP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint8_t *smem_a = smem;
  uint8_t *smem_b = smem + kStages * C::kABytes;
  uint8_t *store_s = smem + kStages * C::kStageBytes;  // [4 warps][4 KB], 1024-byte aligned
  float *epi_s = reinterpret_cast<float *>(store_s + C::kStoreBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(epi_s) + C::kEpiBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kStages;
  uint64_t *tmem_full_bar = bars + 2 * kStages;
  uint64_t *tmem_empty_bar = bars + 2 * kStages + 2;
  uint64_t *drain_bar = bars + 2 * kStages + 4;
  uint64_t *pfull_bar = bars + 2 * kStages + 5;        // W4: [kStages], per CTA
  uint32_t *tmem_ptr_s = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 5 + (W4 ? kStages : 0));
  volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_ptr_s + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int num_m = (p.M + C::BMP - 1) / C::BMP, num_n = (p.N + BNP - 1) / BNP;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), W4 ? 1 + 2 * 2 : 1);  // TMA + the two warps of one converter group in each CTA
      mbar_init(smem_u32(&empty_bar[s]), 1);
      if (W4) mbar_init(smem_u32(&pfull_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 8);
    }
    mbar_init(smem_u32(drain_bar), 1);
    *abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_ptr_s)),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();  // both CTAs' barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr_s;
  // Programmatic dependent launch: the next kernel of the stream may start its own
  // set-up now; it waits (as the roles below do) before touching dependent data.
  pdl_launch_dependents();

  if (warp == 0) {
    // ---------------------------------------------- producer (both CTAs)
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      pdl_wait();  // the operands may come from the kernel before this one
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < num_tiles; t += num_pairs) {
        const int m0 = (t / num_n) * C::BMP + (int)rank * 128;
        const int n0 = (t % num_n) * BNP + (int)rank * 128;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_s)) {
            ok = false;
            break;
          }
          // bytes of both CTAs are counted on the leader's barrier
          const uint32_t fb = map_to_cta(smem_u32(&full_bar[stage]), 0);
          if (leader) mbar_expect_tx(smem_u32(&full_bar[stage]), 2 * (W4 ? C::kABytes : C::kStageBytes));
          tma_load_2d_pair(smem_u32(smem_a + stage * C::kABytes), &tma_a, fb, kb * BK, m0);
          if (W4) {  // this CTA's packed int4 rows: its own slot and barrier
            const uint32_t pb = smem_u32(&pfull_bar[stage]);
            mbar_expect_tx(pb, C::kPBytes);
            tma_load_2d(smem_u32(smem_b + stage * C::kBBytes + C::kPOff), &tma_b, pb, kb * (BK / 2), n0);
          } else {
            tma_load_2d_pair(smem_u32(smem_b + stage * C::kBBytes), &tma_b, fb, kb * BK, n0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          // gave up: the full barrier lives in the leader, so the peer cannot watch
          // it; let copies already issued land before this CTA tears down (~1 ms)
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {
          }
          break;
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------- MMA issuer (leader CTA only)
    // (the whole warp walks the loop, one elected lane issues: see elect_one)
    if (leader) {
      const uint32_t issuer = elect_one();
      const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      constexpr uint32_t idesc = make_idesc(256, BNP);
      int stage = 0;
      uint32_t phase = 0, handover = 0;
      bool ok = true;
      for (int t = pair; t < num_tiles && ok; t += num_pairs) {
        const uint32_t buf = handover & 1u;
        if (!mbar_wait(smem_u32(&tmem_empty_bar[buf]), ((handover >> 1) & 1u) ^ 1u, abort_s)) {
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&full_bar[stage]), phase, abort_s)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_desc = make_smem_desc(smem_u32(smem_a + stage * C::kABytes));
          const uint64_t b_desc = make_smem_desc(smem_u32(smem_b + stage * C::kBBytes));
          const uint32_t empty_l = smem_u32(&empty_bar[stage]), empty_r = map_to_cta(empty_l, 1);
          if (issuer) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              tc_mma_i8_pair(tmem_base_u + buf * BNP, a_desc + (uint64_t)(k * (UMMA_K >> 4)),
                             b_desc + (uint64_t)(k * (UMMA_K >> 4)), idesc, (kb | k) ? 1u : 0u);
            tc_commit_pair(empty_l);
            tc_commit_pair(empty_r);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          const uint32_t tfull_l = smem_u32(&tmem_full_bar[buf]), tfull_r = map_to_cta(tfull_l, 1);
          if (issuer) {
            tc_commit_pair(tfull_l);
            tc_commit_pair(tfull_r);
          }
          ++handover;
        }
      }
      if (issuer) tc_commit_pair(smem_u32(drain_bar));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(drain_bar), 0) && clock64() - t0 < kWaitCycles) {
        }
      }
    }
  } else if (warp >= 6) {
    // ---------------------------------------------- int4 -> int8 converters (W4 only, both CTAs)
    if constexpr (W4) {
      pdl_wait();  // the packed rows may come from a repacking kernel just before this one
      const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
      // groups of two warps take the stages in turn (three stages in flight; one warp per stage and
      // six in flight measured 3 % slower, one group of four warps 11 % slower)
      constexpr int kGroups = kConvThreadsPair / 64;
      static_assert(kStages % kGroups == 0, "the converter groups must divide the stage count");
      const int ctid = (int)threadIdx.x - kThreads, grp = ctid >> 6;
      w4_converter<128, 64, kStages>(my_tiles * num_kb, smem_b, C::kBBytes, C::kPOff, pfull_bar,
                                     map_to_cta(smem_u32(&full_bar[0]), 0), abort_s, ctid & 63, 15 - grp, grp,
                                     kGroups);
    }
  } else {
    // ---------------------------------------------- epilogue (both CTAs)
    pdl_wait();
    const int q = warp & 3;
    float *sw_s = epi_s + (warp - 2) * 2 * BNP;
    float *bias_s = sw_s + BNP;
    uint32_t handover = 0;
    for (int t = pair; t < num_tiles; t += num_pairs) {
      const int m0 = (t / num_n) * C::BMP + (int)rank * 128, n0 = (t % num_n) * BNP;
      const int m = m0 + q * 32 + lane;
      const bool row_ok = m < p.M;
      float sa_m = 0.0f;
      if (EPI != (int)Epi::kRawInt32) {
        sa_m = row_ok ? __ldg(p.sa + m) : 0.0f;
        __syncwarp();
        for (int j = lane; j < BNP; j += 32) {
          const int n = n0 + j;
          sw_s[j] = n < p.N ? sw_load(p.sw, p.sw_half, n) : 0.0f;
          bias_s[j] = (p.bias != nullptr && n < p.N) ? __half2float(p.bias[n]) : 0.0f;
        }
        __syncwarp();
      }
      const uint32_t buf = handover & 1u;
      uint32_t got = 0;
      if (lane == 0) got = mbar_wait(smem_u32(&tmem_full_bar[buf]), (handover >> 1) & 1u, abort_s);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      epilogue_tile<EPI, BNP>(p, &tma_c, tmem_base + ((uint32_t)(q * 32) << 16) + buf * BNP, m, m0 + q * 32, n0,
                              W4 ? sa_m * kW4Unscale : sa_m, sw_s, bias_s, store_s + (warp - 2) * 4096, lane);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tmem_empty_bar[buf]), 0));
      ++handover;
    }
  }

  if (warp >= 2 && warp < 6 && lane == 0) tma_store_wait_read();

  // ---- teardown: nobody leaves while its partner may still read its shared
  // memory (the leader's MMAs do) or signal its barriers
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                 "r"((uint32_t)C::kTmemCols)
                 : "memory");
  }
}

// ------------------------------------------------ wide per-group kernel (1 CTA)
// Same operand pipeline as gemm_tc_kernel on a 128 x 128 tile, but the accumulator
// is handed over every `gs` of K: the MMA issuer cycles
// through FOUR 128-column TMEM buffers group by group, and the epilogue promotes
// each group to fp32 registers, accf = fma(float(acc_g), sw[g, n], accf), while the
// next groups' MMAs run (pergroup_int8_gemm.metal:99-172 does the same flush once
// per group).  Four buffers so that three groups of MMAs can be in flight while one
// is promoted.  A single CTA per tile on purpose: with a CTA pair every hand-over
// needs two cross-SM barrier round trips (~1 us each, measured), which at one
// hand-over per 128 bytes of K costs more than the pair saves in operand traffic.
// Sixteen epilogue warps per CTA: warp e reads TMEM lane quarter (warp & 3) and owns
// 32 columns of the tile; four warps share each scheduler - while one waits on its
// TMEM load or a barrier the others do arithmetic.  (Eight warps of 64 columns left
// the schedulers idle two thirds of the time.)  The accumulator is read in the
// 16x256b shape: a lane then holds 4 rows x 8 columns, needs 8 of a group's 32 scales
// (two 16-byte shared-memory reads) and keeps 32 fp32 partial sums as 16 packed pairs.
// Lane l fetches the group scale of column l of its warp four groups ahead into
// registers - a scale row is a dependent L2 / DRAM access per group, fetched one group
// ahead its latency would set the pace - and publishes it, converted to fp32 once, to
// the warp through a shared-memory slot.  The promotion (int->float convert + FMA per
// element and group) is CUDA-core work on top of the tensor work.  What a group costs
// is the length of ONE warp's instruction stream for it (every warp handles every
// group, and a warp issues about once in seven cycles next to its three neighbours),
// so both sides are written for few instructions per group: the epilogue loop has no
// index arithmetic and one warp barrier, the MMA issue loop is specialised on the
// number of MMAs per group.  Measured at M=8192, N=10240, K=2560: 1130 cycles per
// group at gs = 128 with the promotion, 880 without it (operand delivery).
constexpr int kThreadsPg = 64 + 16 * 32;
template <bool W4 = false>
struct CfgPgT {
  static constexpr int BMP = 128, BNP = 128;
  // W4: an even stage count, so that the two converter warps can each take every other stage
  static constexpr int kStages = W4 ? 4 : 5;
  static constexpr int kPBytes = 128 * (BK / 2);  // W4: packed int4 rows of a stage, in the upper half of its B tile
  static constexpr int kBufs = 4;           // TMEM accumulator buffers of BNP columns
  static constexpr int kABytes = 128 * BK;
  static constexpr int kBBytes = 128 * BK;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kStoreBytes = 8 * 4096;        // one output box per pair of epilogue warps
  static constexpr int kScaleAhead = 4;               // group-scale rows in flight per lane
  static constexpr int kScaleBytes = 16 * 2 * 32 * 4; // per warp: two slots of 32 fp32 scales
  static constexpr int kBiasBytes = 16 * 32 * 4;      // per warp: 32 fp32 bias values
  static constexpr int kBarBytes = (2 * kStages + 2 * kBufs + 1 + (W4 ? kStages : 0)) * 8 + 16;
  static constexpr int kPOff = kBBytes - kPBytes;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kStoreBytes + kScaleBytes + kBiasBytes + kBarBytes + 1024;
};
using CfgPairPg = CfgPgT<false>;

// acc <- fma(float(i0), s, acc.lo), fma(float(i1), s, acc.hi) for two int32 group sums of one
// output column: two conversions and one packed two-lane fp32 fma, each lane an IEEE
// round-to-nearest operation, so the result equals the scalar fmaf() of the oracle bit for
// bit.  sc2 = {s, s} is formed once per group by the caller.  (The conversion by a
// magic-number add - bits of i + 0x4B400000 are the float 12582912 + i - needs an integer
// add and a packed subtraction per pair and measured 3-30 % slower in this loop.)
__device__ __forceinline__ uint64_t promote2(uint32_t i0, uint32_t i1, uint64_t sc2, uint64_t acc) {
  asm("{\n\t.reg .f32 a, b;\n\t.reg .b64 t;\n\t"
      "cvt.rn.f32.s32 a, %1;\n\t"
      "cvt.rn.f32.s32 b, %2;\n\t"
      "mov.b64 t, {a, b};\n\t"
      "fma.rn.f32x2 %0, t, %3, %0;\n\t}"
      : "+l"(acc)
      : "r"(i0), "r"(i1), "l"(sc2));
  return acc;
}
__device__ __forceinline__ float2 unpack2(uint64_t v) { return *reinterpret_cast<const float2 *>(&v); }
// {x, x} as one 64-bit register pair the compiler cannot take apart again
__device__ __forceinline__ uint64_t splat2(float x) {
  uint64_t r;
  asm volatile("mov.b64 %0, {%1, %1};" : "=l"(r) : "f"(x));
  return r;
}

// W4: two more warps (18, 19) expand the packed int4 weight rows of every stage - see w4_converter.
constexpr int kConvThreadsPg = 64;
template <bool W4 = false>
__global__ void __launch_bounds__(W4 ? kThreadsPg + kConvThreadsPg : kThreadsPg, 1)
gemm_tc_pg_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                       const __grid_constant__ CUtensorMap tma_c, const TcParams p) {
  using C = CfgPgT<W4>;
  constexpr int kStages = C::kStages;
  constexpr int BNP = C::BNP;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint8_t *smem_a = smem;
  uint8_t *smem_b = smem + kStages * C::kABytes;
  uint8_t *store_s = smem + kStages * C::kStageBytes;
  float *scale_s = reinterpret_cast<float *>(store_s + C::kStoreBytes);
  float *bias_all = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(scale_s) + C::kScaleBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(bias_all) + C::kBiasBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kStages;
  constexpr int kBufs = C::kBufs;
  uint64_t *tmem_full_bar = bars + 2 * kStages;
  uint64_t *tmem_empty_bar = bars + 2 * kStages + kBufs;
  uint64_t *drain_bar = bars + 2 * kStages + 2 * kBufs;
  uint64_t *pfull_bar = bars + 2 * kStages + 2 * kBufs + 1;  // W4: [kStages]
  uint32_t *tmem_ptr_s = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 2 * kBufs + 1 + (W4 ? kStages : 0));
  volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_ptr_s + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x, num_pairs = gridDim.x;  // tile index start / stride
  const int num_m = (p.M + C::BMP - 1) / C::BMP, num_n = (p.N + BNP - 1) / BNP;
  const int num_tiles = num_m * num_n;
  // split-K: p.M counts the row tiles of all K pieces; tile row mt covers rows
  // (mt % split_mtiles) * 128 of the matrix and K blocks (mt / split_mtiles) * kb_per_split
  // onwards, all pieces the same whole number of groups; its fp32 partial sums (before
  // the row scale and the bias) go to the piece's slab
  const bool split = p.split_mtiles > 0;
  const int num_kb = split ? p.kb_per_split : (p.K + BK - 1) / BK;
  const int groups = split ? p.kb_per_split * BK / p.gs : p.K / p.gs;
  const int mma_per_group = p.gs / UMMA_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), W4 ? 1 + 1 : 1);  // TMA + the converter warp that owns the stage
      mbar_init(smem_u32(&empty_bar[s]), 1);
      if (W4) mbar_init(smem_u32(&pfull_bar[s]), 1);
    }
    for (int b = 0; b < kBufs; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 16);  // one arrival per epilogue warp
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
  // Programmatic dependent launch: the next kernel of the stream may start its own
  // set-up now; it waits (as the roles below do) before touching dependent data.
  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      pdl_wait();  // the operands may come from the kernel before this one
      int stage = 0;
      uint32_t phase = 0;
      for (int t = pair; t < num_tiles; t += num_pairs) {
        const int mt = t / num_n;
        const int m0 = (split ? mt % p.split_mtiles : mt) * C::BMP;
        const int kb0 = split ? (mt / p.split_mtiles) * num_kb : 0;
        const int n0 = (t % num_n) * BNP;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_s)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, W4 ? C::kABytes : C::kStageBytes);
          tma_load_2d(smem_u32(smem_a + stage * C::kABytes), &tma_a, fb, (kb0 + kb) * BK, m0);
          if (W4) {
            const uint32_t pb = smem_u32(&pfull_bar[stage]);
            mbar_expect_tx(pb, C::kPBytes);
            tma_load_2d(smem_u32(smem_b + stage * C::kBBytes + C::kPOff), &tma_b, pb, (kb0 + kb) * (BK / 2), n0);
          } else {
            tma_load_2d(smem_u32(smem_b + stage * C::kBBytes), &tma_b, fb, (kb0 + kb) * BK, n0);
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {
          }
          break;
        }
      }
    }
  } else if (warp == 1) {
    {
      const uint32_t issuer = elect_one();
      const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
      // The issuing thread shares its scheduler with four promotion warps that are busy
      // all the time, so every instruction it executes between two MMAs costs several
      // cycles of tensor-pipe time: the loop is specialised on the MMAs per group (2, 4
      // or 8 for gs = 64, 128, 256) so that the group structure is resolved at compile
      // time, descriptors are formed by one addition, and the only run-time quantities
      // per K block are the stage and the accumulator hand-over count.
      // the weight tile is the 128-row operand and the activation tile the column operand:
      // the accumulator is the transpose of the output tile (see the promotion warps)
      constexpr uint32_t idesc = make_idesc(BNP, C::BMP);
      const uint64_t a_desc0 = make_smem_desc(smem_u32(smem_a));
      const uint64_t b_desc0 = make_smem_desc(smem_u32(smem_b));
      const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
      const uint32_t tfull0 = smem_u32(tmem_full_bar), tempty0 = smem_u32(tmem_empty_bar);
      // MMAs of the last K block (2 or 4); K pieces are whole K blocks
      const int last_nk = split ? BK / UMMA_K : (p.K - (num_kb - 1) * BK) / UMMA_K;
      auto issue = [&](auto mpg_c) {
        constexpr int MPG = decltype(mpg_c)::value;
        int stage = 0;
        uint32_t phase = 0, handover = 0;
        for (int t = pair; t < num_tiles; t += num_pairs) {
          for (int kb = 0; kb < num_kb; ++kb) {
            if (!mbar_wait(full0 + 8u * stage, phase, abort_s)) return;
            tc_fence_after();
            const uint64_t a_desc = a_desc0 + (uint64_t)(stage * (C::kABytes >> 4));
            const uint64_t b_desc = b_desc0 + (uint64_t)(stage * (C::kBBytes >> 4));
            const int nk = kb == num_kb - 1 ? last_nk : BK / UMMA_K;
            if constexpr (MPG == 2) {
              // gs = 64: the two groups of a K block go side by side into ONE buffer of 256
              // columns (two such buffers) and are handed over together - half the barrier
              // rounds per group for the promotion warps and for this loop
              const uint32_t buf = handover & 1u;
              if (!mbar_wait(tempty0 + 8u * buf, ((handover >> 1) & 1u) ^ 1u, abort_s)) return;
              tc_fence_after();
              if (issuer) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  if (2 * h < nk) {
                    const uint32_t d = tmem_base_u + buf * (2 * BNP) + h * BNP;
                    tc_mma_i8(d, b_desc + (uint64_t)(4 * h), a_desc + (uint64_t)(4 * h), idesc, 0u);
                    tc_mma_i8(d, b_desc + (uint64_t)(4 * h + 2), a_desc + (uint64_t)(4 * h + 2), idesc, 1u);
                  }
                }
                tc_commit(tfull0 + 8u * buf);
              }
              ++handover;
              // the K block ends with the hand-over: the first epilogue warp frees the stage
            } else if constexpr (MPG == 4) {
              // gs = 128: two K blocks (two groups) per hand-over, side by side in one buffer of
              // 256 columns; the last hand-over of an odd block count brings one
              const bool first = (kb & 1) == 0, last = (kb & 1) == 1 || kb == num_kb - 1;
              const uint32_t buf = handover & 1u;
              if (first) {
                if (!mbar_wait(tempty0 + 8u * buf, ((handover >> 1) & 1u) ^ 1u, abort_s)) return;
                tc_fence_after();
              }
              if (issuer) {
                const uint32_t d = tmem_base_u + buf * (2 * BNP) + (uint32_t)(kb & 1) * BNP;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                  tc_mma_i8(d, b_desc + (uint64_t)(2 * k), a_desc + (uint64_t)(2 * k), idesc, k == 0 ? 0u : 1u);
                if (last) tc_commit(tfull0 + 8u * buf);
                else tc_commit(empty0 + 8u * stage);  // the stage is free once these MMAs retire
              }
              if (last) ++handover;
            } else {
              const bool opens = MPG == 4 || (kb & 1) == 0;   // first K block of a group
              const bool closes = MPG == 4 || (kb & 1) == 1;  // last K block of a group
              const uint32_t buf = handover % kBufs;
              if (opens) {
                if (!mbar_wait(tempty0 + 8u * buf, ((handover / kBufs) & 1u) ^ 1u, abort_s)) return;
                tc_fence_after();
              }
              if (issuer) {
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)
                  tc_mma_i8(tmem_base_u + buf * BNP, b_desc + (uint64_t)(2 * k), a_desc + (uint64_t)(2 * k), idesc,
                            (k == 0 && opens) ? 0u : 1u);
                if (closes) tc_commit(tfull0 + 8u * buf);
                else tc_commit(empty0 + 8u * stage);  // the stage is free once these MMAs retire
              }
              if (closes) ++handover;
            }
            if (++stage == kStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      };
      if (mma_per_group == 2) issue(std::integral_constant<int, 2>{});
      else if (mma_per_group == 4) issue(std::integral_constant<int, 4>{});
      else issue(std::integral_constant<int, 8>{});
      if (issuer) tc_commit(smem_u32(drain_bar));
      {
        const long long t0 = clock64();
        while (!mbar_try_wait(smem_u32(drain_bar), 0) && clock64() - t0 < kWaitCycles) {
        }
      }
    }
  } else if (warp >= 18) {
    if constexpr (W4) {
      pdl_wait();
      const int my_tiles = pair < num_tiles ? (num_tiles - pair + num_pairs - 1) / num_pairs : 0;
      // each of the two converter warps takes every other stage (see w4_converter)
      static_assert(kStages % (kConvThreadsPg / 32) == 0, "the converter warps must divide the stage count");
      const int ctid = (int)threadIdx.x - kThreadsPg, grp = ctid >> 5;
      w4_converter<128, 32, kStages>(my_tiles * num_kb, smem_b, C::kBBytes, C::kPOff, pfull_bar,
                                     smem_u32(&full_bar[0]), abort_s, ctid & 31, 15 - grp, grp, kConvThreadsPg / 32);
    }
  } else {
    pdl_wait();
    // The accumulator is the TRANSPOSE of the output tile: TMEM lane = weight row (output
    // column n), TMEM column = activation row m (the MMA takes the weight tile as its
    // 128-row operand).  With one TMEM lane per thread (the 32x32b load shape, three times
    // the read rate of the 16x256b shape) all 32 values a thread receives belong to ONE
    // output column, so the group scale sw[g, n] is a single register of that thread:
    // no staging of scales through shared memory, no exchange between lanes.
    const int e = warp - 2;             // 0..15
    const int q = warp & 3;             // the TMEM lane quarter this warp can read: 32 output columns
    const int ch = e >> 2;              // its 32-column chunk of the accumulator: 32 activation rows
    const int hq = q & 1;               // which half of the pair's 64-column output box
    const int pr = ch * 2 + (q >> 1);   // warps (q even, ch) and (q odd, ch) fill one 32-row x 128-byte output box
    float *sa_s = bias_all + e * 32;    // the row scales of this warp's 32 activation rows
    uint8_t *stage_buf = store_s + pr * 4096;
    constexpr int kAhead = C::kScaleAhead;
    // Every instruction of the group loop is executed by 16 warps per group and the warps
    // of a scheduler take turns, so the loop is kept short: specialised on the scale type,
    // a running pointer instead of index arithmetic, and what does not change in the loop is
    // computed here and made opaque, so that it is held in a register instead of being
    // derived again from the thread index in every pass.
    uint32_t fwd = e == 0 && lane == 0, lane0 = lane == 0;
    uint32_t tfull0 = smem_u32(tmem_full_bar), tempty0 = smem_u32(tmem_empty_bar);
    uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + ch * 32;
    asm volatile("" : "+r"(fwd), "+r"(lane0), "+r"(tfull0), "+r"(tempty0), "+r"(taddr0));
    const size_t sw_pitch = (size_t)p.N * (p.sw_half ? 2 : 4);
    auto epilogue = [&](auto half_c) {
      constexpr bool kHalf = decltype(half_c)::value;
      auto to_f32 = [](uint32_t raw) {
        return kHalf ? __half2float(__ushort_as_half((unsigned short)raw)) : __uint_as_float(raw);
      };
      uint32_t handover = 0, kb_base = 0;  // kb_base: K blocks of the tiles before this one
      bool ok = true;
      // No early exit from this loop: the two warps of a pair meet at named barriers
      // once per tile, so a warp that gave up keeps walking the tiles without waiting.
      for (int t = pair; t < num_tiles; t += num_pairs) {
        const int mt = t / num_n;
        const int piece = split ? mt / p.split_mtiles : 0;
        const int m0 = (split ? mt % p.split_mtiles : mt) * C::BMP;
        const int nt0 = (t % num_n) * BNP;
        const int mrow0 = m0 + ch * 32;        // first activation row of this warp
        const int ncol = nt0 + q * 32 + lane;  // the output column of this lane
        const int m_lim = split ? p.M_real : p.M;
        __syncwarp();
        sa_s[lane] = (!split && mrow0 + lane < m_lim) ? __ldg(p.sa + mrow0 + lane) : 0.0f;
        const float bias_n = (p.bias != nullptr && ncol < p.N) ? __half2float(p.bias[ncol]) : 0.0f;
        // Group scales: the lane fetches sw[g, n] kAhead groups before its use (a scale row
        // is a dependent L2 / DRAM access per group; fetched one group ahead its latency
        // would set the pace of the kernel) and keeps the raw bits in registers.
        // Columns past N read column N - 1: their results are never stored.
        const char *swp = reinterpret_cast<const char *>(p.sw) + (size_t)min(ncol, p.N - 1) * (kHalf ? 2 : 4) +
                          (size_t)piece * (size_t)groups * sw_pitch;
        uint32_t pre[kAhead];
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          pre[i] = 0u;
          if (i < groups)
            pre[i] = kHalf ? (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(swp))
                           : __ldg(reinterpret_cast<const uint32_t *>(swp));
          swp += sw_pitch;
        }
        // fp32 partial sums of column n for the 32 activation rows, as packed pairs (rows 2i, 2i + 1)
        uint64_t acc2[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) acc2[i] = 0ull;
        if (ok && p.gs <= 128) {
          // gs = 64 / 128: one hand-over brings two groups (columns 0..127 and 128..255 of one of
          // two 256-column buffers; the last one of an odd group count brings one) - the two
          // groups of a K block (gs = 64) or two K blocks (gs = 128)
          for (int g = 0; g < groups; g += 2) {
            const uint32_t buf = handover & 1u;
            const uint32_t full_b = tfull0 + 8u * buf, par = (handover >> 1) & 1u;
            if (!__all_sync(0xffffffffu, mbar_try_wait(full_b, par))) {
              uint32_t got = 0;
              if (lane0) got = mbar_wait(full_b, par, abort_s);
              if (!__shfl_sync(0xffffffffu, got, 0)) { ok = false; break; }
            }
            tc_fence_after();
            if (fwd) {
              // the MMAs of the hand-over have completed: the shared-memory stage of its (last) K
              // block is free (gs = 128: the first block's stage was freed by the issuing thread)
              const int kb_last = p.gs == 64 ? (g >> 1) : min(g + 1, groups - 1);
              mbar_arrive_relaxed(smem_u32(&empty_bar[(kb_base + (uint32_t)kb_last) % kStages]));
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              if (g + j < groups) {
                uint32_t r[32];
                tc_ld32(taddr0 + buf * (2 * BNP) + j * BNP, r);
                const uint64_t sc2 = splat2(W4 ? to_f32(pre[0]) * kW4Unscale : to_f32(pre[0]));
#pragma unroll
                for (int i = 0; i + 1 < kAhead; ++i) pre[i] = pre[i + 1];
                if (g + j + kAhead < groups)
                  pre[kAhead - 1] = kHalf ? (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(swp))
                                          : __ldg(reinterpret_cast<const uint32_t *>(swp));
                swp += sw_pitch;
                tc_wait_ld();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc2[i] = promote2(r[2 * i], r[2 * i + 1], sc2, acc2[i]);
              }
            }
            tc_fence_before();
            __syncwarp();  // every lane has read the buffer
            if (lane0) mbar_arrive_relaxed(tempty0 + 8u * buf);
            ++handover;
          }
        } else if (ok) {
          for (int g = 0; g < groups; ++g) {
            const uint32_t buf = handover % kBufs;
            const uint32_t full_b = tfull0 + 8u * buf, par = (handover / kBufs) & 1u;
            if (!__all_sync(0xffffffffu, mbar_try_wait(full_b, par))) {
              uint32_t got = 0;
              if (lane0) got = mbar_wait(full_b, par, abort_s);
              if (!__shfl_sync(0xffffffffu, got, 0)) { ok = false; break; }
            }
            tc_fence_after();
            if (fwd) {
              // the MMAs of this group have completed; if it was the last one of its K block
              // the block's shared-memory stage is free for the producer
              const int kend = (g + 1) * p.gs;
              if ((kend % BK) == 0 || g == groups - 1)
                mbar_arrive_relaxed(smem_u32(&empty_bar[(kb_base + (uint32_t)((kend - 1) / BK)) % kStages]));
            }
            uint32_t r[32];
            tc_ld32(taddr0 + buf * BNP, r);
            const uint64_t sc2 = splat2(W4 ? to_f32(pre[0]) * kW4Unscale : to_f32(pre[0]));
#pragma unroll
            for (int i = 0; i + 1 < kAhead; ++i) pre[i] = pre[i + 1];
            if (g + kAhead < groups)
              pre[kAhead - 1] = kHalf ? (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(swp))
                                      : __ldg(reinterpret_cast<const uint32_t *>(swp));
            swp += sw_pitch;
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) acc2[i] = promote2(r[2 * i], r[2 * i + 1], sc2, acc2[i]);
            tc_fence_before();
            __syncwarp();  // every lane has read the buffer
            if (lane0) mbar_arrive_relaxed(tempty0 + 8u * buf);
            ++handover;
          }
        }
        kb_base += (uint32_t)num_kb;
        if (split) {
          // fp32 partial sums of this K piece to its slab [piece][row][N]: a warp store is 32
          // consecutive columns of one row
          if (ok && ncol < p.N) {
            float *slab = reinterpret_cast<float *>(p.out) + (int64_t)piece * p.split_mtiles * C::BMP * p.N + ncol;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const float2 a = unpack2(acc2[i]);
              const int m = mrow0 + 2 * i;
              if (m < m_lim) slab[(int64_t)m * p.N] = a.x;
              if (m + 1 < m_lim) slab[(int64_t)(m + 1) * p.N] = a.y;
            }
          }
          continue;
        }
        // ---- final scale by sa[m], add bias, store this warp's 32 rows x 32 columns
        __syncwarp();
        // rows mrow0 + 4 i .. + 3 of column ncol (sa_s: the same address in every lane, a broadcast)
        auto finish4 = [&](int i, __half (&h)[4]) {
          const float4 sa4 = *reinterpret_cast<const float4 *>(sa_s + 4 * i);
          const float2 a0 = unpack2(acc2[2 * i]), a1 = unpack2(acc2[2 * i + 1]);
          h[0] = __float2half_rn(__fmaf_rn(a0.x, sa4.x, bias_n));
          h[1] = __float2half_rn(__fmaf_rn(a0.y, sa4.y, bias_n));
          h[2] = __float2half_rn(__fmaf_rn(a1.x, sa4.z, bias_n));
          h[3] = __float2half_rn(__fmaf_rn(a1.y, sa4.w, bias_n));
        };
        if (p.tma_store) {
          // the pair's previous box must have been read out of the staging buffer
          if (hq == 0 && lane == 0) tma_store_wait_read();
          group_bar_sync(1 + pr, 64);
          // box row = 128 bytes = the 64 columns of the two warps, 16-byte chunks swizzled by
          // the row; the 32 lanes of a store write 64 consecutive bytes of one row
          uint8_t *dst = stage_buf + (lane & 7) * 2;
          const int chunk = hq * 4 + (lane >> 3);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __half h[4];
            finish4(i, h);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const int j = 4 * i + jj;
              *reinterpret_cast<__half *>(dst + j * 128 + ((chunk ^ (j & 7)) << 4)) = h[jj];
            }
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          group_bar_sync(1 + pr, 64);
          const int nbox = nt0 + (q >> 1) * 64;
          if (hq == 0 && lane == 0 && ok && nbox < p.N && mrow0 < p.M) {
            tma_store_2d(&tma_c, smem_u32(stage_buf), nbox, mrow0);
            tma_store_commit();
          }
        } else if (ok && ncol < p.N) {
          // rows whose pitch TMA cannot describe: element stores, 32 consecutive columns per warp store
          __half *ocol = reinterpret_cast<__half *>(p.out) + ncol;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            __half h[4];
            finish4(i, h);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
              if (mrow0 + 4 * i + jj < p.M) ocol[(int64_t)(mrow0 + 4 * i + jj) * p.N] = h[jj];
          }
        }
      }
    };
    if (p.sw_half) epilogue(std::true_type{});
    else epilogue(std::false_type{});
  }

  if (warp >= 2 && warp < 18 && lane == 0) tma_store_wait_read();
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

// ------------------------------------------------ per-group kernel, 128 x 256 tile (1 CTA)
// The same transposed accumulator and per-group promotion as gemm_tc_pg_kernel on a tile of 128
// weight rows (output columns) x 256 activation rows: 48 KB of operands per K block feed 32 K
// outputs where the 128 x 128 tile pulls 32 KB for 16 K, and every weight tile is fetched half as
// often.  The accumulator is two independent halves (activation rows 0..127 and 128..255), each
// with its own two 128-column TMEM buffers (one group per hand-over), its own barriers and its
// own eight promotion warps holding 64 fp32 partial sums per thread; the MMAs of a K block go to
// the two halves one after the other.  The accumulator is read 16 words at a time: 64 partial
// sums and a 32-word load do not fit the 96 registers a thread of 18 warps gets (giving the
// promotion warps more with setmaxnreg made the compiler spill in the control warps instead), so
// a group costs a warp four load round trips and the promotion, not the operands, sets the pace:
// faster than the 128 x 128 kernel only for weights of ~48 MB and more (see launch_gemm_tc).
// Results leave the registers as 2-byte stores, 32 consecutive output columns of one row per warp
// store (64 bytes, two whole sectors): no staging buffer, the shared memory holds four 48 KB
// operand stages.  int8 weights, no split-K; the other cases stay with gemm_tc_pg_kernel.
struct CfgPg2 {
  static constexpr int BMP = 256, BNP = 128;
  static constexpr int kStages = 4;
  static constexpr int kABytes = 256 * BK;  // activations: two boxes of 128 rows
  static constexpr int kBBytes = 128 * BK;  // weights
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kScaleAhead = 3;
  static constexpr int kSaBytes = 16 * 64 * 4;  // per promotion warp: the row scales of its 64 activation rows
  static constexpr int kBarBytes = (2 * kStages + 4 + 4 + 1) * 8 + 16;
  static constexpr int kSmemBytes = kStages * kStageBytes + kSaBytes + kBarBytes + 1024;
};

constexpr int kLd = 16;  // accumulator words per TMEM load of a promotion warp
__global__ void __launch_bounds__(kThreadsPg, 1)
gemm_tc_pg2_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                   const TcParams p) {
  using C = CfgPg2;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                              ~(uintptr_t)1023);
  uint8_t *smem_a = smem;
  uint8_t *smem_b = smem + kStages * C::kABytes;
  float *sa_all = reinterpret_cast<float *>(smem + kStages * C::kStageBytes);
  uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sa_all) + C::kSaBytes);
  uint64_t *full_bar = bars;
  uint64_t *empty_bar = bars + kStages;
  uint64_t *tmem_full_bar = bars + 2 * kStages;       // [half][buffer]
  uint64_t *tmem_empty_bar = bars + 2 * kStages + 4;  // [half][buffer]
  uint64_t *drain_bar = bars + 2 * kStages + 8;
  uint32_t *tmem_ptr_s = reinterpret_cast<uint32_t *>(bars + 2 * kStages + 9);
  volatile int *abort_s = reinterpret_cast<volatile int *>(tmem_ptr_s + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cta = blockIdx.x, num_ctas = gridDim.x;
  const int num_m = (p.M + C::BMP - 1) / C::BMP, num_n = (p.N + C::BNP - 1) / C::BNP;
  const int num_tiles = num_m * num_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int groups = p.K / p.gs;
  const int mma_per_group = p.gs / UMMA_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(smem_u32(&tmem_full_bar[b]), 1);
      mbar_init(smem_u32(&tmem_empty_bar[b]), 8);  // one arrival per promotion warp of the half
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
  pdl_launch_dependents();
  if (warp == 0) {
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_a)) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tma_b)) : "memory");
      pdl_wait();  // the operands may come from the kernel before this one
      int stage = 0;
      uint32_t phase = 0;
      for (int t = cta; t < num_tiles; t += num_ctas) {
        const int m0 = (t / num_n) * C::BMP, n0 = (t % num_n) * C::BNP;
        bool ok = true;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&empty_bar[stage]), phase ^ 1u, abort_s)) {
            ok = false;
            break;
          }
          const uint32_t fb = smem_u32(&full_bar[stage]);
          mbar_expect_tx(fb, C::kStageBytes);
          // rows past M (a whole box of them, too) arrive as zeros and count their bytes
          tma_load_2d(smem_u32(smem_b + stage * C::kBBytes), &tma_b, fb, kb * BK, n0);
          tma_load_2d(smem_u32(smem_a + stage * C::kABytes), &tma_a, fb, kb * BK, m0);
          tma_load_2d(smem_u32(smem_a + stage * C::kABytes + 128 * BK), &tma_a, fb, kb * BK, m0 + 128);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) {
          const long long t0 = clock64();
          while (clock64() - t0 < 2000000ll) {
          }
          break;
        }
      }
    }
  } else if (warp == 1) {
    // (the whole warp walks the loop, one elected lane issues: see elect_one)
    const uint32_t issuer = elect_one();
    const uint32_t tmem_base_u = __shfl_sync(0xffffffffu, tmem_base, 0);
    // the weight tile is the 128-row operand, 128 activation rows the column operand
    constexpr uint32_t idesc = make_idesc(128, 128);
    const uint64_t a_desc0 = make_smem_desc(smem_u32(smem_a));
    const uint64_t b_desc0 = make_smem_desc(smem_u32(smem_b));
    const uint32_t full0 = smem_u32(full_bar), empty0 = smem_u32(empty_bar);
    const uint32_t tfull0 = smem_u32(tmem_full_bar), tempty0 = smem_u32(tmem_empty_bar);
    const int last_nk = (p.K - (num_kb - 1) * BK) / UMMA_K;  // MMAs of the last K block (2 or 4)
    auto issue = [&](auto mpg_c) {
      constexpr int MPG = decltype(mpg_c)::value;  // MMAs per group: 2, 4 or 8 (gs = 64, 128, 256)
      constexpr int kPerPass = MPG == 2 ? 2 : 4;   // MMAs per half and pass over a K block
      int stage = 0;
      uint32_t phase = 0, hand0 = 0, hand1 = 0;    // hand-overs of the two halves so far
      for (int t = cta; t < num_tiles; t += num_ctas) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(full0 + 8u * stage, phase, abort_s)) return;
          tc_fence_after();
          const uint64_t a_desc = a_desc0 + (uint64_t)(stage * (C::kABytes >> 4));
          const uint64_t b_desc = b_desc0 + (uint64_t)(stage * (C::kBBytes >> 4));
          const int nk = kb == num_kb - 1 ? last_nk : BK / UMMA_K;
          const bool opens = MPG != 8 || (kb & 1) == 0;   // first K block of a group
          const bool closes = MPG != 8 || (kb & 1) == 1;  // last K block of a group
#pragma unroll
          for (int h = 0; h < (MPG == 2 ? 2 : 1); ++h) {  // the groups of the K block (gs = 64: two)
            if (kPerPass * h < nk) {
#pragma unroll
              for (int s = 0; s < 2; ++s) {               // the two halves of the activation rows
                const uint32_t hand = s == 0 ? hand0 : hand1;
                const uint32_t buf = hand & 1u, bar = (uint32_t)(2 * s) + buf;
                if (opens) {
                  if (!mbar_wait(tempty0 + 8u * bar, ((hand >> 1) & 1u) ^ 1u, abort_s)) return;
                  tc_fence_after();
                }
                if (issuer) {
                  const uint32_t d = tmem_base_u + (uint32_t)(s * 256) + buf * 128u;
#pragma unroll
                  for (int k = 0; k < kPerPass; ++k) {
                    const uint64_t ko = (uint64_t)(2 * (kPerPass * h + k));
                    tc_mma_i8(d, b_desc + ko, a_desc + (uint64_t)(s * ((128 * BK) >> 4)) + ko, idesc,
                              (k == 0 && opens) ? 0u : 1u);
                  }
                  if (closes) tc_commit(tfull0 + 8u * bar);
                }
                if (closes) {
                  if (s == 0) ++hand0;
                  else ++hand1;
                }
              }
            }
          }
          if (issuer) tc_commit(empty0 + 8u * stage);  // the stage is free once these MMAs retire
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    };
    if (mma_per_group == 2) issue(std::integral_constant<int, 2>{});
    else if (mma_per_group == 4) issue(std::integral_constant<int, 4>{});
    else issue(std::integral_constant<int, 8>{});
    if (issuer) tc_commit(smem_u32(drain_bar));
    {
      const long long t0 = clock64();
      while (!mbar_try_wait(smem_u32(drain_bar), 0) && clock64() - t0 < kWaitCycles) {
      }
    }
  } else {
    pdl_wait();
    // TMEM lane = weight row (output column n), TMEM column = activation row m: a thread's
    // values of a group all belong to one output column and share one group scale.
    const int e = warp - 2;        // 0..15
    const int half = e >> 3;       // activation rows 0..127 or 128..255 of the tile
    const int q = warp & 3;        // the TMEM lane quarter this warp can read: 32 output columns
    const int ch = (e >> 2) & 1;   // its 64 columns of the half's accumulator: 64 activation rows
    float *sa_s = sa_all + e * 64;
    constexpr int kAhead = C::kScaleAhead;
    uint32_t lane0 = lane == 0;
    uint32_t tfull0 = smem_u32(tmem_full_bar + 2 * half), tempty0 = smem_u32(tmem_empty_bar + 2 * half);
    uint32_t taddr0 = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(half * 256 + ch * 64);
    asm volatile("" : "+r"(lane0), "+r"(tfull0), "+r"(tempty0), "+r"(taddr0));
    const uint32_t sw_pitch = (uint32_t)p.N * (p.sw_half ? 2u : 4u);  // the scale matrix is far below 4 GB
    auto epilogue = [&](auto half_c) {
      constexpr bool kHalf = decltype(half_c)::value;
      auto to_f32 = [](uint32_t raw) {
        return kHalf ? __half2float(__ushort_as_half((unsigned short)raw)) : __uint_as_float(raw);
      };
      uint32_t handover = 0;
      for (int t = cta; t < num_tiles; t += num_ctas) {
        // (row scales, bias and the row / column numbers are formed after the groups: nothing of the
        // tile's epilogue is held in registers through the group loop)
        // the lane fetches sw[g, n] kAhead groups before its use and keeps the raw bits in registers;
        // columns past N read column N - 1 (their results are never stored)
        const int ncol_s = (t % num_n) * C::BNP + q * 32 + lane;
        uint32_t swo = (uint32_t)min(ncol_s, p.N - 1) * (kHalf ? 2u : 4u);  // byte offset into the scale matrix
        auto scale_at = [&](uint32_t off) {
          const char *a = reinterpret_cast<const char *>(p.sw) + off;
          return kHalf ? (uint32_t)__ldg(reinterpret_cast<const unsigned short *>(a))
                       : __ldg(reinterpret_cast<const uint32_t *>(a));
        };
        uint32_t pre[kAhead];
#pragma unroll
        for (int i = 0; i < kAhead; ++i) {
          pre[i] = 0u;
          if (i < groups) pre[i] = scale_at(swo);
          swo += sw_pitch;
        }
        // fp32 partial sums of column n for the 64 activation rows, as packed pairs (rows 2i, 2i + 1)
        uint64_t acc2[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc2[i] = 0ull;
        for (int g = 0; g < groups; ++g) {
          const uint32_t buf = handover & 1u;
          const uint32_t full_b = tfull0 + 8u * buf, par = (handover >> 1) & 1u;
          if (!__all_sync(0xffffffffu, mbar_try_wait(full_b, par))) {
            uint32_t got = 0;
            if (lane0) got = mbar_wait(full_b, par, abort_s);
            if (!__shfl_sync(0xffffffffu, got, 0)) return;
          }
          tc_fence_after();
          const uint64_t sc2 = splat2(to_f32(pre[0]));
#pragma unroll
          for (int i = 0; i + 1 < kAhead; ++i) pre[i] = pre[i + 1];
          if (g + kAhead < groups) pre[kAhead - 1] = scale_at(swo);
          swo += sw_pitch;
#pragma unroll
          for (int c = 0; c < 64 / kLd; ++c) {
            uint32_t r[kLd];
            tc_ldn(taddr0 + buf * 128u + (uint32_t)(c * kLd), r);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < kLd / 2; ++i)
              acc2[(kLd / 2) * c + i] = promote2(r[2 * i], r[2 * i + 1], sc2, acc2[(kLd / 2) * c + i]);
          }
          tc_fence_before();
          __syncwarp();  // every lane has read the buffer
          if (lane0) mbar_arrive_relaxed(tempty0 + 8u * buf);
          ++handover;
        }
        // ---- final scale by sa[m], add bias, store this warp's 64 rows x 32 columns
        const int mrow0 = (t / num_n) * C::BMP + half * 128 + ch * 64;  // first activation row of this warp
        const int ncol = (t % num_n) * C::BNP + q * 32 + lane;          // the output column of this lane
        const float bias_n = (p.bias != nullptr && ncol < p.N) ? __half2float(p.bias[ncol]) : 0.0f;
        __syncwarp();
        sa_s[lane] = mrow0 + lane < p.M ? __ldg(p.sa + mrow0 + lane) : 0.0f;
        sa_s[32 + lane] = mrow0 + 32 + lane < p.M ? __ldg(p.sa + mrow0 + 32 + lane) : 0.0f;
        __syncwarp();
        if (ncol < p.N) {
          __half *ocol = reinterpret_cast<__half *>(p.out) + ncol;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // rows mrow0 + 4 i .. + 3 (sa_s: the same address in every lane, a broadcast)
            const float4 sa4 = *reinterpret_cast<const float4 *>(sa_s + 4 * i);
            const float2 a0 = unpack2(acc2[2 * i]), a1 = unpack2(acc2[2 * i + 1]);
            const int m = mrow0 + 4 * i;
            if (m < p.M) ocol[(int64_t)m * p.N] = __float2half_rn(__fmaf_rn(a0.x, sa4.x, bias_n));
            if (m + 1 < p.M) ocol[(int64_t)(m + 1) * p.N] = __float2half_rn(__fmaf_rn(a0.y, sa4.y, bias_n));
            if (m + 2 < p.M) ocol[(int64_t)(m + 2) * p.N] = __float2half_rn(__fmaf_rn(a1.x, sa4.z, bias_n));
            if (m + 3 < p.M) ocol[(int64_t)(m + 3) * p.N] = __float2half_rn(__fmaf_rn(a1.y, sa4.w, bias_n));
          }
        }
      }
    };
    if (p.sw_half) epilogue(std::true_type{});
    else epilogue(std::false_type{});
  }

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
// Name of the tensor-core kernel this thread launched last (for reports: which kernel a
// timed figure belongs to is read from the dispatch, not assumed).
thread_local const char *t_last_kernel = "";

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

// A tensor map is a pure function of (base pointer, shape, box, element type), and
// encoding one costs about a microsecond on the host - three of them per launch are a
// visible part of a small-M call outside a CUDA graph.  Each host thread keeps the
// maps it encoded last in a small direct-mapped table keyed by those arguments.
struct MapKey {
  const void *base;
  int64_t rows, cols;
  int box_rows, kind;  // kind: 0 int8 operand, 1 fp16 output, 2 int32 output
  bool operator==(const MapKey &o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows && kind == o.kind;
  }
};
struct MapSlot {
  MapKey key{nullptr, 0, 0, 0, -1};
  CUtensorMap map;
};
constexpr int kMapSlots = 64;
MapSlot *map_slot(const MapKey &k) {
  thread_local MapSlot table[kMapSlots];
  uint64_t h = reinterpret_cast<uintptr_t>(k.base) >> 4;
  h ^= (uint64_t)k.rows * 0x9E3779B97F4A7C15ull;
  h ^= (uint64_t)k.cols * 0xC2B2AE3D27D4EB4Full;
  h ^= (uint64_t)(k.box_rows * 4 + k.kind) * 0x165667B19E3779F9ull;
  return &table[(h >> 20) % kMapSlots];
}

// 2-D int8 tensor map over a row-major [rows, K] matrix, box [box_rows x 128 bytes],
// 128-byte swizzle, zero fill outside the matrix.
int make_map(CUtensorMap *map, const void *base, int64_t rows, int64_t K, int box_rows) {
  const MapKey key{base, rows, K, box_rows, 0};
  MapSlot *slot = map_slot(key);
  if (slot->key == key) {
    *map = slot->map;
    return CIDER_OK;
  }
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
  slot->key = key;
  slot->map = *map;
  return CIDER_OK;
}

// 2-D map over packed int4 weight rows [rows, K/2 bytes]: box [box_rows x 64 bytes] (the 128 k
// of one stage), no swizzle (the converter reads whole 16-byte pieces of consecutive rows),
// zero fill outside (rows past N are never stored; k past K meets zero activations).
int make_packed_map(CUtensorMap *map, const void *base, int64_t rows, int64_t K, int box_rows) {
  const MapKey key{base, rows, K / 2, box_rows, 3};
  MapSlot *slot = map_slot(key);
  if (slot->key == key) {
    *map = slot->map;
    return CIDER_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)(K / 2), (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(K / 2)};
  cuuint32_t box[2] = {(cuuint32_t)(BK / 2), (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled (packed rows) failed with CUresult " + std::to_string((int)r));
  slot->key = key;
  slot->map = *map;
  return CIDER_OK;
}

// 2-D map of the [M, N] output for TMA stores: boxes of 32 rows x 128 bytes
// (64 fp16 or 32 int32 columns), 128-byte swizzle.  When the output cannot take
// TMA stores (p.tma_store == 0) the kernel never touches the map; the A map is
// passed in its place.
int make_out_map(CUtensorMap *map, const GemmArgs &g) {
  const bool raw = g.epi == Epi::kRawInt32;
  const int64_t cols = g.rowmax != nullptr ? g.N / 2 : g.N;  // SwiGLU epilogue: half as many output columns
  const MapKey key{g.out, g.M, cols, 32, raw ? 2 : 1};
  MapSlot *slot = map_slot(key);
  if (slot->key == key) {
    *map = slot->map;
    return CIDER_OK;
  }
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  const cuuint64_t esz = raw ? 4 : 2;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)g.M};
  cuuint64_t strides[1] = {(cuuint64_t)cols * esz};
  cuuint32_t box[2] = {(cuuint32_t)(128 / esz), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, raw ? CU_TENSOR_MAP_DATA_TYPE_INT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, g.out, dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(CIDER_E_CUDA, "cuTensorMapEncodeTiled (output) failed with CUresult " + std::to_string((int)r));
  slot->key = key;
  slot->map = *map;
  return CIDER_OK;
}

template <int BN, int EPI, bool W4 = false>
int launch_cfg(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  using C = Cfg<BN, W4>;
  auto kern = gemm_tc_kernel<BN, EPI, W4>;
  constexpr int kThreadsK = W4 ? kThreads + conv_threads<BN>() : kThreads;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc shared-memory attribute");
  if (rc) return rc;
  CUtensorMap ma, mb;
  rc = make_map(&ma, g.a, g.M, g.K, BM);
  if (rc) return rc;
  rc = W4 ? make_packed_map(&mb, g.w4rows, g.N, g.K, BN) : make_map(&mb, g.b, g.N, g.K, BN);
  if (rc) return rc;
  CUtensorMap mc = ma;
  if (p.tma_store && (rc = make_out_map(&mc, g))) return rc;
  const int64_t tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  t_last_kernel = W4 ? "gemm_tc_kernel<128x128, int4 weights expanded in shared memory>"
                     : (BN == 256 ? "gemm_tc_kernel<128x256>" : (BN == 192 ? "gemm_tc_kernel<128x192>"
                        : (BN == 128 ? "gemm_tc_kernel<128x128>" : "gemm_tc_kernel<128x64>")));
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreadsK), (size_t)C::kSmemBytes, st, ma, mb, mc, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc launch");
  return check_cuda(cudaGetLastError(), "gemm_tc launch");
}

// Number of CTA pairs that can be resident at once (a pair needs two SMs of one
// cluster-capable group); queried once per kernel and device.
template <int EPI, bool W4 = false>
int launch_pair(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  using C = CfgPairT<W4>;
  auto kern = gemm_tc_pair_kernel<EPI, W4>;
  constexpr int kThreadsK = W4 ? kThreads + kConvThreadsPair : kThreads;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc_pair shared-memory attribute");
  if (rc) return rc;
  // resident CTA pairs of this kernel on the current device, queried once per device
  static std::atomic<int> max_pairs_dev[64];
  const int dev = current_device() & 63;
  int max_pairs = max_pairs_dev[dev].load(std::memory_order_acquire);
  if (max_pairs == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74, 1, 1);
    cfg.blockDim = dim3(kThreadsK, 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) max_pairs = n;
    else { cudaGetLastError(); max_pairs = sm_count(dev) / 2; }
    max_pairs_dev[dev].store(max_pairs, std::memory_order_release);
  }
  CUtensorMap ma, mb;
  rc = make_map(&ma, g.a, g.M, g.K, 128);
  if (rc) return rc;
  rc = W4 ? make_packed_map(&mb, g.w4rows, g.N, g.K, 128) : make_map(&mb, g.b, g.N, g.K, 128);
  if (rc) return rc;
  CUtensorMap mc = ma;
  if (p.tma_store && (rc = make_out_map(&mc, g))) return rc;
  const int64_t tiles = ((g.M + C::BMP - 1) / C::BMP) * ((g.N + C::BNP - 1) / C::BNP);
  const unsigned pairs = (unsigned)(tiles < max_pairs ? tiles : max_pairs);
  t_last_kernel = W4 ? "gemm_tc_pair_kernel<256x256 per CTA pair, cta_group::2, int4 weights expanded in shared memory>"
                     : "gemm_tc_pair_kernel<256x256 per CTA pair, cta_group::2>";
  cudaError_t le = launch_kernel(kern, dim3(2 * pairs), dim3(kThreadsK), (size_t)C::kSmemBytes, st, ma, mb, mc, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc_pair launch");
  return check_cuda(cudaGetLastError(), "gemm_tc_pair launch");
}

template <bool W4 = false>
int launch_pg_wide_impl(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  using C = CfgPgT<W4>;
  auto kern = gemm_tc_pg_kernel<W4>;
  constexpr int kThreadsK = W4 ? kThreadsPg + kConvThreadsPg : kThreadsPg;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc_pg shared-memory attribute");
  if (rc) return rc;
  CUtensorMap ma, mb;
  rc = make_map(&ma, g.a, g.M, g.K, C::BMP);
  if (rc) return rc;
  rc = W4 ? make_packed_map(&mb, g.w4rows, g.N, g.K, C::BNP) : make_map(&mb, g.b, g.N, g.K, C::BNP);
  if (rc) return rc;
  CUtensorMap mc = ma;
  if (p.tma_store && (rc = make_out_map(&mc, g))) return rc;
  const int64_t tiles = ((g.M + C::BMP - 1) / C::BMP) * ((g.N + C::BNP - 1) / C::BNP);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  t_last_kernel = W4 ? "gemm_tc_pg_kernel<128x128, per-group promotion, int4 weights expanded in shared memory>"
                     : "gemm_tc_pg_kernel<128x128, per-group promotion>";
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreadsK), (size_t)C::kSmemBytes, st, ma, mb, mc, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc_pg launch");
  return check_cuda(cudaGetLastError(), "gemm_tc_pg launch");
}

int launch_pg2(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  using C = CfgPg2;
  auto kern = gemm_tc_pg2_kernel;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc_pg2 shared-memory attribute");
  if (rc) return rc;
  CUtensorMap ma, mb;
  rc = make_map(&ma, g.a, g.M, g.K, 128);
  if (rc) return rc;
  rc = make_map(&mb, g.b, g.N, g.K, 128);
  if (rc) return rc;
  const int64_t tiles = ((g.M + C::BMP - 1) / C::BMP) * ((g.N + C::BNP - 1) / C::BNP);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  t_last_kernel = "gemm_tc_pg2_kernel<128 output columns x 256 rows, per-group promotion in two half-tiles>";
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreadsPg), (size_t)C::kSmemBytes, st, ma, mb, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc_pg2 launch");
  return check_cuda(cudaGetLastError(), "gemm_tc_pg2 launch");
}

int launch_pg_wide(const GemmArgs &g, const TcParams &p, cudaStream_t st) {
  if (p.w4 != nullptr)
    return launch_pg_wide_impl<true>(g, p, st);
  return launch_pg_wide_impl<false>(g, p, st);
}

template <int EPI>
int launch_epi(const GemmArgs &g, const TcParams &p, int bn, cudaStream_t st) {
  switch (bn) {
    case 256: return launch_cfg<256, EPI>(g, p, st);
    case 192: return launch_cfg<192, EPI>(g, p, st);
    case 128: return launch_cfg<128, EPI>(g, p, st);
    default: return launch_cfg<64, EPI>(g, p, st);
  }
}

// ---- split-K for few output tiles (small M): slabs of int32 partial sums, then this
// kernel: sum over the splits (exact), per-channel dequant with the operation order of
// the fused epilogue, fp16 store.  One thread per 8 consecutive columns of a row.
__global__ void __launch_bounds__(256)
splitk_finish_kernel(const int32_t *__restrict__ slabs, int splits, int64_t slab_elems, const float *__restrict__ sa,
                     const float *__restrict__ sw, const __half *__restrict__ bias, __half *__restrict__ y, int M,
                     int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t chunks = (int64_t)M * (N / 8);
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(c / (N / 8)), n = (int)(c % (N / 8)) * 8;
    int acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const int32_t *src = slabs + (int64_t)m * N + n;
    for (int s = 0; s < splits; ++s) {
      const int4 lo = __ldcg(reinterpret_cast<const int4 *>(src + s * slab_elems));
      const int4 hi = __ldcg(reinterpret_cast<const int4 *>(src + s * slab_elems) + 1);
      acc[0] += lo.x; acc[1] += lo.y; acc[2] += lo.z; acc[3] += lo.w;
      acc[4] += hi.x; acc[5] += hi.y; acc[6] += hi.z; acc[7] += hi.w;
    }
    const float sa_m = sa[m];
    const float4 s0 = *reinterpret_cast<const float4 *>(sw + n), s1 = *reinterpret_cast<const float4 *>(sw + n + 4);
    const float swv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    float bv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) bv[i] = __half2float(bias[n + i]);
    }
    uint32_t o[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float v0 = __fmaf_rn(__fmul_rn(__int2float_rn(acc[2 * i]), sa_m), swv[2 * i], bv[2 * i]);
      const float v1 = __fmaf_rn(__fmul_rn(__int2float_rn(acc[2 * i + 1]), sa_m), swv[2 * i + 1], bv[2 * i + 1]);
      const __half2 h = __floats2half2_rn(v0, v1);
      o[i] = *reinterpret_cast<const uint32_t *>(&h);
    }
    *reinterpret_cast<uint4 *>(y + (int64_t)m * N + n) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The per-group counterpart: the slabs hold fp32 partial sums of whole K-groups (group scales
// applied, row scale and bias not yet); summed in piece order, so the result is deterministic;
// the fp32 additions associate differently from the unsplit kernel's running sum (last-bit
// differences in fp32, far below fp16 resolution).  One thread per 4 consecutive columns.
__global__ void __launch_bounds__(256)
pg_splitk_finish_kernel(const float *__restrict__ slabs, int splits, int64_t slab_elems, const float *__restrict__ sa,
                        const __half *__restrict__ bias, __half *__restrict__ y, int M, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t chunks = (int64_t)M * (N / 4);
  for (int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * blockDim.x) {
    const int m = (int)(c / (N / 4)), n = (int)(c % (N / 4)) * 4;
    const float *src = slabs + (int64_t)m * N + n;
    float4 acc = __ldcg(reinterpret_cast<const float4 *>(src));
    for (int s = 1; s < splits; ++s) {
      const float4 v = __ldcg(reinterpret_cast<const float4 *>(src + s * slab_elems));
      acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    const float sa_m = sa[m];
    float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (bias != nullptr) {
#pragma unroll
      for (int i = 0; i < 4; ++i) b[i] = __half2float(bias[n + i]);
    }
    const __half2 h0 = __floats2half2_rn(__fmaf_rn(acc.x, sa_m, b[0]), __fmaf_rn(acc.y, sa_m, b[1]));
    const __half2 h1 = __floats2half2_rn(__fmaf_rn(acc.z, sa_m, b[2]), __fmaf_rn(acc.w, sa_m, b[3]));
    *reinterpret_cast<uint2 *>(y + (int64_t)m * N + n) =
        make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
  }
}

template <bool W4>
int launch_pg_splitk_impl(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st) {
  using C = CfgPgT<W4>;
  auto kern = gemm_tc_pg_kernel<W4>;
  constexpr int kThreadsK = W4 ? kThreadsPg + kConvThreadsPg : kThreadsPg;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc_pg shared-memory attribute");
  if (rc) return rc;
  TcParams p;
  p.out = slabs; p.sa = g.sa; p.sw = g.sw; p.bias = nullptr;
  p.M = pl.splits * pl.m_pad; p.N = (int)g.N; p.K = (int)g.K; p.gs = g.gs; p.sw_half = g.sw_is_half ? 1 : 0;
  p.vec_store = 1; p.tma_store = 0; p.w4 = W4 ? g.w4rows : nullptr; p.reduce_out = 0; p.M_real = (int)g.M;
  p.split_mtiles = pl.m_pad / 128; p.kb_per_split = pl.kb_per_split; p.rowmax = nullptr; p.out_cols = (int)g.N;
  CUtensorMap ma, mb;
  if ((rc = make_map(&ma, g.a, g.M, g.K, C::BMP))) return rc;  // rows past M read as zero
  rc = W4 ? make_packed_map(&mb, g.w4rows, g.N, g.K, C::BNP) : make_map(&mb, g.b, g.N, g.K, C::BNP);
  if (rc) return rc;
  const int64_t tiles = (int64_t)(p.M / 128) * ((g.N + C::BNP - 1) / C::BNP);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  t_last_kernel = W4 ? "gemm_tc_pg_kernel<128x128, per-group promotion, int4 weights> split-K, fp32 slabs"
                     : "gemm_tc_pg_kernel<128x128, per-group promotion> split-K, fp32 slabs";
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreadsK), (size_t)C::kSmemBytes, st, ma, mb, ma, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc_pg split-K launch");
  const int64_t chunks = g.M * (g.N / 4);
  int64_t blocks = (chunks + 255) / 256;
  if (blocks > 8 * (int64_t)sms) blocks = 8 * (int64_t)sms;
  le = launch_kernel(pg_splitk_finish_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0, st,
                     static_cast<const float *>(slabs), pl.splits, (int64_t)pl.m_pad * g.N, g.sa, g.bias,
                     static_cast<__half *>(g.out), (int)g.M, (int)g.N);
  if (le != cudaSuccess) return check_cuda(le, "per-group split-K finish launch");
  return check_cuda(cudaGetLastError(), "gemm_tc_pg split-K launch");
}

}  // namespace

static std::atomic<int> g_tile_mode{0};  // 0 auto, 1 single-CTA, 3 CTA pair
static std::atomic<int> g_force_bn{0};

// Split-K plan for the per-group linear on int8 weights: K is cut into equal pieces of
// an even number of 128-wide K blocks (so every piece holds whole groups for gs = 64, 128 and 256
// alike and the workspace does not depend on gs); each (tile, piece) is a CTA of the per-group
// kernel writing fp32 partial sums to its slab.  Taken when the tiles fill at most half of the
// 148 SMs.
SplitKPlan plan_pg_splitk(int64_t M, int64_t N, int64_t K) {
  SplitKPlan best;
  if (M < 2 || M > 512 || N % 8 != 0 || K % (2 * BK) != 0 || K < 8 * BK) return best;
  const int64_t units = K / (2 * BK);  // pairs of K blocks
  const int64_t m_pad = (M + 127) / 128 * 128;
  const int64_t tiles = (m_pad / 128) * ((N + 127) / 128);
  int64_t s = 148 / tiles;
  if (s > 16) s = 16;
  if (s > units / 2) s = units / 2;  // at least four K blocks per piece
  while (s >= 2 && units % s != 0) --s;
  if (s < 2) return best;
  best.splits = (int)s;
  best.kb_per_split = (int)(2 * units / s);
  best.m_pad = (int)m_pad;
  best.bn = 128;
  best.bytes = (size_t)(s * m_pad * N) * sizeof(float);
  return best;
}

int launch_gemm_tc_pg_splitk(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st) {
  const auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (!gemm_tc_eligible(g) || g.epi != Epi::kPerGroup || g.w4rows != nullptr || pl.splits < 2 || slabs == nullptr ||
      !a16(slabs) ||
      (reinterpret_cast<uintptr_t>(g.out) & 7u) || (pl.kb_per_split * BK) % g.gs != 0)
    return fail(CIDER_E_SHAPE, "gemm_tc per-group split-K: shape or alignment not supported");
  if (g_tile_mode.load(std::memory_order_relaxed) == 1) return launch_gemm_tc(g, st);  // a test asked for the narrow kernel
  return launch_pg_splitk_impl<false>(g, pl, slabs, st);
}

// Split-K plan for the per-channel linear: with M <= 512 rows and few 128 x 128 output tiles most
// SMs would idle while every busy one pulls all of A through its own L2 port; the K range is cut
// into `splits` pieces, each (tile, piece) a CTA of the raw-int32 kernel writing its own slab.
// Fixed at 148 SMs (the only part this library is built for) so that the workspace size is a pure
// function of the shape.
SplitKPlan plan_splitk(int64_t M, int64_t N, int64_t K) {
  SplitKPlan best;
  if (M < 2 || M > 512 || N % 8 != 0 || K % 16 != 0 || K < 8 * BK) return best;
  const int64_t num_kb = (K + BK - 1) / BK;
  const int64_t m_pad = (M + 127) / 128 * 128;
  // estimated bytes through one SM's L2 port: the operand stages of its CTA plus its share of
  // the slab traffic (written once, read once); the unsplit 128-wide tiling is the baseline
  const int64_t tiles128 = (m_pad / 128) * ((N + 127) / 128);
  int64_t best_cost = ((tiles128 + 147) / 148) * num_kb * (BM + 128) * BK;
  for (int bn = 128; bn <= 256; bn += 128) {
    const int64_t tiles = (m_pad / 128) * ((N + bn - 1) / bn);
    int64_t s = 148 / tiles;
    if (s > num_kb / 4) s = num_kb / 4;
    if (s > 16) s = 16;
    if (s < 2) continue;
    const int64_t kbs = (num_kb + s - 1) / s;
    s = (num_kb + kbs - 1) / kbs;
    if (s < 2) continue;
    const int64_t slab = s * m_pad * N * (int64_t)sizeof(int32_t);
    const int64_t cost = kbs * (BM + bn) * BK + 2 * slab / 148 + 400000;  // + the finishing launch
    if (cost < best_cost) {
      best_cost = cost;
      best.splits = (int)s;
      best.kb_per_split = (int)kbs;
      best.m_pad = (int)m_pad;
      best.bn = bn;
      best.bytes = (size_t)slab;
    }
  }
  return best;
}

template <int BN>
int launch_splitk_bn(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st);

int launch_gemm_tc_splitk(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st) {
  if (!gemm_tc_eligible(g) || g.epi != Epi::kPerChannel || pl.splits < 2 || slabs == nullptr ||
      (reinterpret_cast<uintptr_t>(slabs) & 15u) || (reinterpret_cast<uintptr_t>(g.out) & 15u) ||
      (reinterpret_cast<uintptr_t>(g.sw) & 15u))
    return fail(CIDER_E_SHAPE, "gemm_tc split-K: shape or alignment not supported");
  return pl.bn == 256 ? launch_splitk_bn<256>(g, pl, slabs, st) : launch_splitk_bn<128>(g, pl, slabs, st);
}

template <int BN>
int launch_splitk_bn(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_tc_kernel<BN, (int)Epi::kRawInt32>;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc shared-memory attribute");
  if (rc) return rc;
  TcParams p;
  p.out = slabs; p.sa = nullptr; p.sw = nullptr; p.bias = nullptr;
  p.M = pl.splits * pl.m_pad; p.N = (int)g.N; p.K = (int)g.K; p.gs = 0; p.sw_half = 0;
  p.vec_store = 1; p.tma_store = 1; p.w4 = nullptr; p.reduce_out = 0; p.M_real = 0;
  p.split_mtiles = pl.m_pad / 128; p.kb_per_split = pl.kb_per_split; p.rowmax = nullptr; p.out_cols = (int)g.N;
  CUtensorMap ma, mb, mc;
  if ((rc = make_map(&ma, g.a, g.M, g.K, BM))) return rc;  // rows past M read as zero
  if ((rc = make_map(&mb, g.b, g.N, g.K, BN))) return rc;
  GemmArgs og;
  og.out = slabs; og.M = p.M; og.N = g.N; og.epi = Epi::kRawInt32;
  if ((rc = make_out_map(&mc, og))) return rc;
  const int64_t tiles = (int64_t)(p.M / 128) * ((g.N + BN - 1) / BN);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, ma, mb, mc, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc split-K launch");
  const int64_t chunks = g.M * (g.N / 8);
  int64_t blocks = (chunks + 255) / 256;
  if (blocks > 8 * (int64_t)sms) blocks = 8 * (int64_t)sms;
  le = launch_kernel(splitk_finish_kernel, dim3((unsigned)blocks), dim3(256), (size_t)0, st,
                     static_cast<const int32_t *>(slabs), pl.splits, (int64_t)pl.m_pad * g.N, g.sa,
                     static_cast<const float *>(g.sw), g.bias, static_cast<__half *>(g.out), (int)g.M, (int)g.N);
  if (le != cudaSuccess) return check_cuda(le, "split-K finish launch");
  return check_cuda(cudaGetLastError(), "gemm_tc split-K launch");
}

// Raw int32 product with split-K and no scratch: zero the result, then every (tile, piece)
// CTA of the raw-int32 kernel adds its partial tile with TMA reduce-adds.
template <int BN>
int launch_raw_splitk_bn(const GemmArgs &g, TcParams p, const SplitKPlan &pl, cudaStream_t st) {
  using C = Cfg<BN>;
  auto kern = gemm_tc_kernel<BN, (int)Epi::kRawInt32>;
  static std::atomic<unsigned long long> attr_done{0};
  int rc = ensure_dynamic_smem(kern, C::kSmemBytes, attr_done, "gemm_tc shared-memory attribute");
  if (rc) return rc;
  if ((rc = check_cuda(cudaMemsetAsync(g.out, 0, (size_t)g.M * (size_t)g.N * sizeof(int32_t), st),
                       "int8_matmul_int32 split-K: zeroing the result")))
    return rc;
  p.M_real = (int)g.M;
  p.M = pl.splits * pl.m_pad;
  p.reduce_out = 1;
  p.split_mtiles = pl.m_pad / 128;
  p.kb_per_split = pl.kb_per_split;
  CUtensorMap ma, mb, mc;
  if ((rc = make_map(&ma, g.a, g.M, g.K, BM))) return rc;  // rows past M read as zero
  if ((rc = make_map(&mb, g.b, g.N, g.K, BN))) return rc;
  if ((rc = make_out_map(&mc, g))) return rc;               // the real [M, N] int32 result
  const int64_t tiles = (int64_t)(p.M / 128) * ((g.N + BN - 1) / BN);
  const int sms = sm_count(current_device());
  const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
  t_last_kernel = BN == 256 ? "gemm_tc_kernel<128x256> split-K, TMA reduce-add" : "gemm_tc_kernel<128x128> split-K, TMA reduce-add";
  cudaError_t le = launch_kernel(kern, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, st, ma, mb, mc, p);
  if (le != cudaSuccess) return check_cuda(le, "gemm_tc raw split-K launch");
  return check_cuda(cudaGetLastError(), "gemm_tc raw split-K launch");
}

int launch_raw_splitk(const GemmArgs &g, const TcParams &p, const SplitKPlan &pl, cudaStream_t st) {
  return pl.bn == 256 ? launch_raw_splitk_bn<256>(g, p, pl, st) : launch_raw_splitk_bn<128>(g, p, pl, st);
}

// Kernel selection override for the tests (set_tile_override, reached through the
// testing header only): tile 128 forces the single-CTA 128-row kernel, tile 2 the
// CTA-pair kernel, bn forces the single-CTA kernel's N tile (per-group on int8 weights:
// bn 128 the 128 x 128 kernel, bn 256 the 128 x 256 one); 0 lets the heuristic
// choose.  Every choice computes the same results.

int set_tile_override(int tile, int bn) {
  if ((tile != 0 && tile != 128 && tile != 2) || (bn != 0 && bn != 64 && bn != 128 && bn != 192 && bn != 256))
    return fail(CIDER_E_INVALID, "set_tile_override: tile must be 0, 128 or 2 and bn 0, 64, 128, 192 or 256");
  g_tile_mode.store(tile == 128 ? 1 : (tile == 2 ? 3 : 0));
  g_force_bn.store(bn);
  return CIDER_OK;
}

bool gemm_tc_eligible(const GemmArgs &g) {
  auto a16 = [](const void *q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
  if (g.packed4 != nullptr || g.a == nullptr) return false;
  if (g.w4rows != nullptr) {
    // packed int4 rows: whole 16-byte chunks per row and stage, fused epilogues only
    if (g.b != nullptr || (g.K % 32) != 0 || !a16(g.w4rows) || g.epi == Epi::kRawInt32) return false;
  } else if (g.b == nullptr) {
    return false;
  }
  if (g.M < 1 || g.N < 1 || g.K < BK || (g.K % 16) != 0) return false;
  if (g.M > (1 << 30) || g.N > (1 << 30) || g.K > (1 << 30)) return false;
  if (((g.M + BM - 1) / BM) * ((g.N + 63) / 64) > (int64_t)(1u << 30)) return false;
  if (!a16(g.a) || (g.b != nullptr && !a16(g.b))) return false;
  if (g.epi == Epi::kPerGroup && (g.gs % 64 != 0 || g.K % g.gs != 0)) return false;
  return true;
}

int launch_gemm_tc(const GemmArgs &g, cudaStream_t st) {
  if (!gemm_tc_eligible(g)) return fail(CIDER_E_SHAPE, "gemm_tc: shape or alignment not supported");
  TcParams p;
  p.split_mtiles = 0; p.kb_per_split = 0; p.reduce_out = 0; p.M_real = 0;
  p.out = g.out; p.sa = g.sa; p.sw = g.sw; p.bias = g.bias;
  p.M = (int)g.M; p.N = (int)g.N; p.K = (int)g.K; p.gs = g.gs; p.sw_half = g.sw_is_half;
  p.w4 = g.w4rows;
  const bool w4 = g.w4rows != nullptr;
  const bool swiglu = g.rowmax != nullptr;
  if (swiglu && (g.epi != Epi::kPerChannel || w4 || g.N % 64 != 0))
    return fail(CIDER_E_SHAPE, "gemm_tc: the SwiGLU epilogue takes per-channel int8 weights with N a multiple of 64");
  p.rowmax = g.rowmax;
  p.out_cols = swiglu ? (int)(g.N / 2) : (int)g.N;
  const bool o16 = (reinterpret_cast<uintptr_t>(g.out) & 15u) == 0;
  p.vec_store = g.epi == Epi::kRawInt32 ? (o16 && g.N % 4 == 0) : (o16 && p.out_cols % 8 == 0);
  const int tile_mode = g_tile_mode.load(std::memory_order_relaxed);
  const int64_t tiles256 = ((g.M + 255) / 256) * ((g.N + 255) / 256);
  const int sms = sm_count(current_device());
  // per-group: the 128 x 128 kernel also when its tiles do not fill the machine - the
  // 128 x 64 path of the generic kernel fetches its group scales with a dependent
  // global load per hand-over and is an order of magnitude slower per group
  const bool pg_wide = g.epi == Epi::kPerGroup && (tile_mode != 1 || w4);
  // TMA stores need 16-byte aligned rows
  p.tma_store = (p.vec_store && (g.epi != Epi::kPerGroup || pg_wide)) ? 1 : 0;
  // N tile of the single-CTA kernel: the candidate with the smallest estimated time,
  // waves x (K blocks x cycles per block + epilogue cycles), constants fitted to
  // measured launches of small problems (a K block of a 128 x 64 / 128 / 192 / 256 tile
  // costs about 535 / 560 / 665 / 770 cycles: the narrower tiles do not get cheaper in
  // proportion, so fewer, wider tiles win unless they leave a whole wave mostly idle)
  const int64_t num_m = (g.M + BM - 1) / BM;
  const int64_t num_kb = (g.K + BK - 1) / BK;
  int bn = 256;
  int64_t best = -1;
  {
    const int cand[4] = {256, 192, 128, 64};
    const int64_t c_kb[4] = {770, 665, 560, 535}, c_epi[4] = {1000, 1150, 1300, 750};
    for (int i = 0; i < 4; ++i) {
      if (w4 && cand[i] != 128) continue;  // the int4 converters of the single-CTA kernel: 128-column tiles
      if (swiglu && cand[i] % 128 != 0) continue;  // the SwiGLU epilogue works on 128 accumulator columns at a time
      const int64_t tiles = num_m * ((g.N + cand[i] - 1) / cand[i]);
      const int64_t waves = (tiles + sms - 1) / sms;
      const int64_t cost = waves * (num_kb * c_kb[i] + c_epi[i]);
      if (best < 0 || cost < best) {
        best = cost;
        bn = cand[i];
      }
    }
  }
  const int force_bn = g_force_bn.load(std::memory_order_relaxed);
  if (!w4 && (force_bn == 64 || force_bn == 128 || force_bn == 192 || force_bn == 256) && !(swiglu && force_bn % 128 != 0))
    bn = force_bn;
  // CTA-pair kernel once its 256 x 256 tiles fill the machine twice over (with fewer
  // tiles the 74 pairs quantise into waves worse than 148 single CTAs do)
  // (int4 weights: the pair kernel from one wave of its tiles on - its single-CTA form only
  // has 128 x 128 tiles, which are the better choice for a handful of tiles only)
  // Below that the same estimate decides: a K block of a pair's 256 x 256 tile costs about 610
  // cycles (each CTA takes 32 KB per K block from L2 where a single 128 x 256 CTA takes 48 KB for
  // half the work), its epilogue 1600, and the cluster launch about 4000 once - with a long K
  // and tiles for one or two rounds of the 74 pairs that undercuts the single-CTA tilings
  // (measured: M=3455 over [2048, 6144] 44.6 -> 35.9 us, M=2048 over [4096, 12288] 87.3 -> 69.1 us).
  const int64_t pairs = sms / 2 > 0 ? sms / 2 : 1;
  const int64_t cost_pair = ((tiles256 + pairs - 1) / pairs) * (num_kb * 610 + 1600) + 4000;
  const bool pair_by_cost = tile_mode == 0 && force_bn == 0 && !w4 && best > 0 && cost_pair < best;
  if (g.epi != Epi::kPerGroup && tile_mode != 1 &&
      (tile_mode == 3 || pair_by_cost || tiles256 >= 2 * (int64_t)sms || (w4 && 2 * tiles256 >= (int64_t)sms))) {
    if (w4) return launch_pair<(int)Epi::kPerChannel, true>(g, p, st);
    return g.epi == Epi::kRawInt32 ? launch_pair<(int)Epi::kRawInt32>(g, p, st)
                                   : launch_pair<(int)Epi::kPerChannel>(g, p, st);
  }
  if (w4 && g.epi == Epi::kPerChannel) return launch_cfg<128, (int)Epi::kPerChannel, true>(g, p, st);
  if (g.epi == Epi::kRawInt32 && tile_mode == 0 && force_bn == 0 && p.tma_store) {
    // few output tiles and a long K: cut K into pieces that add into the zeroed result
    const SplitKPlan pl = plan_splitk(g.M, g.N, g.K);
    if (pl.splits >= 2) return launch_raw_splitk(g, p, pl, st);
  }
  switch (g.epi) {
    case Epi::kRawInt32: return launch_epi<(int)Epi::kRawInt32>(g, p, bn, st);
    case Epi::kPerChannel: return launch_epi<(int)Epi::kPerChannel>(g, p, bn, st);
    default:
      // per-group: the 128 x 128 kernel with sixteen promotion warps; the generic
      // kernel's 128 x 64 per-group path only when the tile override asks for it
      if (pg_wide) {
        // the 128 x 256 tile for int8 weights of 48 MB and more, once its tiles fill the machine:
        // measured at M = 16384, 128 x 128 -> 128 x 256: [4096, 12288] 1388 -> 1195 us (gs = 128),
        // 2675 -> 2271 us (gs = 64); [24576, 4096] 2996 -> 2733 and 5507 -> 4832 us.  Smaller weights
        // are faster on the 128 x 128 tile ([10240, 2560] at M = 8192: 319 against 367 us).
        const int64_t tiles_tall = ((g.M + 255) / 256) * ((g.N + 127) / 128);
        const bool big_weights = g.N * g.K >= (int64_t)48 << 20;
        if (!w4 && (force_bn == 256 || (force_bn == 0 && tile_mode == 0 && big_weights && tiles_tall >= (int64_t)sms)))
          return launch_pg2(g, p, st);
        return launch_pg_wide(g, p, st);
      }
      return launch_cfg<64, (int)Epi::kPerGroup>(g, p, st);
  }
}

const char *last_gemm_kernel() { return t_last_kernel; }

int read_device_status(unsigned int *out) {
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return check_cuda(e, "device synchronize");
  int rc = check_cuda(cudaMemcpyFromSymbol(out, g_device_status, sizeof(unsigned int)), "read status");
  if (rc) return rc;
  unsigned int v = 0;
  if ((rc = read_gemv_status(&v))) return rc;
  *out |= v;
  if ((rc = read_glue_status(&v))) return rc;
  *out |= v;
  if ((rc = read_peer_status(&v))) return rc;
  *out |= v;
  if ((rc = read_sdpa_status(&v))) return rc;
  *out |= v;
  return CIDER_OK;
}

int clear_device_status() {
  unsigned int z = 0;
  int rc = check_cuda(cudaMemcpyToSymbol(g_device_status, &z, sizeof(z)), "clear status");
  if (!rc) rc = clear_gemv_status();
  if (!rc) rc = clear_glue_status();
  if (!rc) rc = clear_peer_status();
  return rc ? rc : clear_sdpa_status();
}

}  // namespace cider
