// Shared declarations for the cider_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>
#include <string>

#include "../../include/cider_b200.h"
#include "../../include/cider_b200_testing.h"

namespace cider {

// ---- host-side error plumbing -------------------------------------------
// Every C-ABI entry point returns a status code; the message of the last
// failure on the calling thread is kept for cider_last_error().
void set_error(const std::string &msg);
int fail(int code, const std::string &msg);
int check_cuda(cudaError_t e, const char *what);

int sm_count(int device);
int current_device();

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device):
// the attribute is per device, and one process may drive several GPUs.
// `done` is a bit mask of devices already set, one static mask per kernel.
template <typename Kern>
int ensure_dynamic_smem(Kern kern, int bytes, std::atomic<unsigned long long> &done, const char *what) {
  const int dev = current_device();
  const unsigned long long bit = 1ull << (dev & 63);
  if (done.load(std::memory_order_acquire) & bit) return CIDER_OK;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return check_cuda(e, what);
  // these kernels live on shared memory, not on L1: ask for the largest carve-out
  // (it is what lets two half-SM launches share an SM)
  e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  if (e != cudaSuccess) return check_cuda(e, what);
  done.fetch_or(bit, std::memory_order_release);
  return CIDER_OK;
}

// Programmatic dependent launch (PDL).  When enabled (cider_set_programmatic_launch)
// the small kernels of a decode step are launched with the programmatic stream
// serialization attribute: the next kernel may start while the previous one is
// still running, and itself waits (pdl_wait) before it touches anything the
// previous kernel produced.  That hides the launch latency and, for the
// matrix-vector kernel, lets the weight stream start early.  Kernels launched
// without the attribute see both device calls as no-ops.
bool pdl_enabled();
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// silu(g) = g * sigmoid(g) rounded to fp16, the first of the two roundings of an
// fp16 SwiGLU.  One definition for every kernel that applies it (stand-alone,
// fused into the quantiser, fused into the M == 1 prologue) so that fused and
// unfused paths agree bit for bit.  ex2.approx / rcp.approx: their ~1e-7 relative
// error is far below the fp16 rounding that follows, and the full-precision expf +
// division made the fused SwiGLU quantiser compute-bound (33 us where the bytes
// take 7).
__device__ __forceinline__ float silu_to_half(float g) {
  return __half2float(__float2half_rn(__fdividef(g, 1.0f + __expf(-g))));
}

// ---- the per-token quantiser's element arithmetic (one definition for every kernel that
// quantises: the row kernels, the fused all-reduce + norm + quantiser)
// round-half-away-from-zero of v = xf * inv as a word whose LOW BYTE is the int8 result.
// floor(|v| + 0.5) with the addition rounded DOWN is exact for every fp32 v (a
// round-to-nearest add would turn the largest float below 0.5 into 1.0).  The floor and the
// float->int conversion are additions of 2^23 and 1.5 * 2^23 (for 0 <= t < 2^22 the sum
// t + 2^23, rounded down, is 2^23 + floor(t); the bits of 1.5 * 2^23 + i end in the two's
// complement of i), which run on the FMA pipe: the conversion instruction has a quarter
// of its rate and the integer select / min / max of the obvious form made the ALU pipe the
// limit of this kernel.  |v| <= 127.00003 for every finite row (inv = 1 / (amax / 127)), so
// the clamp to [-128, 127] of the reference never acts and is not spelled out.
__device__ __forceinline__ int quant_one(float xf, float inv) {
  const float v = __fmul_rn(xf, inv);
  const float t = __fadd_rd(fabsf(v), 0.5f);
  const float m = __fadd_rn(__fadd_rd(t, 8388608.0f), -8388608.0f);  // floor(t), exact
  return __float_as_int(__fadd_rn(copysignf(m, v), 12582912.0f));
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d) {
  uint32_t lo = __byte_perm((uint32_t)a, (uint32_t)b, 0x0040);
  uint32_t hi = __byte_perm((uint32_t)c, (uint32_t)d, 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

// Per-head RMSNorm + rotate-half rope of one head of 128 values by a HALF-warp: lane hl
// (0..15) owns the 8 consecutive elements d = 8 hl .. 8 hl + 7 in `raw`; lanes 0..7 hold the
// first half of the head, lanes 8..15 the elements d + 64, so the rotary partner is 8 lanes
// away.  y = half(x * rsqrt(mean(x^2) + eps) * w) (rounded to fp16 as an unfused norm would),
// o[d] = y[d]*cos - y[d+64]*sin, o[d+64] = y[d+64]*cos + y[d]*sin in fp32, rounded once.
// cs[i] = (cos, sin) of frequency slot i = d mod 64.  hmask names the 16 lanes of the half.
// One definition for the stand-alone rope kernel and the attention kernel's fused prologue,
// so that both produce the same bits.
__device__ __forceinline__ uint4 norm_rope_head128(const uint4 raw, const __half *norm_w, const float2 *cs, float eps,
                                                   int hl, unsigned hmask) {
  const int d0 = 8 * hl, i0 = d0 & 63;
  const bool second = hl >= 8;
  const __half2 *hx = reinterpret_cast<const __half2 *>(&raw);
  float x[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(hx[j]);
    x[2 * j] = f.x;
    x[2 * j + 1] = f.y;
  }
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(x[j], x[j], ss);
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(hmask, ss, o);
  const float r = 1.0f / sqrtf(ss / 128.0f + eps);
  const uint4 wraw = *reinterpret_cast<const uint4 *>(norm_w + d0);
  const __half2 *hw = reinterpret_cast<const __half2 *>(&wraw);
  uint32_t ybits[4];
  float y[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 w = __half22float2(hw[j]);
    const __half2 h = __floats2half2_rn(__fmul_rn(__fmul_rn(x[2 * j], r), w.x), __fmul_rn(__fmul_rn(x[2 * j + 1], r), w.y));
    ybits[j] = *reinterpret_cast<const uint32_t *>(&h);
    const float2 f = __half22float2(h);
    y[2 * j] = f.x;
    y[2 * j + 1] = f.y;
  }
  uint4 outv;
  __half2 *oh = reinterpret_cast<__half2 *>(&outv);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t ob = __shfl_xor_sync(hmask, ybits[j], 8);  // the partner's rounded values
    const float2 ot = __half22float2(*reinterpret_cast<const __half2 *>(&ob));
    const float2 c0 = cs[i0 + 2 * j], c1 = cs[i0 + 2 * j + 1];  // (cos, sin)
    const float a = second ? __fadd_rn(__fmul_rn(y[2 * j], c0.x), __fmul_rn(ot.x, c0.y))
                           : __fsub_rn(__fmul_rn(y[2 * j], c0.x), __fmul_rn(ot.x, c0.y));
    const float b = second ? __fadd_rn(__fmul_rn(y[2 * j + 1], c1.x), __fmul_rn(ot.y, c1.y))
                           : __fsub_rn(__fmul_rn(y[2 * j + 1], c1.x), __fmul_rn(ot.y, c1.y));
    oh[j] = __floats2half2_rn(a, b);
  }
  return outv;
}

template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                          Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (pdl_enabled()) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// Epilogue selection for the integer GEMM kernels.
enum class Epi : int {
  kRawInt32 = 0,    // C int32 [M,N]                      (S2)
  kPerChannel = 1,  // half(fma(float(acc)*sa[m], sw[n], bias[n]))   (S3)
  kPerGroup = 2,    // accf = fma(float(acc_g), sw[g,n], accf); half(fma(accf, sa[m], bias[n]))  (S4)
};

struct GemmArgs {
  const int8_t *a = nullptr;   // [M,K] int8 activations
  const int8_t *b = nullptr;   // [N,K] int8 weights (null when packed4 is set)
  const uint8_t *packed4 = nullptr;  // [K/2,N] packed int4 weights (generic kernel only)
  const uint8_t *w4rows = nullptr;   // [N,K/2] packed int4 weight rows (tensor-core kernels; b is null)
  void *out = nullptr;         // int32 [M,N] or half [M,N]
  const float *sa = nullptr;   // [M]
  const void *sw = nullptr;    // [N] fp32, or [K/gs,N] fp32/fp16
  int sw_is_half = 0;
  const __half *bias = nullptr;  // [N] or null
  int64_t M = 0, N = 0, K = 0;
  int gs = 0;
  Epi epi = Epi::kRawInt32;
  // SwiGLU epilogue (per-channel, tensor-core kernels): the weight rows come as blocks of
  // 32 gate rows followed by their 32 up rows, the output is half(half(silu(g)) * u), [M, N/2],
  // and every row's largest |output| is raised into rowmax[m] (fp32 bits, atomicMax as unsigned)
  float *rowmax = nullptr;
};

// kernels (each returns a cider status code)
int launch_quantize_per_token(const __half *x, int64_t M, int64_t K, int64_t ldx,
                              int8_t *q, float *scale, cudaStream_t st);
// the same with every aligned run of 8 values stored as k0 k2 k4 k6 k1 k3 k5 k7 (the order the
// W4A8 converters of the tensor-core kernels produce the weights in); _ok: shapes it takes
bool quantize_perm8_ok(const __half *x, int64_t K, int64_t ldx, const int8_t *q);
int launch_quantize_per_token_perm8(const __half *x, int64_t M, int64_t K, int64_t ldx, int8_t *q, float *scale,
                                    cudaStream_t st);
int launch_permute8(int8_t *q, int64_t bytes, cudaStream_t st);  // the same permutation, in place
int launch_row_absmax(const __half *x, int64_t M, int64_t K, int64_t ldx, float *amax, cudaStream_t st);
int launch_quantize_given_amax(const __half *x, int64_t M, int64_t K, int64_t ldx, const float *amax, int8_t *q,
                               float *scale, cudaStream_t st, bool reset_amax = false);
int launch_quantize_heads(const __half *a, int64_t B, int64_t heads, int64_t T, int64_t D, int8_t *q,
                          float *scale, cudaStream_t st);
int launch_silu_mul_quant(const __half *gate_up, int64_t M, int64_t inter, int8_t *q, float *scale,
                          cudaStream_t st);
int launch_rmsnorm_quant(const __half *x, const __half *w, float eps, int64_t M, int64_t K,
                         __half *y_or_null, int8_t *q, float *scale, cudaStream_t st);
int launch_add_rmsnorm_quant(__half *x, const __half *delta, const __half *w, float eps, int64_t M,
                             int64_t K, __half *y_or_null, int8_t *q_or_null, float *scale_or_null,
                             cudaStream_t st);
int launch_qk_norm_rope_append(const __half *qkv, const __half *qw, const __half *kw, const float *inv_freq,
                               const int8_t *axis, const int *pos3, int pos_stride, const int *base_dev,
                               int base_host, float eps, __half *q_out, __half *k_cache, __half *v_cache,
                               int64_t B, int64_t T, int nq, int nkv, int64_t Tcap, cudaStream_t st);
int launch_silu_mul(const __half *gu, __half *act, int64_t M, int64_t inter, cudaStream_t st);
int launch_gemm_generic(const GemmArgs &g, cudaStream_t st);
bool gemm_tc_eligible(const GemmArgs &g);
// split-K of the per-channel linear at small M (see gemm_tc.cu): splits == 0 means "do not split"
struct SplitKPlan {
  int splits = 0, kb_per_split = 0, m_pad = 0, bn = 128;
  size_t bytes = 0;  // int32 slabs [splits][m_pad][N]
};
SplitKPlan plan_splitk(int64_t M, int64_t N, int64_t K);
int launch_gemm_tc_splitk(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st);
// per-group counterpart: equal K pieces of whole groups, fp32 slabs, summed in piece order
SplitKPlan plan_pg_splitk(int64_t M, int64_t N, int64_t K);
int launch_gemm_tc_pg_splitk(const GemmArgs &g, const SplitKPlan &pl, void *slabs, cudaStream_t st);
int launch_gemm_tc(const GemmArgs &g, cudaStream_t st);
int set_tile_override(int tile, int bn);  // tests only
const char *last_gemm_kernel();
int launch_gemv(const __half *x, const int8_t *w, const void *sw, int sw_is_half, int gs,
                const __half *bias, __half *y, int64_t N, int64_t K, cudaStream_t st);
int launch_gemv_fused(const __half *x, int mode, const __half *delta, const __half *norm_w, float eps,
                      __half *x_out, const int8_t *w, const void *sw, int sw_is_half, int gs,
                      const __half *bias, __half *y, int64_t N, int64_t K, cudaStream_t st);
// w4: the weight rows are packed int4 ([N, K/2] bytes, high nibble = even k, value + 8)
bool smallm_eligible(int64_t M, int64_t N, int64_t K, int gs, const void *xq, const void *w, const void *sw,
                     bool w4 = false);
int launch_smallm(const int8_t *xq, const float *sa, const int8_t *w, const void *sw, int sw_is_half, int gs,
                  const __half *bias, __half *y, int64_t M, int64_t N, int64_t K, cudaStream_t st,
                  bool w4 = false);
int launch_repack_w4(const uint8_t *packed_kn, uint8_t *w_nk4, int64_t N, int64_t K, cudaStream_t st);
int launch_unpack_w4_nk(const uint8_t *w_nk4, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st);
int launch_unpack_w4(const uint8_t *packed, int8_t *w_nk, int64_t N, int64_t K, cudaStream_t st);
int launch_sdpa_decode(const __half *q, const __half *kc, const __half *vc, __half *out,
                       int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T, int64_t Tcap,
                       float scale, void *workspace, size_t ws_bytes, const int *length_dev,
                       unsigned int *tickets, cudaStream_t st);
int launch_sdpa_decode_fused(const __half *qkv, const __half *q_norm_w, const __half *k_norm_w, const float *inv_freq,
                             const int8_t *axis, const int *pos3, int pos_stride, float eps, __half *kc, __half *vc,
                             __half *out, int64_t B, int64_t Hq, int64_t Hkv, int64_t T, int64_t Tcap, float scale,
                             void *workspace, size_t ws_bytes, const int *length_dev, unsigned int *tickets,
                             cudaStream_t st);
int set_sdpa_kernel(int mode);  // tests only
int read_sdpa_status(unsigned int *out);
int clear_sdpa_status();
size_t sdpa_decode_workspace_bytes(int64_t B, int64_t Hq, int64_t Hkv, int64_t D, int64_t T);

// Device-side status word: kernels whose waits are bounded record here when a
// wait ran out instead of spinning for ever.  0 = clean.
int read_gemv_status(unsigned int *out);
int clear_gemv_status();
int read_glue_status(unsigned int *out);
int clear_glue_status();
int read_peer_status(unsigned int *out);
int clear_peer_status();
int read_device_status(unsigned int *out);
int clear_device_status();

constexpr unsigned kStatusWaitTimeout = 1u;   // an mbarrier wait ran out
constexpr unsigned kStatusBadTmem = 2u;
constexpr unsigned kStatusKvOverflow = 4u;    // a KV-cache append fell outside the cache and was skipped
constexpr unsigned kStatusPeerTimeout = 8u;   // a bounded wait on another GPU's flag ran out

}  // namespace cider
