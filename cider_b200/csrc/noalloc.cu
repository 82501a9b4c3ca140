// cider_perchannel_linear_noalloc: the W8A8 per-channel linear for callers that
// cannot hand the library a scratch buffer because they cannot allocate device
// memory at the point of the call: code running under someone else's memory
// budget (a plugin inside a server whose pool is fully carved up at start-up),
// a real-time or interrupt-like path where cudaMalloc's implicit device
// synchronisation is not acceptable, or a host runtime with no allocator of its
// own to lend a buffer from.
//
// The regular entry point (cider_perchannel_linear) needs scratch for the int8
// copy of the activations and their per-row scales.  Here that scratch is a
// fixed array inside the library image, so every GPU that loads the library
// holds kScratchBytes of it until the process exits, and problems larger than
// the array are refused.
//
// What a user has to know:
//   * capacity: M*K <= 8 MiB and M <= 16384 (M > 1); M == 1 needs no scratch
//     and has no limit;
//   * the first call on each device looks up the array's device address
//     (cudaGetSymbolAddress) - make that first call outside any stream capture;
//   * every call on a device uses the SAME array.  It still holds the previous
//     call's bytes; nothing in it has to start at zero, because the quantiser
//     overwrites every byte the GEMM will read (rows past M are never read: the
//     GEMM's loads are bounded by M).  Two calls that may run at the same time
//     on one GPU (different streams, different host threads) race on it - order
//     them on one stream or use the regular entry point with separate buffers;
//   * no cudaMalloc, cudaFree or other allocating routine is called;
//   * results are the bits of cider_perchannel_linear.  Speed differs in one case:
//     shapes for which the regular entry point splits K (M <= 512, few output tiles,
//     long K) run unsplit here, since the split needs int32 slabs that do not fit the
//     array; expect those calls to take up to twice as long.
#include <mutex>

#include "common.cuh"

constexpr size_t kMaxActBytes = 8u << 20;   // int8 activations, M*K
constexpr size_t kMaxRows = 16384;          // fp32 row scales
constexpr size_t kScratchBytes = kMaxActBytes + kMaxRows * sizeof(float);

// The scratch itself.  In host code this name is only a handle for the runtime's
// symbol table, never an address a kernel may be given; the address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

namespace cider {
namespace {

constexpr int kMaxDev = 64;
std::mutex g_mu;
unsigned char *g_scratch_ptr[kMaxDev] = {nullptr};

// Device address of the scratch array on the CURRENT device, resolved once per
// device.
int scratch_for_current_device(unsigned char **out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return check_cuda(e, "perchannel_linear_noalloc: cudaGetDevice");
  if (dev < 0 || dev >= kMaxDev)
    return fail(CIDER_E_UNSUPPORTED, "perchannel_linear_noalloc: device index out of range");
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_ptr[dev] == nullptr) {
    unsigned char *p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_noalloc_scratch);
    if (e != cudaSuccess) return check_cuda(e, "perchannel_linear_noalloc: cudaGetSymbolAddress");
    if (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 255u))
      return fail(CIDER_E_CUDA, "perchannel_linear_noalloc: scratch symbol has no usable address");
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return CIDER_OK;
}

}  // namespace
}  // namespace cider

using namespace cider;

extern "C" int cider_perchannel_linear_noalloc(const void *x, const void *w, const float *sw,
                                               const void *bias, void *y, int64_t M, int64_t N,
                                               int64_t K, void *stream) {
  if (M < 0 || N <= 0 || K <= 0)
    return fail(CIDER_E_INVALID, "perchannel_linear_noalloc: need M >= 0, N > 0, K > 0");
  if (N > ((int64_t)1 << 30) || K > ((int64_t)1 << 30) || M > ((int64_t)1 << 30))
    return fail(CIDER_E_INVALID, "perchannel_linear_noalloc: dimension exceeds 2^30");
  if (M == 0) return CIDER_OK;
  if (!x || !w || !sw || !y) return fail(CIDER_E_INVALID, "perchannel_linear_noalloc: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (M == 1)  // matrix-vector path: activations are not quantised, no scratch at all
    return launch_gemv(static_cast<const __half *>(x), static_cast<const int8_t *>(w), sw, 0, 0,
                       static_cast<const __half *>(bias), static_cast<__half *>(y), N, K, st);
  if ((size_t)M > kMaxRows || (size_t)M * (size_t)K > kMaxActBytes)
    return fail(CIDER_E_WORKSPACE,
                "perchannel_linear_noalloc: M=" + std::to_string(M) + ", K=" + std::to_string(K) +
                    " exceeds the built-in scratch (M*K <= " + std::to_string(kMaxActBytes) +
                    " and M <= " + std::to_string(kMaxRows) +
                    "); use cider_perchannel_linear with a caller-provided workspace");
  unsigned char *scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  int8_t *a_q = reinterpret_cast<int8_t *>(scratch);
  float *sa = reinterpret_cast<float *>(scratch + kMaxActBytes);
  rc = launch_quantize_per_token(static_cast<const __half *>(x), M, K, K, a_q, sa, st);
  if (rc) return rc;
  // From here on the call is the regular one on pre-quantised activations: the same
  // kernel choice (weight-streaming kernel for a handful of rows, tensor-core tiles
  // otherwise, the testing backend override honoured).  The one form it never takes is
  // the split-K plan of cider_perchannel_linear, whose int32 slabs would need more
  // scratch than this array has.
  return cider_linear_prequantized(a_q, sa, w, sw, CIDER_F32, 0, bias, y, M, N, K, stream);
}
