// cider_perchannel_linear_host: the W8A8 per-channel linear for callers whose
// activations and results live in HOST memory.  The reference runs on unified
// memory (an MLX array is addressable by CPU and GPU alike), so a program that
// adopts this library from the reference's side of the boundary holds host
// pointers; on a discrete GPU the copies across PCIe then cost ~20x the linear
// itself (M=8192, N=10240, K=2560: 42 MB up, 168 MB down, 0.19 ms of kernels).
// This entry hides what can be hidden: the rows are cut into chunks and the
// three steps of a chunk - copy in, quantise + GEMM, copy out - run on three
// streams, so that the upload of chunk i+1 and the download of chunk i-1 (PCIe is
// full duplex) overlap the kernels of chunk i.  The call then takes about as
// long as the larger of the two transfers instead of their sum.
//
// Staging buffers (two of each: fp16 rows in, int8 rows + scales, fp16 rows out)
// belong to the library, one set per device, allocated on first use and grown
// on demand; calls on one device are serialised by a mutex.  Arithmetic per row
// is that of cider_perchannel_linear for M > 1 (a chunk of one row is still
// quantised: the M == 1 matrix-vector semantics apply only when the whole call
// has M == 1), so the result is bit-identical to the device-buffer entry.
#include <mutex>

#include "common.cuh"

namespace cider {
namespace {

constexpr int kMaxDev = 64;
constexpr int kSlots = 2;

struct HostPipe {
  bool ready = false;
  cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
  cudaEvent_t ev_start = nullptr, ev_in[kSlots] = {}, ev_run[kSlots] = {}, ev_out[kSlots] = {};
  void *x_dev[kSlots] = {}, *q_dev[kSlots] = {}, *y_dev[kSlots] = {};
  float *sa_dev[kSlots] = {};
  size_t x_cap = 0, q_cap = 0, y_cap = 0, sa_cap = 0;
};
std::mutex g_mu[kMaxDev];
HostPipe g_pipe[kMaxDev];

int grow(void **p, size_t *cap, size_t need, bool shared_cap) {
  if (need <= *cap && *p != nullptr) return CIDER_OK;
  if (*p != nullptr) {
    cudaError_t e = cudaFree(*p);
    if (e != cudaSuccess) return check_cuda(e, "perchannel_linear_host: cudaFree");
    *p = nullptr;
  }
  cudaError_t e = cudaMalloc(p, need);
  if (e != cudaSuccess) return check_cuda(e, "perchannel_linear_host: cudaMalloc");
  if (!shared_cap) *cap = need;
  return CIDER_OK;
}

int ensure_pipe(HostPipe &hp, size_t x_bytes, size_t q_bytes, size_t sa_bytes, size_t y_bytes) {
  cudaError_t e;
  if (!hp.ready) {
    if ((e = cudaStreamCreateWithFlags(&hp.s_in, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&hp.s_run, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaStreamCreateWithFlags(&hp.s_out, cudaStreamNonBlocking)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: stream creation");
    if ((e = cudaEventCreateWithFlags(&hp.ev_start, cudaEventDisableTiming)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: event creation");
    for (int i = 0; i < kSlots; ++i) {
      if ((e = cudaEventCreateWithFlags(&hp.ev_in[i], cudaEventDisableTiming)) != cudaSuccess ||
          (e = cudaEventCreateWithFlags(&hp.ev_run[i], cudaEventDisableTiming)) != cudaSuccess ||
          (e = cudaEventCreateWithFlags(&hp.ev_out[i], cudaEventDisableTiming)) != cudaSuccess)
        return check_cuda(e, "perchannel_linear_host: event creation");
    }
    hp.ready = true;
  }
  // a buffer about to be replaced may still be in use by an earlier call
  if (x_bytes > hp.x_cap || q_bytes > hp.q_cap || sa_bytes > hp.sa_cap || y_bytes > hp.y_cap) {
    if ((e = cudaStreamSynchronize(hp.s_in)) != cudaSuccess || (e = cudaStreamSynchronize(hp.s_run)) != cudaSuccess ||
        (e = cudaStreamSynchronize(hp.s_out)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: stream synchronize");
  }
  int rc;
  for (int i = 0; i < kSlots; ++i) {
    if ((rc = grow(&hp.x_dev[i], &hp.x_cap, x_bytes, i + 1 < kSlots))) return rc;
    if ((rc = grow(&hp.q_dev[i], &hp.q_cap, q_bytes, i + 1 < kSlots))) return rc;
    if ((rc = grow(reinterpret_cast<void **>(&hp.sa_dev[i]), &hp.sa_cap, sa_bytes, i + 1 < kSlots))) return rc;
    if ((rc = grow(&hp.y_dev[i], &hp.y_cap, y_bytes, i + 1 < kSlots))) return rc;
  }
  return CIDER_OK;
}

}  // namespace
}  // namespace cider

using namespace cider;

extern "C" int cider_perchannel_linear_host(const void *x_host, const void *w, const float *sw, const void *bias,
                                            void *y_host, int64_t M, int64_t N, int64_t K, int64_t chunk_rows,
                                            void *stream) {
  if (M < 0 || N < 1 || K < 1) return fail(CIDER_E_INVALID, "perchannel_linear_host: bad dimensions");
  if (M == 0) return CIDER_OK;
  if (!x_host || !w || !sw || !y_host) return fail(CIDER_E_INVALID, "perchannel_linear_host: null pointer");
  if (chunk_rows < 0) return fail(CIDER_E_INVALID, "perchannel_linear_host: chunk_rows must be >= 0");
  const int dev = current_device();
  if (dev < 0 || dev >= kMaxDev) return fail(CIDER_E_UNSUPPORTED, "perchannel_linear_host: device index out of range");
  if (chunk_rows == 0) {
    // about 16 MB of output per chunk: long enough transfers to run PCIe at its
    // rate, short enough that the first upload and the last download - the parts
    // nothing overlaps - stay small
    chunk_rows = (16ll << 20) / (2 * N);
    chunk_rows = chunk_rows / 128 * 128;
    if (chunk_rows < 128) chunk_rows = 128;
  }
  if (chunk_rows > M) chunk_rows = M;
  cudaStream_t user = static_cast<cudaStream_t>(stream);
  std::lock_guard<std::mutex> lock(g_mu[dev]);
  HostPipe &hp = g_pipe[dev];
  int rc = ensure_pipe(hp, (size_t)chunk_rows * K * 2, (size_t)chunk_rows * K, (size_t)chunk_rows * sizeof(float),
                       (size_t)chunk_rows * N * 2);
  if (rc) return rc;
  cudaError_t e;
  // everything below is ordered after the work already queued on the caller's stream
  if ((e = cudaEventRecord(hp.ev_start, user)) != cudaSuccess) return check_cuda(e, "perchannel_linear_host: event record");
  if ((e = cudaStreamWaitEvent(hp.s_in, hp.ev_start, 0)) != cudaSuccess ||
      (e = cudaStreamWaitEvent(hp.s_run, hp.ev_start, 0)) != cudaSuccess ||
      (e = cudaStreamWaitEvent(hp.s_out, hp.ev_start, 0)) != cudaSuccess)
    return check_cuda(e, "perchannel_linear_host: stream wait");
  const char *xh = static_cast<const char *>(x_host);
  char *yh = static_cast<char *>(y_host);
  int64_t done = 0;
  for (int64_t c = 0; done < M; ++c) {
    const int slot = (int)(c % kSlots);
    const int64_t rows = M - done < chunk_rows ? M - done : chunk_rows;
    // copy in: the slot's fp16 rows were last read by the quantiser of chunk c - 2
    // (or by an earlier call: waiting on an event that was never recorded is a no-op)
    if ((e = cudaStreamWaitEvent(hp.s_in, hp.ev_run[slot], 0)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: stream wait");
    if ((e = cudaMemcpyAsync(hp.x_dev[slot], xh + (size_t)done * K * 2, (size_t)rows * K * 2, cudaMemcpyHostToDevice,
                             hp.s_in)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: upload");
    if ((e = cudaEventRecord(hp.ev_in[slot], hp.s_in)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: event record");
    // kernels: the slot's output rows were last read by the download of chunk c - 2
    if ((e = cudaStreamWaitEvent(hp.s_run, hp.ev_in[slot], 0)) != cudaSuccess ||
        (e = cudaStreamWaitEvent(hp.s_run, hp.ev_out[slot], 0)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: stream wait");
    if (M == 1) {
      rc = cider_perchannel_linear(hp.x_dev[slot], w, sw, bias, hp.y_dev[slot], 1, N, K, nullptr, 0, hp.s_run);
    } else {
      rc = cider_quantize_per_token(hp.x_dev[slot], rows, K, K, hp.q_dev[slot], hp.sa_dev[slot], hp.s_run);
      if (!rc)
        rc = cider_linear_prequantized(hp.q_dev[slot], hp.sa_dev[slot], w, sw, CIDER_F32, 0, bias, hp.y_dev[slot],
                                       rows, N, K, hp.s_run);
    }
    if (rc) return rc;
    if ((e = cudaEventRecord(hp.ev_run[slot], hp.s_run)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: event record");
    // copy out
    if ((e = cudaStreamWaitEvent(hp.s_out, hp.ev_run[slot], 0)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: stream wait");
    if ((e = cudaMemcpyAsync(yh + (size_t)done * N * 2, hp.y_dev[slot], (size_t)rows * N * 2, cudaMemcpyDeviceToHost,
                             hp.s_out)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: download");
    if ((e = cudaEventRecord(hp.ev_out[slot], hp.s_out)) != cudaSuccess)
      return check_cuda(e, "perchannel_linear_host: event record");
    done += rows;
  }
  // the caller's stream continues once the last rows have reached host memory
  // (downloads complete in order on one stream, so the last event covers all)
  const int last = (int)(((M + chunk_rows - 1) / chunk_rows - 1) % kSlots);
  if ((e = cudaStreamWaitEvent(user, hp.ev_out[last], 0)) != cudaSuccess)
    return check_cuda(e, "perchannel_linear_host: stream wait");
  return CIDER_OK;
}
