// One-shot all-reduce (sum) of a small fp16 message over peer-mapped memory, for the
// exchange step of the tensor-parallel decoder: after a row-parallel o_proj / down_proj
// every rank holds a partial [M, hidden] result and needs the sum.  At decode sizes the
// message is a few KB to 64 KB, so the cost of a library all-reduce is its launch and
// protocol latency, and a library call cannot be replayed inside this library's CUDA
// graph of the decode step.  The reference has no multi-device path; this follows the
// generation loop it would sit in (vlm_service/custom_qwen3vl.py:660-679).
//
// Protocol (one kernel launch per rank, no host round trip, NVLink peer stores only):
//   every rank owns an "inbox" in its own memory that all peers have mapped:
//       header  flags[2][8][32] u32, counter[32] u32                (4 KB)
//       data    [2 parities][8 source ranks][slot_bytes]
//   CTA c of rank r handles a fixed slice of the message:
//     1. seq = counter[c] + 1 (local, advanced once per call; all ranks make the same calls,
//        so their counters agree), parity = seq & 1;
//     2. push: its slice of the local partial is stored into data[parity][r] of every PEER's
//        inbox (plain 16-byte stores through the peer mapping);
//     3. publish: __syncthreads, one thread issues a system-scope fence and stores seq into
//        flags[parity][r][c] of every peer with release semantics;
//     4. wait: thread q spins (acquire loads of its OWN memory) until flags[parity][q][c] ==
//        seq; the spin is bounded - when it runs out the kernel records kStatusPeerTimeout,
//        skips the sum and returns;
//     5. sum: fp32, in ascending rank order with the local partial at its own position, so
//        every rank computes the same bits; the result is rounded to fp16 once.
//   Two parities: a rank can be at most one call ahead of a peer (it cannot finish call k+1
//   without that peer's flag for k+1, which the peer sends only after it has finished reading
//   call k's data), so the slots written by call k+2 are never still being read.
// No multicast, no multimem, no load from a peer: peers are only ever written to.
//
// The kernel never waits for another CTA of its own GPU, only for peers' flags.  For a
// one-GPU test the ranks are emulated as ONE cooperative launch (gridDim.y = world), which
// guarantees that the CTAs that wait for one another are resident together.
#include <cstring>

#include "common.cuh"

namespace cider {

__device__ unsigned int g_peer_status = 0;

namespace {

constexpr int kMaxWorld = 8;
constexpr int kMaxCtas = 32;
constexpr int kPeerThreads = 256;
constexpr size_t kHeaderBytes = 4096;
constexpr long long kDefaultWaitCycles = 2000000000ll;  // about a second

struct PeerParams {
  unsigned char *inbox[kMaxWorld];  // every rank's inbox as mapped in this process
  const __half *in[kMaxWorld];      // real launch: only [rank] is used
  __half *out[kMaxWorld];
  long long count;                  // halves, a multiple of 8
  size_t slot_bytes;
  long long wait_cycles;
  int world, rank;                  // rank < 0: emulated, the rank is blockIdx.y
  int absent;                       // emulated only: this rank does not take part (-1: none)
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t *p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t *p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__global__ void __launch_bounds__(kPeerThreads)
peer_allreduce_kernel(const PeerParams p) {
  __shared__ uint32_t seq_s;
  __shared__ int ok_s;
  pdl_launch_dependents();
  const int rank = p.rank >= 0 ? p.rank : (int)blockIdx.y;
  if (rank == p.absent) return;
  const int c = blockIdx.x, tid = threadIdx.x;
  uint32_t *hdr = reinterpret_cast<uint32_t *>(p.inbox[rank]);
  uint32_t *counter = hdr + 2 * kMaxWorld * kMaxCtas;
  if (tid == 0) {
    seq_s = counter[c] + 1;
    ok_s = 1;
  }
  __syncthreads();
  const uint32_t seq = seq_s;
  const int par = (int)(seq & 1u);
  pdl_wait();  // the partial comes from the kernel before this one

  const long long vecs = p.count / 8;  // 16-byte vectors
  const long long per = (vecs + gridDim.x - 1) / gridDim.x;
  const long long v0 = (long long)c * per, v1 = min(vecs, v0 + per);
  const uint4 *in = reinterpret_cast<const uint4 *>(p.in[rank]);
  const size_t slot = (size_t)par * kMaxWorld * p.slot_bytes;

  // 2. push the local slice into every peer's inbox
  for (long long v = v0 + tid; v < v1; v += kPeerThreads) {
    const uint4 x = in[v];
    for (int q = 0; q < p.world; ++q) {
      if (q == rank) continue;
      uint4 *dst = reinterpret_cast<uint4 *>(p.inbox[q] + kHeaderBytes + slot + (size_t)rank * p.slot_bytes);
      dst[v] = x;
    }
  }
  __syncthreads();
  // 3. publish
  if (tid == 0) {
    __threadfence_system();
    for (int q = 0; q < p.world; ++q) {
      if (q == rank) continue;
      uint32_t *f = reinterpret_cast<uint32_t *>(p.inbox[q]) + ((size_t)par * kMaxWorld + rank) * kMaxCtas + c;
      st_release_sys(f, seq);
    }
  }
  // 4. bounded wait for every peer's flag in this rank's own inbox
  if (tid < p.world && tid != rank) {
    const uint32_t *f = hdr + ((size_t)par * kMaxWorld + tid) * kMaxCtas + c;
    const long long t0 = clock64();
    while (ld_acquire_sys(f) != seq) {
      if (clock64() - t0 > p.wait_cycles) {
        ok_s = 0;
        atomicOr(&g_peer_status, kStatusPeerTimeout);
        break;
      }
    }
  }
  __syncthreads();
  if (ok_s) {
    // 5. sum in ascending rank order (the same bits on every rank)
    const unsigned char *mine = p.inbox[rank] + kHeaderBytes + slot;
    uint4 *out = reinterpret_cast<uint4 *>(p.out[rank]);
    for (long long v = v0 + tid; v < v1; v += kPeerThreads) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int q = 0; q < p.world; ++q) {
        const uint4 x = q == rank ? in[v]
                                  : __ldcg(reinterpret_cast<const uint4 *>(mine + (size_t)q * p.slot_bytes) + v);
        const __half2 *h = reinterpret_cast<const __half2 *>(&x);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
          acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
        }
      }
      uint4 o;
      __half2 *oh = reinterpret_cast<__half2 *>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
      out[v] = o;
    }
  }
  if (tid == 0) counter[c] = seq;  // advance also after a time-out: the call was made
}

// ---- the same exchange fused with what follows it in a decoder layer: the all-reduced
// partial output of a row-parallel linear is the residual delta, x <- half(x + delta), and the
// RMSNorm of x (optionally quantised per token) is the next linear's input.  One CTA per row
// (the norm and the absmax are row reductions), K / 8 threads, each owning 8 consecutive
// elements from the push to the quantised store; the row never goes back to global memory
// between the exchange and the norm.  Arithmetic of the unfused kernels: fp32 sum in rank
// order rounded to fp16 (cider_allreduce_f16), fp16 residual add, norm rounded to fp16 before
// it is quantised (cider_add_rmsnorm_quant).
struct PeerNormParams {
  PeerParams pp;          // in[] = the partial outputs [M, K]; out[] = the residual stream x [M, K], in place
  const __half *norm_w[kMaxWorld];
  __half *y[kMaxWorld];   // optional fp16 norm output
  int8_t *q[kMaxWorld];   // optional int8 norm output ...
  float *scale[kMaxWorld];  // ... with its per-row scale
  float eps;
  int K;
};

__global__ void __launch_bounds__(1024)
peer_allreduce_norm_kernel(const PeerNormParams np) {
  const PeerParams &p = np.pp;
  __shared__ uint32_t seq_s;
  __shared__ int ok_s;
  __shared__ float red_s[32];
  pdl_launch_dependents();
  const int rank = p.rank >= 0 ? p.rank : (int)blockIdx.y;
  if (rank == p.absent) return;
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nvec = np.K / 8, nwarps = (blockDim.x + 31) >> 5;
  const bool active = tid < nvec;
  uint32_t *hdr = reinterpret_cast<uint32_t *>(p.inbox[rank]);
  uint32_t *counter = hdr + 2 * kMaxWorld * kMaxCtas;
  if (tid == 0) {
    seq_s = counter[row] + 1;
    ok_s = 1;
  }
  __syncthreads();
  const uint32_t seq = seq_s;
  const int par = (int)(seq & 1u);
  pdl_wait();
  const size_t slot = (size_t)par * kMaxWorld * p.slot_bytes;
  const long long v = (long long)row * nvec + tid;
  uint4 mine = make_uint4(0, 0, 0, 0);
  if (active) {
    mine = reinterpret_cast<const uint4 *>(p.in[rank])[v];
    for (int q = 0; q < p.world; ++q) {
      if (q == rank) continue;
      reinterpret_cast<uint4 *>(p.inbox[q] + kHeaderBytes + slot + (size_t)rank * p.slot_bytes)[v] = mine;
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    for (int q = 0; q < p.world; ++q) {
      if (q == rank) continue;
      st_release_sys(reinterpret_cast<uint32_t *>(p.inbox[q]) + ((size_t)par * kMaxWorld + rank) * kMaxCtas + row, seq);
    }
  }
  if (tid < p.world && tid != rank) {
    const uint32_t *f = hdr + ((size_t)par * kMaxWorld + tid) * kMaxCtas + row;
    const long long t0 = clock64();
    while (ld_acquire_sys(f) != seq) {
      if (clock64() - t0 > p.wait_cycles) {
        ok_s = 0;
        atomicOr(&g_peer_status, kStatusPeerTimeout);
        break;
      }
    }
  }
  __syncthreads();
  if (!ok_s) {
    if (tid == 0) counter[row] = seq;
    return;
  }
  // ---- delta = half(sum over ranks in order); x <- half(x + delta)
  float xf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  uint4 *xrow = reinterpret_cast<uint4 *>(p.out[rank]);
  if (active) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    const unsigned char *inb = p.inbox[rank] + kHeaderBytes + slot;
    for (int q = 0; q < p.world; ++q) {
      const uint4 x = q == rank ? mine : __ldcg(reinterpret_cast<const uint4 *>(inb + (size_t)q * p.slot_bytes) + v);
      const __half2 *h = reinterpret_cast<const __half2 *>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
      }
    }
    const uint4 xr = xrow[v];
    const __half2 *hx = reinterpret_cast<const __half2 *>(&xr);
    uint4 xo;
    __half2 *ho = reinterpret_cast<__half2 *>(&xo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 d = __half22float2(__floats2half2_rn(acc[2 * j], acc[2 * j + 1]));  // the all-reduce's fp16 result
      const float2 a = __half22float2(hx[j]);
      ho[j] = __floats2half2_rn(__fadd_rn(a.x, d.x), __fadd_rn(a.y, d.y));
      const float2 f = __half22float2(ho[j]);
      xf[2 * j] = f.x;
      xf[2 * j + 1] = f.y;
    }
    xrow[v] = xo;
  }
  // ---- RMSNorm of the updated row
  float ss = 0.0f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(xf[j], xf[j], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (lane == 0) red_s[warp] = ss;
  __syncthreads();
  ss = 0.0f;
  for (int w = 0; w < nwarps; ++w) ss += red_s[w];
  const float r = 1.0f / sqrtf(ss / (float)np.K + np.eps);
  float nf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  float amax = 0.0f;
  if (active) {
    const uint4 wr = reinterpret_cast<const uint4 *>(np.norm_w[rank])[tid];
    const __half2 *hw = reinterpret_cast<const __half2 *>(&wr);
    uint4 yo;
    __half2 *hy = reinterpret_cast<__half2 *>(&yo);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 w = __half22float2(hw[j]);
      hy[j] = __floats2half2_rn(__fmul_rn(__fmul_rn(xf[2 * j], r), w.x), __fmul_rn(__fmul_rn(xf[2 * j + 1], r), w.y));
      const float2 f = __half22float2(hy[j]);
      nf[2 * j] = f.x;
      nf[2 * j + 1] = f.y;
      amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
    if (np.y[rank] != nullptr) reinterpret_cast<uint4 *>(np.y[rank])[v] = yo;
  }
  if (np.q[rank] != nullptr) {
    // ---- per-token quantiser of the fp16 norm output (the arithmetic of quantize_rows_kernel)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();  // red_s is reused
    if (lane == 0) red_s[warp] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < nwarps; ++w) amax = fmaxf(amax, red_s[w]);
    float sc = __fdiv_rn(amax, 127.0f);
    if (sc == 0.0f) sc = 1.0f;
    const float inv = __fdiv_rn(1.0f, sc);
    if (tid == 0) np.scale[rank][row] = sc;
    if (active) {
      const uint32_t lo = pack4(quant_one(nf[0], inv), quant_one(nf[1], inv), quant_one(nf[2], inv), quant_one(nf[3], inv));
      const uint32_t hi = pack4(quant_one(nf[4], inv), quant_one(nf[5], inv), quant_one(nf[6], inv), quant_one(nf[7], inv));
      reinterpret_cast<uint2 *>(np.q[rank])[v] = make_uint2(lo, hi);
    }
  }
  if (tid == 0) counter[row] = seq;
}

size_t slot_bytes_of(size_t inbox_bytes) {
  if (inbox_bytes <= kHeaderBytes) return 0;
  return (inbox_bytes - kHeaderBytes) / (2 * kMaxWorld) / 256 * 256;
}

int fill_params(PeerParams *p, int64_t count, int world, void *const *inboxes, size_t inbox_bytes,
                int64_t wait_cycles, const char *op) {
  if (world < 2 || world > kMaxWorld)
    return fail(CIDER_E_INVALID, std::string(op) + ": world must be 2.." + std::to_string(kMaxWorld));
  if (count <= 0 || count % 8 != 0)
    return fail(CIDER_E_SHAPE, std::string(op) + ": count must be a positive multiple of 8 halves");
  if (!inboxes) return fail(CIDER_E_INVALID, std::string(op) + ": null inbox table");
  p->slot_bytes = slot_bytes_of(inbox_bytes);
  if ((size_t)count * 2 > p->slot_bytes)
    return fail(CIDER_E_WORKSPACE, std::string(op) + ": message of " + std::to_string(count * 2) +
                                       " bytes exceeds the inbox slot of " + std::to_string(p->slot_bytes));
  for (int q = 0; q < kMaxWorld; ++q) {
    p->inbox[q] = nullptr;
    p->in[q] = nullptr;
    p->out[q] = nullptr;
  }
  for (int q = 0; q < world; ++q) {
    if (!inboxes[q] || (reinterpret_cast<uintptr_t>(inboxes[q]) & 255u))
      return fail(CIDER_E_INVALID, std::string(op) + ": inbox pointers must be non-null and 256-byte aligned");
    p->inbox[q] = static_cast<unsigned char *>(inboxes[q]);
  }
  p->count = count;
  p->world = world;
  p->wait_cycles = wait_cycles > 0 ? wait_cycles : kDefaultWaitCycles;
  p->absent = -1;
  return CIDER_OK;
}

unsigned grid_for(int64_t count) {
  const int64_t vecs = count / 8;
  int64_t ctas = (vecs + kPeerThreads - 1) / kPeerThreads;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  return (unsigned)ctas;
}

}  // namespace

int read_peer_status(unsigned int *out) {
  return check_cuda(cudaMemcpyFromSymbol(out, g_peer_status, sizeof(unsigned int)), "read peer status");
}
int clear_peer_status() {
  unsigned int z = 0;
  return check_cuda(cudaMemcpyToSymbol(g_peer_status, &z, sizeof(z)), "clear peer status");
}

}  // namespace cider

using namespace cider;

extern "C" {

size_t cider_peer_max_bytes(size_t inbox_bytes) { return slot_bytes_of(inbox_bytes); }

int cider_peer_alloc(size_t bytes, void **ptr, unsigned char *handle64) {
  if (!ptr || !handle64) return fail(CIDER_E_INVALID, "peer_alloc: null pointer");
  if (slot_bytes_of(bytes) == 0) return fail(CIDER_E_INVALID, "peer_alloc: inbox too small (needs > 4 KB + 16 slots)");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  void *p = nullptr;
  int rc = check_cuda(cudaMalloc(&p, bytes), "peer_alloc: cudaMalloc");
  if (rc) return rc;
  if ((rc = check_cuda(cudaMemset(p, 0, bytes), "peer_alloc: cudaMemset"))) {
    cudaFree(p);
    return rc;
  }
  cudaIpcMemHandle_t h;
  if ((rc = check_cuda(cudaIpcGetMemHandle(&h, p), "peer_alloc: cudaIpcGetMemHandle"))) {
    cudaFree(p);
    return rc;
  }
  memcpy(handle64, &h, 64);
  *ptr = p;
  return CIDER_OK;
}

int cider_peer_open(const unsigned char *handle64, void **ptr) {
  if (!ptr || !handle64) return fail(CIDER_E_INVALID, "peer_open: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return check_cuda(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess), "peer_open: cudaIpcOpenMemHandle");
}

int cider_peer_close(void *ptr) {
  if (!ptr) return CIDER_OK;
  return check_cuda(cudaIpcCloseMemHandle(ptr), "peer_close: cudaIpcCloseMemHandle");
}

int cider_peer_free(void *ptr) {
  if (!ptr) return CIDER_OK;
  return check_cuda(cudaFree(ptr), "peer_free: cudaFree");
}

int cider_peer_reset(void *own_inbox, void *stream) {
  if (!own_inbox) return fail(CIDER_E_INVALID, "peer_reset: null pointer");
  return check_cuda(cudaMemsetAsync(own_inbox, 0, kHeaderBytes, static_cast<cudaStream_t>(stream)), "peer_reset");
}

int cider_allreduce_f16(const void *in, void *out, int64_t count, int rank, int world, void *const *inboxes,
                        size_t inbox_bytes, int64_t wait_cycles, void *stream) {
  PeerParams p;
  int rc = fill_params(&p, count, world, inboxes, inbox_bytes, wait_cycles, "allreduce_f16");
  if (rc) return rc;
  if (rank < 0 || rank >= world) return fail(CIDER_E_INVALID, "allreduce_f16: rank out of range");
  if (!in || !out) return fail(CIDER_E_INVALID, "allreduce_f16: null pointer");
  if ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u)
    return fail(CIDER_E_ALIGNMENT, "allreduce_f16: in / out must be 16-byte aligned");
  p.rank = rank;
  p.in[rank] = static_cast<const __half *>(in);
  p.out[rank] = static_cast<__half *>(out);
  return check_cuda(launch_kernel(peer_allreduce_kernel, dim3(grid_for(count)), dim3(kPeerThreads), 0,
                                  static_cast<cudaStream_t>(stream), p),
                    "allreduce_f16 launch");
}

static int fill_norm(PeerNormParams *np, int64_t M, int64_t K, float eps, int world, void *const *inboxes,
                     size_t inbox_bytes, int64_t wait_cycles, const char *op) {
  if (M <= 0 || M > kMaxCtas) return fail(CIDER_E_SHAPE, std::string(op) + ": 1 <= M <= " + std::to_string(kMaxCtas));
  if (K <= 0 || K % 8 != 0 || K > 8192) return fail(CIDER_E_SHAPE, std::string(op) + ": K must be a multiple of 8, at most 8192");
  int rc = fill_params(&np->pp, M * K, world, inboxes, inbox_bytes, wait_cycles, op);
  if (rc) return rc;
  for (int q = 0; q < kMaxWorld; ++q) {
    np->norm_w[q] = nullptr;
    np->y[q] = nullptr;
    np->q[q] = nullptr;
    np->scale[q] = nullptr;
  }
  np->eps = eps;
  np->K = (int)K;
  return CIDER_OK;
}

static unsigned norm_threads(int64_t K) { return (unsigned)(((K / 8) + 31) / 32 * 32); }

int cider_allreduce_add_rmsnorm_quant(const void *partial, void *x, const void *norm_w, float eps, int64_t M, int64_t K,
                                      void *y, void *q, float *scale, int rank, int world, void *const *inboxes,
                                      size_t inbox_bytes, int64_t wait_cycles, void *stream) {
  PeerNormParams np;
  int rc = fill_norm(&np, M, K, eps, world, inboxes, inbox_bytes, wait_cycles, "allreduce_add_rmsnorm_quant");
  if (rc) return rc;
  if (rank < 0 || rank >= world) return fail(CIDER_E_INVALID, "allreduce_add_rmsnorm_quant: rank out of range");
  if (!partial || !x || !norm_w) return fail(CIDER_E_INVALID, "allreduce_add_rmsnorm_quant: null pointer");
  if (!y && !q) return fail(CIDER_E_INVALID, "allreduce_add_rmsnorm_quant: neither an fp16 nor an int8 output given");
  if (q && !scale) return fail(CIDER_E_INVALID, "allreduce_add_rmsnorm_quant: int8 output without a scale output");
  for (const void *ptr : {partial, (const void *)x, norm_w, (const void *)y})
    if (reinterpret_cast<uintptr_t>(ptr) & 15u)
      return fail(CIDER_E_ALIGNMENT, "allreduce_add_rmsnorm_quant: fp16 buffers must be 16-byte aligned");
  if (reinterpret_cast<uintptr_t>(q) & 7u) return fail(CIDER_E_ALIGNMENT, "allreduce_add_rmsnorm_quant: q must be 8-byte aligned");
  np.pp.rank = rank;
  np.pp.in[rank] = static_cast<const __half *>(partial);
  np.pp.out[rank] = static_cast<__half *>(x);
  np.norm_w[rank] = static_cast<const __half *>(norm_w);
  np.y[rank] = static_cast<__half *>(y);
  np.q[rank] = static_cast<int8_t *>(q);
  np.scale[rank] = scale;
  return check_cuda(launch_kernel(peer_allreduce_norm_kernel, dim3((unsigned)M), dim3(norm_threads(K)), 0,
                                  static_cast<cudaStream_t>(stream), np),
                    "allreduce_add_rmsnorm_quant launch");
}

int cider_testing_allreduce_norm_emulated(const void *const *partials, void *const *xs, const void *norm_w, float eps,
                                          int64_t M, int64_t K, void *const *ys, void *const *qs, float *const *scales,
                                          int world, void *const *inboxes, size_t inbox_bytes, void *stream) {
  PeerNormParams np;
  int rc = fill_norm(&np, M, K, eps, world, inboxes, inbox_bytes, 0, "allreduce_norm_emulated");
  if (rc) return rc;
  if (!partials || !xs || !norm_w || !ys || !qs || !scales) return fail(CIDER_E_INVALID, "allreduce_norm_emulated: null pointer");
  for (int r = 0; r < world; ++r) {
    np.pp.in[r] = static_cast<const __half *>(partials[r]);
    np.pp.out[r] = static_cast<__half *>(xs[r]);
    np.norm_w[r] = static_cast<const __half *>(norm_w);
    np.y[r] = static_cast<__half *>(ys[r]);
    np.q[r] = static_cast<int8_t *>(qs[r]);
    np.scale[r] = scales[r];
  }
  np.pp.rank = -1;
  void *args[] = {&np};
  return check_cuda(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(peer_allreduce_norm_kernel),
                                                dim3((unsigned)M, (unsigned)world), dim3(norm_threads(K)), args, 0,
                                                static_cast<cudaStream_t>(stream)),
                    "allreduce_norm_emulated launch");
}

int cider_testing_allreduce_emulated(const void *const *ins, void *const *outs, int64_t count, int world,
                                     void *const *inboxes, size_t inbox_bytes, int64_t wait_cycles, int absent_rank,
                                     void *stream) {
  PeerParams p;
  int rc = fill_params(&p, count, world, inboxes, inbox_bytes, wait_cycles, "allreduce_emulated");
  if (rc) return rc;
  if (!ins || !outs) return fail(CIDER_E_INVALID, "allreduce_emulated: null pointer");
  for (int q = 0; q < world; ++q) {
    if (!ins[q] || !outs[q]) return fail(CIDER_E_INVALID, "allreduce_emulated: null pointer");
    p.in[q] = static_cast<const __half *>(ins[q]);
    p.out[q] = static_cast<__half *>(outs[q]);
  }
  p.rank = -1;
  p.absent = absent_rank;
  // the ranks wait for one another inside one launch: all their CTAs must be resident
  // together, which a cooperative launch guarantees (or refuses)
  void *args[] = {&p};
  return check_cuda(cudaLaunchCooperativeKernel(reinterpret_cast<void *>(peer_allreduce_kernel),
                                                dim3(grid_for(count), (unsigned)world), dim3(kPeerThreads), args, 0,
                                                static_cast<cudaStream_t>(stream)),
                    "allreduce_emulated launch");
}

}  // extern "C"
