// micro-benchmark: how fast can 26 MB be read once per launch, by method
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <vector>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok;
}
__device__ __forceinline__ bool bwait(uint32_t bar, uint32_t parity) {
  long long t0 = clock64();
  while (!try_wait(bar, parity)) if (clock64() - t0 > 2000000000ll) return false;
  return true;
}
__global__ void k_empty(int *out) { if (threadIdx.x == 0 && blockIdx.x == 9999) out[0] = 1; }

__global__ void __launch_bounds__(1024) k_ldg(const uint4 *__restrict__ src, size_t n16, unsigned *out) {
  unsigned acc = 0;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 a = __ldcs(src + i), b = __ldcs(src + i + stride), c = __ldcs(src + i + 2 * stride), d = __ldcs(src + i + 3 * stride);
    acc ^= a.x ^ a.y ^ a.z ^ a.w ^ b.x ^ b.y ^ b.z ^ b.w ^ c.x ^ c.y ^ c.z ^ c.w ^ d.x ^ d.y ^ d.z ^ d.w;
  }
  for (; i < n16; i += stride) { uint4 a = __ldcs(src + i); acc ^= a.x ^ a.y ^ a.z ^ a.w; }
  if (acc == 0x12345678u) out[0] = acc;
}

// bulk ring: producer thread + 8 consumer warps; consumers read one uint4 per lane per stage (touch) or all
template <int TOUCH>
__global__ void __launch_bounds__(288, 1) k_ring(const uint8_t *__restrict__ src, size_t total, int stage_bytes, int stages, int interleave, unsigned *out) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full_bar[32], empty_bar[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const size_t nblk = total / stage_bytes;  // stage-sized blocks overall
  // contiguous: CTA b takes blocks [b*per, ...); interleaved: blocks b, b+grid, ...
  const size_t per = (nblk + gridDim.x - 1) / gridDim.x;
  size_t first, step, count;
  if (interleave) { first = blockIdx.x; step = gridDim.x; count = blockIdx.x < nblk ? (nblk - blockIdx.x + gridDim.x - 1) / gridDim.x : 0; }
  else { first = blockIdx.x * per; step = 1; count = first < nblk ? (nblk - first < per ? nblk - first : per) : 0; }
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_bar[s])), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty_bar[s])), "r"(8) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 8) {
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      for (size_t it = 0; it < count; ++it) {
        if (!bwait(smem_u32(&empty_bar[stage]), phase ^ 1u)) return;
        uint32_t fb = smem_u32(&full_bar[stage]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(stage_bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(ring + (size_t)stage * stage_bytes)),
                     "l"(src + (first + it * step) * stage_bytes), "r"(stage_bytes), "r"(fb) : "memory");
        if (++stage == stages) { stage = 0; phase ^= 1u; }
      }
    }
    return;
  }
  unsigned acc = 0;
  int stage = 0; uint32_t phase = 0;
  for (size_t it = 0; it < count; ++it) {
    uint32_t got = 0;
    if (lane == 0) got = bwait(smem_u32(&full_bar[stage]), phase);
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) return;
    const uint4 *p = reinterpret_cast<const uint4 *>(ring + (size_t)stage * stage_bytes);
    if (TOUCH) { uint4 a = p[threadIdx.x]; acc ^= a.x ^ a.y ^ a.z ^ a.w; }
    else { for (int i = threadIdx.x; i < stage_bytes / 16; i += 256) { uint4 a = p[i]; acc ^= a.x ^ a.y ^ a.z ^ a.w; } }
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty_bar[stage])) : "memory");
    if (++stage == stages) { stage = 0; phase ^= 1u; }
  }
  if (acc == 0x12345678u) out[0] = acc;
}

// ring whose stage is R separate row copies of RB bytes (dst stride RB + pad), issued by R lanes at once
__global__ void __launch_bounds__(288, 1) k_rows(const uint8_t *__restrict__ src, size_t total, int R, int RB, int pad, int stages, unsigned *out) {
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ uint64_t full_bar[32], empty_bar[32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int stage_src = R * RB, stage_dst = R * (RB + pad);
  const size_t nblk = total / stage_src;
  const size_t first = blockIdx.x, step = gridDim.x, count = blockIdx.x < nblk ? (nblk - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&full_bar[s])), "r"(1) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&empty_bar[s])), "r"(8) : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 8) {
    int stage = 0; uint32_t phase = 0;
    for (size_t it = 0; it < count; ++it) {
      uint32_t got = 0;
      if (lane == 0) got = bwait(smem_u32(&empty_bar[stage]), phase ^ 1u);
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) return;
      uint32_t fb = smem_u32(&full_bar[stage]);
      if (lane == 0) asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fb), "r"(stage_src) : "memory");
      __syncwarp();
      if (lane < R)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(ring + (size_t)stage * stage_dst + (size_t)lane * (RB + pad))),
                     "l"(src + (first + it * step) * stage_src + (size_t)lane * RB), "r"(RB), "r"(fb) : "memory");
      if (++stage == stages) { stage = 0; phase ^= 1u; }
    }
    return;
  }
  unsigned acc = 0;
  int stage = 0; uint32_t phase = 0;
  for (size_t it = 0; it < count; ++it) {
    uint32_t got = 0;
    if (lane == 0) got = bwait(smem_u32(&full_bar[stage]), phase);
    got = __shfl_sync(0xffffffffu, got, 0);
    if (!got) return;
    const uint4 *p = reinterpret_cast<const uint4 *>(ring + (size_t)stage * stage_dst);
    uint4 a = p[threadIdx.x]; acc ^= a.x ^ a.y ^ a.z ^ a.w;
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty_bar[stage])) : "memory");
    if (++stage == stages) { stage = 0; phase ^= 1u; }
  }
  if (acc == 0x12345678u) out[0] = acc;
}

int main() {
  const size_t W = 10240ull * 2560;  // bytes per "weight"
  const int copies = 16;
  uint8_t *buf; unsigned *out;
  CK(cudaMalloc(&buf, W * copies)); CK(cudaMalloc(&out, 64));
  CK(cudaMemset(buf, 1, W * copies));
  cudaStream_t st; CK(cudaStreamCreate(&st));
  CK(cudaFuncSetAttribute(k_ring<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  CK(cudaFuncSetAttribute(k_ring<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  CK(cudaFuncSetAttribute(k_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
  struct V { const char *name; int kind; int a, b, c, d; };
  std::vector<V> vs = {
    {"empty 148x288", 0, 0, 0, 0, 0},
    {"ldg grid=148x1 1024thr", 1, 148, 1024, 0, 0},
    {"ldg grid=148x2 1024thr", 1, 296, 1024, 0, 0},
    {"ldg grid=148x4 512thr", 1, 592, 512, 0, 0},
    {"ldg grid=148x8 256thr", 1, 1184, 256, 0, 0},
    {"ring contig 20K x8 full", 2, 20480, 8, 0, 0},
    {"ring contig 20K x8 touch", 2, 20480, 8, 0, 1},
    {"ring inter  20K x8 full", 2, 20480, 8, 1, 0},
    {"ring inter  20K x8 touch", 2, 20480, 8, 1, 1},
    {"ring inter  40K x4 touch", 2, 40960, 4, 1, 1},
    {"ring inter  10K x16 touch", 2, 10240, 16, 1, 1},
    {"ring inter  5K x32 touch", 2, 5120, 32, 1, 1},
    {"ring contig 10K x16 touch", 2, 10240, 16, 0, 1},
    {"ring inter 20K x4 touch (80K)", 2, 20480, 4, 1, 1},
    {"ring inter 10K x4 touch (40K)", 2, 10240, 4, 1, 1},
    {"rows 8 x 2560 pad64, 8 stages", 3, 8, 2560, 64, 8},
    {"rows 8 x 2048 pad64, 8 stages", 3, 8, 2048, 64, 8},
    {"rows 16 x 2048 pad64, 4 stages", 3, 16, 2048, 64, 4},
    {"rows 16 x 2560 pad64, 4 stages", 3, 16, 2560, 64, 4},
    {"rows 8 x 1024 pad64, 16 stages", 3, 8, 1024, 64, 16},
    {"rows 16 x 512 pad64, 16 stages", 3, 16, 512, 64, 16},
    {"rows 1 x 20480 pad0, 8 stages", 3, 1, 20480, 0, 8},
    {"rows 2 x 10240 pad64, 8 stages", 3, 2, 10240, 64, 8},
    {"rows 4 x 5120 pad64, 8 stages", 3, 4, 5120, 64, 8},
  };
  for (auto &v : vs) {
    auto launch = [&](int i) {
      const uint8_t *src = buf + (size_t)(i % copies) * W;
      if (v.kind == 0) k_empty<<<148, 288, 0, st>>>((int *)out);
      else if (v.kind == 1) k_ldg<<<v.a, v.b, 0, st>>>((const uint4 *)src, W / 16, out);
      else if (v.kind == 3) k_rows<<<148, 288, (size_t)v.a * (v.b + v.c) * v.d, st>>>(src, W, v.a, v.b, v.c, v.d, out);
      else if (v.d) k_ring<1><<<148, 288, (size_t)v.a * v.b, st>>>(src, W, v.a, v.b, v.c, out);
      else k_ring<0><<<148, 288, (size_t)v.a * v.b, st>>>(src, W, v.a, v.b, v.c, out);
    };
    for (int i = 0; i < 4; ++i) launch(i);
    CK(cudaStreamSynchronize(st));
    cudaGraph_t g; cudaGraphExec_t ge;
    CK(cudaStreamBeginCapture(st, cudaStreamCaptureModeGlobal));
    for (int i = 0; i < copies; ++i) launch(i);
    CK(cudaStreamEndCapture(st, &g));
    CK(cudaGraphInstantiate(&ge, g, 0));
    CK(cudaGraphLaunch(ge, st)); CK(cudaStreamSynchronize(st));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    float best = 1e9, sum = 0;
    for (int r = 0; r < 10; ++r) {
      CK(cudaEventRecord(e0, st)); CK(cudaGraphLaunch(ge, st)); CK(cudaEventRecord(e1, st)); CK(cudaEventSynchronize(e1));
      float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); sum += ms; if (ms < best) best = ms;
    }
    printf("%-34s avg %.2f us  min %.2f us per launch  (%.0f GB/s)\n", v.name, sum / 10 * 1e3 / copies, best * 1e3 / copies, W / (best * 1e-3 / copies) / 1e9);
    CK(cudaGraphExecDestroy(ge)); CK(cudaGraphDestroy(g));
  }
  CK(cudaGetLastError());
  return 0;
}
