// micro-benchmark: rate of tcgen05.ld (TMEM -> registers) on one SM.
// W warps per TMEM lane quarter (4W warps in all) each read a 32-lane x 32-column block
// (4 KB per warp and iteration) in a loop: either one 32x32b.x32 load or two 16x256b.x4
// loads, each batch followed by tcgen05.wait::ld, optionally with `depth` batches in
// flight before the wait (more registers).  Reports cycles per 64 KB read by the SM
// (= one 128 x 128 int32 accumulator), the quantity a per-group epilogue pays per group.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void ld16(uint32_t taddr, uint32_t *r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.16x256b.x4.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shape 0: 32x32b.x32, 1: 2 x 16x256b.x4;  depth 1 or 2 batches before each wait
template <int kShape, int kDepth>
__global__ void __launch_bounds__(512, 1) k_ld(int warps, int iters, long long *out, uint32_t *sink) {
  __shared__ uint32_t tmem_ptr;
  const int warp = threadIdx.x >> 5;
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_ptr)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = tmem_ptr;
  long long t0 = 0, t1 = 0;
  if (warp < warps) {
    const int q = warp & 3, ch = warp >> 2;  // lane quarter, 32-column chunk
    uint32_t x = 0;
    t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      uint32_t r[kDepth][32];
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        // walk over the 512 columns so that consecutive batches read different data
        const uint32_t col = (uint32_t)((ch * 32 + (it * kDepth + d) * 128) & 511);
        const uint32_t ta = tb + ((uint32_t)(q * 32) << 16) + col;
        if (kShape == 0) {
          ld32(ta, r[d]);
        } else {
          ld16(ta, r[d]);
          ld16(ta + (16u << 16), r[d] + 16);
        }
      }
      wait_ld();
#pragma unroll
      for (int d = 0; d < kDepth; ++d)
#pragma unroll
        for (int i = 0; i < 32; i += 8) x ^= r[d][i];
    }
    t1 = clock64();
    if (x == 0x12345678u) sink[threadIdx.x] = x;
  }
  if ((threadIdx.x & 31) == 0 && warp < warps) {
    out[2 * warp] = t0;
    out[2 * warp + 1] = t1;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512u) : "memory");
}

template <int kShape, int kDepth>
int run(int warps, long long *d_out, uint32_t *d_sink) {
  const int iters = 4096 / kDepth;
  long long h[32];
  k_ld<kShape, kDepth><<<1, 512>>>(warps, iters, d_out, d_sink);
  CK(cudaDeviceSynchronize());
  k_ld<kShape, kDepth><<<1, 512>>>(warps, iters, d_out, d_sink);
  CK(cudaDeviceSynchronize());
  CK(cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost));
  long long lo = h[0], hi = h[1];
  for (int w = 0; w < warps; ++w) {
    lo = h[2 * w] < lo ? h[2 * w] : lo;
    hi = h[2 * w + 1] > hi ? h[2 * w + 1] : hi;
  }
  const double cycles = (double)(hi - lo);
  const double bytes = (double)warps * 4096.0 * 4096.0;  // 4 KB per warp and batch, 4096 batches
  printf("%-14s depth %d  %2d warps: %7.1f cycles per 64 KB, %6.1f B/clk/SM, %6.1f cycles per batch and warp\n",
         kShape == 0 ? "32x32b.x32" : "2x16x256b.x4", kDepth, warps, cycles / (bytes / 65536.0), bytes / cycles,
         cycles / 4096.0);
  return 0;
}

int main() {
  long long *d_out;
  uint32_t *d_sink;
  CK(cudaMalloc(&d_out, 64 * sizeof(long long)));
  CK(cudaMalloc(&d_sink, 512 * sizeof(uint32_t)));
  for (int warps : {4, 8, 16}) {
    if (run<0, 1>(warps, d_out, d_sink)) return 1;
    if (run<1, 1>(warps, d_out, d_sink)) return 1;
    if (run<0, 2>(warps, d_out, d_sink)) return 1;
    if (run<1, 2>(warps, d_out, d_sink)) return 1;
  }
  return 0;
}
