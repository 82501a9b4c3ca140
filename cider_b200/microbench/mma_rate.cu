// micro-benchmark: issue rate of tcgen05.mma kind::i8, cta_group::1, M=128, N in {64,128,256}, K=32
// operands sit in shared memory (zeros), no TMA traffic, no epilogue.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t a) {
  uint64_t d = (uint64_t)((a >> 4) & 0x3FFFu); d |= (uint64_t)1 << 16; d |= (uint64_t)(1024 >> 4) << 32; d |= (uint64_t)1 << 46; d |= (uint64_t)2 << 61; return d;
}
__host__ __device__ constexpr uint32_t make_idesc(int m, int n) { return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24); }
__device__ __forceinline__ void mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ uint32_t try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok; asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory"); return ok;
}
// mode bit0: alternate between two accumulators; bit1: commit after every 4 MMAs (to a barrier nobody waits on);
// bit2: rotate over 4 different operand stages (distinct smem addresses)
__global__ void __launch_bounds__(128, 1) k_mma(int N, int iters, int mode, long long *out) {
  extern __shared__ uint8_t raw[];
  uint8_t *smem = (uint8_t *)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_ptr;
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 4 * (16384 + 32768) / 16; i += blockDim.x) reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0x01010101, 0x01010101, 0x01010101, 0x01010101);
  if (threadIdx.x == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar[0])), "r"(1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(&bar[1])), "r"(1 << 20) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_ptr)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tb = tmem_ptr;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc(128, N);
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      const int st = (mode & 4) ? (it & 3) : 0;
      const uint64_t a = make_smem_desc(smem_u32(smem + st * (16384 + 32768)));
      const uint64_t b = make_smem_desc(smem_u32(smem + st * (16384 + 32768) + 16384));
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t d = tb + ((mode & 1) ? (uint32_t)((k & 1) * 256) : 0u);
        mma(d, a + (uint64_t)(k * 2), b + (uint64_t)(k * 2), idesc, (it | k) ? 1u : 0u);
      }
      if (mode & 2) commit(smem_u32(&bar[1]));
    }
    const long long t1 = clock64();
    commit(smem_u32(&bar[0]));
    long long tw = clock64();
    while (!try_wait(smem_u32(&bar[0]), 0) && clock64() - tw < 2000000000ll) {}
    const long long t2 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tb), "r"(512u) : "memory");
  }
}
int main() {
  long long *out; CK(cudaMalloc(&out, 64));
  const size_t smem = 4 * (16384 + 32768) + 1024;
  CK(cudaFuncSetAttribute(k_mma, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const int iters = 2000;
  for (int grid : {1, 148}) for (int N : {64, 128, 256}) for (int mode : {0, 1, 2, 4, 6}) {
    k_mma<<<grid, 128, smem>>>(N, iters, mode, out);
    CK(cudaDeviceSynchronize());
    k_mma<<<grid, 128, smem>>>(N, iters, mode, out);
    CK(cudaDeviceSynchronize());
    long long h[2]; CK(cudaMemcpy(h, out, 16, cudaMemcpyDeviceToHost));
    printf("grid %3d N=%3d mode=%d: issue %.1f cycles/MMA, complete %.1f cycles/MMA (ideal %.0f)\n", grid, N, mode, (double)h[0] / (4.0 * iters), (double)h[1] / (4.0 * iters), 128.0 * N * 32 / 8192.0);
  }
  return 0;
}
