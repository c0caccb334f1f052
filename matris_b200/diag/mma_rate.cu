// Diagnostic (not part of the library): raw issue rate of tcgen05.mma kind::tf32 / kind::f16 with operands
// resident in shared / tensor memory, SS and TS forms, N = 128 / 256.  Gives the tensor-pipe peak the GEMM is
// judged against.  Build and run on a B200:
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 matris_b200/diag/mma_rate.cu -o /tmp/mma_rate && /tmp/mma_rate
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
template <int KIND, int TS>  // KIND 0: tf32, 1: f16(bf16)
__device__ __forceinline__ void mma(uint32_t d, uint32_t ta, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  if (KIND == 0) {
    if (TS) asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;}" :: "r"(d), "r"(ta), "l"(db), "r"(idesc), "r"(acc) : "memory");
    else asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;}" :: "r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
  } else {
    if (TS) asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;}" :: "r"(d), "r"(ta), "l"(db), "r"(idesc), "r"(acc) : "memory");
    else asm volatile("{.reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;}" :: "r"(d), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
  }
}
template <int KIND, int TS, int N>
__global__ void k(int iters, long long* out) {
  extern __shared__ uint8_t raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t bar; __shared__ uint32_t slot;
  for (int i = threadIdx.x; i < 48 * 1024 / 4; i += blockDim.x) ((float*)smem)[i] = 0.f;
  if (threadIdx.x == 0) { asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(smem_u32(&bar))); asm volatile("fence.mbarrier_init.release.cluster;"); }
  if (threadIdx.x < 32) { asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" :: "r"(smem_u32(&slot))); asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;"); }
  asm volatile("fence.proxy.async.shared::cta;"); asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads(); asm volatile("tcgen05.fence::after_thread_sync;");
  uint32_t tb = slot;
  const uint32_t fmt = KIND == 0 ? 2u : 1u;
  const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(N >> 3) << 17) | ((128u >> 4) << 24);
  if (threadIdx.x == 0) {
    uint64_t da = umma_desc(smem_u32(smem)), db = umma_desc(smem_u32(smem + 16384));
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) mma<KIND, TS>(tb, tb + 256 + 8 * kk, da + 2 * kk, db + 2 * kk, idesc, 1u);
    }
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(&bar)) : "memory");
    uint32_t ok = 0; int spins = 0;
    while (!ok && spins < (1 << 26)) { asm volatile("{.reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p;}" : "=r"(ok) : "r"(smem_u32(&bar)), "r"(0u) : "memory"); ++spins; }
    long long t1 = clock64();
    if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = ok; }
  }
  asm volatile("tcgen05.fence::before_thread_sync;"); __syncthreads();
  if (threadIdx.x < 32) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" :: "r"(tb));
}
template <int KIND, int TS, int N> void run(const char* name, int ctas) {
  long long* d; cudaMalloc(&d, 16); cudaMemset(d, 0, 16);
  int iters = 2000; size_t sm = 49 * 1024 + 1024;
  cudaFuncSetAttribute(k<KIND, TS, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm);
  k<KIND, TS, N><<<ctas, 128, sm>>>(iters, d);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[2]; cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  double cyc = (double)h[0] / (iters * 4);
  double macs = 128.0 * N * (KIND == 0 ? 8 : 16);
  printf("%-28s ctas=%d err=%s ok=%lld cycles/MMA=%.1f MAC/clk/SM=%.0f  -> %.0f TFLOP/s at 148 SMs x 1.9 GHz\n", name, ctas, cudaGetErrorString(e), h[1], cyc, macs / cyc, 2 * macs / cyc * 148 * 1.9e9 / 1e12);
  cudaFree(d);
}
int main() {
  run<0, 0, 128>("tf32 SS N=128", 148); run<0, 1, 128>("tf32 TS N=128", 148);
  run<0, 0, 256>("tf32 SS N=256", 148); run<0, 1, 256>("tf32 TS N=256", 148);
  run<1, 0, 128>("bf16 SS N=128", 148); run<1, 0, 256>("bf16 SS N=256", 148); run<1, 1, 256>("bf16 TS N=256", 148);
  run<0, 1, 128>("tf32 TS N=128 1 CTA", 1);
  return 0;
}
