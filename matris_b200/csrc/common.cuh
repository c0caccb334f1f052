// Shared helpers for the matris_b200 CUDA sources (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include "matris_b200.h"

namespace mb {

// last CUDA error text, per host thread
void set_cuda_error(cudaError_t e, const char* where);

#define MB_CUDA_CHECK(expr)                                  \
  do {                                                       \
    cudaError_t _e = (expr);                                 \
    if (_e != cudaSuccess) {                                 \
      mb::set_cuda_error(_e, #expr);                         \
      return MB_ERR_CUDA;                                    \
    }                                                        \
  } while (0)

#define MB_LAUNCH_CHECK(name)                                \
  do {                                                       \
    cudaError_t _e = cudaGetLastError();                     \
    if (_e != cudaSuccess) {                                 \
      mb::set_cuda_error(_e, name);                          \
      return MB_ERR_CUDA;                                    \
    }                                                        \
  } while (0)

static inline int cdiv(long long a, long long b) { return (int)((a + b - 1) / b); }

// exclusive scan of n int32 values into out[0..n] (out[n] = total); tmp holds
// mb_graph_scan_tmp_len(n) ints.  in may alias out.
int scan_exclusive(const int32_t* in, int32_t* out, int64_t n, int32_t* tmp, cudaStream_t s);

// accurate expf on purpose: these feed fp32-tolerance parity checks
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
// d/dx [x * sigmoid(x)] = s * (1 + x * (1 - s))   (matris/model/op/fused_silu_op.py:5-13)
__device__ __forceinline__ float silu_grad_f(float x) {
  const float s = 1.0f / (1.0f + expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

// Fast variants for the GEMM prologue / epilogue, where the transcendental cost is paid per operand element:
// ex2.approx-based exponential and an approximate division (a few ulp each, far inside the fp32-tolerance gates).
__device__ __forceinline__ float silu_fast_f(float x) { return __fdividef(x, 1.0f + __expf(-x)); }
__device__ __forceinline__ float silu_grad_fast_f(float x) {
  const float s = __fdividef(1.0f, 1.0f + __expf(-x));
  return s * (1.0f + x * (1.0f - s));
}

__device__ __forceinline__ float sigmoid_fast_f(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace mb
