// Version, status strings and the per-thread CUDA error record of the C ABI.
#include <stdio.h>
#include "common.cuh"

namespace mb {
static thread_local char g_cuda_error[512] = "";
void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorString(e), cudaGetErrorName(e));
}
}  // namespace mb

extern "C" int mb_version(void) { return MB_VERSION; }

extern "C" const char* mb_last_cuda_error(void) { return mb::g_cuda_error; }

extern "C" const char* mb_status_string(int status) {
  switch (status) {
    case MB_OK: return "ok";
    case MB_ERR_INVALID: return "invalid argument";
    case MB_ERR_CUDA: return "CUDA runtime error";
    case MB_ERR_OVERFLOW: return "count or periodic image index out of range";
    case MB_ERR_UNPAIRED: return "directed edge without a reverse edge";
    case MB_ERR_ISOLATED: return "isolated atom: no neighbour inside the cutoff";
    case MB_ERR_TOO_LARGE: return "problem exceeds the fixed capacity of this allocation-free entry point";
    case MB_ERR_CAPACITY: return "capacity buffer too small";
    default: return "unknown status";
  }
}
