// Shared helpers for the forward-Laplacian kernels: error reporting across the C ABI,
// launch checks and small device utilities.  Everything here is internal to the shared
// library; the exported surface is declared in include/folx_b200.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/folx_b200.h"

namespace fl {

// Records a message that fl_last_error() returns on the calling thread.
void set_error(const char* fmt, ...);

inline int32_t cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return FL_ECUDA;
}

#define FL_CHECK_LAUNCH(what)                              \
  do {                                                     \
    cudaError_t e__ = cudaGetLastError();                  \
    if (e__ != cudaSuccess) return fl::cuda_fail(e__, what); \
  } while (0)

#define FL_CUDA(call)                                      \
  do {                                                     \
    cudaError_t e__ = (call);                              \
    if (e__ != cudaSuccess) return fl::cuda_fail(e__, #call); \
  } while (0)

#define FL_REQUIRE(cond, code, ...)  \
  do {                               \
    if (!(cond)) {                   \
      fl::set_error(__VA_ARGS__);    \
      return (code);                 \
    }                                \
  } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device ordinal).
int sm_count();

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float4 ld_stream(const float4* p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream(float4* p, float4 v) { __stcs(p, v); }

}  // namespace fl
