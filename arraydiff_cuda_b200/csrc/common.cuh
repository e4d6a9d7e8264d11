// Shared helpers for the sm_100a kernels: status codes, launch accounting, dtype access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "arraydiff_b200.h"

namespace adk {

// Every kernel launch of the library goes through this counter so that callers can
// report how many of OUR kernels ran inside a timed region.
extern unsigned long long g_launch_count;
inline void count_launch(unsigned long long n = 1) { __atomic_fetch_add(&g_launch_count, n, __ATOMIC_RELAXED); }

// Which kernel family the calling thread's most recent ad_conv2d_* call launched (ad_conv2d_last_kernel).
enum { kConvNone = 0, kConvDirectF32 = 1, kConvTcGeneral = 2, kConvTcRow = 3 };
extern thread_local int g_last_conv_kernel;

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? AD_OK : AD_ERR_CUDA;
}

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int elem_size(int dtype) { return dtype == AD_F32 ? 4 : (dtype == AD_BF16 ? 2 : 0); }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline unsigned grid_for(size_t work_items, unsigned per_block, unsigned max_blocks_per_sm = 8) {
  size_t b = (work_items + per_block - 1) / per_block;
  size_t cap = (size_t)kNumSMs * max_blocks_per_sm;
  if (b > cap) b = cap;
  if (b < 1) b = 1;
  return (unsigned)b;
}

// ---- typed element access (device) ----
template <typename T> __device__ __forceinline__ float ld_f(const T* p);
template <> __device__ __forceinline__ float ld_f<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_f<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st_f(T* p, float v);
template <> __device__ __forceinline__ void st_f<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_f<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Dispatch a callable templated on the element type.
#define AD_DISPATCH_DTYPE(dtype, ...)                                   \
  do {                                                                  \
    if ((dtype) == AD_F32) { using T = float; __VA_ARGS__; }            \
    else if ((dtype) == AD_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return AD_ERR_UNSUPPORTED;                                     \
  } while (0)

}  // namespace adk
