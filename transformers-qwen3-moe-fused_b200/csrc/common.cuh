// Shared helpers for the libmoe_b200 kernels: status codes, dtype dispatch, scalar
// conversion and the small device utilities every translation unit needs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moe_b200.h"

#define MOE_API extern "C" __attribute__((visibility("default")))

namespace moe {

inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? MOE_OK : (int)e; }

// Status of the launch that was just enqueued (does not synchronise).
inline int launch_status() { return cuda_status(cudaGetLastError()); }

__host__ __device__ inline bool is_float_dtype(int d) { return d == MOE_F32 || d == MOE_BF16 || d == MOE_F16; }
__host__ __device__ inline bool is_int_dtype(int d) { return d == MOE_I32 || d == MOE_I64; }
__host__ __device__ inline size_t dtype_size(int d) {
  switch (d) {
    case MOE_F32: case MOE_I32: return 4;
    case MOE_BF16: case MOE_F16: return 2;
    case MOE_I64: return 8;
  }
  return 0;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// Read element i of an int32 / int64 vector chosen at run time.
__device__ __forceinline__ int64_t load_index(const void* p, int is64, int64_t i) {
  return is64 ? ((const int64_t*)p)[i] : (int64_t)((const int32_t*)p)[i];
}

inline int sm_count() {
  // Cached per device; immutable after the first query.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace moe

// Run `body` with `T` bound to the C++ type of a floating dtype code.
#define MOE_DISPATCH_FLOAT(code, T, ...)                                  \
  do {                                                                    \
    if ((code) == MOE_F32) { using T = float; __VA_ARGS__ }               \
    else if ((code) == MOE_BF16) { using T = __nv_bfloat16; __VA_ARGS__ } \
    else if ((code) == MOE_F16) { using T = __half; __VA_ARGS__ }         \
    else return MOE_ERR_DTYPE;                                            \
  } while (0)
