// Shared helpers for the xopes_b200 kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/xopes_b200.h"

namespace la {

template <typename T> struct Cvt;
template <> struct Cvt<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
};
template <> struct Cvt<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
};
template <> struct Cvt<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
};

static inline size_t dtype_size(int dtype) { return dtype == LA_F32 ? 4 : 2; }

// Text of the last CUDA error this library met on the calling thread (la_debug_last_cuda_error).
char *last_cuda_error_buf();
static inline void note_cuda_error(cudaError_t e, const char *where) {
  snprintf(last_cuda_error_buf(), 256, "%s: %s", where, cudaGetErrorString(e));
}

// Launch-error check that never synchronises: reports configuration errors only.
static inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) note_cuda_error(e, "kernel launch");
  return e == cudaSuccess ? LA_OK : LA_ERR_CUDA;
}

// Address (on the current device) of the watchdog word that la_device_status() reads.
// Defined in api.cu; kernels that can time out receive it as a parameter.
int *status_word_ptr();

}  // namespace la
