// Pieces shared by the tcgen05 chunk kernels: 16-bit pack/unpack, packed fp32 helpers, tensor-map
// construction.
#pragma once
#include <cuda.h>
#include <type_traits>
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace la {
namespace tile {

template <typename T> struct Fmt;
template <> struct Fmt<__nv_bfloat16> {
  static constexpr uint32_t kAB = 1;  // tcgen05 kind::f16 operand format code
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&u));
  }
  // y * (hi + lo) on a packed pair, rounded once more than the exact product: the factor is
  // carried as a 16-bit value plus its 16-bit remainder, so no unpacking to fp32 is needed
  static __device__ __forceinline__ uint32_t scale(uint32_t y, uint32_t hi, uint32_t lo) {
    const __nv_bfloat162 yy = *reinterpret_cast<__nv_bfloat162 *>(&y);
    const __nv_bfloat162 r = __hfma2(yy, *reinterpret_cast<__nv_bfloat162 *>(&hi),
                                     __hmul2(yy, *reinterpret_cast<__nv_bfloat162 *>(&lo)));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
};
template <> struct Fmt<__half> {
  static constexpr uint32_t kAB = 0;
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&v);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<__half2 *>(&u));
  }
  static __device__ __forceinline__ uint32_t scale(uint32_t y, uint32_t hi, uint32_t lo) {
    const __half2 yy = *reinterpret_cast<__half2 *>(&y);
    const __half2 r = __hfma2(yy, *reinterpret_cast<__half2 *>(&hi), __hmul2(yy, *reinterpret_cast<__half2 *>(&lo)));
    return *reinterpret_cast<const uint32_t *>(&r);
  }
};

// Four consecutive features of one row of a decay tile as TMA left it in shared memory (128-byte
// swizzle, rows of 128 bytes): fp32 tiles are four boxes of 32 features, 16-bit tiles two boxes of
// 64.  d0 is a multiple of 4; box_bytes is the size of one box (128 rows x 128 B).
template <typename T, bool LD16>
__device__ __forceinline__ float4 decay_quad(const uint8_t *tile, int row, int d0, uint32_t box_bytes) {
  if (!LD16) {
    return *reinterpret_cast<const float4 *>(tile + (uint32_t)(d0 >> 5) * box_bytes + (uint32_t)row * 128u +
                                             ((uint32_t)(((d0 & 31) >> 2) ^ (row & 7)) << 4));
  }
  const uint2 raw = *reinterpret_cast<const uint2 *>(tile + (uint32_t)(d0 >> 6) * box_bytes + (uint32_t)row * 128u +
                                                     ((uint32_t)(((d0 & 63) >> 3) ^ (row & 7)) << 4) +
                                                     (uint32_t)((d0 & 4) << 1));
  const float2 lo = Fmt<T>::unpack(raw.x), hi = Fmt<T>::unpack(raw.y);
  return make_float4(lo.x, lo.y, hi.x, hi.y);
}

__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 f2(uint32_t lo, uint32_t hi) {
  return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}
__device__ __forceinline__ float ex2(float x) {  // 2^x, one MUFU op; 2^(-inf) = 0, 2^(+big) = +inf
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// log2(sigmoid(x)) = min(x, 0) log2(e) - log2(1 + 2^(-|x| log2(e))): the log decay, in log2 units, of a
// decay that is given as the pre-activation of a logsigmoid (no overflow for any x).
__device__ __forceinline__ float log2_sigmoid(float x) {
  const float l2e = 1.4426950408889634f;
  const float t = ex2(-fabsf(x) * l2e);
  // log2(1 + t): the series where 1 + t would round t away (decays close to 1)
  const float l1p = t < 0.00390625f ? t * l2e * (1.f - t * (0.5f - t * 0.33333334f)) : lg2(1.f + t);
  return fminf(x, 0.f) * l2e - l1p;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void *p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// (B, N, H, F) tensor of 16-bit (dtype LA_BF16 / LA_F16) or fp32 (LA_F32) elements, F <= 128
// features per head.  One box = 128 tokens x 128 bytes of one head (64 16-bit or 32 fp32 features),
// 128-byte swizzle; where a box reaches past feature F - 1 a load fills zeros and a store clips.
inline int make_map(CUtensorMap *m, const void *ptr, int dtype, int B, int N, int H, int F = 128) {
  EncodeTiledFn enc = encode_fn();
  if (enc == nullptr) return LA_ERR_CUDA;
  // The encoder is a driver call and needs this thread to have the device's context current; a
  // thread that has made no runtime call yet (an autograd worker, say) has none until the runtime
  // binds it, which this no-op does.  Once per thread.
  static thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
  if (reinterpret_cast<uintptr_t>(ptr) & 15u) return LA_ERR_MISALIGNED;
  const cuuint64_t esz = dtype == LA_F32 ? 4 : 2;
  const cuuint64_t f = (cuuint64_t)F;
  const cuuint64_t dims[4] = {f, (cuuint64_t)H, (cuuint64_t)N, (cuuint64_t)B};
  const cuuint64_t strides[3] = {f * esz, (cuuint64_t)H * f * esz, (cuuint64_t)N * H * f * esz};
  const cuuint32_t box[4] = {(cuuint32_t)(128 / esz), 1, 128, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt = dtype == LA_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : dtype == LA_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult r = enc(m, dt, 4, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) snprintf(last_cuda_error_buf(), 256, "cuTensorMapEncodeTiled: CUresult %d (ptr %p, B %d N %d H %d)", (int)r, ptr, B, N, H);
  return r == CUDA_SUCCESS ? LA_OK : LA_ERR_CUDA;
}

}  // namespace tile
}  // namespace la
