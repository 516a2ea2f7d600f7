// Shared helpers for the sm_100a kernels of the tensor-parallel decoder-layer path.
//
// Numeric convention (restated from the reference's scalar types): the
// reference instantiates its kernels with c10::Half / c10::BFloat16, whose
// binary operators compute in fp32 and round the result to the 16-bit type
// (round-to-nearest-even).  `rt<T>()` below is that rounding step, so an
// expression such as `a * b - c * d` on the reference's scalar type is written
// here as rt<T>(rt<T>(a*b) - rt<T>(c*d)) on floats.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/sarathi_b200.h"

namespace sb200 {

// ---------------------------------------------------------------- error text
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define SB_CHECK_ARG(cond, ...)                         \
  do {                                                  \
    if (!(cond)) {                                      \
      ::sb200::set_error(__VA_ARGS__);                  \
      return SB200_ERR_INVALID_ARGUMENT;                \
    }                                                   \
  } while (0)

#define SB_CHECK_LAUNCH(what)                                         \
  do {                                                                \
    cudaError_t e__ = cudaGetLastError();                             \
    if (e__ != cudaSuccess) return ::sb200::cuda_fail(e__, what);     \
  } while (0)

#define SB_CUDA(call)                                                 \
  do {                                                                \
    cudaError_t e__ = (call);                                         \
    if (e__ != cudaSuccess) return ::sb200::cuda_fail(e__, #call);    \
  } while (0)

// ------------------------------------------------------------- dtype helpers
template <typename T> struct DT;
template <> struct DT<float> {
  static constexpr int id = SB200_F32;
  __device__ __forceinline__ static float to_f(float v) { return v; }
  __device__ __forceinline__ static float from_f(float v) { return v; }
};
template <> struct DT<__half> {
  static constexpr int id = SB200_F16;
  __device__ __forceinline__ static float to_f(__half v) { return __half2float(v); }
  __device__ __forceinline__ static __half from_f(float v) { return __float2half_rn(v); }
};
template <> struct DT<__nv_bfloat16> {
  static constexpr int id = SB200_BF16;
  __device__ __forceinline__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ __forceinline__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// Round an fp32 value to T and bring it back to fp32: one "operator result" of
// the reference's 16-bit scalar types.  Identity for float.
template <typename T> __device__ __forceinline__ float rt(float v) { return DT<T>::to_f(DT<T>::from_f(v)); }
template <> __device__ __forceinline__ float rt<float>(float v) { return v; }

__host__ __device__ inline size_t dtype_size(int dt) { return dt == SB200_F32 ? 4 : 2; }

// 16-byte vector of T.
template <typename T> struct Vec16 {
  static constexpr int N = 16 / sizeof(T);
  union { uint4 raw; T v[16 / sizeof(T)]; };
};

template <typename T>
__device__ __forceinline__ Vec16<T> ld16(const T* p) {
  Vec16<T> r; r.raw = *reinterpret_cast<const uint4*>(p); return r;
}
template <typename T>
__device__ __forceinline__ void st16(T* p, const Vec16<T>& v) {
  *reinterpret_cast<uint4*>(p) = v.raw;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Sum over the CTA; every thread gets the result. `red` needs 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (warp == 0) {
    t = warp_sum(t);
    if (lane == 0) red[32] = t;
  }
  __syncthreads();
  return red[32];
}

__host__ __device__ inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per process).
int sm_count();

#define SB_DISPATCH_FLOAT(dt, ...)                                            \
  switch (dt) {                                                               \
    case SB200_F32: { using scalar_t = float; __VA_ARGS__; break; }           \
    case SB200_F16: { using scalar_t = __half; __VA_ARGS__; break; }          \
    case SB200_BF16: { using scalar_t = __nv_bfloat16; __VA_ARGS__; break; }  \
    default:                                                                  \
      ::sb200::set_error("unsupported dtype id %d", (int)(dt));               \
      return SB200_ERR_UNSUPPORTED;                                           \
  }

}  // namespace sb200
