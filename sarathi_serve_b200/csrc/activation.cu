// silu_and_mul, gelu_new, gelu_fast: flat element-wise kernels over [T, d].
//
// Grid-stride over 16-byte vectors (any T, d); a scalar tail covers rows whose
// length is not a multiple of the vector width.  The arithmetic restates the
// reference's expressions on its 16-bit scalar types (each operator result
// rounded to T): csrc/activation_kernels.cu:8-25 (silu_and_mul), :86-102 (GELUs).
#include "common.cuh"

namespace sb200 {

template <typename T> __device__ __forceinline__ float silu_mul_op(float g, float u) {
  // (T)(g / (1 + expf(-g))) * u, product rounded to T
  const float s = rt<T>(g / (1.0f + expf(-g)));
  return rt<T>(s * u);
}

template <typename T> __device__ __forceinline__ float gelu_new_op(float x) {
  const float x3 = rt<T>(rt<T>(x * x) * x);
  const float inner = rt<T>(x + rt<T>(0.044715f * x3));
  const float t = rt<T>(tanhf(rt<T>(0.79788456f * inner)));
  return rt<T>(rt<T>(rt<T>(0.5f) * x) * rt<T>(rt<T>(1.0f) + t));
}

template <typename T> __device__ __forceinline__ float gelu_fast_op(float x) {
  const float a = rt<T>(x * 0.79788456f);
  const float b = rt<T>(rt<T>(1.0f) + rt<T>(rt<T>(0.044715f * x) * x));
  const float t = rt<T>(tanhf(rt<T>(a * b)));
  return rt<T>(rt<T>(rt<T>(0.5f) * x) * rt<T>(rt<T>(1.0f) + t));
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
silu_and_mul_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t T_, int64_t d) {
  constexpr int N = Vec16<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  if constexpr (VEC) {
    // four vectors per thread and step, all eight loads issued before the first use: the kernel is a pure
    // stream, so what matters is the number of bytes in flight per SM
    constexpr int U = 4;
    const int64_t vpr = d / N, total = T_ * vpr;
    for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
      Vec16<T> g[U], u[U];
      int64_t off_in[U], off_out[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int64_t i = i0 + stride * k;
        if (i < total) {
          const int64_t t = i / vpr, c = (i - t * vpr) * N;
          off_in[k] = t * 2 * d + c;
          off_out[k] = t * d + c;
          g[k] = ld16(in + off_in[k]);
          u[k] = ld16(in + off_in[k] + d);
        }
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        if (i0 + stride * k < total) {
          Vec16<T> o;
#pragma unroll
          for (int j = 0; j < N; ++j)
            o.v[j] = DT<T>::from_f(silu_mul_op<T>(DT<T>::to_f(g[k].v[j]), DT<T>::to_f(u[k].v[j])));
          st16(out + off_out[k], o);
        }
      }
    }
  } else {
    const int64_t total = T_ * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
      const int64_t t = i / d, c = i - t * d;
      out[i] = DT<T>::from_f(silu_mul_op<T>(DT<T>::to_f(in[t * 2 * d + c]), DT<T>::to_f(in[t * 2 * d + d + c])));
    }
  }
}

template <typename T, int OP, bool VEC>
__global__ void __launch_bounds__(256)
unary_kernel(T* __restrict__ out, const T* __restrict__ in, int64_t total) {
  constexpr int N = Vec16<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (VEC) {
    for (int64_t i = i0; i < total / N; i += stride) {
      const Vec16<T> x = ld16(in + i * N);
      Vec16<T> o;
#pragma unroll
      for (int j = 0; j < N; ++j) {
        const float f = DT<T>::to_f(x.v[j]);
        o.v[j] = DT<T>::from_f(OP == 0 ? gelu_new_op<T>(f) : gelu_fast_op<T>(f));
      }
      st16(out + i * N, o);
    }
    for (int64_t i = total / N * N + i0; i < total; i += stride) {
      const float f = DT<T>::to_f(in[i]);
      out[i] = DT<T>::from_f(OP == 0 ? gelu_new_op<T>(f) : gelu_fast_op<T>(f));
    }
  } else {
    for (int64_t i = i0; i < total; i += stride) {
      const float f = DT<T>::to_f(in[i]);
      out[i] = DT<T>::from_f(OP == 0 ? gelu_new_op<T>(f) : gelu_fast_op<T>(f));
    }
  }
}

static int grid_for(int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  const int64_t cap = (int64_t)sm_count() * 8;  // 8 resident CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}

template <typename T>
static int launch_silu(void* out, const void* in, int64_t T_, int64_t d, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  const bool vec = (d % N == 0) && aligned16(out) && aligned16(in);
  if (vec)
    silu_and_mul_kernel<T, true><<<grid_for(T_ * (d / N), 256), 256, 0, s>>>((T*)out, (const T*)in, T_, d);
  else
    silu_and_mul_kernel<T, false><<<grid_for(T_ * d, 256), 256, 0, s>>>((T*)out, (const T*)in, T_, d);
  SB_CHECK_LAUNCH("silu_and_mul_kernel");
  return SB200_OK;
}

template <typename T, int OP>
static int launch_unary(void* out, const void* in, int64_t total, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  const bool vec = aligned16(out) && aligned16(in);
  if (vec)
    unary_kernel<T, OP, true><<<grid_for(total / N + 1, 256), 256, 0, s>>>((T*)out, (const T*)in, total);
  else
    unary_kernel<T, OP, false><<<grid_for(total, 256), 256, 0, s>>>((T*)out, (const T*)in, total);
  SB_CHECK_LAUNCH("activation unary_kernel");
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_silu_and_mul(void* out, const void* in, int64_t T, int64_t d, int dtype,
                                  sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && d >= 0, "silu_and_mul: bad shape T=%lld d=%lld", (long long)T, (long long)d);
  if (T == 0 || d == 0) return SB200_OK;
  SB_CHECK_ARG(out && in, "silu_and_mul: null pointer");
  SB_DISPATCH_FLOAT(dtype, return (launch_silu<scalar_t>(out, in, T, d, (cudaStream_t)stream)));
  return SB200_OK;
}

extern "C" int sb200_gelu_new(void* out, const void* in, int64_t T, int64_t d, int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && d >= 0, "gelu_new: bad shape");
  if (T == 0 || d == 0) return SB200_OK;
  SB_CHECK_ARG(out && in, "gelu_new: null pointer");
  SB_DISPATCH_FLOAT(dtype, return (launch_unary<scalar_t, 0>(out, in, T * d, (cudaStream_t)stream)));
  return SB200_OK;
}

extern "C" int sb200_gelu_fast(void* out, const void* in, int64_t T, int64_t d, int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && d >= 0, "gelu_fast: bad shape");
  if (T == 0 || d == 0) return SB200_OK;
  SB_CHECK_ARG(out && in, "gelu_fast: null pointer");
  SB_DISPATCH_FLOAT(dtype, return (launch_unary<scalar_t, 1>(out, in, T * d, (cudaStream_t)stream)));
  return SB200_OK;
}
