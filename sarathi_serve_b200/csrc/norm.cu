// RMSNorm and residual-add + RMSNorm for [T, H] rows (HBM-bound row kernels).
//
// One CTA per token row.  The row is read once with 16-byte loads, held in
// registers across the block reduction and written once, so the kernel moves
// the algorithmic (2*T*H + H) * sizeof(T) bytes (4*T*H + H for the add variant).
// Semantics follow the reference kernel (csrc/layernorm_kernels.cu:10-35):
// sum of squares in fp32, inv = rsqrtf(var / H + eps), and the product
// x * inv is rounded to T BEFORE the multiply by the weight.
#include "common.cuh"

namespace sb200 {

constexpr int kNormMaxVec = 4;  // 16-byte vectors cached per thread

template <typename T, bool ADD, bool VEC>
__global__ void __launch_bounds__(1024)
rms_norm_kernel(T* __restrict__ out, T* resid_out, const T* x, const T* resid,
                const T* __restrict__ w, float eps, int H) {
  __shared__ float red[33];
  constexpr int N = Vec16<T>::N;
  const int64_t row = blockIdx.x;
  const T* xr = x + row * H;
  const T* rr = ADD ? resid + row * H : nullptr;
  T* orow = out + row * H;
  T* zrow = ADD ? resid_out + row * H : nullptr;
  float ss = 0.f;

  if constexpr (VEC) {
    Vec16<T> cache[kNormMaxVec];
    const int nvec = H / N;
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = i * blockDim.x + threadIdx.x;
      if (v < nvec) {
        cache[i] = ld16(xr + v * N);
        if constexpr (ADD) {
          Vec16<T> r = ld16(rr + v * N);
#pragma unroll
          for (int j = 0; j < N; ++j)
            cache[i].v[j] = DT<T>::from_f(DT<T>::to_f(cache[i].v[j]) + DT<T>::to_f(r.v[j]));
          st16(zrow + v * N, cache[i]);
        }
#pragma unroll
        for (int j = 0; j < N; ++j) {
          const float f = DT<T>::to_f(cache[i].v[j]);
          ss += f * f;
        }
      }
    }
    ss = block_sum(ss, red);
    const float inv = rsqrtf(ss / (float)H + eps);
#pragma unroll
    for (int i = 0; i < kNormMaxVec; ++i) {
      const int v = i * blockDim.x + threadIdx.x;
      if (v < nvec) {
        Vec16<T> wv = ld16(w + v * N), o;
#pragma unroll
        for (int j = 0; j < N; ++j)
          o.v[j] = DT<T>::from_f(rt<T>(DT<T>::to_f(cache[i].v[j]) * inv) * DT<T>::to_f(wv.v[j]));
        st16(orow + v * N, o);
      }
    }
  } else {
    // Generic path: any H / alignment; the row is re-read from L1/L2.
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
      float f = DT<T>::to_f(xr[i]);
      if constexpr (ADD) {
        f = rt<T>(f + DT<T>::to_f(rr[i]));
        zrow[i] = DT<T>::from_f(f);
      }
      ss += f * f;
    }
    ss = block_sum(ss, red);  // also orders the zrow writes before the re-read below
    const float inv = rsqrtf(ss / (float)H + eps);
    const T* src = ADD ? zrow : xr;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
      orow[i] = DT<T>::from_f(rt<T>(DT<T>::to_f(src[i]) * inv) * DT<T>::to_f(w[i]));
  }
}

template <typename T, bool ADD>
static int launch_norm(void* out, void* resid_out, const void* x, const void* resid, const void* w,
                       float eps, int64_t T_, int64_t H, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  bool vec = (H % N == 0) && aligned16(out) && aligned16(x) && aligned16(w) &&
             (!ADD || (aligned16(resid) && aligned16(resid_out)));
  int threads = 0;
  if (vec) {
    const int64_t nvec = H / N;
    // fewest vectors per thread that keep the CTA at >= 128 threads when possible
    int per = 1;
    while (per < kNormMaxVec && (nvec + per - 1) / per > 512) ++per;
    int64_t t = (nvec + per - 1) / per;
    t = (t + 31) / 32 * 32;
    if (t > 1024 || t * kNormMaxVec < nvec) vec = false;
    threads = (int)t;
  }
  if (!vec) threads = (int)((H < 1024 ? (H + 31) / 32 * 32 : 1024));
  dim3 grid((unsigned)T_);
  if (vec)
    rms_norm_kernel<T, ADD, true><<<grid, threads, 0, s>>>((T*)out, (T*)resid_out, (const T*)x,
                                                           (const T*)resid, (const T*)w, eps, (int)H);
  else
    rms_norm_kernel<T, ADD, false><<<grid, threads, 0, s>>>((T*)out, (T*)resid_out, (const T*)x,
                                                            (const T*)resid, (const T*)w, eps, (int)H);
  SB_CHECK_LAUNCH("rms_norm_kernel");
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_rms_norm(void* out, const void* x, const void* w, float eps, int64_t T, int64_t H,
                              int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && H > 0 && H <= INT32_MAX && T <= INT32_MAX, "rms_norm: bad shape T=%lld H=%lld",
               (long long)T, (long long)H);
  if (T == 0) return SB200_OK;
  SB_CHECK_ARG(out && x && w, "rms_norm: null pointer");
  SB_DISPATCH_FLOAT(dtype, return (launch_norm<scalar_t, false>(out, nullptr, x, nullptr, w, eps, T, H,
                                                               (cudaStream_t)stream)));
  return SB200_OK;
}

extern "C" int sb200_fused_add_rms_norm(void* out, void* residual_out, const void* x, const void* residual,
                                        const void* w, float eps, int64_t T, int64_t H, int dtype,
                                        sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && H > 0 && H <= INT32_MAX && T <= INT32_MAX,
               "fused_add_rms_norm: bad shape T=%lld H=%lld", (long long)T, (long long)H);
  if (T == 0) return SB200_OK;
  SB_CHECK_ARG(out && residual_out && x && residual && w, "fused_add_rms_norm: null pointer");
  SB_CHECK_ARG(out != x && out != residual, "fused_add_rms_norm: out must not alias an input");
  SB_DISPATCH_FLOAT(dtype, return (launch_norm<scalar_t, true>(out, residual_out, x, residual, w, eps, T, H,
                                                              (cudaStream_t)stream)));
  return SB200_OK;
}
