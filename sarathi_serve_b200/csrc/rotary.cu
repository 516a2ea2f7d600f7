// In-place rotary position embedding on strided q / k rows.
//
// Flat grid-stride over (token, head, 16-byte vector of rotation pairs); q and
// k heads are one index space so a single launch covers both.  Restates
// csrc/pos_encoding_kernels.cu:8-76 of the reference: the cache row for
// positions[t] holds cos | sin (rot_dim/2 each) in the model dtype; NeoX style
// pairs element i with i + rot_dim/2, GPT-J style pairs 2i with 2i+1; each
// product and each sum is rounded to T like the reference's scalar operators.
#include "common.cuh"

namespace sb200 {

template <typename T>
__device__ __forceinline__ void rot_pair(float x, float y, float c, float s, float& xo, float& yo) {
  xo = rt<T>(rt<T>(x * c) - rt<T>(y * s));
  yo = rt<T>(rt<T>(y * c) + rt<T>(x * s));
}

template <typename T, bool NEOX, bool VEC>
__global__ void __launch_bounds__(256)
rotary_kernel(const int64_t* __restrict__ positions, T* q, T* k, const T* __restrict__ cache,
              int64_t T_, int nq, int nkv, int head_size, int rot_dim, int64_t q_stride, int64_t k_stride) {
  constexpr int N = Vec16<T>::N;
  const int half = rot_dim / 2;
  const int heads = nq + nkv;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // work items per head: NeoX -> half/N vectors of x (and the matching y vectors);
  // GPT-J -> rot_dim/N vectors of interleaved pairs; scalar -> half pairs.
  const int per_head = VEC ? (NEOX ? half / N : rot_dim / N) : half;
  const int64_t total = T_ * heads * per_head;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t th = i / per_head;
    const int j = (int)(i - th * per_head);
    const int64_t t = th / heads;
    const int h = (int)(th - t * heads);
    T* base = (h < nq) ? q + t * q_stride + (int64_t)h * head_size
                       : k + t * k_stride + (int64_t)(h - nq) * head_size;
    const T* cs = cache + positions[t] * rot_dim;
    if constexpr (VEC && NEOX) {
      Vec16<T> x = ld16(base + j * N), y = ld16(base + half + j * N);
      const Vec16<T> c = ld16(cs + j * N), s = ld16(cs + half + j * N);
#pragma unroll
      for (int e = 0; e < N; ++e) {
        float xo, yo;
        rot_pair<T>(DT<T>::to_f(x.v[e]), DT<T>::to_f(y.v[e]), DT<T>::to_f(c.v[e]), DT<T>::to_f(s.v[e]), xo, yo);
        x.v[e] = DT<T>::from_f(xo);
        y.v[e] = DT<T>::from_f(yo);
      }
      st16(base + j * N, x);
      st16(base + half + j * N, y);
    } else if constexpr (VEC && !NEOX) {
      Vec16<T> xy = ld16(base + j * N);
#pragma unroll
      for (int e = 0; e < N / 2; ++e) {
        const int p = j * (N / 2) + e;  // pair index
        float xo, yo;
        rot_pair<T>(DT<T>::to_f(xy.v[2 * e]), DT<T>::to_f(xy.v[2 * e + 1]), DT<T>::to_f(cs[p]),
                    DT<T>::to_f(cs[half + p]), xo, yo);
        xy.v[2 * e] = DT<T>::from_f(xo);
        xy.v[2 * e + 1] = DT<T>::from_f(yo);
      }
      st16(base + j * N, xy);
    } else {
      const int xi = NEOX ? j : 2 * j, yi = NEOX ? half + j : 2 * j + 1;
      float xo, yo;
      rot_pair<T>(DT<T>::to_f(base[xi]), DT<T>::to_f(base[yi]), DT<T>::to_f(cs[j]), DT<T>::to_f(cs[half + j]), xo, yo);
      base[xi] = DT<T>::from_f(xo);
      base[yi] = DT<T>::from_f(yo);
    }
  }
}

template <typename T>
static int launch_rotary(const int64_t* positions, void* q, void* k, const void* cache, int64_t T_, int nq,
                         int nkv, int head_size, int rot_dim, int64_t qs, int64_t ks, bool neox, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  const int half = rot_dim / 2;
  const int unit = neox ? half : rot_dim;  // contiguous run that must split into 16-byte vectors
  const bool vec = (unit % N == 0) && (head_size % N == 0) && (rot_dim % N == 0) && (half % N == 0 || !neox) &&
                   aligned16(q) && (nkv == 0 || aligned16(k)) && aligned16(cache) && (qs % N == 0) &&
                   (nkv == 0 || ks % N == 0);
  const int per_head = vec ? (neox ? half / N : rot_dim / N) : half;
  const int64_t total = T_ * (nq + nkv) * per_head;
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  T* kq = (T*)q; T* kk = (T*)k; const T* kc = (const T*)cache;
#define SB_ROT(NE, VE) \
  rotary_kernel<T, NE, VE><<<(int)blocks, 256, 0, s>>>(positions, kq, kk, kc, T_, nq, nkv, head_size, rot_dim, qs, ks)
  if (neox) { if (vec) SB_ROT(true, true); else SB_ROT(true, false); }
  else      { if (vec) SB_ROT(false, true); else SB_ROT(false, false); }
#undef SB_ROT
  SB_CHECK_LAUNCH("rotary_kernel");
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_rotary_embedding(const int64_t* positions, void* query, void* key, int64_t T, int num_heads,
                                      int num_kv_heads, int head_size, int rot_dim, int64_t q_stride,
                                      int64_t k_stride, const void* cos_sin_cache, int is_neox, int dtype,
                                      sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && num_heads >= 0 && num_kv_heads >= 0 && head_size > 0, "rotary_embedding: bad shape");
  SB_CHECK_ARG(rot_dim > 0 && rot_dim % 2 == 0 && rot_dim <= head_size,
               "rotary_embedding: rot_dim=%d must be even and <= head_size=%d", rot_dim, head_size);
  if (T == 0 || num_heads + num_kv_heads == 0) return SB200_OK;
  SB_CHECK_ARG(positions && query && cos_sin_cache && (key || num_kv_heads == 0), "rotary_embedding: null pointer");
  SB_CHECK_ARG(q_stride >= (int64_t)num_heads * head_size && (num_kv_heads == 0 || k_stride >= (int64_t)num_kv_heads * head_size),
               "rotary_embedding: row stride smaller than the row");
  SB_DISPATCH_FLOAT(dtype, return (launch_rotary<scalar_t>(positions, query, key, cos_sin_cache, T, num_heads,
                                                          num_kv_heads, head_size, rot_dim, q_stride, k_stride,
                                                          is_neox != 0, (cudaStream_t)stream)));
  return SB200_OK;
}
