// Vocabulary-parallel embedding lookup: out[t, :] = weight[ids[t] - vocab_start, :] when ids[t] lies in
// this rank's slice [vocab_start, vocab_end) of the vocabulary, zeros otherwise.
//
// Restates VocabParallelEmbedding.forward of the reference
// (tensor_parallel/layers.py:147-177): its mask / clone / F.embedding / masked_fill sequence is one
// pass here; the sum over the ranks that follows is the all-reduce of comm.cu.  Pure data movement:
// T*H*s bytes read and written, 16-byte vectors, several rows in flight per thread.
#include "common.cuh"

namespace sb200 {

template <typename T, bool VEC>
__global__ void __launch_bounds__(256)
vocab_embedding_kernel(T* __restrict__ out, const int64_t* __restrict__ ids, const T* __restrict__ weight, int64_t T_,
                       int64_t H, int64_t vocab_start, int64_t vocab_end) {
  constexpr int N = Vec16<T>::N;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t i_first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if constexpr (VEC) {
    constexpr int U = 4;
    const int64_t vpr = H / N, total = T_ * vpr;
    for (int64_t i0 = i_first; i0 < total; i0 += stride * U) {
      Vec16<T> v[U];
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int64_t i = i0 + stride * k;
        v[k].raw = make_uint4(0u, 0u, 0u, 0u);
        if (i < total) {
          const int64_t t = i / vpr, c = (i - t * vpr) * N;
          const int64_t id = ids[t];
          if (id >= vocab_start && id < vocab_end) v[k] = ld16(weight + (id - vocab_start) * H + c);
        }
      }
#pragma unroll
      for (int k = 0; k < U; ++k) {
        const int64_t i = i0 + stride * k;
        if (i < total) st16(out + i * N, v[k]);
      }
    }
  } else {
    const int64_t total = T_ * H;
    for (int64_t i = i_first; i < total; i += stride) {
      const int64_t t = i / H, c = i - t * H;
      const int64_t id = ids[t];
      T val;
      if (id >= vocab_start && id < vocab_end) val = weight[(id - vocab_start) * H + c];
      else val = DT<T>::from_f(0.f);
      out[i] = val;
    }
  }
}

template <typename T>
static int launch_vocab_embedding(void* out, const int64_t* ids, const void* weight, int64_t T_, int64_t H,
                                  int64_t v0, int64_t v1, cudaStream_t s) {
  constexpr int N = Vec16<T>::N;
  const bool vec = (H % N == 0) && aligned16(out) && aligned16(weight);
  const int64_t items = vec ? (T_ * (H / N) + 3) / 4 : T_ * H;
  int64_t blocks = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  if (vec)
    vocab_embedding_kernel<T, true><<<(int)blocks, 256, 0, s>>>((T*)out, ids, (const T*)weight, T_, H, v0, v1);
  else
    vocab_embedding_kernel<T, false><<<(int)blocks, 256, 0, s>>>((T*)out, ids, (const T*)weight, T_, H, v0, v1);
  SB_CHECK_LAUNCH("vocab_embedding_kernel");
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_vocab_embedding(void* out, const int64_t* ids, const void* weight, int64_t T, int64_t H,
                                     int64_t vocab_start, int64_t vocab_end, int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && H >= 0, "vocab_embedding: bad shape T=%lld H=%lld", (long long)T, (long long)H);
  SB_CHECK_ARG(vocab_start >= 0 && vocab_end >= vocab_start, "vocab_embedding: bad vocabulary range [%lld, %lld)",
               (long long)vocab_start, (long long)vocab_end);
  if (T == 0 || H == 0) return SB200_OK;
  SB_CHECK_ARG(out && ids && (weight || vocab_end == vocab_start), "vocab_embedding: null pointer");
  SB_DISPATCH_FLOAT(dtype, return (launch_vocab_embedding<scalar_t>(out, ids, weight, T, H, vocab_start, vocab_end,
                                                                    (cudaStream_t)stream)));
  return SB200_OK;
}
