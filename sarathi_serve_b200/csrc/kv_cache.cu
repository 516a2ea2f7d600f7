// Append of a step's keys and values to the paged KV cache, the step that sits between the qkv
// projection and attention.
//
// Replaces what the reference does in its attention wrapper before it calls attention
// (sarathi/model_executor/attention/flashinfer_attention_wrapper.py:253-270): three `.contiguous()`
// reshapes of q / k / v and flashinfer's append_paged_kv_cache (flashinfer-python, pinned 0.4.1 in the
// reference's requirements.txt:18) into a cache of layout [pages, 2, page_size, kv_heads, head_dim]
// (:69-77; "NHD").  Entry i of the batch belongs to request b = batch_indices[i] and is the token at
// position p = positions[i] of that request; its page is kv_indices[kv_indptr[b] + p / page_size] and its
// slot inside the page is p % page_size; keys go to cache[page, 0, slot], values to cache[page, 1, slot].
//
// Two kernels: `kv_slots_kernel` turns (batch_indices, positions, page table) into one row index per
// token, and `kv_append_kernel` copies strided k / v rows (views of the fused qkv buffer; no
// `.contiguous()` copy) to those rows.  The qkv GEMM can also store k and v there from its epilogue
// (gemm_sm100.cuh), in which case only the first kernel runs.
#include "common.cuh"

namespace sb200 {

// slots[i] = page * (2 * page_size) + slot: the row of cache seen as [pages * 2 * page_size, kv_heads * head_dim]
// that receives token i's key; its value goes page_size rows further.  -1 for entries with a negative
// batch index (padding tokens).
__global__ void kv_slots_kernel(int64_t* __restrict__ slots, const int32_t* __restrict__ batch_indices,
                                const int32_t* __restrict__ positions, const int32_t* __restrict__ kv_indices,
                                const int32_t* __restrict__ kv_indptr, int64_t n, int page_size) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int b = batch_indices[i];
  if (b < 0) { slots[i] = -1; return; }
  const int p = positions[i];
  const int64_t page = kv_indices[kv_indptr[b] + p / page_size];
  slots[i] = page * (2 * (int64_t)page_size) + (p % page_size);
}

template <typename T>
__global__ void __launch_bounds__(256)
kv_append_kernel(T* __restrict__ cache, const T* __restrict__ k, int64_t ldk, const T* __restrict__ v, int64_t ldv,
                 const int64_t* __restrict__ slots, int64_t n, int row_elems, int page_size) {
  constexpr int N = Vec16<T>::N;
  const int nvec = row_elems / N;
  const int64_t total = n * nvec * 2, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t t = i / (2 * nvec);
    const int r = (int)(i - t * 2 * nvec);
    const int which = r / nvec, vec = r - which * nvec;  // 0: key, 1: value
    const int64_t s = slots[t];
    if (s < 0) continue;
    const T* src = (which ? v + t * ldv : k + t * ldk) + (int64_t)vec * N;
    st16(cache + (s + (which ? page_size : 0)) * row_elems + (int64_t)vec * N, ld16(src));
  }
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_kv_cache_slots(int64_t* slots, const int32_t* batch_indices, const int32_t* positions,
                                    const int32_t* kv_indices, const int32_t* kv_indptr, int64_t n, int page_size,
                                    sb200_stream_t stream) {
  SB_CHECK_ARG(n >= 0 && page_size > 0, "kv_cache_slots: bad sizes");
  if (n == 0) return SB200_OK;
  SB_CHECK_ARG(slots && batch_indices && positions && kv_indices && kv_indptr, "kv_cache_slots: null pointer");
  kv_slots_kernel<<<(int)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(slots, batch_indices, positions, kv_indices,
                                                                            kv_indptr, n, page_size);
  SB_CHECK_LAUNCH("kv_slots_kernel");
  return SB200_OK;
}

extern "C" int sb200_kv_cache_append(void* cache, const void* k, int64_t ldk, const void* v, int64_t ldv,
                                     const int64_t* slots, int64_t n, int num_kv_heads, int head_dim, int page_size,
                                     int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(n >= 0 && num_kv_heads > 0 && head_dim > 0 && page_size > 0, "kv_cache_append: bad sizes");
  if (n == 0) return SB200_OK;
  SB_CHECK_ARG(cache && k && v && slots, "kv_cache_append: null pointer");
  const int64_t row = (int64_t)num_kv_heads * head_dim;
  const size_t es = dtype_size(dtype);
  SB_CHECK_ARG((row * es) % 16 == 0 && (ldk * es) % 16 == 0 && (ldv * es) % 16 == 0 && ldk >= row && ldv >= row &&
                   aligned16(cache) && aligned16(k) && aligned16(v),
               "kv_cache_append: rows must be 16-byte aligned multiples of 16 bytes");
  int64_t blocks = (n * 2 * (row / (16 / (int64_t)es)) + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  SB_DISPATCH_FLOAT(dtype, (kv_append_kernel<scalar_t><<<(int)blocks, 256, 0, (cudaStream_t)stream>>>(
                               (scalar_t*)cache, (const scalar_t*)k, ldk, (const scalar_t*)v, ldv, slots, n, (int)row,
                               page_size)));
  SB_CHECK_LAUNCH("kv_append_kernel");
  return SB200_OK;
}
