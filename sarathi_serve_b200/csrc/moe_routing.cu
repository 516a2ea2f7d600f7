// MoE routing: fused softmax + top-k gating, and the block-aligned counting sort.
//
// topk_softmax restates csrc/moe_topk_softmax_kernels.cu of the reference.  The
// selected expert ids must equal the reference's bit for bit, which pins the
// floating-point evaluation order of the softmax: per-thread sequential sums
// over the same element groups, the same xor-butterfly across the threads of a
// row, max-subtracted expf, multiply by the reciprocal of the sum
// (:259-318), then k rounds of arg-max with the lowest index winning ties
// (:325-377).  On top of that this kernel reads fp16/bf16 logits directly
// (the reference casts with `.float()` first, fused_moe.py:367) and can
// renormalise the selected weights in the same launch (fused_moe.py:371-372).
//
// moe_align_block_size restates csrc/moe_align_block_size_kernels.cu:23-109
// (one CTA of `num_experts` threads there) as a warp-segmented stable counting
// sort: every warp owns a contiguous segment of slots, counts per expert with
// warp match operations, a scan over segments turns counts into start offsets,
// and a second walk scatters slot indices in order.  With a caller-provided
// scratch buffer the segments spread over many CTAs (three launches); without
// one a single 1024-thread CTA does the whole job in shared memory.
#include "common.cuh"

#include <cub/block/block_reduce.cuh>
#include <float.h>
#include <mutex>

namespace sb200 {

// ============================================================ topk_softmax

template <typename TIn> __device__ __forceinline__ float load_logit(const TIn* p, int64_t i) { return DT<TIn>::to_f(p[i]); }

template <int E> struct TopkLayout {
  static constexpr int ELTS_PER_LDG = (E < 4) ? E : 4;  // floats fetched as one group
  static constexpr int VECS = (E / (ELTS_PER_LDG * 32)) > 1 ? (E / (ELTS_PER_LDG * 32)) : 1;
  static constexpr int VPT = VECS * ELTS_PER_LDG;       // values per thread
  static constexpr int TPR = E / VPT;                   // threads per row
  static constexpr int ROWS_PER_WARP = 32 / TPR;
};

template <int E, typename TIn, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
topk_softmax_pow2_kernel(const TIn* __restrict__ gating, float* __restrict__ weights, int32_t* __restrict__ ids,
                         int32_t* __restrict__ src_rows, int64_t num_rows, int k, int renorm) {
  using L = TopkLayout<E>;
  constexpr int VPT = L::VPT, TPR = L::TPR, EPL = L::ELTS_PER_LDG, LDGS = L::VECS;
  constexpr int COLS_PER_GROUP = EPL * TPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = ((int64_t)blockIdx.x * WARPS + warp) * L::ROWS_PER_WARP + lane / TPR;
  if (row >= num_rows) return;  // whole row groups leave together (TPR divides 32)
  const int g = lane % TPR;
  const int first_col = g * EPL;

  float v[VPT];
#pragma unroll
  for (int l = 0; l < LDGS; ++l)
#pragma unroll
    for (int e = 0; e < EPL; ++e) v[l * EPL + e] = load_logit(gating, row * E + l * COLS_PER_GROUP + first_col + e);

  float mx = v[0];
#pragma unroll
  for (int i = 1; i < VPT; ++i) mx = max(mx, v[i]);
#pragma unroll
  for (int m = TPR / 2; m > 0; m >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, m, TPR));

  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    v[i] = expf(v[i] - mx);
    sum += v[i];
  }
#pragma unroll
  for (int m = TPR / 2; m > 0; m >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m, TPR);
  const float rcp = 1.f / sum;
#pragma unroll
  for (int i = 0; i < VPT; ++i) v[i] = v[i] * rcp;

  float picked_sum = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    float best = v[0];
    int expert = first_col;
#pragma unroll
    for (int l = 0; l < LDGS; ++l)
#pragma unroll
      for (int e = 0; e < EPL; ++e) {
        const float val = v[l * EPL + e];
        if (val > best) { best = val; expert = first_col + l * COLS_PER_GROUP + e; }
      }
#pragma unroll
    for (int m = TPR / 2; m > 0; m >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, m, TPR);
      const int oe = __shfl_xor_sync(0xffffffffu, expert, m, TPR);
      if (ob > best || (ob == best && oe < expert)) { best = ob; expert = oe; }
    }
    if (g == 0) {
      const int64_t o = row * k + kk;
      weights[o] = best;
      ids[o] = expert;
      if (src_rows) src_rows[o] = (int32_t)(kk * num_rows + row);
    }
    picked_sum += best;
    if (kk + 1 < k) {
      const int grp = expert / COLS_PER_GROUP;
      if (g == (expert / EPL) % TPR) v[grp * EPL + expert % EPL] = -10000.f;
    }
  }
  if (renorm && g == 0) {
    // Same thread wrote the k weights above; sequential sum in selection order.
    for (int kk = 0; kk < k; ++kk) weights[row * k + kk] = weights[row * k + kk] / picked_sum;
  }
}

// Any number of experts: one CTA per row, probabilities kept in shared memory.
// Sum order = strided per-thread accumulation + cub::BlockReduce<float,256>,
// as in moeSoftmax (csrc/moe_topk_softmax_kernels.cu:50-106).
template <typename TIn>
__global__ void __launch_bounds__(256)
topk_softmax_generic_kernel(const TIn* __restrict__ gating, float* __restrict__ weights, int32_t* __restrict__ ids,
                            int32_t* __restrict__ src_rows, int64_t num_rows, int E, int k, int renorm) {
  constexpr int TPB = 256;
  using BlockReduce = cub::BlockReduce<float, TPB>;
  __shared__ typename BlockReduce::TempStorage tmp;
  __shared__ float s_max, s_norm;
  __shared__ float s_bestv[TPB / 32];
  __shared__ int s_beste[TPB / 32];
  __shared__ int s_pick;
  extern __shared__ float probs[];
  const int64_t row = blockIdx.x;
  float t = -FLT_MAX;
  for (int i = threadIdx.x; i < E; i += TPB) t = max(load_logit(gating, row * E + i), t);
  const float m = BlockReduce(tmp).Reduce(t, cub::Max());
  if (threadIdx.x == 0) s_max = m;
  __syncthreads();
  t = 0.f;
  for (int i = threadIdx.x; i < E; i += TPB) t += expf(load_logit(gating, row * E + i) - s_max);
  const float Z = BlockReduce(tmp).Reduce(t, cub::Sum());
  if (threadIdx.x == 0) s_norm = 1.f / Z;
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += TPB) probs[i] = expf(load_logit(gating, row * E + i) - s_max) * s_norm;
  __syncthreads();
  float picked_sum = 0.f;
  for (int kk = 0; kk < k; ++kk) {
    float best = -1.f;
    int expert = 0x7fffffff;
    for (int i = threadIdx.x; i < E; i += TPB) {
      const float p = probs[i];
      if (p > best) { best = p; expert = i; }  // ascending i: first maximum wins
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, expert, o);
      if (ob > best || (ob == best && oe < expert)) { best = ob; expert = oe; }
    }
    if ((threadIdx.x & 31) == 0) { s_bestv[threadIdx.x >> 5] = best; s_beste[threadIdx.x >> 5] = expert; }
    __syncthreads();
    if (threadIdx.x == 0) {
      for (int w = 1; w < TPB / 32; ++w)
        if (s_bestv[w] > best || (s_bestv[w] == best && s_beste[w] < expert)) { best = s_bestv[w]; expert = s_beste[w]; }
      if (expert == 0x7fffffff) expert = 0;  // k > E: the reference's arg-max also falls back to key 0
      const int64_t o = row * k + kk;
      weights[o] = best;
      ids[o] = expert;
      if (src_rows) src_rows[o] = (int32_t)(kk * num_rows + row);
      picked_sum += best;
      s_pick = expert;
    }
    __syncthreads();
    if (threadIdx.x == 0 && s_pick < E) probs[s_pick] = -2.f;  // below the -1 start value: never picked again
    __syncthreads();
  }
  if (renorm && threadIdx.x == 0)
    for (int kk = 0; kk < k; ++kk) weights[row * k + kk] = weights[row * k + kk] / picked_sum;
}

template <int E, typename TIn>
static void launch_topk_pow2(const void* g, float* w, int32_t* ids, int32_t* src, int64_t T_, int k, int renorm,
                             cudaStream_t s) {
  constexpr int WARPS = 4;
  const int64_t rows_per_cta = WARPS * TopkLayout<E>::ROWS_PER_WARP;
  const int64_t blocks = (T_ + rows_per_cta - 1) / rows_per_cta;
  topk_softmax_pow2_kernel<E, TIn, WARPS><<<(unsigned)blocks, WARPS * 32, 0, s>>>((const TIn*)g, w, ids, src, T_, k, renorm);
}

template <typename TIn>
static int launch_topk(const void* g, float* w, int32_t* ids, int32_t* src, int64_t T_, int E, int k, int renorm,
                       cudaStream_t s) {
  switch (E) {
#define SB_CASE(n) case n: launch_topk_pow2<n, TIn>(g, w, ids, src, T_, k, renorm, s); break;
    SB_CASE(1) SB_CASE(2) SB_CASE(4) SB_CASE(8) SB_CASE(16) SB_CASE(32) SB_CASE(64) SB_CASE(128) SB_CASE(256)
#undef SB_CASE
    default: {
      const size_t smem = (size_t)E * sizeof(float);
      if (smem > 160 * 1024) {
        set_error("topk_softmax: num_experts=%d too large", E);
        return SB200_ERR_UNSUPPORTED;
      }
      if (smem > 40 * 1024)
        SB_CUDA(cudaFuncSetAttribute(topk_softmax_generic_kernel<TIn>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      topk_softmax_generic_kernel<TIn><<<(unsigned)T_, 256, smem, s>>>((const TIn*)g, w, ids, src, T_, E, k, renorm);
    }
  }
  SB_CHECK_LAUNCH("topk_softmax kernel");
  return SB200_OK;
}

// ===================================================== moe_align_block_size

template <typename TI> __device__ __forceinline__ int load_id(const void* p, int64_t i) { return (int)((const TI*)p)[i]; }

__device__ __forceinline__ int load_id_any(const void* p, int itype, int64_t i) {
  switch (itype) {
    case SB200_I32: return load_id<int32_t>(p, i);
    case SB200_I64: return load_id<int64_t>(p, i);
    case SB200_I16: return load_id<int16_t>(p, i);
    case SB200_I8: return load_id<int8_t>(p, i);
    default: return load_id<uint8_t>(p, i);
  }
}

// Walk one warp-owned segment [lo, hi) 32 slots at a time.  COUNT: add the
// per-expert population of the segment into cnt[].  Otherwise scatter slot
// indices to base[e] + cnt[e]++ in slot order (cnt = running start offsets).
template <bool COUNT>
__device__ __forceinline__ void walk_segment(const void* ids, int itype, int64_t lo, int64_t hi, int E, int* cnt,
                                             const int* base, int32_t* sorted) {
  const int lane = threadIdx.x & 31;
  for (int64_t s = lo; s < hi; s += 32) {
    const int64_t i = s + lane;
    int e = -1;
    if (i < hi) {
      e = load_id_any(ids, itype, i);
      if (e < 0 || e >= E) e = -1;  // ids outside [0, E) are ignored (the reference leaves them undefined)
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0) {
      if (COUNT) {
        if (rank == 0) cnt[e] += __popc(peers);
      } else {
        const int start = cnt[e];
        sorted[base[e] + start + rank] = (int32_t)i;
        __syncwarp(peers);
        if (rank == 0) cnt[e] = start + __popc(peers);
      }
    }
    __syncwarp();
  }
}

__device__ __forceinline__ int find_expert(const int* cumsum, int E, int pos) {
  // largest e with cumsum[e] <= pos, skipping empty experts (cumsum[e] == cumsum[e+1])
  int lo = 0, hi = E;  // invariant: cumsum[lo] <= pos < cumsum[hi]
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cumsum[mid] <= pos) lo = mid; else hi = mid;
  }
  return lo;
}

// Single CTA (32 warps = 32 segments), everything in shared memory.
// smem ints: cnt[32][E] | cumsum[E+1]
__global__ void __launch_bounds__(1024)
moe_align_single_kernel(const void* ids, int itype, int64_t numel, int E, int block, int32_t* sorted,
                        int64_t sorted_cap, int32_t* expert_ids, int64_t expert_cap, int32_t* num_post_pad) {
  extern __shared__ int sm[];
  int* cnt = sm;                 // [32][E]
  int* cumsum = sm + 32 * E;     // [E+1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 32 * E; i += 1024) cnt[i] = 0;
  for (int64_t i = threadIdx.x; i < sorted_cap; i += 1024) sorted[i] = (int32_t)numel;
  __syncthreads();
  const int64_t seg = (numel + 31) / 32;
  const int64_t lo = min((int64_t)warp * seg, numel), hi = min(lo + seg, numel);
  walk_segment<true>(ids, itype, lo, hi, E, cnt + warp * E, nullptr, nullptr);
  __syncthreads();
  // exclusive scan over the 32 segments for every expert: one warp per expert, lane = segment
  for (int e = warp; e < E; e += 32) {
    const int c = cnt[lane * E + e];
    int incl = c;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int n = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += n;
    }
    cnt[lane * E + e] = incl - c;
    if (lane == 31) cumsum[e + 1] = (incl + block - 1) / block * block;  // padded total of expert e
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    cumsum[0] = 0;
    for (int e = 1; e <= E; ++e) cumsum[e] += cumsum[e - 1];
    *num_post_pad = cumsum[E];
  }
  __syncthreads();
  const int nblk = cumsum[E] / block;
  for (int b = threadIdx.x; b < nblk && b < expert_cap; b += 1024) expert_ids[b] = find_expert(cumsum, E, b * block);
  walk_segment<false>(ids, itype, lo, hi, E, cnt + warp * E, cumsum, sorted);
}

// ---- multi-CTA path: scratch ints = counts[nseg][E] | cumsum[E+1]
__global__ void __launch_bounds__(256)
moe_align_count_kernel(const void* ids, int itype, int64_t numel, int E, int64_t seg_len, int nseg, int* scratch,
                       int32_t* sorted, int64_t sorted_cap) {
  const int64_t gtid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, gsz = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = gtid; i < sorted_cap; i += gsz) sorted[i] = (int32_t)numel;
  const int seg = (int)(gtid >> 5);
  if (seg >= nseg) return;
  int* cnt = scratch + (int64_t)seg * E;
  const int lane = threadIdx.x & 31;
  for (int e = lane; e < E; e += 32) cnt[e] = 0;
  __syncwarp();
  const int64_t lo = min((int64_t)seg * seg_len, numel), hi = min(lo + seg_len, numel);
  walk_segment<true>(ids, itype, lo, hi, E, cnt, nullptr, nullptr);
}

__global__ void __launch_bounds__(1024)
moe_align_scan_kernel(int E, int block, int nseg, int* scratch, int32_t* expert_ids, int64_t expert_cap,
                      int32_t* num_post_pad) {
  int* cumsum = scratch + (int64_t)nseg * E;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int e = warp; e < E; e += 32) {
    int carry = 0;
    for (int s0 = 0; s0 < nseg; s0 += 32) {
      const int s = s0 + lane;
      const int c = (s < nseg) ? scratch[(int64_t)s * E + e] : 0;
      int incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
      }
      if (s < nseg) scratch[(int64_t)s * E + e] = carry + incl - c;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) cumsum[e + 1] = (carry + block - 1) / block * block;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    cumsum[0] = 0;
    for (int e = 1; e <= E; ++e) cumsum[e] += cumsum[e - 1];
    *num_post_pad = cumsum[E];
  }
  __syncthreads();
  const int nblk = cumsum[E] / block;
  for (int b = threadIdx.x; b < nblk && b < expert_cap; b += 1024) expert_ids[b] = find_expert(cumsum, E, b * block);
}

__global__ void __launch_bounds__(256)
moe_align_scatter_kernel(const void* ids, int itype, int64_t numel, int E, int64_t seg_len, int nseg, int* scratch,
                         int32_t* sorted) {
  const int seg = (int)(((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5);
  if (seg >= nseg) return;
  const int64_t lo = min((int64_t)seg * seg_len, numel), hi = min(lo + seg_len, numel);
  walk_segment<false>(ids, itype, lo, hi, E, scratch + (int64_t)seg * E, scratch + (int64_t)nseg * E, sorted);
}

struct AlignPlan { int nseg; int64_t seg_len; };
static AlignPlan align_plan(int64_t numel) {
  // segments of >= 256 slots, at most 8 warps per CTA on every SM
  int64_t nseg = (numel + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (nseg > cap) nseg = cap;
  if (nseg < 1) nseg = 1;
  int64_t seg_len = (numel + nseg - 1) / nseg;
  seg_len = (seg_len + 31) / 32 * 32;
  return {(int)nseg, seg_len};
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_topk_softmax(float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices,
                                  const void* gating, int gating_dtype, int64_t T, int E, int k, int renormalize,
                                  sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && E > 0 && k > 0, "topk_softmax: bad shape T=%lld E=%d k=%d", (long long)T, E, k);
  SB_CHECK_ARG(T * (int64_t)k <= INT32_MAX, "topk_softmax: T*k overflows int32 row indices");
  if (T == 0) return SB200_OK;
  SB_CHECK_ARG(topk_weights && topk_ids && gating, "topk_softmax: null pointer");
  SB_DISPATCH_FLOAT(gating_dtype, return (launch_topk<scalar_t>(gating, topk_weights, topk_ids, token_expert_indices,
                                                               T, E, k, renormalize, (cudaStream_t)stream)));
  return SB200_OK;
}

extern "C" int64_t sb200_moe_align_scratch_bytes(int64_t numel, int num_experts) {
  if (numel < 0 || num_experts <= 0) return 0;
  const AlignPlan p = align_plan(numel);
  return ((int64_t)p.nseg * num_experts + num_experts + 1) * (int64_t)sizeof(int);
}

extern "C" int sb200_moe_align_block_size(const void* topk_ids, int ids_itype, int64_t numel, int num_experts,
                                          int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                          int32_t* expert_ids, int64_t expert_ids_capacity,
                                          int32_t* num_tokens_post_pad, void* scratch, int64_t scratch_bytes,
                                          sb200_stream_t stream) {
  const int E = num_experts;
  SB_CHECK_ARG(numel >= 0 && E > 0 && block_size > 0, "moe_align_block_size: bad shape numel=%lld E=%d block=%d",
               (long long)numel, E, block_size);
  SB_CHECK_ARG(ids_itype >= SB200_I32 && ids_itype <= SB200_U8, "moe_align_block_size: bad index type %d", ids_itype);
  SB_CHECK_ARG(numel + (int64_t)E * block_size <= INT32_MAX, "moe_align_block_size: sizes overflow int32");
  SB_CHECK_ARG(sorted_token_ids && expert_ids && num_tokens_post_pad && (topk_ids || numel == 0),
               "moe_align_block_size: null pointer");
  // worst case of the padded length: every expert non-empty and one past a block boundary
  const int64_t worst = numel + (int64_t)(E < numel ? E : numel) * (block_size - 1);
  SB_CHECK_ARG(sorted_capacity >= worst, "moe_align_block_size: sorted_token_ids holds %lld < %lld entries",
               (long long)sorted_capacity, (long long)worst);
  SB_CHECK_ARG(expert_ids_capacity >= (worst + block_size - 1) / block_size,
               "moe_align_block_size: expert_ids holds %lld entries, %lld needed", (long long)expert_ids_capacity,
               (long long)((worst + block_size - 1) / block_size));
  cudaStream_t s = (cudaStream_t)stream;
  const AlignPlan p = align_plan(numel);
  const int64_t need = ((int64_t)p.nseg * E + E + 1) * (int64_t)sizeof(int);
  const bool multi = scratch != nullptr && scratch_bytes >= need && numel > 8192;
  if (!multi) {
    const size_t smem = ((size_t)32 * E + E + 1) * sizeof(int);
    if (smem > 200 * 1024) {
      set_error("moe_align_block_size: num_experts=%d needs a scratch buffer (shared memory exceeded)", E);
      return SB200_ERR_UNSUPPORTED;
    }
    if (smem > 40 * 1024)
      SB_CUDA(cudaFuncSetAttribute(moe_align_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    moe_align_single_kernel<<<1, 1024, smem, s>>>(topk_ids, ids_itype, numel, E, block_size, sorted_token_ids,
                                                  sorted_capacity, expert_ids, expert_ids_capacity,
                                                  num_tokens_post_pad);
    SB_CHECK_LAUNCH("moe_align_single_kernel");
    return SB200_OK;
  }
  int* scr = (int*)scratch;
  const int ctas = (p.nseg + 7) / 8;
  moe_align_count_kernel<<<ctas, 256, 0, s>>>(topk_ids, ids_itype, numel, E, p.seg_len, p.nseg, scr,
                                              sorted_token_ids, sorted_capacity);
  SB_CHECK_LAUNCH("moe_align_count_kernel");
  moe_align_scan_kernel<<<1, 1024, 0, s>>>(E, block_size, p.nseg, scr, expert_ids, expert_ids_capacity,
                                           num_tokens_post_pad);
  SB_CHECK_LAUNCH("moe_align_scan_kernel");
  moe_align_scatter_kernel<<<ctas, 256, 0, s>>>(topk_ids, ids_itype, numel, E, p.seg_len, p.nseg, scr,
                                                sorted_token_ids);
  SB_CHECK_LAUNCH("moe_align_scatter_kernel");
  return SB200_OK;
}

// ------------------------------------------------------------------------------------------
// sb200_moe_align_block_size_noalloc: the multi-CTA sort above, for callers that must not
// allocate.  Some hosts of this library cannot hand it a scratch buffer and cannot call
// cudaMalloc at the point where they route tokens: a serving worker that has already given
// every free byte of the GPU to its KV cache, code that runs between other streams' kernels
// where the device-wide synchronisation inside cudaMalloc / cudaFree would stall them, or a
// plugin boundary that only passes inputs and outputs through.  For them the per-segment
// counters live in a fixed array that is part of the library image: every GPU that loads
// the library holds these 258 KiB until the process exits.
//
// Limits: numel <= SB200_ALIGN_NOALLOC_MAX_SLOTS and num_experts <= SB200_ALIGN_NOALLOC_MAX_EXPERTS;
// larger inputs are refused with SB200_ERR_UNSUPPORTED.
//
// The array is shared by every call on a device and keeps the previous call's contents.
// Nothing in it needs clearing between calls: the count kernel zeroes each segment's
// counters before counting and the scan kernel rewrites every prefix entry it later reads.
// Two calls that overlap on the GPU (different streams, or different threads without
// ordering) would race on it; issue them on one stream or order them with events.
//
// The first call on each device looks up the array's device address (with that device
// current); make that first call outside any stream capture.
constexpr int kNoAllocMaxSegments = SB200_ALIGN_NOALLOC_MAX_SLOTS / 256;
constexpr int kNoAllocScratchInts = kNoAllocMaxSegments * SB200_ALIGN_NOALLOC_MAX_EXPERTS + SB200_ALIGN_NOALLOC_MAX_EXPERTS + 1 + 63;
static __device__ __align__(256) int g_align_noalloc_scratch[kNoAllocScratchInts];

namespace sb200 {
constexpr int kMaxDevices = 64;
static int* g_noalloc_ptr[kMaxDevices];  // device address of the array, per device ordinal
static std::mutex g_noalloc_mutex;

// In host code the array's name is only a handle for the runtime, not a device address:
// the address a kernel can use comes from cudaGetSymbolAddress, once per device.
static int noalloc_scratch(int** out) {
  int dev = -1;
  SB_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < kMaxDevices, "moe_align_block_size_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_align_noalloc_scratch);
    if (e != cudaSuccess) return cuda_fail(e, "cudaGetSymbolAddress(g_align_noalloc_scratch)");
    g_noalloc_ptr[dev] = static_cast<int*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return SB200_OK;
}
}  // namespace sb200

extern "C" int sb200_moe_align_block_size_noalloc(const void* topk_ids, int ids_itype, int64_t numel, int num_experts,
                                                  int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                                  int32_t* expert_ids, int64_t expert_ids_capacity,
                                                  int32_t* num_tokens_post_pad, sb200_stream_t stream) {
  const int E = num_experts;
  SB_CHECK_ARG(numel >= 0 && E > 0 && block_size > 0, "moe_align_block_size_noalloc: bad shape numel=%lld E=%d block=%d",
               (long long)numel, E, block_size);
  if (numel > SB200_ALIGN_NOALLOC_MAX_SLOTS || E > SB200_ALIGN_NOALLOC_MAX_EXPERTS) {
    set_error("moe_align_block_size_noalloc: numel=%lld / num_experts=%d exceed the built-in scratch (at most %d slots, "
              "%d experts); use sb200_moe_align_block_size with a caller-provided scratch buffer",
              (long long)numel, E, SB200_ALIGN_NOALLOC_MAX_SLOTS, SB200_ALIGN_NOALLOC_MAX_EXPERTS);
    return SB200_ERR_UNSUPPORTED;
  }
  SB_CHECK_ARG(ids_itype >= SB200_I32 && ids_itype <= SB200_U8, "moe_align_block_size_noalloc: bad index type %d", ids_itype);
  SB_CHECK_ARG(numel + (int64_t)E * block_size <= INT32_MAX, "moe_align_block_size_noalloc: sizes overflow int32");
  SB_CHECK_ARG(sorted_token_ids && expert_ids && num_tokens_post_pad && (topk_ids || numel == 0),
               "moe_align_block_size_noalloc: null pointer");
  const int64_t worst = numel + (int64_t)(E < numel ? E : numel) * (block_size - 1);
  SB_CHECK_ARG(sorted_capacity >= worst, "moe_align_block_size_noalloc: sorted_token_ids holds %lld < %lld entries",
               (long long)sorted_capacity, (long long)worst);
  SB_CHECK_ARG(expert_ids_capacity >= (worst + block_size - 1) / block_size,
               "moe_align_block_size_noalloc: expert_ids holds %lld entries, %lld needed", (long long)expert_ids_capacity,
               (long long)((worst + block_size - 1) / block_size));
  int* scr = nullptr;
  const int rc = noalloc_scratch(&scr);
  if (rc) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  AlignPlan p = align_plan(numel);
  if (p.nseg > kNoAllocMaxSegments) {  // cannot happen below the slot limit; kept as a guard on the array bound
    set_error("moe_align_block_size_noalloc: internal segment count %d exceeds %d", p.nseg, kNoAllocMaxSegments);
    return SB200_ERR_UNSUPPORTED;
  }
  const int ctas = (p.nseg + 7) / 8;
  moe_align_count_kernel<<<ctas, 256, 0, s>>>(topk_ids, ids_itype, numel, E, p.seg_len, p.nseg, scr, sorted_token_ids,
                                              sorted_capacity);
  SB_CHECK_LAUNCH("moe_align_count_kernel (noalloc)");
  moe_align_scan_kernel<<<1, 1024, 0, s>>>(E, block_size, p.nseg, scr, expert_ids, expert_ids_capacity,
                                           num_tokens_post_pad);
  SB_CHECK_LAUNCH("moe_align_scan_kernel (noalloc)");
  moe_align_scatter_kernel<<<ctas, 256, 0, s>>>(topk_ids, ids_itype, numel, E, p.seg_len, p.nseg, scr,
                                                sorted_token_ids);
  SB_CHECK_LAUNCH("moe_align_scatter_kernel (noalloc)");
  return SB200_OK;
}
