// Mixture-of-experts expert GEMMs on the tcgen05 kernel (grouped mode of gemm_sm100.cuh).
//
// Replaces the reference's Triton grouped GEMM and the glue around it
// (layers/fused_moe/fused_moe.py:15-148 fused_moe_kernel, :411-544 fused_experts):
//   gather : xs[r, :] = x[sorted_ids[r] / top_k, :]         (expert-sorted, block-padded rows)
//   GEMM 1 : act[r, :] = silu(xs[r] W13[e]_gate^T) * (xs[r] W13[e]_up^T)   (SiLU*mul in the epilogue)
//   GEMM 2 : out3[slot(r), :] = (act[r] W2[e]^T) * topk_weight[slot(r)]    (scaled + scattered in the epilogue)
//   sum    : out[t, :] = sum_j out3[t*k + j, :]              (or fused into the all-reduce push, comm.cu)
// with e = expert_ids[r / block] and block = 128 rows = one tile row block, so a tile never mixes experts.
#include "gemm_host.cuh"

namespace sb200 {

constexpr int kMoeBlockRows = 128;

template <typename T>
__global__ void __launch_bounds__(256)
moe_gather_kernel(T* __restrict__ out, const T* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                  const int32_t* __restrict__ num_post_pad, int64_t rows_cap, int64_t num_slots, int H, int top_k) {
  constexpr int N = Vec16<T>::N;
  const int nvec = H / N;
  const int64_t rows = min((int64_t)*num_post_pad, rows_cap);
  const int64_t total = rows * nvec;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t r = i / nvec;
    const int v = (int)(i - r * nvec);
    const int32_t slot = sorted_ids[r];
    Vec16<T> val;
    if (slot >= 0 && slot < num_slots) val = ld16(x + (int64_t)(slot / top_k) * H + (int64_t)v * N);
    else val.raw = make_uint4(0, 0, 0, 0);  // padding rows are zero: their products vanish
    st16(out + r * H + (int64_t)v * N, val);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_sum_kernel(T* __restrict__ out, const T* __restrict__ in3, const T* __restrict__ residual, int64_t T_, int k, int H) {
  constexpr int N = Vec16<T>::N;
  const int nvec = H / N;
  const int64_t total = T_ * nvec, stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t t = i / nvec;
    const int v = (int)(i - t * nvec);
    float acc[N];
#pragma unroll
    for (int j = 0; j < N; ++j) acc[j] = 0.f;
    for (int s = 0; s < k; ++s) {
      const Vec16<T> a = ld16(in3 + ((t * k + s) * (int64_t)H) + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] += DT<T>::to_f(a.v[j]);
    }
    Vec16<T> o;
    if (residual) {  // the layer's `residual + hidden_states` on the rounded sum (models/mixtral.py:257)
      const Vec16<T> r = ld16(residual + t * H + (int64_t)v * N);
#pragma unroll
      for (int j = 0; j < N; ++j) o.v[j] = DT<T>::from_f(DT<T>::to_f(r.v[j]) + rt<T>(acc[j]));
    } else {
#pragma unroll
      for (int j = 0; j < N; ++j) o.v[j] = DT<T>::from_f(acc[j]);
    }
    st16(out + t * H + (int64_t)v * N, o);
  }
}

static int grid_1d(int64_t items) {
  int64_t b = (items + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  if (b > cap) b = cap;
  return (int)(b < 1 ? 1 : b);
}

static int moe_gemm(int epi, void* out, int64_t ldo, const void* a, const void* w, const int32_t* expert_ids,
                    const int32_t* num_post_pad, const int32_t* sorted_ids, const float* topk_w, int64_t rows_cap,
                    int64_t num_slots, int E, int64_t N, int64_t K, int dtype, uint32_t* status, int tile_cfg,
                    cudaStream_t s) {
  SB_CHECK_ARG(dtype == SB200_BF16 || dtype == SB200_F16, "moe GEMMs support bf16/fp16");
  SB_CHECK_ARG(rows_cap > 0 && rows_cap % kMoeBlockRows == 0, "moe GEMM: the row capacity must be a multiple of %d",
               kMoeBlockRows);
  SB_CHECK_ARG(out && a && w && expert_ids && num_post_pad && E > 0 && N > 0 && K > 0, "moe GEMM: bad arguments");
  // One accumulator per tile and whole tiles only; a tile is one row block of one expert: 128 rows on a single
  // CTA (configurations 1xxx) or 256 rows on a CTA pair (3xxx; each CTA of a pair loads half of the weight tile,
  // and the L2 -> shared-memory feed is what bounds these GEMMs), so the caller aligns the expert blocks to the
  // tile's rows.
  int cfg = tile_cfg;
  if (cfg == 0) {
    const GemmPlan p0 = plan_gemm(epi == EPI_MOE_SCATTER ? EPI_STORE : epi, rows_cap, N, K, 128, 0, 0);
    int bn = p0.bn ? p0.bn : 128;
    cfg = bn + 1000;
  }
  const int mode = (cfg / 1000) % 100;
  SB_CHECK_ARG((mode == 1 || mode == 3) && cfg < 100000,
               "moe GEMM: only whole-tile configurations with one accumulator (1xxx: one CTA, 3xxx: CTA pairs)");
  const int block = mode == 3 ? 2 * kMoeBlockRows : kMoeBlockRows;
  SB_CHECK_ARG(rows_cap % block == 0, "moe GEMM: the row capacity must be a multiple of the %d-row expert blocks", block);
  const GemmPlan plan = plan_gemm(epi == EPI_MOE_SCATTER ? EPI_STORE : epi, rows_cap, N, K, 128, cfg, 0);
  SB_CHECK_ARG(plan.bn != 0 && plan.mi == 1 && plan.cta2 == (mode == 3 ? 1 : 0), "moe GEMM: no tile shape for configuration %d", cfg);
  GemmArgs g = {};
  g.M = (int)rows_cap; g.N = (int)N; g.K = (int)K;
  g.out = out; g.ldo = ldo; g.status = status; g.head_size = 128;
  g.expert_ids = expert_ids; g.num_post_pad = num_post_pad; g.rows_per_expert = (int)N;
  g.sorted_ids = sorted_ids; g.topk_w = topk_w; g.num_slots = (int)num_slots;
  CommView cv = {};
  ReduceArgs ra = {};
  // B = the stacked expert weights seen as one [E * N, K] matrix
  return run_gemm_sm100(dtype, epi, plan, a, K, w, K, g, nullptr, cv, ra, s, (int64_t)E * N);
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_moe_block_rows(void) { return kMoeBlockRows; }

extern "C" int sb200_moe_gather_rows(void* out, const void* x, const int32_t* sorted_ids, const int32_t* num_post_pad,
                                     int64_t rows_cap, int64_t T, int64_t H, int top_k, int dtype,
                                     sb200_stream_t stream) {
  SB_CHECK_ARG(out && x && sorted_ids && num_post_pad && rows_cap >= 0 && T >= 0 && H > 0 && top_k > 0,
               "moe_gather_rows: bad arguments");
  SB_CHECK_ARG((H * dtype_size(dtype)) % 16 == 0 && aligned16(out) && aligned16(x), "moe_gather_rows: rows must be 16-byte multiples");
  if (rows_cap == 0) return SB200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = grid_1d(rows_cap * (H / (16 / (int64_t)dtype_size(dtype))));
  SB_DISPATCH_FLOAT(dtype, (moe_gather_kernel<scalar_t><<<grid, 256, 0, s>>>((scalar_t*)out, (const scalar_t*)x, sorted_ids,
                                                                            num_post_pad, rows_cap, T * top_k, (int)H, top_k)));
  SB_CHECK_LAUNCH("moe_gather_kernel");
  return SB200_OK;
}

extern "C" int sb200_moe_gemm1(void* act_out, const void* xs, const void* w13, const int32_t* expert_ids,
                               const int32_t* num_post_pad, int64_t rows_cap, int E, int64_t two_d, int64_t K, int dtype,
                               uint32_t* status, int tile_cfg, sb200_stream_t stream) {
  SB_CHECK_ARG(two_d % 2 == 0, "moe_gemm1: the stacked gate/up width must be even");
  return moe_gemm(EPI_SILU_MUL, act_out, two_d / 2, xs, w13, expert_ids, num_post_pad, nullptr, nullptr, rows_cap, 0, E,
                  two_d, K, dtype, status, tile_cfg, (cudaStream_t)stream);
}

extern "C" int sb200_moe_gemm2(void* out3, const void* act, const void* w2, const int32_t* expert_ids,
                               const int32_t* num_post_pad, const int32_t* sorted_ids, const float* topk_w,
                               int64_t rows_cap, int64_t num_slots, int E, int64_t H, int64_t d, int dtype,
                               uint32_t* status, int tile_cfg, sb200_stream_t stream) {
  SB_CHECK_ARG(sorted_ids && topk_w && num_slots > 0, "moe_gemm2: bad arguments");
  return moe_gemm(EPI_MOE_SCATTER, out3, H, act, w2, expert_ids, num_post_pad, sorted_ids, topk_w, rows_cap, num_slots, E,
                  H, d, dtype, status, tile_cfg, (cudaStream_t)stream);
}

extern "C" int sb200_moe_sum(void* out, const void* in3, const void* residual, int64_t T, int top_k, int64_t H,
                             int dtype, sb200_stream_t stream) {
  SB_CHECK_ARG(out && in3 && T >= 0 && top_k > 0 && H > 0, "moe_sum: bad arguments");
  SB_CHECK_ARG((H * dtype_size(dtype)) % 16 == 0 && aligned16(out) && aligned16(in3) &&
                   (!residual || aligned16(residual)), "moe_sum: rows must be 16-byte multiples");
  if (T == 0) return SB200_OK;
  cudaStream_t s = (cudaStream_t)stream;
  const int grid = grid_1d(T * (H / (16 / (int64_t)dtype_size(dtype))));
  SB_DISPATCH_FLOAT(dtype, (moe_sum_kernel<scalar_t><<<grid, 256, 0, s>>>((scalar_t*)out, (const scalar_t*)in3,
                                                                         (const scalar_t*)residual, T, top_k, (int)H)));
  SB_CHECK_LAUNCH("moe_sum_kernel");
  return SB200_OK;
}
