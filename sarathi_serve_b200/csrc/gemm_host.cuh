// Host-side declarations shared by gemm.cu (launch logic) and comm.cu (the
// row-parallel entry point builds its GemmArgs/ReduceArgs and calls in here).
#pragma once

#include "gemm_sm100.cuh"

namespace sb200 {

int make_tmap_2d(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int64_t cols, int64_t ld_elems,
                 int box_rows, int box_cols);
// First bytes of a split-K workspace hold the per-(tile, slot) arrival counters (zero between launches).
constexpr size_t kWsCounterBytes = 64 * 1024;

struct GemmPlan {
  int cta2, mi, bn, units, tiles_full;
  int rem_splits;  // S of the tile configuration: about S units share a tile of the last partial round
  int rem_units;   // units the k-blocks of that round are spread over (= its tiles when nothing is cut)
  int stages, m_tiles, n_tiles, k_blocks;
  int cluster_split;  // > 1: one tile per cluster of that many CTA pairs, K split between the pairs (MODE 5)
  double est_clocks;
};
// tile_cfg: 0 = choose; else BN + 1000*MODE + 100000*S (MODE 1|2: one CTA, 3|4: CTA pairs; S >= 2: the tiles of the last partial round are cut along K so that about S units share one; MODE 5: CTA pairs, every tile computed by a cluster of S = 2 or 4 pairs that split its k-blocks and combine their accumulators through distributed shared memory -- for problems with at most #SMs / (2 S) tiles).  ws_bytes: split-K workspace available (0 = none).
GemmPlan plan_gemm(int epi, int64_t M, int64_t N, int64_t K, int head_size, int tile_cfg, size_t ws_bytes, int neox = 1);
uint32_t gemm_push_increments(const GemmPlan& p, int64_t M, int64_t lo, int64_t hi);
int run_gemm_sm100(int dtype, int epi, const GemmPlan& plan, const void* x, int64_t ldx, const void* w, int64_t ldw,
                   GemmArgs g, void* workspace, const CommView& cv, const ReduceArgs& ra, cudaStream_t s,
                   int64_t b_rows = 0);  // b_rows: rows of the B matrix when it is taller than g.N (stacked experts)
int run_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* B, int64_t ldb, const float* bias,
                 int M, int N, int K, cudaStream_t s);

}  // namespace sb200
