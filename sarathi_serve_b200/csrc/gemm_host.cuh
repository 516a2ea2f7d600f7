// Host-side declarations shared by gemm.cu (launch logic) and comm.cu (the
// row-parallel entry point builds its GemmArgs/ReduceArgs and calls in here).
#pragma once

#include "gemm_sm100.cuh"

namespace sb200 {

int make_tmap_2d(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int64_t cols, int64_t ld_elems,
                 int box_rows, int box_cols);
int choose_bn(int epi, int64_t M, int64_t N, int head_size, int tile_n);
int run_gemm_sm100(int dtype, int epi, int tile_n, const void* x, int64_t ldx, const void* w, int64_t ldw, GemmArgs g,
                   const CommView& cv, const ReduceArgs& ra, cudaStream_t s);
int run_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* B, int64_t ldb, const float* bias,
                 int M, int N, int K, cudaStream_t s);

}  // namespace sb200
