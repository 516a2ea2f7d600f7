// Host side of the dense projections: TMA descriptors, tile selection, launch
// of the tcgen05 kernel (gemm_sm100.cuh) for bf16/fp16, and a plain FFMA kernel
// for fp32 (the fp32 configuration is a parity case, not a throughput target).
#include "gemm_host.cuh"

#include <mutex>

namespace sb200 {

// ------------------------------------------------------- driver entry point
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* map, int dtype, const void* ptr, int64_t rows, int64_t cols, int64_t ld_elems,
                 int box_rows, int box_cols) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    set_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    return SB200_ERR_CUDA;
  }
  const size_t es = dtype_size(dtype);
  SB_CHECK_ARG(aligned16(ptr), "GEMM operand pointer %p is not 16-byte aligned", ptr);
  SB_CHECK_ARG((ld_elems * es) % 16 == 0, "GEMM operand row stride (%lld elements) is not a multiple of 16 bytes",
               (long long)ld_elems);
  SB_CHECK_ARG(rows > 0 && cols > 0 && ld_elems >= cols, "GEMM operand shape rows=%lld cols=%lld ld=%lld",
               (long long)rows, (long long)cols, (long long)ld_elems);
  const CUtensorMapDataType dt = dtype == SB200_BF16  ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                 : dtype == SB200_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)(ld_elems * es)};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  const CUresult r = fn(map, dt, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("cuTensorMapEncodeTiled failed with CUresult %d (rows=%lld cols=%lld ld=%lld box=%dx%d)", (int)r,
              (long long)rows, (long long)cols, (long long)ld_elems, box_rows, box_cols);
    return SB200_ERR_CUDA;
  }
  return SB200_OK;
}

// ------------------------------------------------------------ tile selection
int choose_bn(int epi, int64_t M, int64_t N, int head_size, int tile_n) {
  const int64_t m_tiles = (M + kBM - 1) / kBM;
  const int sms = sm_count();
  auto allowed = [&](int bn) {
    if (epi == EPI_ROTARY) return bn % head_size == 0;
    return true;
  };
  if (tile_n == 64 || tile_n == 128 || tile_n == 256) return allowed(tile_n) ? tile_n : 0;
  // Largest tile that still gives every SM a tile; otherwise the smallest allowed tile.
  const int cands[3] = {256, 128, 64};
  int smallest = 0;
  for (int bn : cands) {
    if (!allowed(bn)) continue;
    smallest = bn;
    const int64_t cols_per_tile = (epi == EPI_SILU_MUL) ? bn / 2 : bn;
    const int64_t out_cols = (epi == EPI_SILU_MUL) ? N / 2 : N;
    const int64_t tiles = m_tiles * ((out_cols + cols_per_tile - 1) / cols_per_tile);
    if (tiles >= sms) return bn;
  }
  return smallest;
}

template <typename T, int BN, int EPI>
static int launch_sm100(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const CommView& cv,
                        const ReduceArgs& ra, cudaStream_t s) {
  using S = GemmSmem<BN>;
  auto kern = gemm_sm100_kernel<T, BN, EPI>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal));
    configured_dev = dev;
  }
  const int tiles = g.m_tiles * g.n_tiles;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (EPI == EPI_PUSH && grid < 1) grid = 1;
  kern<<<grid, kGemmThreads, S::kTotal, s>>>(ta, tb, g, cv, ra);
  SB_CHECK_LAUNCH("gemm_sm100_kernel");
  return SB200_OK;
}

template <typename T, int EPI>
static int dispatch_bn(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const CommView& cv,
                       const ReduceArgs& ra, cudaStream_t s) {
  switch (bn) {
    case 64: return launch_sm100<T, 64, EPI>(ta, tb, g, cv, ra, s);
    case 128: return launch_sm100<T, 128, EPI>(ta, tb, g, cv, ra, s);
    case 256: return launch_sm100<T, 256, EPI>(ta, tb, g, cv, ra, s);
  }
  set_error("unsupported GEMM tile width %d", bn);
  return SB200_ERR_UNSUPPORTED;
}

template <typename T>
static int dispatch_epi(int epi, int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g,
                        const CommView& cv, const ReduceArgs& ra, cudaStream_t s) {
  switch (epi) {
    case EPI_STORE: return dispatch_bn<T, EPI_STORE>(bn, ta, tb, g, cv, ra, s);
    case EPI_ROTARY: return dispatch_bn<T, EPI_ROTARY>(bn, ta, tb, g, cv, ra, s);
    case EPI_SILU_MUL: return dispatch_bn<T, EPI_SILU_MUL>(bn, ta, tb, g, cv, ra, s);
    case EPI_PUSH: return dispatch_bn<T, EPI_PUSH>(bn, ta, tb, g, cv, ra, s);
  }
  set_error("unknown GEMM epilogue %d", epi);
  return SB200_ERR_INVALID_ARGUMENT;
}

int run_gemm_sm100(int dtype, int epi, int tile_n, const void* x, int64_t ldx, const void* w, int64_t ldw,
                   GemmArgs g, const CommView& cv, const ReduceArgs& ra, cudaStream_t s) {
  const int bn = choose_bn(epi, g.M, g.N, g.head_size, tile_n);
  SB_CHECK_ARG(bn != 0, "no GEMM tile width fits epilogue %d (head_size=%d, tile_n=%d)", epi, g.head_size, tile_n);
  const int out_cols_per_tile = (epi == EPI_SILU_MUL) ? bn / 2 : bn;
  const int64_t out_cols = (epi == EPI_SILU_MUL) ? g.N / 2 : g.N;
  g.m_tiles = (g.M + kBM - 1) / kBM;
  g.n_tiles = (int)((out_cols + out_cols_per_tile - 1) / out_cols_per_tile);
  g.k_blocks = (g.K + kBK - 1) / kBK;
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, dtype, x, g.M, g.K, ldx, kBM, kBK);
  if (rc) return rc;
  rc = make_tmap_2d(&tb, dtype, w, g.N, g.K, ldw, (epi == EPI_SILU_MUL) ? bn / 2 : bn, kBK);
  if (rc) return rc;
  if (dtype == SB200_BF16) return dispatch_epi<__nv_bfloat16>(epi, bn, ta, tb, g, cv, ra, s);
  if (dtype == SB200_F16) return dispatch_epi<__half>(epi, bn, ta, tb, g, cv, ra, s);
  set_error("tcgen05 GEMM supports bf16/fp16 only");
  return SB200_ERR_UNSUPPORTED;
}

// --------------------------------------------------------------- fp32 (FFMA)
// C[M,N] = A[M,K] * B[N,K]^T (+bias), 64x64 tiles, 4x4 outputs per thread.
__global__ void __launch_bounds__(256)
gemm_f32_kernel(float* __restrict__ C, int64_t ldc, const float* __restrict__ A, int64_t lda,
                const float* __restrict__ B, int64_t ldb, const float* __restrict__ bias, int M, int N, int K) {
  __shared__ float sa[16][64 + 1], sb[16][64 + 1];
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = threadIdx.x; i < 64 * 16; i += 256) {
      const int r = i >> 4, kk = i & 15;
      sa[kk][r] = (m0 + r < M && k0 + kk < K) ? A[(int64_t)(m0 + r) * lda + k0 + kk] : 0.f;
      sb[kk][r] = (n0 + r < N && k0 + kk < K) ? B[(int64_t)(n0 + r) * ldb + k0 + kk] : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = sa[kk][ty * 4 + i]; b[i] = sb[kk][tx * 4 + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int m = m0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (m < M && n < N) C[(int64_t)m * ldc + n] = acc[i][j] + (bias ? bias[n] : 0.f);
    }
}

int run_gemm_f32(float* C, int64_t ldc, const float* A, int64_t lda, const float* B, int64_t ldb, const float* bias,
                 int M, int N, int K, cudaStream_t s) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  gemm_f32_kernel<<<grid, 256, 0, s>>>(C, ldc, A, lda, B, ldb, bias, M, N, K);
  SB_CHECK_LAUNCH("gemm_f32_kernel");
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_gemm_colpar(void* out, int64_t ldo, const void* x, int64_t ldx, const void* w, int64_t ldw,
                                 const void* bias, int64_t T, int64_t N, int64_t K, int dtype, int epilogue,
                                 const sb200_rotary_args* rot, uint32_t* status, int tile_n, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && N > 0 && K > 0 && T <= INT32_MAX && N <= INT32_MAX && K <= INT32_MAX,
               "gemm_colpar: bad shape T=%lld N=%lld K=%lld", (long long)T, (long long)N, (long long)K);
  if (T == 0) return SB200_OK;
  SB_CHECK_ARG(out && x && w, "gemm_colpar: null pointer");
  SB_CHECK_ARG(epilogue >= SB200_EPI_NONE && epilogue <= SB200_EPI_SILU_MUL, "gemm_colpar: bad epilogue %d", epilogue);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SB200_F32) {
    SB_CHECK_ARG(epilogue == SB200_EPI_NONE, "gemm_colpar: fp32 supports only the plain epilogue (compose the "
                 "rotary / silu_and_mul kernels after it)");
    return run_gemm_f32((float*)out, ldo, (const float*)x, ldx, (const float*)w, ldw, (const float*)bias, (int)T,
                        (int)N, (int)K, s);
  }
  GemmArgs g = {};
  g.M = (int)T; g.N = (int)N; g.K = (int)K;
  g.out = out; g.ldo = ldo; g.bias = bias; g.status = status;
  g.head_size = 128;
  int epi = EPI_STORE;
  if (epilogue == SB200_EPI_ROTARY) {
    SB_CHECK_ARG(rot && rot->positions && rot->cos_sin_cache, "gemm_colpar: rotary epilogue needs positions and cache");
    SB_CHECK_ARG(bias == nullptr, "gemm_colpar: rotary epilogue does not take a bias");
    SB_CHECK_ARG(rot->rot_dim == rot->head_size, "gemm_colpar: fused rotary needs rot_dim == head_size");
    SB_CHECK_ARG(rot->head_size == 64 || rot->head_size == 128 || rot->head_size == 256,
                 "gemm_colpar: fused rotary supports head_size 64/128/256, got %d", rot->head_size);
    SB_CHECK_ARG(rot->rot_cols % rot->head_size == 0 && rot->rot_cols <= N && N % rot->head_size == 0,
                 "gemm_colpar: rot_cols=%d / N=%lld must be multiples of head_size", rot->rot_cols, (long long)N);
    SB_CHECK_ARG(aligned16(rot->cos_sin_cache), "gemm_colpar: cos_sin_cache must be 16-byte aligned");
    g.positions = rot->positions; g.cos_sin = rot->cos_sin_cache; g.head_size = rot->head_size;
    g.rot_cols = rot->rot_cols; g.is_neox = rot->is_neox;
    epi = EPI_ROTARY;
  } else if (epilogue == SB200_EPI_SILU_MUL) {
    SB_CHECK_ARG(bias == nullptr, "gemm_colpar: silu_and_mul epilogue does not take a bias");
    SB_CHECK_ARG(N % 2 == 0, "gemm_colpar: silu_and_mul epilogue needs an even N");
    epi = EPI_SILU_MUL;
  }
  CommView cv = {};
  ReduceArgs ra = {};
  return run_gemm_sm100(dtype, epi, tile_n, x, ldx, w, ldw, g, cv, ra, s);
}
