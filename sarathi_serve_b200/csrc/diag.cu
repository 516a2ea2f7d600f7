// Measurement of the tcgen05.mma issue / completion rate on the current GPU: the two constants the tile
// planner of gemm.cu is built on (clocks per MMA of a single CTA, M = 128, and of a CTA pair, M = 256, as a
// function of N).  Both operands sit in shared memory for the whole run -- nothing is loaded inside the
// timed loop, so the figure is the tensor pipe's, not the operand feed's.  One thread issues `iters`
// k-blocks of four MMAs (K = 16 each) into one accumulator and commits once at the end; the clock is read
// before the first issue, after the last issue and after the commit has arrived.
// No counterpart in the reference (its GEMMs are cuBLAS calls).
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sb200 {

constexpr int kDiagStage = 48 * 1024;  // A tile (128 x 64 bf16) at offset 0, B tile (<= 256 x 64) at 16 KiB

template <bool PAIR>
__global__ void __launch_bounds__(128, 1) mma_rate_kernel(long long* out, int N, int iters) {
  extern __shared__ __align__(1024) uint8_t diag_smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)diag_smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t final_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag_s;
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
  for (int i = threadIdx.x; i < 4 * kDiagStage / 4; i += blockDim.x) ((uint32_t*)smem)[i] = 0;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&final_bar, 1);
    abort_flag_s = 0;
    ptx::mbar_fence_init();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncthreads();
  if (threadIdx.x < 32) {
    if (PAIR) { ptx::tmem_alloc_pair(&tmem_slot, 512); ptx::tmem_relinquish_pair(); }
    else      { ptx::tmem_alloc(&tmem_slot, 512);      ptx::tmem_relinquish(); }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();
  ptx::tc_fence_after();
  const uint32_t tmem = tmem_slot;
  volatile int* abort_flag = &abort_flag_s;
  if (threadIdx.x == 0) {
    long long t0 = clock64(), t1 = t0;
    if (rank == 0) {
      const uint32_t idesc = ptx::make_idesc(1, N, PAIR ? 256 : 128);
      for (int it = 0; it < iters; ++it) {
        const uint32_t sa = ptx::smem_u32(smem + (size_t)(it & 3) * kDiagStage);
        const uint64_t da = ptx::make_smem_desc_sw128(sa), db = ptx::make_smem_desc_sw128(sa + 16384);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          if (PAIR) ptx::umma_f16_pair(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, acc);
          else ptx::umma_f16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, acc);
        }
      }
      if (PAIR) ptx::umma_commit_pair(&final_bar); else ptx::umma_commit(&final_bar);
      t1 = clock64();
    }
    const bool ok = ptx::mbar_wait(&final_bar, 0, abort_flag);  // (both CTAs of a pair: the commit arrives on both)
    const long long t2 = clock64();
    if (rank == 0) { out[0] = t1 - t0; out[1] = ok ? t2 - t0 : -1; }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (PAIR) ptx::cluster_sync_all();
  if (threadIdx.x < 32) {
    ptx::tc_fence_after();
    if (PAIR) ptx::tmem_dealloc_pair(tmem, 512); else ptx::tmem_dealloc(tmem, 512);
  }
}

template <bool PAIR>
static int run_mma_rate(int n, int iters, long long* dev_out, cudaStream_t s) {
  auto kern = mma_rate_kernel<PAIR>;
  const int smem = 4 * kDiagStage + 1024;
  SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(PAIR ? 2 : 1);
  cfg.blockDim = dim3(128);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = PAIR ? 2 : 1;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kern, dev_out, n, iters));
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int sb200_diag_mma_rate(int pair, int n, int iters, int64_t* dev_clocks, sb200_stream_t stream) {
  SB_CHECK_ARG(n >= 16 && n <= 256 && n % 16 == 0 && (!pair || n % 32 == 0), "diag_mma_rate: N must be a multiple of 16 (32 for pairs) in [16, 256]");
  SB_CHECK_ARG(iters > 0 && iters <= (1 << 20) && dev_clocks, "diag_mma_rate: bad arguments");
  static_assert(sizeof(long long) == sizeof(int64_t), "clock type");
  return pair ? run_mma_rate<true>(n, iters, (long long*)dev_clocks, (cudaStream_t)stream)
              : run_mma_rate<false>(n, iters, (long long*)dev_clocks, (cudaStream_t)stream);
}
