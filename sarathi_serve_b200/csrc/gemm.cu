// Host side of the dense projections: TMA descriptors, tile selection, launch
// of the tcgen05 kernel (gemm_sm100.cuh) for bf16/fp16, and a plain FFMA kernel
// for fp32 (the fp32 configuration is a parity case, not a throughput target).
#include "gemm_host.cuh"

#include <mutex>
#include <stdlib.h>

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

// Clusters of `cluster_ctas` GEMM CTAs (one CTA per SM) that can be resident at the same time.  A cluster must
// sit inside one GPC, so this is less than #SMs / cluster_ctas when the GPCs' SM counts are not multiples of the
// cluster size.  It matters for the row-parallel kernel: its CTAs wait, after their tiles, for flags that depend
// on every tile of the launch, so all clusters of a launch must be resident together -- one that is still
// queued behind waiting CTAs would never start.  Asked of the runtime once per device and cluster size; without
// a device (planning on a CPU-only host) the estimate is three quarters of #SMs / cluster_ctas.
static int max_coresident_clusters(int cluster_ctas) {
  static std::mutex mu;
  static int cached[64][17];
  int dev = 0;
  const bool have_dev = cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64;
  if (cluster_ctas < 2 || cluster_ctas > 16) return sm_count();
  if (!have_dev) { cudaGetLastError(); return sm_count() / cluster_ctas * 3 / 4; }
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev][cluster_ctas] > 0) return cached[dev][cluster_ctas];
  auto kern = gemm_sm100_kernel<__nv_bfloat16, EPI_PUSH, true, 1>;
  int n = 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(cluster_ctas * 32);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = kSmemBudget;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster_ctas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = sm_count() / cluster_ctas * 3 / 4;
  }
  cached[dev][cluster_ctas] = n;
  return n;
}

// ------------------------------------------------------------ tile selection
// Analytical choice of (CTA pairing, MI, BN, scheduling): estimated SM clocks of the slowest unit.
//   main loop per k-block = max(tensor time, shared-memory traffic of the stage at 128 B/clk
//   (TMA writes + operand reads of the MMAs), L2 -> shared-memory time of the stage);
//   data-parallel: whole tiles per unit (no fix-up, but units may get unequal tile counts);
//   stream-K: every unit gets the same number of k-blocks and tiles cut along K are summed
//   through the workspace by the last unit to arrive.
GemmPlan plan_gemm(int epi, int64_t M, int64_t N, int64_t K, int head_size, int tile_cfg, size_t ws_bytes, int neox) {
  GemmPlan best = {};
  const int sms = sm_count();
  const int k_blocks = (int)((K + kBK - 1) / kBK);
  const int64_t out_cols = (epi == EPI_SILU_MUL) ? N / 2 : N;
  // explicit configuration: BN + 1000*MODE + 100000*S.  MODE = 1|2: accumulators of one CTA;
  // 3|4: CTA pairs with 1|2 accumulators.  S = 0|1: whole tiles per unit; S >= 2: cut along K so
  // that about S units share a tile.
  int f_bn = 0, f_mode = 0, f_s = 0;
  if (tile_cfg > 0) {
    f_s = tile_cfg / 100000;
    f_mode = (tile_cfg / 1000) % 100;
    f_bn = tile_cfg % 1000;
    if (f_mode == 0) f_mode = 1;
    if (f_s == 0) f_s = 1;
  }
  if (f_mode == 5) {
    // cluster K-split: explicit configurations only (the autotuner times them against the others)
    GemmPlan p = {};
    const int bn = f_bn, sp = f_s;
    const bool rot_ok = epi != EPI_ROTARY || bn % head_size == 0 || (neox && bn < head_size && bn == 64 && head_size % bn == 0);
    const bool shape_ok = bn >= 32 && bn <= 256 && bn % 64 == 0 && (sp == 2 || sp == 4) && rot_ok;
    if (!shape_ok) return p;
    const int m_tiles = (int)((M + 255) / 256);
    const int cols_per_tile = (epi == EPI_SILU_MUL) ? bn / 2 : bn;
    const int n_tiles = (int)((out_cols + cols_per_tile - 1) / cols_per_tile);
    const int64_t tiles = (int64_t)m_tiles * n_tiles;
    const int stages = gemm_max_stages(1, bn, 1);
    // room in every CTA's stage ring for the chunks it sends and the chunks it receives
    const bool split_tile = epi == EPI_ROTARY && bn < head_size;
    const int units_of_tile = (epi == EPI_SILU_MUL || split_tile) ? bn / 64 : bn / 32;
    const size_t exchange = 2 * (size_t)(sp - 1) * xchg_area_bytes(units_of_tile, sp, (epi == EPI_SILU_MUL || epi == EPI_ROTARY) ? 2 : 1);
    if (tiles * 2 * sp > sms || k_blocks < sp || stages < 2 || exchange > (size_t)stages * gemm_stage_bytes(1, bn, 1)) return p;
    // row-parallel kernel: its CTAs wait for one another, so every cluster must be resident; and clusters of
    // four pairs are not used with it (on two ranks that combination left an owner's flag unset in the
    // owner-reduce scheme -- the bounded wait reported it -- while clusters of two pairs pass every case)
    if (epi == EPI_PUSH && (sp != 2 || tiles > max_coresident_clusters(2 * sp))) return p;
    p.cta2 = 1; p.mi = 1; p.bn = bn; p.units = (int)tiles; p.tiles_full = (int)tiles; p.rem_splits = 1; p.rem_units = 0;
    p.stages = stages; p.m_tiles = m_tiles; p.n_tiles = n_tiles; p.k_blocks = k_blocks; p.cluster_split = sp;
    p.est_clocks = 9000.0 + (double)((k_blocks + sp - 1) / sp) * (2.0 * bn > 260.0 ? 2.0 * bn : 260.0) + exchange / 2.0 / 64.0;
    return p;
  }
  double best_cost = 1e30;
  for (int mode = 1; mode <= 4; ++mode) {
    if (f_mode && mode != f_mode) continue;
    const int cta2 = mode >= 3 ? 1 : 0;
    const int mi = cta2 ? mode - 2 : mode;
    for (int bn = 32; bn <= 256; bn += 32) {
      if (f_bn && bn != f_bn) continue;
      // rotary: whole heads per tile, or (NeoX) a 64-column slice of both halves of a head
      if (epi == EPI_ROTARY && bn % head_size != 0 && !(neox && bn < head_size && bn == 64 && head_size % bn == 0)) continue;
      if (epi == EPI_SILU_MUL && bn % 64 != 0) continue;
      if (cta2 && bn % 64 != 0) continue;  // each CTA of a pair keeps bn/2 rows of B: whole 32-column chunks
      if (!f_bn && bn < 64) continue;
      const int stages = gemm_max_stages(mi, bn, cta2);
      if (stages < 2) continue;
      const int bm = (cta2 ? 256 : 128) * mi;
      const int m_tiles = (int)((M + bm - 1) / bm);
      const int cols_per_tile = (epi == EPI_SILU_MUL) ? bn / 2 : bn;
      const int n_tiles = (int)((out_cols + cols_per_tile - 1) / cols_per_tile);
      const int64_t tiles = (int64_t)m_tiles * n_tiles;
      if (!f_mode && bm > 128 && M <= bm / 2) continue;  // half of the tile would be empty
      int units_max = cta2 ? sms / 2 : sms;     // CTAs or CTA pairs that run at once
      if (cta2 && epi == EPI_PUSH && max_coresident_clusters(2) < units_max) units_max = max_coresident_clusters(2);
      const int64_t total = tiles * k_blocks;
      // per-k-block clocks of one SM (constants fitted to the measured times of the full kernels on B200):
      //   one CTA: about 616 clocks per k-block whatever N <= 256 -- not the tensor pipe (the MMA-rate probe of
      //   diag.cu shows N/2 clocks per MMA for one CTA as for a pair) but the operand feed: a single-CTA stage
      //   of 128 + N rows crosses L2 -> shared memory at ~50 B/clk/SM with every SM pulling;
      //   a CTA pair loads half of the B tile per SM and reaches the nominal N/2 clocks per MMA down to a
      //   floor of ~65; its 256x256 tiles are again bound by the feed (64 B/clk needed), and shared memory
      //   itself (fill + operand reads) is modelled too.
      const double stage = gemm_stage_bytes(mi, bn, cta2);
      const double mma_nominal = cta2 ? 2.0 * mi * bn : 616.0 * mi;
      const double mma_floor = cta2 ? 260.0 * mi : 616.0 * mi;
      const double b_rows = cta2 ? bn / 2.0 : bn;
      const double smem_rd = mi * (128 + b_rows) * kBK * 2;
      double per_kb = mma_nominal > mma_floor ? mma_nominal : mma_floor;
      if ((stage + smem_rd) / 100.0 > per_kb) per_kb = (stage + smem_rd) / 100.0;
      if (stage / 50.0 > per_kb) per_kb = stage / 50.0;
      const int64_t busy_sms = (tiles < units_max ? tiles : units_max) * (cta2 ? 2 : 1);
      if (busy_sms > sms / 2) per_kb *= 1.0 + 0.25 * (double)(busy_sms - sms / 2) / (sms / 2);  // L2 contention
      if (mi == 2) per_kb *= 1.4;  // single-buffered accumulators, shallow ring: measured well above the model
      const double epi_units = (mi == 2 ? bn / 32.0 : bn / 64.0);
      const double epi_c = epi_units * 450.0 + 400.0;
      const bool dbuf = mi * bn * 2 <= 512;
      const int64_t G = tiles < units_max ? tiles : units_max;
      const int64_t tiles_full = (tiles / G) * G, rem = tiles - tiles_full;
      const double full_item = dbuf ? (k_blocks * per_kb > epi_c ? k_blocks * per_kb : epi_c) : k_blocks * per_kb + epi_c;
      for (int sp = 1; sp <= 8; ++sp) {  // about sp units share a tile of the last partial round
        if (f_s && sp != f_s) continue;
        const int64_t rem_t = rem ? rem : (tiles < units_max ? tiles : 0);  // fewer tiles than units: all are "the last round"
        const int64_t full_rounds = tiles < units_max ? 0 : tiles_full / G;
        int64_t units = G, gs = rem_t;
        double cost = 9000.0 + (dbuf ? epi_c : 0.0) + full_rounds * full_item;
        if (sp == 1) {
          if (rem_t) cost += full_item;
        } else {
          if (rem_t == 0) continue;  // nothing to cut
          const int64_t W = rem_t * k_blocks;
          gs = rem_t * sp < units_max ? rem_t * sp : units_max;
          if (gs > W / 2) gs = W / 2;          // at least two k-blocks per unit
          if (gs <= rem_t) continue;           // degenerates to whole tiles
          if (!sk_fits_32bit(k_blocks, rem_t, gs)) continue;  // the kernel's scheduling arithmetic is 32-bit
          if (tiles < units_max) units = gs;
          const size_t need = kWsCounterBytes + (size_t)(gs + rem_t) * bm * bn * sizeof(float);
          if (need > ws_bytes || (size_t)rem_t * 32 * sizeof(uint32_t) > kWsCounterBytes) continue;
          const double share = (double)((W + gs - 1) / gs);
          // every range leaves an fp32 partial tile in L2 and reads one tile's worth back (measured ~20 B/clk/SM
          // with all SMs at it); a unit whose range straddles two tiles does that twice
          const double segs = (gs % rem_t == 0) ? 1.0 : 2.0;
          const double fix = 1500.0 + segs * 51.0 * bn;
          cost += share * per_kb + (dbuf ? 300.0 : epi_c) + fix;
        }
        if (cost < best_cost) {
          best_cost = cost;
          best.cta2 = cta2; best.mi = mi; best.bn = bn;
          best.units = (int)units;
          best.tiles_full = (tiles >= units_max) ? (int)tiles_full : 0;
          best.rem_splits = sp; best.rem_units = (int)gs;
          best.stages = stages; best.m_tiles = m_tiles; best.n_tiles = n_tiles; best.k_blocks = k_blocks;
          best.cluster_split = 1;
          best.est_clocks = cost;
        }
      }
    }
  }
  // a forced cut along K that is impossible (workspace too small, or it degenerates to whole tiles)
  if (best.bn == 0 && tile_cfg >= 100000) return plan_gemm(epi, M, N, K, head_size, tile_cfg % 100000, ws_bytes, neox);
  return best;
}

// Arrivals the row-parallel kernel of a rank counts for the rank that owns
// rows [lo, hi): one per (tile, epilogue slot whose 32 rows overlap the range), times the number of
// K-parts for tiles that are cut or split inside a cluster (every part finishes a share of such a tile and
// reports it).
uint32_t gemm_push_increments(const GemmPlan& p, int64_t M, int64_t lo, int64_t hi) {
  if (hi <= lo) return 0;
  const int bm = (p.cta2 ? 256 : 128) * p.mi;
  const uint32_t slots_per_group = p.mi == 1 ? 2u : 1u;  // warps of a tile that cover the same 32 rows
  const int64_t tiles = (int64_t)p.m_tiles * p.n_tiles;
  uint64_t total = 0;
  for (int mt = 0; mt < p.m_tiles; ++mt) {
    const int64_t r0 = (int64_t)mt * bm, r1 = (r0 + bm < M ? r0 + bm : M);
    uint32_t groups = 0;
    for (int64_t g0 = r0; g0 < r1; g0 += 32) {
      const int64_t g1 = (g0 + 32 < r1 ? g0 + 32 : r1);
      if (g0 < hi && g1 > lo) ++groups;
    }
    if (!groups) continue;
    // tiles mt, mt + m_tiles, ... : whole ones below tiles_full, cut ones from there on
    uint64_t weight = 0;
    for (int64_t t = mt; t < tiles; t += p.m_tiles) {
      int first = 0, parts = 1;
      if (t >= p.tiles_full) sk_tile_parts(p.k_blocks, (int)(tiles - p.tiles_full), p.rem_units, (int)(t - p.tiles_full), &first, &parts);
      if (p.cluster_split > 1) parts = p.cluster_split;  // every pair of the cluster finishes a share of the tile
      weight += (uint64_t)parts;
    }
    total += (uint64_t)groups * slots_per_group * weight;
  }
  return (uint32_t)total;
}

// Programmatic dependent launch of the GEMM kernels: off unless SB200_PDL=1.  Measured on the TP=1 layer
// step it gains about 1 us of 244 (only GEMM -> GEMM boundaries overlap, and a CTA of the next kernel cannot
// become resident before a CTA of this one has left its SM), so it is not worth a default.
static bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB200_PDL");
    v = (e && atoi(e) != 0) ? 1 : 0;
  }
  return v != 0;
}

// Distance (k-blocks) of the L2 prefetch of weight boxes; SB200_L2_PREFETCH overrides (0 disables).
static int l2_prefetch_distance() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("SB200_L2_PREFETCH");
    v = e ? atoi(e) : 0;
    if (v < 0) v = 0;
  }
  return v;
}

template <typename T, int EPI, bool CTA2, int MI>
static int launch_sm100(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const CommView& cv,
                        const ReduceArgs& ra, cudaStream_t s) {
  auto kern = gemm_sm100_kernel<T, EPI, CTA2, MI>;
  static thread_local int configured_dev = -1;
  int dev = 0;
  SB_CUDA(cudaGetDevice(&dev));
  if (configured_dev != dev) {
    SB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget));
    configured_dev = dev;
  }
  const int smem = g.stages * gemm_stage_bytes(g.mi, g.bn, CTA2 ? 1 : 0) + kBarrierBytes + kEpiStageBytes + 1024;
  int grid = g.units;
  if (grid < 1) grid = 1;
  const int pairs_per_unit = (CTA2 && g.cluster_split > 1) ? g.cluster_split : 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(CTA2 ? 2 * pairs_per_unit * grid : grid);
  cfg.blockDim = dim3(kGemmThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTA2 ? 2 * pairs_per_unit : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: the prologue (barriers, TMEM, tensor maps) may run while the previous
  // kernel of the stream finishes; the kernel waits for it before its first global access
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  SB_CUDA(cudaLaunchKernelEx(&cfg, kern, ta, tb, g, cv, ra));
  return SB200_OK;
}

template <typename T, int EPI>
static int launch_mode(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const CommView& cv,
                       const ReduceArgs& ra, cudaStream_t s) {
  if (g.cta2) return g.mi == 2 ? launch_sm100<T, EPI, true, 2>(ta, tb, g, cv, ra, s) : launch_sm100<T, EPI, true, 1>(ta, tb, g, cv, ra, s);
  return g.mi == 2 ? launch_sm100<T, EPI, false, 2>(ta, tb, g, cv, ra, s) : launch_sm100<T, EPI, false, 1>(ta, tb, g, cv, ra, s);
}

template <typename T>
static int dispatch_epi(int epi, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g,
                        const CommView& cv, const ReduceArgs& ra, cudaStream_t s) {
  switch (epi) {
    case EPI_STORE: return launch_mode<T, EPI_STORE>(ta, tb, g, cv, ra, s);
    case EPI_ROTARY: return launch_mode<T, EPI_ROTARY>(ta, tb, g, cv, ra, s);
    case EPI_SILU_MUL: return launch_mode<T, EPI_SILU_MUL>(ta, tb, g, cv, ra, s);
    case EPI_PUSH: return launch_mode<T, EPI_PUSH>(ta, tb, g, cv, ra, s);
    case EPI_MOE_SCATTER: return launch_mode<T, EPI_MOE_SCATTER>(ta, tb, g, cv, ra, s);
  }
  set_error("unknown GEMM epilogue %d", epi);
  return SB200_ERR_INVALID_ARGUMENT;
}

int run_gemm_sm100(int dtype, int epi, const GemmPlan& plan, const void* x, int64_t ldx, const void* w, int64_t ldw,
                   GemmArgs g, void* workspace, const CommView& cv, const ReduceArgs& ra, cudaStream_t s,
                   int64_t b_rows) {
  SB_CHECK_ARG(plan.bn != 0, "no GEMM tile shape fits epilogue %d (head_size=%d)", epi, g.head_size);
  g.cta2 = plan.cta2;
  g.mi = plan.mi; g.bn = plan.bn; g.units = plan.units; g.tiles_full = plan.tiles_full;
  g.rem_units = plan.rem_units;
  g.cluster_split = plan.cluster_split > 1 ? plan.cluster_split : 1;
  g.l2_prefetch = l2_prefetch_distance();
  g.stages = plan.stages; g.m_tiles = plan.m_tiles; g.n_tiles = plan.n_tiles; g.k_blocks = plan.k_blocks;
  if (plan.rem_units > (int)((int64_t)plan.m_tiles * plan.n_tiles - plan.tiles_full)) {
    SB_CHECK_ARG(workspace && aligned16(workspace), "cutting tiles along K needs an aligned workspace");
    g.ws_counters = reinterpret_cast<uint32_t*>(workspace);
    g.ws = reinterpret_cast<float*>(reinterpret_cast<char*>(workspace) + kWsCounterBytes);
  }
  CUtensorMap ta, tb;
  int rc = make_tmap_2d(&ta, dtype, x, g.M, g.K, ldx, 128, kBK);
  if (rc) return rc;
  g.rot_split = (epi == EPI_ROTARY && plan.bn < g.head_size) ? 1 : 0;
  rc = make_tmap_2d(&tb, dtype, w, b_rows > 0 ? b_rows : g.N, g.K, ldw,
                    (epi == EPI_SILU_MUL || plan.cta2 || g.rot_split) ? plan.bn / 2 : plan.bn, kBK);
  if (rc) return rc;
  if (dtype == SB200_BF16) return dispatch_epi<__nv_bfloat16>(epi, ta, tb, g, cv, ra, s);
  if (dtype == SB200_F16) return dispatch_epi<__half>(epi, ta, tb, g, cv, ra, s);
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
                                 const void* bias, const void* residual, int64_t ldr, int64_t T, int64_t N, int64_t K,
                                 int dtype, int epilogue,
                                 const sb200_rotary_args* rot, uint32_t* status, int tile_cfg, void* workspace,
                                 int64_t workspace_bytes, sb200_stream_t stream) {
  SB_CHECK_ARG(T >= 0 && N > 0 && K > 0 && T <= INT32_MAX && N <= INT32_MAX && K <= INT32_MAX,
               "gemm_colpar: bad shape T=%lld N=%lld K=%lld", (long long)T, (long long)N, (long long)K);
  if (T == 0) return SB200_OK;
  SB_CHECK_ARG(out && x && w, "gemm_colpar: null pointer");
  SB_CHECK_ARG(epilogue >= SB200_EPI_NONE && epilogue <= SB200_EPI_SILU_MUL, "gemm_colpar: bad epilogue %d", epilogue);
  SB_CHECK_ARG(residual == nullptr || (epilogue == SB200_EPI_NONE && dtype != SB200_F32 && ldr >= N),
               "gemm_colpar: a residual goes with the plain epilogue of the bf16 / fp16 kernel only (ldr >= N)");
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
  g.residual = residual; g.ldr = ldr;
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
    if (rot->kv_cache) {
      const int64_t kvc = (int64_t)rot->num_kv_heads * rot->head_size;
      SB_CHECK_ARG(rot->kv_slots && rot->kv_page_size > 0 && rot->num_kv_heads > 0 && kvc <= rot->rot_cols &&
                       rot->rot_cols + kvc <= N && aligned16(rot->kv_cache),
                   "gemm_colpar: fused KV-cache append needs slots, a page size, and k / v column blocks of "
                   "num_kv_heads * head_size columns at [rot_cols - that, rot_cols + that)");
      g.kv_cache = rot->kv_cache; g.kv_slots = rot->kv_slots; g.kv_page_size = rot->kv_page_size;
      g.kv_cols = (int)kvc; g.q_cols = rot->rot_cols - (int)kvc;
    }
    epi = EPI_ROTARY;
  } else if (epilogue == SB200_EPI_SILU_MUL) {
    SB_CHECK_ARG(bias == nullptr, "gemm_colpar: silu_and_mul epilogue does not take a bias");
    SB_CHECK_ARG(N % 2 == 0, "gemm_colpar: silu_and_mul epilogue needs an even N");
    epi = EPI_SILU_MUL;
  }
  CommView cv = {};
  ReduceArgs ra = {};
  const GemmPlan plan = plan_gemm(epi, T, N, K, g.head_size, tile_cfg, workspace ? (size_t)workspace_bytes : 0,
                                  epi == EPI_ROTARY ? g.is_neox : 1);
  return run_gemm_sm100(dtype, epi, plan, x, ldx, w, ldw, g, workspace, cv, ra, s);
}

#ifdef SB200_TRACE
// profiling builds only: the phase time stamps (ns) CTA 0 of the last 64 GEMM launches recorded, and the launch count
extern "C" int sb200_debug_gemm_trace(unsigned long long* host_out /*[64][16]*/, unsigned int* launches) {
  SB_CUDA(cudaDeviceSynchronize());
  SB_CUDA(cudaMemcpyFromSymbol(host_out, g_gemm_trace, sizeof(unsigned long long) * 64 * 16));
  SB_CUDA(cudaMemcpyFromSymbol(launches, g_gemm_trace_launch, sizeof(unsigned int)));
  return SB200_OK;
}
#endif

// The tile shape and schedule sb200_gemm_colpar / sb200_gemm_rowpar would use (for tuning and tests).
// out[0..11] = cta2, mi, bn, units, tiles_full, rem_splits, rem_units, stages, m_tiles, n_tiles, k_blocks, cluster_split.
extern "C" int sb200_gemm_plan(int epilogue, int64_t T, int64_t N, int64_t K, int head_size, int tile_cfg,
                               int64_t workspace_bytes, int* out) {
  SB_CHECK_ARG(out != nullptr && T > 0 && N > 0 && K > 0, "gemm_plan: bad arguments");
  const int epi = epilogue == SB200_EPI_ROTARY ? EPI_ROTARY : epilogue == SB200_EPI_SILU_MUL ? EPI_SILU_MUL
                  : epilogue == 3 ? EPI_PUSH : EPI_STORE;
  const GemmPlan p = plan_gemm(epi, T, N, K, head_size ? head_size : 128, tile_cfg, (size_t)workspace_bytes);
  const int v[12] = {p.cta2, p.mi, p.bn, p.units, p.tiles_full, p.rem_splits, p.rem_units, p.stages, p.m_tiles,
                     p.n_tiles, p.k_blocks, p.cluster_split > 1 ? p.cluster_split : 1};
  for (int i = 0; i < 12; ++i) out[i] = v[i];
  return p.bn ? SB200_OK : SB200_ERR_UNSUPPORTED;
}

// Arrivals the row-parallel kernel of one rank counts for the owner of rows [lo, hi) under the schedule
// sb200_gemm_plan reports for (T, N, K, tile_cfg) -- what sb200_gemm_rowpar writes into the kernel's
// expected counts.  Host-only, for tests of that bookkeeping; no counterpart in the reference.
extern "C" int64_t sb200_gemm_rowpar_arrivals(int64_t T, int64_t N, int64_t K, int tile_cfg, int64_t workspace_bytes,
                                              int64_t lo, int64_t hi) {
  if (T <= 0 || N <= 0 || K <= 0) return -1;
  const GemmPlan p = plan_gemm(EPI_PUSH, T, N, K, 128, tile_cfg, (size_t)workspace_bytes);
  if (!p.bn) return -1;
  return (int64_t)gemm_push_increments(p, T, lo, hi);
}
