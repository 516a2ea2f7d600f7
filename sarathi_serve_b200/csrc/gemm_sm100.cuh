// Persistent, warp-specialised bf16/fp16 GEMM for sm_100a:
//   C[M, N] = A[M, K] * B[N, K]^T        (both operands K-major, fp32 accumulate)
// TMA (128-byte swizzle) feeds a multi-stage shared-memory ring, one elected
// thread issues tcgen05.mma into TMEM accumulators, and eight epilogue warps
// drain TMEM with tcgen05.ld.  Row-major nn.Linear weights [out, in] are
// consumed as the K-major B operand as they are.
//
// Tile shape is a run-time choice of the host (gemm.cu):
//   BM = 128 * MI rows  (MI = 1 or 2 accumulators that share every B tile: with
//                        MI = 2 each weight byte crosses L2 -> shared memory
//                        half as often per flop); 256 * MI rows for CTA pairs,
//   BN = 32..256 columns in steps of 32 (UMMA N),
//   scheduling: whole tiles go round-robin to the G scheduling units (CTAs or
//        CTA pairs) for as many full rounds as there are; the tiles of the
//        last, partial round (all tiles, when there are fewer than G) can be
//        cut along K into S parts so that they still occupy all units.  Every
//        part leaves an fp32 partial tile in a workspace, and the last one to
//        arrive (per 32-row slot) sums the parts in part order and runs the
//        epilogue.  So neither wave quantisation nor a small tile count leaves
//        SMs idle, and the result does not depend on arrival order.
// When MI * BN <= 256 the accumulators are double buffered in TMEM and the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Roles (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..9 = epilogue.  Epilogue warp w may read TMEM lanes 32*(w%4)..+31
// (rows of a 128-row accumulator); the two warps that share a lane quarter
// split the work by accumulator (MI = 2) or by alternating work units (MI = 1).
//
// Epilogues (the reference ops they absorb are cited where they are defined):
//   EPI_STORE    out = acc (+ bias)
//   EPI_ROTARY   qkv projection: rotary embedding applied to the q and k heads
//   EPI_SILU_MUL gate_up projection: out[:, j] = silu(gate_j) * up_j
//   EPI_PUSH     row-parallel projection: partial rows go to this rank's heap;
//                the reduce / residual / norm / gather phases of comm.cuh run in
//                the same kernel after the tiles.
//   EPI_MOE_SCATTER  second expert GEMM: row r of the expert-sorted activations is scaled by its
//                routed weight and stored at its (token, k) slot.
// Grouped (mixture-of-experts) mode: when `expert_ids` is set, the rows of A are the
// expert-sorted, block-padded slots of moe_align_block_size (block = tile rows), tile row block
// mt uses the weights of expert expert_ids[mt] (B rows offset by expert * rows_per_expert), and
// row blocks at or beyond *num_post_pad are skipped.
#pragma once

#include "comm.cuh"
#include "sm100_ptx.cuh"

namespace sb200 {

#ifdef SB200_TRACE
// profiling builds: CTA 0 of every GEMM launch records %globaltimer at its phase boundaries, launch after launch
// (slot = launch ordinal modulo 64); read back with sb200_debug_gemm_trace.
__device__ unsigned long long g_gemm_trace[64][16];
__device__ unsigned int g_gemm_trace_launch;
#define SB_GEMM_MARK(slot)                                                                          \
  do {                                                                                              \
    if (blockIdx.x == 0) {                                                                          \
      unsigned long long t__;                                                                       \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__) :: "memory");                           \
      g_gemm_trace[gemm_trace_row % 64][slot] = t__;                                                \
    }                                                                                               \
  } while (0)
#else
#define SB_GEMM_MARK(slot) do { } while (0)
#endif

enum GemmEpilogue { EPI_STORE = 0, EPI_ROTARY = 1, EPI_SILU_MUL = 2, EPI_PUSH = 3, EPI_MOE_SCATTER = 4 };

constexpr int kBK = 64;            // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int kGemmThreads = 320;  // 10 warps
constexpr int kEpiWarps = 8;
constexpr int kSmemBudget = 226 * 1024;  // dynamic shared memory requested (static use is a few bytes)
constexpr int kBarrierBytes = 1024;
constexpr int kEpiWarpStageBytes = 32 * 64;  // per epilogue warp: 32 rows x 32 sixteen-bit values, to transpose stores
constexpr int kEpiStageBytes = 8 * kEpiWarpStageBytes;

struct GemmArgs {
  int M, N, K;             // N counts B rows (for EPI_SILU_MUL: 2*d)
  void* out;               // [M, ldo] (EPI_SILU_MUL: [M, d])
  int64_t ldo;
  const void* bias;        // [N] or null (EPI_STORE only)
  const void* residual;    // [M, ldr] or null (EPI_STORE only): out = residual + round(acc (+ bias))
  int64_t ldr;
  // EPI_ROTARY
  const int64_t* positions;
  const void* cos_sin;     // [max_pos, rot_dim], same dtype as the output
  int head_size;
  int rot_cols;            // columns [0, rot_cols) hold q and k heads, the rest (v) is stored as is
  int is_neox;
  // EPI_ROTARY, optional: the k and v columns of the qkv row are ALSO stored into the paged KV cache
  void* kv_cache;            // [pages, 2, page_size, kv_heads, head_dim] of T, or null
  const int64_t* kv_slots;   // [M] row of the cache seen as [pages * 2 * page_size, kv_cols] for token i's key (-1: skip)
  int kv_page_size;
  int q_cols, kv_cols;       // output columns [q_cols, q_cols + kv_cols) are k, the next kv_cols are v
  int rot_split;           // EPI_ROTARY with bn < head_size (NeoX only): a tile holds bn/2 columns of the first half
                           // of a head followed by the matching bn/2 columns of its second half, so that every
                           // rotation pair (i, i + head_size/2) sits in one accumulator
  // tiling (host-chosen)
  int mi;                  // accumulators per tile (BM = 128 * mi)
  int bn;                  // tile columns
  int units;               // G: scheduling units launched (CTAs, or CTA pairs)
  int tiles_full;          // tiles handed out whole, round-robin (a multiple of units)
  int rem_units;           // units that share the k-blocks of the remaining tiles (= their number: tiles not cut)
  int stages;              // shared-memory ring depth
  int l2_prefetch;         // k-blocks ahead at which the B boxes are prefetched into L2 (0 = off)
  int m_tiles, n_tiles, k_blocks;
  // grouped (MoE) mode
  const int32_t* expert_ids;    // [m_tiles] expert of each row block, or null
  const int32_t* num_post_pad;  // [1] rows in use (device value)
  int rows_per_expert;          // B rows per expert
  const int32_t* sorted_ids;    // EPI_MOE_SCATTER: [rows] (token, k) slot of each sorted row (>= num_slots: padding)
  const float* topk_w;          // EPI_MOE_SCATTER: [num_slots] routed weight of each slot
  int num_slots;
  float* ws;               // partial-tile workspace: [cut tiles * S][BM][bn] fp32
  uint32_t* ws_counters;   // [cut tiles][arrived[16], done[16]], zero between launches
  int cta2;                // 1: tiles of 256 rows computed by CTA pairs (cta_group::2)
  int cluster_split;       // > 1 (CTA pairs, one accumulator, one tile per unit): a cluster of that many CTA pairs
                           // computes ONE tile, pair p the p-th share of its k-blocks; the fp32 accumulators of pairs
                           // 1.. travel to pair 0 through distributed shared memory and pair 0 runs the epilogue
  uint32_t* status;        // device word: first error of this launch (0 = none); may be null
};

// Shared memory of one pipeline stage in one CTA (a CTA of a pair keeps half of the B tile).
__host__ __device__ inline int gemm_stage_bytes(int mi, int bn, int cta2 = 0) {
  return cta2 ? (mi * 128 + bn / 2) * kBK * 2 : (mi * 128 + bn) * kBK * 2;
}
// Cluster K-split: bytes of one pair's share of an accumulator (its units, `chunks_per_unit` 16 KiB chunks each);
// a CTA needs 2 * (split - 1) such areas inside its stage ring (what it sends, what it receives).
__host__ __device__ inline uint32_t xchg_area_bytes(int units, int split, int chunks_per_unit) {
  return (uint32_t)((units + split - 1) / split * chunks_per_unit) * (uint32_t)(128 * 32 * sizeof(float));
}
__host__ __device__ inline int gemm_max_stages(int mi, int bn, int cta2 = 0) {
  int s = (kSmemBudget - kBarrierBytes - kEpiStageBytes - 1024) / gemm_stage_bytes(mi, bn, cta2);
  return s > 8 ? 8 : s;
}

template <typename T> struct Pack2;
template <> struct Pack2<__nv_bfloat16> {
  __device__ __forceinline__ static uint32_t pack(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};
template <> struct Pack2<__half> {
  __device__ __forceinline__ static uint32_t pack(float a, float b) {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
};

// Store 32 consecutive output elements of one row (values already final, fp32).
template <typename T>
__device__ __forceinline__ void store_row32(T* dst, const float* f, int valid_cols, bool vec_ok) {
  if (valid_cols >= 32 && vec_ok) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 u;
      u.x = Pack2<T>::pack(f[q * 8 + 0], f[q * 8 + 1]);
      u.y = Pack2<T>::pack(f[q * 8 + 2], f[q * 8 + 3]);
      u.z = Pack2<T>::pack(f[q * 8 + 4], f[q * 8 + 5]);
      u.w = Pack2<T>::pack(f[q * 8 + 6], f[q * 8 + 7]);
      *reinterpret_cast<uint4*>(dst + q * 8) = u;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < valid_cols) dst[j] = DT<T>::from_f(f[j]);
  }
}

// The same store done by the whole warp.  After a TMEM load a thread holds 32 values of ITS row, so a plain
// per-thread store makes every 16-byte store instruction of the warp touch 32 different 128-byte lines (the
// epilogue of a 128x128 tile then spends ~2000 clocks in the load/store unit).  Here the warp transposes the
// 32 x 64-byte block through its private 2 KiB of shared memory (16-byte chunk c of row r kept at
// c ^ ((r >> 1) & 3): conflict-free both ways) and stores it so that four lanes cover one row's 64 bytes.
// Called by all 32 lanes; `row_ok` = this lane's row is to be stored, `dst` = its first element.
template <typename T>
__device__ __forceinline__ void warp_store_rows32(uint8_t* stage, T* dst, const float* f, int valid_cols, bool vec_ok,
                                                  bool row_ok) {
  const int lane = threadIdx.x & 31;
  if (valid_cols >= 32 && vec_ok) {  // warp-uniform
    const uint32_t sbase = ptx::smem_u32(stage);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const uint32_t a = sbase + (uint32_t)(lane * 64 + ((q ^ ((lane >> 1) & 3)) << 4));
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(Pack2<T>::pack(f[q * 8 + 0], f[q * 8 + 1])),
                   "r"(Pack2<T>::pack(f[q * 8 + 2], f[q * 8 + 3])), "r"(Pack2<T>::pack(f[q * 8 + 4], f[q * 8 + 5])),
                   "r"(Pack2<T>::pack(f[q * 8 + 6], f[q * 8 + 7]))
                   : "memory");
    }
    const unsigned ok_mask = __ballot_sync(0xffffffffu, row_ok);  // (also orders the shared-memory stores above)
    __syncwarp();
    const int chunk = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = i * 8 + (lane >> 2);
      uint4 v;
      const uint32_t a = sbase + (uint32_t)(row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4));
      asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a) : "memory");
      T* p = reinterpret_cast<T*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(dst), row));
      if ((ok_mask >> row) & 1u) *reinterpret_cast<uint4*>(p + chunk * 8) = v;
    }
    __syncwarp();  // the block is read before the warp's next unit overwrites it
  } else if (row_ok) {
    store_row32<T>(dst, f, valid_cols, false);
  }
}

template <typename T>
__device__ __forceinline__ void load_row32(const T* src, float* f) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const Vec16<T> v = ld16(src + q * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[q * 8 + j] = DT<T>::to_f(v.v[j]);
  }
}

// Where an epilogue warp gets the fp32 accumulator chunk (32 columns of its row) from.
struct TmemSource {
  uint32_t row_addr;  // TMEM address of (lane quarter, first column of the accumulator)
  __device__ __forceinline__ void load32(int col, float* f, int /*chunk_of_unit*/ = 0) const {
    uint32_t r[32];
    ptx::tmem_ld_32x32(row_addr + (uint32_t)col, r);
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
  }
};
// Cluster K-split: this pair's accumulator chunk (TMEM) plus the partial accumulators the other pairs of the
// cluster copied into this CTA's shared memory.  An exchanged chunk is a block of [128 rows][32 fp32] = 16 KiB
// (a warp's 32 rows: 4 KiB of it) with the 16-byte pieces of a row permuted (piece j of row r at j ^ (r & 7)):
// the 32 lanes of a warp hold 32 consecutive rows, so its 16-byte accesses touch every bank once per quarter
// warp.  Parts are added in the order of their pairs: the result does not depend on timing.
constexpr uint32_t kXchgChunkBytes = 128 * 32 * sizeof(float);
struct TmemPlusSmemSource {
  uint32_t row_addr;
  const uint8_t* sm;   // this thread's row in the first chunk of the unit, first source pair
  int parts;           // partials in shared memory (cluster_split - 1)
  uint32_t part_bytes; // distance between the source pairs' areas
  __device__ __forceinline__ void load32(int col, float* f, int chunk_of_unit) const {
    uint32_t r[32];
    ptx::tmem_ld_32x32(row_addr + (uint32_t)col, r);
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
    const int sw = (int)(threadIdx.x & 7);
    for (int p = 0; p < parts; ++p) {
      const uint8_t* rowp = sm + (size_t)p * part_bytes + (size_t)chunk_of_unit * kXchgChunkBytes;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float4 v = *reinterpret_cast<const float4*>(rowp + ((j ^ sw) << 4));
        f[4 * j] += v.x; f[4 * j + 1] += v.y; f[4 * j + 2] += v.z; f[4 * j + 3] += v.w;
      }
    }
  }
};
// Scheduling.  Tiles are numbered M-fastest.  With G scheduling units (CTAs or CTA pairs):
//   * the first `tiles_full` tiles (a multiple of G) are handed out round-robin, whole: unit p
//     computes tiles p, p+G, ...  Neighbouring units then work on the M-tiles of the same
//     weight tile at the same time, so a weight tile comes from HBM once and hits in L2 after;
//   * the k-blocks of the remaining R = `rem_tiles` tiles (R < G) form one sequence of
//     W = R * k_blocks items that is cut into Gs >= R equal ranges, one per unit p < Gs:
//     unit p gets [p*W/Gs, (p+1)*W/Gs), which touches one or two tiles.  A tile touched by
//     S > 1 units is "cut": each of them leaves an fp32 partial tile in a workspace slot, and
//     once all S have arrived every one of them sums the slots (in part order) and finishes
//     its share of the tile.  Gs = R: whole tiles, nothing is cut.
// A unit stores the partials of all its ranges before it waits for anybody else's, so the waits
// cannot form a cycle.
struct Sched {
  int G, tiles_full, rem_tiles, Gs, k_blocks;
  int rounds;  // tiles_full / G: whole-tile work items of every unit
};
struct Segment {
  int tile, kb0, kb1;
  int parts;       // units this tile is shared by (1: whole)
  int part_slot;   // workspace slot of this part; the tile's parts are slots first_slot .. first_slot+parts-1
  int first_slot;
  int rem_index;   // index of the tile among the remaining tiles (selects its arrival counters)
  bool valid;
};
// Unit whose range holds item x of the W remaining k-blocks: the p with floor(p*W/Gs) <= x < floor((p+1)*W/Gs).
__host__ __device__ inline int sk_unit_of(long long W, int Gs, long long x) {
  return (int)(((x + 1) * Gs - 1) / W);
}
// First unit and number of units that share remaining tile rt.
__host__ __device__ inline void sk_tile_parts(int k_blocks, int rem_tiles, int Gs, int rt, int* first_unit, int* parts) {
  const long long W = (long long)rem_tiles * k_blocks;
  const int pf = sk_unit_of(W, Gs, (long long)rt * k_blocks);
  const int pl = sk_unit_of(W, Gs, (long long)(rt + 1) * k_blocks - 1);
  *first_unit = pf;
  *parts = pl - pf + 1;
}
// True when the device-side scheduling arithmetic below, which runs in 32 bits (a 64-bit division costs
// the one thread that feeds the pipeline about 0.1 us, and there were six of them on the way to the
// first load), cannot overflow for this plan.
__host__ __device__ inline bool sk_fits_32bit(long long k_blocks, long long rem_tiles, long long Gs) {
  return (rem_tiles + 1) * k_blocks * (Gs + 1) < (1ll << 31);
}
// it-th work item of unit p.
__device__ __forceinline__ Segment segment_of(const Sched& sc, int p, int it) {
  Segment sg;
  sg.valid = true;
  sg.kb0 = 0; sg.kb1 = sc.k_blocks; sg.parts = 1; sg.part_slot = 0; sg.first_slot = 0; sg.rem_index = 0;
  if (it < sc.rounds) {
    sg.tile = p + it * sc.G;
    return sg;
  }
  sg.valid = false;
  if (p >= sc.Gs || sc.rem_tiles == 0) return sg;
  if (sc.Gs == sc.rem_tiles) {  // nothing is cut: unit p has the whole remaining tile p
    if (it > sc.rounds) return sg;
    sg.valid = true;
    sg.tile = sc.tiles_full + p;
    sg.rem_index = p; sg.first_slot = sg.part_slot = 2 * p;
    return sg;
  }
  const unsigned kbs = (unsigned)sc.k_blocks, Gs = (unsigned)sc.Gs;
  const unsigned W = (unsigned)sc.rem_tiles * kbs;
  const unsigned b0 = (unsigned)p * W / Gs, b1 = (unsigned)(p + 1) * W / Gs;
  const unsigned rt = b0 / kbs + (unsigned)(it - sc.rounds);
  if (rt >= (unsigned)sc.rem_tiles) return sg;
  const unsigned t0 = rt * kbs;
  const unsigned lo = b0 > t0 ? b0 : t0, hi = b1 < t0 + kbs ? b1 : t0 + kbs;
  if (lo >= hi) return sg;
  const unsigned pf = ((t0 + 1u) * Gs - 1u) / W, pl = ((t0 + kbs) * Gs - 1u) / W;  // sk_tile_parts in 32 bits
  sg.valid = true;
  sg.tile = sc.tiles_full + (int)rt;
  sg.kb0 = (int)(lo - t0);
  sg.kb1 = (int)(hi - t0);
  sg.parts = (int)(pl - pf + 1u);
  sg.first_slot = (int)(pf + rt);
  sg.part_slot = p + (int)rt;
  sg.rem_index = (int)rt;
  return sg;
}
// True when some tile of this launch is cut along K (its parts meet in the workspace).
__device__ __forceinline__ bool has_cut_tiles(const Sched& sc) { return sc.Gs > sc.rem_tiles; }

// Partial tiles are kept column-major in the workspace ([BN columns][BM rows] fp32): the 32 lanes
// of an epilogue warp hold 32 consecutive rows, so every load / store instruction of a warp moves
// one full 128-byte line and the 32 instructions of a chunk are independent of each other.
struct WorkspaceSource {
  const float* ws;       // first slot of the tile's parts, at this thread's row
  size_t slot_stride;    // floats per slot (BM * BN)
  int bm;                // rows of the tile = stride between columns
  int parts;
  __device__ __forceinline__ void load32(int col, float* f, int /*chunk_of_unit*/ = 0) const {
#pragma unroll
    for (int j = 0; j < 32; ++j) f[j] = 0.f;
    int i = 0;
    for (; i + 1 < parts; i += 2) {  // two parts in flight; the order of the additions stays 0, 1, 2, ...
      const float* p0 = ws + (size_t)i * slot_stride + (size_t)col * bm;
      const float* p1 = p0 + slot_stride;
      float a[32], b[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) { a[j] = __ldcg(p0 + (size_t)j * bm); b[j] = __ldcg(p1 + (size_t)j * bm); }
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = (f[j] + a[j]) + b[j];
    }
    if (i < parts) {
      const float* p0 = ws + (size_t)i * slot_stride + (size_t)col * bm;
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] += __ldcg(p0 + (size_t)j * bm);
    }
  }
};

// Per-thread view of the tile being finished.
template <typename T> struct RowCtx {
  int gm;          // global row of this thread
  bool row_ok;
  int n0;          // first global output column of the tile (for SILU_MUL: first column of d)
  T* out_row;      // out + gm * ldo   (EPI_PUSH: the owner's partial slot row)
  const T* cs;     // rotary: cache row of this token
  const T* res_row;  // EPI_STORE: residual + gm * ldr, or null
  T* kv_row;       // EPI_ROTARY: this token's key row in the paged KV cache, or null
  bool vec_ok;
  float scale;     // EPI_MOE_SCATTER: routed weight of this row's slot
  uint8_t* stage;  // this warp's block of shared memory for warp_store_rows32
};

// Work units of a tile: the chunks an epilogue warp fetches together.
//   STORE / PUSH : unit u = columns [32u, 32u+32)
//   SILU_MUL     : unit u = gate columns [32u, ..) with up columns [bn/2 + 32u, ..)
//   ROTARY       : unit u -> (head = u / upH, j = u % upH), upH = head_size/32 units per head;
//                  for a NeoX-rotated head only j < upH/2 does work (chunks j and j + upH/2).
// (EPI_MOE_SCATTER uses the units of STORE.)
template <int EPI> __device__ __forceinline__ int num_units(const GemmArgs& g) {
  return (EPI == EPI_SILU_MUL || (EPI == EPI_ROTARY && g.rot_split)) ? g.bn / 64 : g.bn / 32;
}
// First output column of tile column block nt.  A split rotary tile (see GemmArgs::rot_split) starts at
// column j * bn/2 of its head and continues at head_size/2 + j * bn/2.
template <int EPI> __device__ __forceinline__ int tile_first_col(const GemmArgs& g, int nt) {
  if (EPI == EPI_SILU_MUL) return nt * (g.bn / 2);
  if (EPI == EPI_ROTARY && g.rot_split) {
    const int tph = g.head_size / g.bn;  // tiles per head
    return (nt / tph) * g.head_size + (nt % tph) * (g.bn / 2);
  }
  return nt * g.bn;
}

// Columns (inside the accumulator) a unit reads; returns how many chunks (0, 1 or 2).
template <int EPI>
__device__ __forceinline__ int unit_chunks(const GemmArgs& g, int n0, int u, int* cols) {
  if (EPI == EPI_SILU_MUL) {
    cols[0] = u * 32;
    cols[1] = g.bn / 2 + u * 32;
    return 2;
  }
  if (EPI == EPI_ROTARY && g.rot_split) {
    cols[0] = u * 32;
    cols[1] = g.bn / 2 + u * 32;
    return 2;
  }
  if (EPI == EPI_ROTARY) {
    const int upH = g.head_size / 32;
    const int head = u / upH, j = u - head * upH;
    const bool rotate = (n0 + head * g.head_size) < g.rot_cols;
    if (rotate && g.is_neox) {
      if (j >= upH / 2) return 0;
      cols[0] = head * g.head_size + j * 32;
      cols[1] = cols[0] + g.head_size / 2;
      return 2;
    }
    cols[0] = u * 32;
    return 1;
  }
  cols[0] = u * 32;
  return 1;
}

// qkv projection with the KV-cache append fused in: the 32 final values of output columns [gn, gn + 32)
// of this thread's token also go to the token's slot of the paged cache when they are k or v columns
// (what flashinfer's append_paged_kv_cache does after the reference's `.contiguous()` copies,
// attention/flashinfer_attention_wrapper.py:253-270).  Head sizes are multiples of 32, so a chunk never
// straddles the k / v boundary.
template <typename T>
__device__ __forceinline__ void store_kv32(const GemmArgs& g, const RowCtx<T>& rc, int gn, const float* f) {
  if (!g.kv_cache || gn < g.q_cols || gn >= g.q_cols + 2 * g.kv_cols) return;  // warp-uniform
  const int c = gn - g.q_cols;
  T* dst = nullptr;
  if (rc.kv_row) dst = c < g.kv_cols ? rc.kv_row + c : rc.kv_row + (int64_t)g.kv_page_size * g.kv_cols + (c - g.kv_cols);
  warp_store_rows32<T>(rc.stage, dst, f, 32, true, rc.row_ok && dst != nullptr);
}

// Finish one unit: fetch its chunk(s) from `src`, apply the epilogue math, store.  Called by all lanes of a warp
// (rows beyond M take part in the loads and in the cooperative store, and store nothing).
template <typename T, int EPI, typename Source>
__device__ __forceinline__ void finish_unit(const GemmArgs& g, const RowCtx<T>& rc, const Source& src, int u) {
  int cols[2];
  const int nch = unit_chunks<EPI>(g, rc.n0, u, cols);
  if (nch == 0) return;
  float a[32];
  src.load32(cols[0], a, 0);  // warp-uniform (TMEM loads are .sync.aligned)
  const int gn = rc.n0 + cols[0];  // the unit's first output column: the same for all lanes
  if constexpr (EPI == EPI_MOE_SCATTER) {
    // Reference: the second fused_moe_kernel launch multiplies the fp32 accumulator by the routed
    // weight before rounding to T (layers/fused_moe/fused_moe.py:130-147, MUL_ROUTED_WEIGHT).
    if (gn < g.N) {
#pragma unroll
      for (int j = 0; j < 32; ++j) a[j] *= rc.scale;
      warp_store_rows32<T>(rc.stage, rc.out_row + gn, a, g.N - gn, rc.vec_ok, rc.row_ok);
    }
  } else if constexpr (EPI == EPI_STORE || EPI == EPI_PUSH) {
    if (gn < g.N) {
      if (EPI == EPI_STORE && g.bias && rc.row_ok) {
        const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (gn + j < g.N) a[j] += DT<T>::to_f(bias[gn + j]);
      }
      if (EPI == EPI_STORE && rc.res_row) {  // (null for rows beyond M)
        // Reference: hidden_states = residual + hidden_states on the rounded projection output
        // (models/llama.py:248,254): one more operator result of the 16-bit type.
        if (g.N - gn >= 32 && rc.vec_ok && ((g.ldr & 7) == 0) && aligned16(g.residual)) {
          float r[32];
          load_row32<T>(rc.res_row + gn, r);
#pragma unroll
          for (int j = 0; j < 32; ++j) a[j] = rt<T>(r[j] + rt<T>(a[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (gn + j < g.N) a[j] = rt<T>(DT<T>::to_f(rc.res_row[gn + j]) + rt<T>(a[j]));
        }
      }
      warp_store_rows32<T>(rc.stage, rc.out_row + gn, a, g.N - gn, rc.vec_ok, rc.row_ok);
    }
  } else if constexpr (EPI == EPI_SILU_MUL) {
    // Reference: gate_up = F.linear(x) rounded to T, then silu_and_mul
    // (csrc/activation_kernels.cu:8-25): out = (T)(silu(gate)) * up.
    float b[32];
    src.load32(cols[1], b, 1);
    const int d = g.N / 2;
    if (gn < d) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float gte = rt<T>(a[j]), up = rt<T>(b[j]);
        const float sl = rt<T>(gte / (1.0f + expf(-gte)));
        a[j] = rt<T>(sl * up);
      }
      warp_store_rows32<T>(rc.stage, rc.out_row + gn, a, d - gn, rc.vec_ok, rc.row_ok);
    }
  } else {  // EPI_ROTARY
    // Reference: F.linear output rounded to T (tensor_parallel/layers.py:278-284), then
    // rotary_embedding in T arithmetic on the q and k heads (csrc/pos_encoding_kernels.cu:8-76).
    if (nch == 2) {  // NeoX pair of chunks: x = global columns gn.., y = x + head_size/2
      float b[32];
      src.load32(cols[1], b, 1);
      if (gn < g.N) {
        const int half = g.head_size / 2;
        const int in_head = gn % g.head_size;  // (whole-head tiles: = cols[0] % head_size)
        if (gn - in_head < g.rot_cols && rc.row_ok) {  // a q or k head; the v heads of a split tile are stored as they are
          float co[32], si[32];
          load_row32<T>(rc.cs + in_head, co);
          load_row32<T>(rc.cs + half + in_head, si);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float x = rt<T>(a[j]), y = rt<T>(b[j]);
            a[j] = rt<T>(rt<T>(x * co[j]) - rt<T>(y * si[j]));
            b[j] = rt<T>(rt<T>(y * co[j]) + rt<T>(x * si[j]));
          }
        }
        warp_store_rows32<T>(rc.stage, rc.out_row + gn, a, g.N - gn, rc.vec_ok, rc.row_ok);
        warp_store_rows32<T>(rc.stage, rc.out_row + gn + half, b, g.N - gn - half, rc.vec_ok, rc.row_ok);
        store_kv32<T>(g, rc, gn, a);
        store_kv32<T>(g, rc, gn + half, b);
      }
    } else if (gn < g.N) {
      const int head0 = (cols[0] / g.head_size) * g.head_size;
      if ((rc.n0 + head0) < g.rot_cols && rc.row_ok) {  // GPT-J style: pairs (2i, 2i+1), cos/sin index = column_in_head / 2
        const int half = g.head_size / 2;
        const int in_head = cols[0] - head0;
#pragma unroll
        for (int j = 0; j < 32; j += 2) {
          const int p = (in_head + j) >> 1;
          const float co = DT<T>::to_f(rc.cs[p]), si = DT<T>::to_f(rc.cs[half + p]);
          const float x = rt<T>(a[j]), y = rt<T>(a[j + 1]);
          a[j] = rt<T>(rt<T>(x * co) - rt<T>(y * si));
          a[j + 1] = rt<T>(rt<T>(y * co) + rt<T>(x * si));
        }
      }
      warp_store_rows32<T>(rc.stage, rc.out_row + gn, a, g.N - gn, rc.vec_ok, rc.row_ok);
      store_kv32<T>(g, rc, gn, a);
    }
  }
}

// Per-thread context of the rows an epilogue warp finishes.
template <typename T, int EPI>
__device__ __forceinline__ RowCtx<T> make_row_ctx(const GemmArgs& g, const CommView& comm, const ReduceArgs& red,
                                                  int gm, int n0, uint8_t* stage) {
  RowCtx<T> rc;
  rc.stage = stage;
  rc.gm = gm;
  rc.row_ok = gm < g.M;
  rc.n0 = n0;
  rc.cs = nullptr;
  rc.res_row = nullptr;
  rc.kv_row = nullptr;
  rc.scale = 1.f;
  if constexpr (EPI == EPI_MOE_SCATTER) {
    int slot = g.num_slots;
    if (rc.row_ok) slot = g.sorted_ids[gm];
    rc.row_ok = rc.row_ok && slot < g.num_slots;  // padding rows produce nothing
    rc.out_row = reinterpret_cast<T*>(g.out) + (size_t)(rc.row_ok ? slot : 0) * g.ldo;
    rc.vec_ok = ((g.ldo & 7) == 0) && aligned16(g.out);
    if (rc.row_ok) rc.scale = g.topk_w[slot];
  } else if constexpr (EPI == EPI_PUSH) {
    // the partial [T, N] of this rank stays in its own heap; the owners of the rows come and read it
    rc.out_row = reinterpret_cast<T*>(partial_of(comm, comm.rank, call_number(comm))) + (size_t)gm * (size_t)g.N;
    rc.vec_ok = (g.N & 7) == 0;
  } else {
    rc.out_row = reinterpret_cast<T*>(g.out) + (size_t)gm * g.ldo;
    rc.vec_ok = ((g.ldo & 7) == 0) && aligned16(g.out);
    if (EPI == EPI_STORE && g.residual && rc.row_ok)
      rc.res_row = reinterpret_cast<const T*>(g.residual) + (size_t)gm * g.ldr;
    if (EPI == EPI_ROTARY && rc.row_ok) {
      rc.cs = reinterpret_cast<const T*>(g.cos_sin) + g.positions[gm] * g.head_size;
      if (g.kv_cache) {
        const int64_t slot = g.kv_slots[gm];
        if (slot >= 0) rc.kv_row = reinterpret_cast<T*>(g.kv_cache) + slot * (int64_t)g.kv_cols;
      }
    }
  }
  return rc;
}

// Row-parallel projection: the 32 rows starting at r_lo of some tile are final in this rank's partial
// region.  Called by all lanes of the storing warp: one arrival per owner of those rows.
__device__ __forceinline__ void push_rows_done(const CommView& comm, const ReduceArgs& red, const GemmArgs& g, int r_lo) {
  const int r_hi = min(g.M, r_lo + 32) - 1;
  if (r_hi < r_lo) return;  // warp-uniform
  if (red.one_shot || red.use_mc) { signal_push_all(comm, red); return; }
  __syncwarp();
  if ((threadIdx.x & 31) == 0)
    for (int o = r_lo / red.rows_per_rank; o <= r_hi / red.rows_per_rank; ++o) signal_push(comm, red, o);
}

// ---------------------------------------------------------------------------
// The kernel.  `comm` / `red` are used only by EPI_PUSH.
//   CTA2 = false: one CTA per tile of 128*MI x BN.
//   CTA2 = true : a cluster of two CTAs per tile of 256 x BN (tcgen05 cta_group::2): CTA r of the
//                 pair loads rows [128r, 128r+128) of the A tile and rows [r*BN/2, (r+1)*BN/2) of the
//                 B tile, the even CTA issues the MMAs for both, each CTA drains its own 128
//                 accumulator rows.  Per SM this halves the shared-memory traffic of the B operand.
template <typename T, int EPI, bool CTA2, int MI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const __grid_constant__ GemmArgs g, const __grid_constant__ CommView comm,
                  const __grid_constant__ ReduceArgs red) {
  constexpr uint32_t kTmemCols = 512;
  const int BN = g.bn;  // (MI is a template parameter: the MMA issue loop must be fully unrolled)
  const int BM = (CTA2 ? 256 : 128) * MI;        // rows of a tile
  const int b_rows = CTA2 ? BN / 2 : BN;         // B rows this CTA keeps in shared memory
  const int a_bytes = MI * 128 * kBK * 2;
  const int stage_bytes = a_bytes + b_rows * kBK * 2;
  const int kStages = g.stages;
  const bool dbuf = (MI * BN * 2) <= (int)kTmemCols;  // room for two sets of accumulators
  const uint32_t idesc = ptx::make_idesc(DT<T>::id == SB200_BF16 ? 1 : 0, BN, CTA2 ? 256 : 128);
  const uint32_t crank = CTA2 ? ptx::cluster_ctarank() : 0u;  // rank in the cluster: pair p = ranks (2p, 2p+1)
  const uint32_t cta_rank = crank & 1u;                        // rank inside the pair
  const uint32_t pair_base = crank & ~1u;                      // cluster rank of this pair's leader
  const bool leader = cta_rank == 0;
  const int ks = (CTA2 && g.cluster_split > 1) ? g.cluster_split : 1;  // CTA pairs per tile (cluster K-split)
  const int kpart = (int)(crank >> 1);                                 // which share of the k-blocks this pair computes
  const int ctas_per_unit = CTA2 ? 2 * ks : 1;
  const int unit_id = (int)blockIdx.x / ctas_per_unit;                 // CTA, CTA pair or cluster of pairs
  const int num_units_grid = (int)gridDim.x / ctas_per_unit;
  const uint16_t pair_mask = (uint16_t)(3u << pair_base);
  // the k-blocks of a work item this pair runs (all of them unless the cluster splits K)
  auto kb_lo = [&](const Segment& sg) { return ks > 1 ? sg.kb0 + (int)((long long)(sg.kb1 - sg.kb0) * kpart / ks) : sg.kb0; };
  auto kb_hi = [&](const Segment& sg) { return ks > 1 ? sg.kb0 + (int)((long long)(sg.kb1 - sg.kb0) * (kpart + 1) / ks) : sg.kb1; };

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)kStages * stage_bytes);
  uint64_t* empty_bar = full_bar + 8;
  uint64_t* tmem_full = empty_bar + 8;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;  // [2]
  uint64_t* xchg_bar = tmem_empty + 2;    // cluster K-split: bytes of the other pairs' partials landing here
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xchg_bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // each epilogue warp's block for the transposing stores (warps 0 and 1 never use theirs)
  uint8_t* epi_stage = smem + (size_t)kStages * stage_bytes + kBarrierBytes + (size_t)((threadIdx.x >> 5) >= 2 ? (threadIdx.x >> 5) - 2 : 0) * kEpiWarpStageBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#ifdef SB200_TRACE
  __shared__ unsigned int gemm_trace_row_s;
  if (blockIdx.x == 0 && threadIdx.x == 0) gemm_trace_row_s = atomicAdd(&g_gemm_trace_launch, 1u);
  unsigned int gemm_trace_row = 0;
  if (threadIdx.x == 0) { gemm_trace_row = gemm_trace_row_s; SB_GEMM_MARK(0); }
#endif
  if constexpr (EPI == EPI_PUSH) trace_mark(red, 0);
  // this unit's work items
  Sched sc;
  sc.G = num_units_grid;
  sc.tiles_full = g.tiles_full;
  sc.rem_tiles = g.m_tiles * g.n_tiles - g.tiles_full;
  sc.Gs = g.rem_units;
  sc.k_blocks = g.k_blocks;
  sc.rounds = g.tiles_full / num_units_grid;
  // Every CTA of this persistent grid is resident from the start, so the next kernel of the stream may be
  // scheduled onto SMs as they become free (its prologue then overlaps this kernel's tail).
  ptx::grid_launch_dependents();

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&tmem_full[b], 1);
      ptx::mbar_init(&tmem_empty[b], CTA2 ? 2 * kEpiWarps : kEpiWarps);  // one arrival per epilogue warp (of both CTAs)
    }
    ptx::mbar_init(xchg_bar, 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    if (CTA2) { ptx::tmem_alloc_pair(tmem_slot, kTmemCols); ptx::tmem_relinquish_pair(); }
    else      { ptx::tmem_alloc(tmem_slot, kTmemCols);      ptx::tmem_relinquish(); }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (CTA2) ptx::cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
#ifdef SB200_TRACE
  gemm_trace_row = gemm_trace_row_s;
  if (threadIdx.x == 0) SB_GEMM_MARK(1);  // prologue done
#endif
  // Nothing above touched global memory: from here on the kernel reads what earlier kernels of the stream wrote.
  ptx::grid_dependency_wait();
  if (threadIdx.x == 0) SB_GEMM_MARK(10);  // after the dependency wait
  // grouped mode: rows of A in use (a device value written by moe_align_block_size earlier in the stream)
  const int rows_in_use = g.expert_ids ? min(g.M, *g.num_post_pad) : g.M;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      SB_GEMM_MARK(14);  // producer entered
      for (int it = 0; ok; ++it) {
        const Segment sg = segment_of(sc, unit_id, it);
        if (!sg.valid) break;
        if (it == 0) SB_GEMM_MARK(15);  // first segment known
        const int mt = sg.tile % g.m_tiles, nt = sg.tile / g.m_tiles;
        int b_row0 = 0;  // grouped mode: first B row of this row block's expert
        if (g.expert_ids) {
          if (mt * BM >= rows_in_use) continue;  // row block beyond the padded slots: every role skips it
          b_row0 = g.expert_ids[mt] * g.rows_per_expert;
        }
        const int p_kb1 = kb_hi(sg);
        for (int kb = kb_lo(sg); kb < p_kb1; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          if (kb == kb_lo(sg) && it == 0) SB_GEMM_MARK(11);  // stage 0 free, about to request it
          uint8_t* sa = stage_base + (size_t)stage * stage_bytes;
          uint8_t* sb = sa + a_bytes;
          const bool halves = (EPI == EPI_SILU_MUL) || (EPI == EPI_ROTARY && g.rot_split);  // B tile = two row blocks
          const int b_first = tile_first_col<EPI>(g, nt);                                  // first row of the first block
          const int b_second = b_first + (EPI == EPI_SILU_MUL ? g.N / 2 : g.head_size / 2);  // ... of the second
          if (g.l2_prefetch > 0 && kb + g.l2_prefetch < p_kb1 && !(EPI == EPI_ROTARY && g.rot_split)) {
            // weights are read once: start their trip from HBM to L2 a few stages early
            const int pk = (kb + g.l2_prefetch) * kBK;
            if (CTA2) {
              ptx::tma_prefetch_l2_2d(&tmap_b, pk, (EPI == EPI_SILU_MUL) ? (int)cta_rank * (g.N / 2) + nt * (BN / 2)
                                                                        : nt * BN + (int)cta_rank * (BN / 2));
            } else {
              ptx::tma_prefetch_l2_2d(&tmap_b, pk, (EPI == EPI_SILU_MUL) ? nt * (BN / 2) : nt * BN);
              if (EPI == EPI_SILU_MUL) ptx::tma_prefetch_l2_2d(&tmap_b, pk, g.N / 2 + nt * (BN / 2));
            }
          }
          if constexpr (CTA2) {
            // both CTAs' bytes are counted on the leader's barrier; only the leader announces them
            const uint32_t bar = ptx::map_to_cta(ptx::smem_u32(&full_bar[stage]), pair_base);
            if (leader) ptx::mbar_expect_tx(&full_bar[stage], (uint32_t)(2 * stage_bytes));
#pragma unroll
            for (int a = 0; a < MI; ++a)  // accumulator a covers tile rows [256a, 256a+256): this CTA's half of them
              ptx::tma_load_2d_pair(sa + a * (128 * kBK * 2), &tmap_a, bar, kb * kBK, mt * BM + a * 256 + (int)cta_rank * 128);
            if (halves)  // even CTA: gate rows (first half of the head), odd CTA: the matching up rows (second half)
              ptx::tma_load_2d_pair(sb, &tmap_b, bar, kb * kBK, b_row0 + (cta_rank ? b_second : b_first));
            else
              ptx::tma_load_2d_pair(sb, &tmap_b, bar, kb * kBK, b_row0 + nt * BN + (int)cta_rank * (BN / 2));
          } else {
            ptx::mbar_expect_tx(&full_bar[stage], (uint32_t)stage_bytes);
#pragma unroll
            for (int a = 0; a < MI; ++a)
              ptx::tma_load_2d(sa + a * (128 * kBK * 2), &tmap_a, &full_bar[stage], kb * kBK, mt * BM + a * 128);
            if (halves) {
              // B tile = BN/2 rows of the gate shard followed by the matching BN/2 rows of the up shard
              // (rotary: of the first and of the second half of the head)
              ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, b_row0 + b_first);
              ptx::tma_load_2d(sb + (BN / 2) * (kBK * 2), &tmap_b, &full_bar[stage], kb * kBK, b_row0 + b_second);
            } else {
              ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, b_row0 + nt * BN);
            }
          }
          if (kb == kb_lo(sg) && it == 0) SB_GEMM_MARK(2);  // first stage requested
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
      SB_GEMM_MARK(3);  // last stage requested
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0 && leader) {
      int stage = 0;
      uint32_t phase = 0;
      int used = 0;  // tiles actually computed (selects the TMEM buffer)
      bool ok = true;
      for (int it = 0; ok; ++it) {
        const Segment sg = segment_of(sc, unit_id, it);
        if (!sg.valid) break;
        if (g.expert_ids && (sg.tile % g.m_tiles) * BM >= rows_in_use) continue;
        const int local = used++;
        const int kb0 = kb_lo(sg), kb1 = kb_hi(sg);
        const int buf = dbuf ? (local & 1) : 0;
        const uint32_t use = (uint32_t)(dbuf ? (local >> 1) : local);  // earlier uses of this buffer
        if (!ptx::mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * MI * BN);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          if (kb == kb0 && it == 0) SB_GEMM_MARK(4);  // first stage arrived
          const uint32_t sa = ptx::smem_u32(stage_base + (size_t)stage * stage_bytes);
          const uint64_t db = ptx::make_smem_desc_sw128(sa + a_bytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzle row: +2 in 16-byte units
            const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
#pragma unroll
            for (int a = 0; a < MI; ++a) {
              const uint64_t da = ptx::make_smem_desc_sw128(sa + a * (128 * kBK * 2));
              if (CTA2) ptx::umma_f16_pair(d_tmem + (uint32_t)(a * BN), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, acc);
              else ptx::umma_f16(d_tmem + (uint32_t)(a * BN), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, acc);
            }
          }
          // frees the smem stage (in both CTAs of a pair) once these MMAs have read it
          if (CTA2) ptx::umma_commit_pair_mask(&empty_bar[stage], pair_mask); else ptx::umma_commit(&empty_bar[stage]);
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {  // accumulators complete
          if (CTA2) ptx::umma_commit_pair_mask(&tmem_full[buf], pair_mask); else ptx::umma_commit(&tmem_full[buf]);
        }
        SB_GEMM_MARK(5);  // last MMA issued
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;            // TMEM lane quarter this warp may read
    const int hsel = (warp - 2) >> 2;  // 0 or 1: which of the two warps of this quarter
    const int slot = (int)cta_rank * 8 + hsel * 4 + q;  // split-K arrival slot of this warp
    const int U = num_units<EPI>(g);
    const int a0 = (MI == 2) ? hsel : 0;                   // accumulator this warp drains
    const int row_in_tile = (CTA2 ? a0 * 256 + (int)cta_rank * 128 : a0 * 128) + q * 32 + lane;
    const int u_first = (MI == 2) ? 0 : hsel, u_step = (MI == 2) ? 1 : 2;
    const uint32_t empty_remote = CTA2 ? ptx::map_to_cta(ptx::smem_u32(&tmem_empty[0]), pair_base) : 0u;
    int used = 0;
    bool ok = true;
    for (int it = 0; ok && ks == 1; ++it) {  // (a cluster K-split finishes its one tile after the role branches)
      const Segment sg = segment_of(sc, unit_id, it);
      if (!sg.valid) break;
      const int tile = sg.tile, S = sg.parts;
      const int mt = tile % g.m_tiles, nt = tile / g.m_tiles;
      if (g.expert_ids && mt * BM >= rows_in_use) continue;
      const int local = used++;
      const int buf = dbuf ? (local & 1) : 0;
      const uint32_t use = (uint32_t)(dbuf ? (local >> 1) : local);
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&tmem_full[buf], use & 1u, abort_flag) ? 1 : 0) != 0;
      if (!ok) break;  // warp-uniform: no lane is left behind in an aligned tcgen05.ld
      ptx::tc_fence_after();
      if (warp == 2 && lane == 0) SB_GEMM_MARK(6);  // accumulators complete (seen by the epilogue)

      const int n0 = tile_first_col<EPI>(g, nt);
      const RowCtx<T> rc = make_row_ctx<T, EPI>(g, comm, red, mt * BM + row_in_tile, n0, epi_stage);
      const TmemSource tsrc{tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)((buf * MI + a0) * BN)};
      if (S == 1) {
        for (int u = u_first; u < U; u += u_step) finish_unit<T, EPI>(g, rc, tsrc, u);
      } else {
        // the tile is cut along K: leave this part in its workspace slot ...
        float* ws_row = g.ws + (size_t)sg.part_slot * BM * BN + row_in_tile;  // column-major slot: (row, col) at col*BM + row
        for (int u = u_first; u < U; u += u_step) {
          int cols[2];
          const int nch = unit_chunks<EPI>(g, n0, u, cols);
          for (int c = 0; c < nch; ++c) {
            float f[32];
            tsrc.load32(cols[c], f);
            float* p = ws_row + (size_t)cols[c] * BM;
#pragma unroll
            for (int j = 0; j < 32; ++j) __stcg(p + (size_t)j * BM, f[j]);
          }
        }
      }

      if (warp == 2 && lane == 0) SB_GEMM_MARK(7);  // this warp's share of the tile stored
      if (warp == 9 && lane == 0) SB_GEMM_MARK(13);
      // TMEM drained: hand the buffer back to the MMA warp (of the leader CTA).
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTA2) ptx::mbar_arrive_cluster(empty_remote + (uint32_t)(buf * 8));
        else ptx::mbar_arrive(&tmem_empty[buf]);
        // a part of a cut tile: tell the tile's other parts that these 32 rows of it are in the workspace
        // (release increment after the __syncwarp: covers the stores of all lanes)
        if (S > 1) arrive_acq_rel(g.ws_counters + (size_t)sg.rem_index * 32 + slot);
      }
      if constexpr (EPI == EPI_PUSH) {
        if (S == 1) push_rows_done(comm, red, g, mt * BM + row_in_tile - lane);
      }
    }

    // Second pass over the cut tiles this unit has a part of: once every part of a tile has left its
    // share for these 32 rows, finish 1/S of the tile's units -- all S parts work on the fix-up at
    // once instead of one of them doing it alone.
    for (int it = sc.rounds; ok && ks == 1 && has_cut_tiles(sc); ++it) {
      const Segment sg = segment_of(sc, unit_id, it);
      if (!sg.valid) break;
      const int S = sg.parts;
      if (S == 1) continue;
      const int mt = sg.tile % g.m_tiles, nt = sg.tile / g.m_tiles;
      if (g.expert_ids && mt * BM >= rows_in_use) continue;
      uint32_t* ctr_arrive = g.ws_counters + (size_t)sg.rem_index * 32 + slot;
      uint32_t* ctr_done = ctr_arrive + 16;
      int arrived = 1;
      if (lane == 0) {
        const long long t0 = clock64();
        while (ld_acquire_gpu(ctr_arrive) < (uint32_t)S) {
          __nanosleep(32);
          if (*abort_flag || clock64() - t0 > ptx::kWaitLimitCycles) { arrived = 0; *abort_flag = 1; break; }
        }
      }
      arrived = __shfl_sync(0xffffffffu, arrived, 0);
      if (!arrived) { ok = false; break; }
      const int n0 = tile_first_col<EPI>(g, nt);
      const RowCtx<T> rc = make_row_ctx<T, EPI>(g, comm, red, mt * BM + row_in_tile, n0, epi_stage);
      {
        const int my_part = sg.part_slot - sg.first_slot;
        const WorkspaceSource wsrc{g.ws + (size_t)sg.first_slot * BM * BN + row_in_tile, (size_t)BM * BN, BM, S};
        int k = 0;
        for (int u = u_first; u < U; u += u_step, ++k)
          if (k % S == my_part) finish_unit<T, EPI>(g, rc, wsrc, u);
      }
      __syncwarp();
      if (lane == 0) {
        if (atomicAdd(ctr_done, 1u) == (uint32_t)(S - 1)) {  // last reader: ready for the next launch
          *ctr_arrive = 0;
          *ctr_done = 0;
        }
      }
      // every part reports its share of these rows: S arrivals per (cut tile, 32-row slot)
      if constexpr (EPI == EPI_PUSH) push_rows_done(comm, red, g, mt * BM + row_in_tile - lane);
    }
  }

  // ------------------------------------------------- cluster K-split: exchange + epilogue
  // The pairs of the cluster hold partial accumulators of the same tile.  The tile's epilogue units are dealt
  // out to the pairs (unit u belongs to pair u % ks).  A pair parks the chunks of the other pairs' units in its
  // own shared memory (the stage ring is free by then) and hands each warp's 4 KiB block to the copy engine,
  // which moves it into the owner's shared memory and counts the bytes on the owner's barrier; a pair finishes
  // its own units from TMEM plus what it received.  The exchange so moves (ks-1)/ks of an accumulator per CTA,
  // in all directions at once, and the epilogue work is split ks ways.
  // Every thread of every CTA of the cluster joins the cluster barrier, whatever happened before (a wait that
  // ran out only makes its warp skip the work after it).
  if constexpr (CTA2 && MI == 1) {
    if (ks > 1) {
      constexpr int kChunksPerUnit = (EPI == EPI_SILU_MUL || EPI == EPI_ROTARY) ? 2 : 1;
      const Segment sg = segment_of(sc, unit_id, 0);  // the unit's one tile
      const int mt = sg.tile % g.m_tiles, nt = sg.tile / g.m_tiles;
      const int q = warp & 3, hsel = (warp - 2) >> 2;
      const int U = num_units<EPI>(g);
      const int row_in_cta = q * 32 + lane;
      const int n0 = tile_first_col<EPI>(g, nt);
      const uint32_t area_bytes = xchg_area_bytes(U, ks, kChunksPerUnit);  // one pair's units of an accumulator
      uint8_t* out_area = stage_base;                                 // [other pair][unit of it][chunk]: what this CTA sends
      uint8_t* in_area = stage_base + (size_t)(ks - 1) * area_bytes;   // [other pair][own unit][chunk]: what it receives
      bool ok = sg.valid;
      if (warp == 2 && lane == 0) {
        // announce the bytes the other pairs will send for this pair's units (before the cluster barrier below,
        // so before any of them can arrive)
        uint32_t chunks = 0;
        for (int u = (int)kpart; u < U; u += ks) {
          int cols[2];
          chunks += (uint32_t)unit_chunks<EPI>(g, n0, u, cols);
        }
        ptx::mbar_expect_tx(xchg_bar, chunks * (uint32_t)(ks - 1) * kXchgChunkBytes);
      }
      if (warp >= 2 && ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(&tmem_full[0], 0u, abort_flag) ? 1 : 0) != 0;
        ptx::tc_fence_after();
      }
      ptx::tc_fence_before();
      __syncthreads();          // (the warps re-converge here: the producer and the MMA issuer ran on one lane)
      ptx::cluster_sync_all();  // every pair's MMAs are complete: the stage buffers of all CTAs are free
      ptx::tc_fence_after();
      if (warp == 2 && lane == 0) SB_GEMM_MARK(6);
      const uint32_t tmem_row = tmem_base + ((uint32_t)(q * 32) << 16);
      // the k-th unit of a pair (u = k * ks + pair) is sent, and later finished, by warp k % 2 of the lane quarter
      if (warp >= 2 && ok) {
        for (int u = 0; u < U; ++u) {
          const int owner = u % ks, k = u / ks;
          if (owner == (int)kpart || (k & 1) != hsel) continue;
          int cols[2];
          const int nch = unit_chunks<EPI>(g, n0, u, cols);
          const int slot_out = owner < (int)kpart ? owner : owner - 1;
          const int slot_in = (int)kpart < owner ? (int)kpart : (int)kpart - 1;  // the owner keeps its sources in pair order
          const uint32_t dst_cta = (uint32_t)(2 * owner) + cta_rank;
          for (int c = 0; c < nch; ++c) {
            const size_t blk = (size_t)(k * kChunksPerUnit + c) * kXchgChunkBytes + (size_t)q * (kXchgChunkBytes / 4);
            uint8_t* mine = out_area + (size_t)slot_out * area_bytes + blk;
            uint32_t r[32];
            ptx::tmem_ld_32x32(tmem_row + (uint32_t)cols[c], r);
            const uint32_t rowp = ptx::smem_u32(mine) + (uint32_t)(lane * 128);
#pragma unroll
            for (int j = 0; j < 8; ++j)
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rowp + (uint32_t)((j ^ (lane & 7)) << 4)), "r"(r[4 * j]),
                           "r"(r[4 * j + 1]), "r"(r[4 * j + 2]), "r"(r[4 * j + 3])
                           : "memory");
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0)
              ptx::bulk_copy_to_cta(ptx::map_to_cta(ptx::smem_u32(in_area + (size_t)slot_in * area_bytes + blk), dst_cta),
                                    ptx::smem_u32(mine), kXchgChunkBytes / 4, ptx::map_to_cta(ptx::smem_u32(xchg_bar), dst_cta));
          }
        }
      }
      if (warp == 2 && lane == 0) SB_GEMM_MARK(7);
      if (warp >= 2 && ok) {
        ok = __all_sync(0xffffffffu, ptx::mbar_wait(xchg_bar, 0u, abort_flag) ? 1 : 0) != 0;  // the partials have landed
        if (warp == 2 && lane == 0) SB_GEMM_MARK(13);
        if (ok) {
          const int row_in_tile = (int)cta_rank * 128 + row_in_cta;
          const RowCtx<T> rc = make_row_ctx<T, EPI>(g, comm, red, mt * BM + row_in_tile, n0, epi_stage);
          for (int u = (int)kpart + hsel * ks; u < U; u += 2 * ks) {
            const TmemPlusSmemSource src{tmem_row, in_area + (size_t)((u / ks) * kChunksPerUnit) * kXchgChunkBytes +
                                                       (size_t)row_in_cta * 128, ks - 1, area_bytes};
            finish_unit<T, EPI>(g, rc, src, u);
          }
          // every warp of every pair reports its share of these 32 rows (also one that had no unit to finish)
          if constexpr (EPI == EPI_PUSH) push_rows_done(comm, red, g, mt * BM + row_in_tile - lane);
        }
      }
    }
  }

  // -------------------------------------------------------------- common exit
  __syncwarp();  // the producer / MMA lanes re-join their warps before the block-wide barrier
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) SB_GEMM_MARK(8);  // all roles done
  if (CTA2) ptx::cluster_sync_all();  // the peer no longer signals our barriers / writes our TMEM
  if (threadIdx.x == 32) SB_GEMM_MARK(12);  // before the TMEM release
  if (warp == 1) {
    ptx::tc_fence_after();
    if (CTA2) ptx::tmem_dealloc_pair(tmem_base, kTmemCols); else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 32) SB_GEMM_MARK(9);  // TMEM released
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      if (g.status) atomicCAS(g.status, 0u, (uint32_t)CS_TIMEOUT_MBARRIER);
      if (EPI == EPI_PUSH) record_status(comm, CS_TIMEOUT_MBARRIER);
    }
    return;
  }

  if constexpr (EPI == EPI_PUSH) {
    trace_mark(red, 1);
    collective_tail<T, kMaxVecPerLaneGemm>(comm, red, blockIdx.x, gridDim.x);
    advance_targets(comm, red);
    trace_mark(red, 6);
  }
}

}  // namespace sb200
