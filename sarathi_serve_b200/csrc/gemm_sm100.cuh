// Persistent, warp-specialised bf16/fp16 GEMM for sm_100a:
//   C[M, N] = A[M, K] * B[N, K]^T        (both operands K-major, fp32 accumulate)
// TMA (128-byte swizzle) feeds a multi-stage shared-memory ring, one elected
// thread issues tcgen05.mma into a double-buffered TMEM accumulator, and four
// epilogue warps drain TMEM with tcgen05.ld while the next tile's main loop
// runs.  Row-major nn.Linear weights [out, in] are consumed as the K-major B
// operand as they are.
//
// Roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (warp w drains TMEM lanes 32*(w%4) .. +31, i.e. rows of
// the 128-row tile).
//
// Epilogues (the reference ops they absorb are cited where they are defined):
//   EPI_STORE    out = acc (+ bias)
//   EPI_ROTARY   qkv projection: rotary embedding applied to the q and k heads
//   EPI_SILU_MUL gate_up projection: out[:, j] = silu(gate_j) * up_j
//   EPI_PUSH     row-parallel projection: partial rows go to the owner rank's
//                reduce slots; the reduce / residual / norm / broadcast phases of
//                comm.cuh run in the same kernel after the tiles.
#pragma once

#include "comm.cuh"
#include "sm100_ptx.cuh"

namespace sb200 {

enum GemmEpilogue { EPI_STORE = 0, EPI_ROTARY = 1, EPI_SILU_MUL = 2, EPI_PUSH = 3 };

constexpr int kBM = 128;          // tile rows  (UMMA M)
constexpr int kBK = 64;           // K elements per stage: 128 bytes of bf16 = one swizzle row
constexpr int kGemmThreads = 192;

struct GemmArgs {
  int M, N, K;             // N counts B rows (for EPI_SILU_MUL: 2*d)
  void* out;               // [M, ldo] (EPI_SILU_MUL: [M, d])
  int64_t ldo;
  const void* bias;        // [N] or null (EPI_STORE only)
  // EPI_ROTARY
  const int64_t* positions;
  const void* cos_sin;     // [max_pos, rot_dim], same dtype as the output
  int head_size;
  int rot_cols;            // columns [0, rot_cols) hold q and k heads, the rest (v) is stored as is
  int is_neox;
  // tiling
  int m_tiles, n_tiles, k_blocks;
  uint32_t* status;        // device word: first error of this launch (0 = none); may be null
};

template <int BN> struct GemmSmem {
  static constexpr int kStageBytesA = kBM * kBK * 2;
  static constexpr int kStageBytesB = BN * kBK * 2;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kStages = (BN == 256) ? 4 : (BN == 128 ? 6 : 8);
  static constexpr int kBarrierBytes = 1024;
  static constexpr int kTotal = kStages * kStageBytes + kBarrierBytes + 1024;  // + alignment slack
};

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

template <typename T>
__device__ __forceinline__ void load_row32(const T* src, float* f) {
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    const Vec16<T> v = ld16(src + q * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[q * 8 + j] = DT<T>::to_f(v.v[j]);
  }
}

// ---------------------------------------------------------------------------
// The kernel.  `comm` / `red` are used only by EPI_PUSH.
template <typename T, int BN, int EPI>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                  const GemmArgs g, const CommView comm, const ReduceArgs red) {
  using S = GemmSmem<BN>;
  constexpr int kStages = S::kStages;
  constexpr uint32_t kTmemCols = 2 * BN;  // two accumulator buffers (power of two >= 32)
  constexpr uint32_t kIdesc = ptx::make_idesc(DT<T>::id == SB200_BF16 ? 1 : 0, BN);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* stage_base = smem;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * S::kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tmem_full = empty_bar + kStages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = g.m_tiles * g.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&full_bar[s], 1);
      ptx::mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&tmem_full[b], 1);
      ptx::mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % g.m_tiles, nt = tile / g.m_tiles;
        for (int kb = 0; kb < g.k_blocks; ++kb) {
          if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
          uint8_t* sa = stage_base + stage * S::kStageBytes;
          uint8_t* sb = sa + S::kStageBytesA;
          ptx::mbar_expect_tx(&full_bar[stage], S::kStageBytes);
          ptx::tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * kBK, mt * kBM);
          if (EPI == EPI_SILU_MUL) {
            // B tile = BN/2 rows of the gate shard followed by the matching BN/2 rows of the up shard
            ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, nt * (BN / 2));
            ptx::tma_load_2d(sb + S::kStageBytesB / 2, &tmap_b, &full_bar[stage], kb * kBK, g.N / 2 + nt * (BN / 2));
          } else {
            ptx::tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * kBK, nt * BN);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        const uint32_t use = (uint32_t)(local >> 1);  // how many times this buffer was used before
        if (!ptx::mbar_wait(&tmem_empty[buf], (use & 1u) ^ 1u, abort_flag)) { ok = false; break; }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
        for (int kb = 0; kb < g.k_blocks; ++kb) {
          if (!ptx::mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t sa = ptx::smem_u32(stage_base + stage * S::kStageBytes);
          const uint64_t da = ptx::make_smem_desc_sw128(sa);
          const uint64_t db = ptx::make_smem_desc_sw128(sa + S::kStageBytesA);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            // advance 16 elements = 32 bytes along K inside the swizzle row: +2 in 16-byte units
            ptx::umma_f16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), kIdesc, (kb | k) ? 1u : 0u);
          }
          ptx::umma_commit(&empty_bar[stage]);  // frees the smem stage once these MMAs have read it
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) ptx::umma_commit(&tmem_full[buf]);  // accumulator complete
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const int mt = tile % g.m_tiles, nt = tile / g.m_tiles;
      const int buf = local & 1;
      const uint32_t use = (uint32_t)(local >> 1);
      ok = __all_sync(0xffffffffu, ptx::mbar_wait(&tmem_full[buf], use & 1u, abort_flag) ? 1 : 0) != 0;
      if (!ok) break;  // warp-uniform: no lane is left behind in an aligned tcgen05.ld
      ptx::tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);
      const int gm = mt * kBM + q * 32 + lane;  // global row of this thread
      const bool row_ok = gm < g.M;
      T* out = reinterpret_cast<T*>(g.out);

      if constexpr (EPI == EPI_STORE) {
        const bool vec_ok = ((g.ldo & 7) == 0) && aligned16(g.out);
        const T* bias = reinterpret_cast<const T*>(g.bias);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_row + c * 32, r);
          const int gn = nt * BN + c * 32;
          if (row_ok && gn < g.N) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
            if (bias) {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (gn + j < g.N) f[j] += DT<T>::to_f(bias[gn + j]);
            }
            store_row32<T>(out + (size_t)gm * g.ldo + gn, f, g.N - gn, vec_ok);
          }
        }
      } else if constexpr (EPI == EPI_ROTARY) {
        // Reference: F.linear output rounded to T (tensor_parallel/layers.py:278-284), then
        // rotary_embedding in T arithmetic on the q and k heads (csrc/pos_encoding_kernels.cu:8-76).
        // Requires BN % head_size == 0, rot_dim == head_size, (head_size/2) % 32 == 0 for NeoX.
        const bool vec_ok = ((g.ldo & 7) == 0) && aligned16(g.out);
        const T* cs = row_ok ? reinterpret_cast<const T*>(g.cos_sin) + g.positions[gm] * g.head_size : nullptr;
        const int half = g.head_size / 2;
        const int chunks_per_head = g.head_size / 32;
#pragma unroll 1
        for (int h0 = 0; h0 < BN; h0 += g.head_size) {
          const int gh = nt * BN + h0;  // first global column of this head
          const bool rotate = gh < g.rot_cols;
          if (rotate && g.is_neox) {
#pragma unroll 1
            for (int c = 0; c < chunks_per_head / 2; ++c) {
              uint32_t rx[32], ry[32];
              ptx::tmem_ld_32x32(t_row + h0 + c * 32, rx);
              ptx::tmem_ld_32x32(t_row + h0 + half + c * 32, ry);
                  if (row_ok && gh < g.N) {
                float co[32], si[32], fx[32], fy[32];
                load_row32<T>(cs + c * 32, co);
                load_row32<T>(cs + half + c * 32, si);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float x = rt<T>(__uint_as_float(rx[j])), y = rt<T>(__uint_as_float(ry[j]));
                  fx[j] = rt<T>(rt<T>(x * co[j]) - rt<T>(y * si[j]));
                  fy[j] = rt<T>(rt<T>(y * co[j]) + rt<T>(x * si[j]));
                }
                store_row32<T>(out + (size_t)gm * g.ldo + gh + c * 32, fx, g.N - (gh + c * 32), vec_ok);
                store_row32<T>(out + (size_t)gm * g.ldo + gh + half + c * 32, fy, g.N - (gh + half + c * 32), vec_ok);
              }
            }
          } else {
#pragma unroll 1
            for (int c = 0; c < chunks_per_head; ++c) {
              uint32_t r[32];
              ptx::tmem_ld_32x32(t_row + h0 + c * 32, r);
                  const int gn = gh + c * 32;
              if (row_ok && gn < g.N) {
                float f[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
                if (rotate) {  // GPT-J style: pairs (2i, 2i+1); cos/sin index = column_in_head / 2
#pragma unroll
                  for (int j = 0; j < 32; j += 2) {
                    const int p = (c * 32 + j) >> 1;
                    const float co = DT<T>::to_f(cs[p]), si = DT<T>::to_f(cs[half + p]);
                    const float x = rt<T>(f[j]), y = rt<T>(f[j + 1]);
                    f[j] = rt<T>(rt<T>(x * co) - rt<T>(y * si));
                    f[j + 1] = rt<T>(rt<T>(y * co) + rt<T>(x * si));
                  }
                }
                store_row32<T>(out + (size_t)gm * g.ldo + gn, f, g.N - gn, vec_ok);
              }
            }
          }
        }
      } else if constexpr (EPI == EPI_SILU_MUL) {
        // Reference: gate_up = F.linear(x) rounded to T, then silu_and_mul
        // (csrc/activation_kernels.cu:8-25): out = (T)(silu(gate)) * up.
        const int d = g.N / 2;
        const bool vec_ok = ((g.ldo & 7) == 0) && aligned16(g.out);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t rg[32], ru[32];
          ptx::tmem_ld_32x32(t_row + c * 32, rg);
          ptx::tmem_ld_32x32(t_row + BN / 2 + c * 32, ru);
          const int gn = nt * (BN / 2) + c * 32;
          if (row_ok && gn < d) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float gte = rt<T>(__uint_as_float(rg[j])), up = rt<T>(__uint_as_float(ru[j]));
              const float sl = rt<T>(gte / (1.0f + expf(-gte)));
              f[j] = rt<T>(sl * up);
            }
            store_row32<T>(out + (size_t)gm * g.ldo + gn, f, d - gn, vec_ok);
          }
        }
      } else {  // EPI_PUSH
        // Partial rows go to the owner's slot [set][src = my rank][local row][H].
        const int owner = row_ok ? gm / red.rows_per_rank : 0;
        const int lr = gm - owner * red.rows_per_rank;
        T* dst_row = row_ok ? reinterpret_cast<T*>(comm.heap[owner] + comm.partial_off[red.set]) +
                                  ((size_t)comm.rank * red.rows_per_rank + lr) * (size_t)g.N
                            : nullptr;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(t_row + c * 32, r);
          const int gn = nt * BN + c * 32;
          if (row_ok && gn < g.N) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(r[j]);
            store_row32<T>(dst_row + gn, f, g.N - gn, (g.N & 7) == 0);
          }
        }
      }

      // TMEM buffer drained: hand it back to the MMA warp.
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&tmem_empty[buf]);

      if constexpr (EPI == EPI_PUSH) {
        // Publish this warp's 32 rows to their owner(s): stores of all lanes first, then one
        // release-increment per owner.  The host's push target counts (32-row group, owner) pairs.
        __threadfence_system();
        __syncwarp();
        if (lane == 0) {
          const int r_lo = mt * kBM + q * 32, r_hi = min(g.M, r_lo + 32) - 1;
          if (r_hi >= r_lo)
            for (int o = r_lo / red.rows_per_rank; o <= r_hi / red.rows_per_rank; ++o)
              red_release_sys_add(comm_counter(comm, o, CC_PUSH0 + red.set), 1u);
        }
      }
    }
  }

  // -------------------------------------------------------------- common exit
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      if (g.status) atomicCAS(g.status, 0u, (uint32_t)CS_TIMEOUT_MBARRIER);
      if (EPI == EPI_PUSH) record_status(comm, CS_TIMEOUT_MBARRIER);
    }
    return;
  }

  if constexpr (EPI == EPI_PUSH) {
    const int warps_per_cta = kGemmThreads / 32;
    reduce_phase<T>(comm, red, blockIdx.x * warps_per_cta + warp, gridDim.x * warps_per_cta);
    if (red.out_copy || red.resid_copy || blockIdx.x == 0) {
      if (finish_phase(comm, red) && (red.out_copy || red.resid_copy))
        copy_out_phase<T>(comm, red, blockIdx.x * kGemmThreads + threadIdx.x, gridDim.x * kGemmThreads);
    }
  }
}

}  // namespace sb200
