// Device-side view of the tensor-parallel communication context and the
// reduce / broadcast phases shared by the fused row-parallel GEMM and the
// standalone all-reduce.
//
// Every rank owns one "symmetric heap" with the same layout, mapped into every
// peer (P2P over NVLink/NVSwitch).  One collective call ("epoch") runs as:
//   push    : each rank writes its partial rows into the OWNER's heap
//             (slot [set][src_rank]), then bumps the owner's push counter;
//   reduce  : the owner waits for all pushes, sums the partials in fp32 (+bias,
//             +residual), optionally RMS-normalises, and stores the finished
//             rows into EVERY rank's output buffers, bumping their done counter;
//   finish  : each rank waits until all rows have landed in its own buffers.
// Row t is owned by rank t / rows_per_rank.  Buffers and counters are double
// buffered by call parity (`set`); counters only ever grow and are compared
// against cumulative targets that live next to them and are advanced on the
// device at the end of each call, so nothing is reset and no per-call value
// comes from the host (a captured CUDA graph of collectives can be replayed).
// Two ranks can be at most one call apart because every call ends with the
// finish wait, which needs every rank's reduce of the same call.
// All waits are bounded; a wait that runs out sets the status word and the
// kernel returns.
#pragma once

#include "common.cuh"

namespace sb200 {

constexpr int kMaxRanks = 8;

// counters (uint32) at the start of each heap
enum CommCounter {
  CC_PUSH0 = 0,   // pushes received, set 0 / 1
  CC_PUSH1 = 1,
  CC_DONE0 = 2,   // finished rows received, set 0 / 1
  CC_DONE1 = 3,
  CC_STATUS = 4,  // first error recorded by a kernel on this rank (0 = none)
  CC_PUSH_TGT0 = 8,   // cumulative number of pushes this rank has been promised, set 0 / 1
  CC_PUSH_TGT1 = 9,   //   (advanced on the device by the last CTA of each collective kernel, so a
  CC_DONE_TGT0 = 10,  //    captured CUDA graph can be replayed: no per-call host value is baked in)
  CC_DONE_TGT1 = 11,
  CC_EXIT_TICKET = 12,  // CTAs of the running collective kernel that have finished
  CC_BARRIER = 16,      // [kMaxRanks] generic barrier slots
  CC_COUNT = 64
};

enum CommStatusCode {
  CS_OK = 0,
  CS_TIMEOUT_MBARRIER = 1,  // pipeline barrier inside a GEMM CTA
  CS_TIMEOUT_PUSH = 2,      // partial rows from a peer never arrived
  CS_TIMEOUT_DONE = 3       // finished rows from a peer never arrived
};

struct CommView {
  int rank;
  int world;
  char* heap[kMaxRanks];   // heap[rank] is local memory, the others are peer mappings
  size_t partial_off[2];   // byte offsets inside a heap
  size_t out_off[2];
  size_t resid_off[2];
  size_t region_bytes;     // capacity of each of the six regions
};

__device__ __forceinline__ uint32_t* comm_counter(const CommView& c, int r, int which) {
  return reinterpret_cast<uint32_t*>(c.heap[r]) + which;
}

// Memory-ordering helpers.  Counters of a multi-rank context are written by peers over NVLink and
// need system scope; a single-rank context (tensor-parallel size 1) stays at GPU scope, which is
// much cheaper.  Polling uses relaxed loads; one acquire fence follows the successful poll.
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed(const uint32_t* p, bool sys) {
  uint32_t v;
  if (sys) asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_scope(bool sys) {
  if (sys) __threadfence_system(); else __threadfence();
}
// Counter increment that publishes the caller's earlier stores; the CALLER has already executed
// fence_scope() after those stores (one fence can cover several increments).
__device__ __forceinline__ void red_add_relaxed(uint32_t* p, uint32_t v, bool sys) {
  if (sys) asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  else asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded spin until *p has reached `target` (wrap-safe).  Returns false on timeout.
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, long long limit_cycles, bool sys) {
  bool ok = true;
  if ((int32_t)(ld_relaxed(p, sys) - target) < 0) {
    const long long t0 = clock64();
    while ((int32_t)(ld_relaxed(p, sys) - target) < 0) {
      __nanosleep(40);
      if (clock64() - t0 > limit_cycles) { ok = false; break; }
    }
  }
  fence_scope(sys);  // acquire: what the counted writers stored is visible from here on
  return ok;
}

__device__ __forceinline__ void record_status(const CommView& c, int code) {
  atomicCAS(comm_counter(c, c.rank, CC_STATUS), 0u, (uint32_t)code);
}

struct ReduceArgs {
  int T, H;               // rows of the whole batch, row length
  int rows_per_rank;      // ownership granule: owner(t) = t / rows_per_rank
  int set;                // call parity
  uint32_t push_per_call; // increments this rank's CC_PUSH[set] receives during this call
  uint32_t done_per_call; // increments this rank's CC_DONE[set] receives during this call (= T)
  const void* bias;       // [H] or null, added after the sum (reference: layers.py:448-453)
  const void* residual;   // [T, H] local tensor or null: z = sum + residual
  const void* norm_w;     // [H] or null: also produce rms_norm(z) * norm_w
  float eps;
  int write_resid_all;    // store z into every rank's resid region (else only the owner's)
  void* out_copy;         // optional local [T, H] tensor that receives the primary result
  void* resid_copy;       // optional local [T, H] tensor that receives z when norm_w != null
  long long wait_cycles;
};

// Primary result = rms_norm(z)*w when norm_w is set, else z.  It goes to the
// `out` region of every rank; z additionally goes to the `resid` region when a
// norm is applied (so the caller gets both the normalised rows and the new residual).
//
// A row is handled by a team of 1, 2, 4 or 8 warps of one CTA (as many as the grid can spare for
// the rows this rank owns); a lane works on batches of kRB 16-byte vectors whose loads are issued
// together, so a row costs a few memory round trips.  The teams' partial sums of squares meet in
// shared memory through named barriers.
constexpr int kRB = 4;
constexpr int kReduceWarps = 8;  // warps of a CTA that take part (warps 0..7)

template <typename T>
__device__ __forceinline__ Vec16<T> ldcg16(const T* p) {
  Vec16<T> r;
  r.raw = __ldcg(reinterpret_cast<const uint4*>(p));
  return r;
}

__device__ __forceinline__ void team_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

template <typename T>
__device__ void reduce_phase(const CommView& c, const ReduceArgs& a, int cta, int num_ctas) {
  constexpr int N = Vec16<T>::N;
  __shared__ float s_ss[kReduceWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp >= kReduceWarps) return;
  const bool sys = c.world > 1;
  const int row0 = c.rank * a.rows_per_rank;
  const int nrows = max(0, min(a.rows_per_rank, a.T - row0));
  // team width: as many warps per row as the grid can spare (power of two, at most a CTA's share)
  int tw = 1;
  while (tw < kReduceWarps && (long long)num_ctas * kReduceWarps >= (long long)nrows * tw * 2) tw <<= 1;
  const int teams_per_cta = kReduceWarps / tw;
  const int team = warp / tw, wt = warp - team * tw;
  const int gteam = cta * teams_per_cta + team, num_teams = num_ctas * teams_per_cta;
  if (gteam >= nrows) return;  // no row for this team: nothing to wait for either
  {
    bool ok = true;
    if (lane == 0) {
      const uint32_t target = *(volatile uint32_t*)comm_counter(c, c.rank, CC_PUSH_TGT0 + a.set) + a.push_per_call;
      ok = wait_counter(comm_counter(c, c.rank, CC_PUSH0 + a.set), target, a.wait_cycles, sys);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok && lane == 0) record_status(c, CS_TIMEOUT_PUSH);
    // (a warp that timed out still walks its rows so that its team mates are not left at a barrier;
    //  the status word tells the host that the results are not to be used)
  }
  const int nvec = a.H / N;
  const T* bias = (const T*)a.bias;
  const T* resid = (const T*)a.residual;
  const T* nw = (const T*)a.norm_w;
  const T* my_partial = (const T*)(c.heap[c.rank] + c.partial_off[a.set]);
  const size_t src_stride = (size_t)a.rows_per_rank * a.H;  // elements between the slots of consecutive source ranks
  const int vstep = 32 * tw;                                // vectors a team covers per step
  for (int lr = gteam; lr < nrows; lr += num_teams) {
    const int t = row0 + lr;
    const size_t row_off = (size_t)t * a.H;
    float ss = 0.f;
    // pass 1: z = round(sum_src partial + bias + residual); z is kept in the local resid/out region
    T* zrow_local = (T*)(c.heap[c.rank] + (nw ? c.resid_off[a.set] : c.out_off[a.set])) + row_off;
    for (int v0 = wt * 32 + lane; v0 < nvec; v0 += vstep * kRB) {
      float acc[kRB][N];
#pragma unroll
      for (int b = 0; b < kRB; ++b)
#pragma unroll
        for (int j = 0; j < N; ++j) acc[b][j] = 0.f;
      Vec16<T> bv[kRB], rv[kRB];
#pragma unroll
      for (int b = 0; b < kRB; ++b) {
        const int v = v0 + vstep * b;
        if (v < nvec) {
          if (bias) bv[b] = ld16(bias + (size_t)v * N);
          if (resid) rv[b] = ld16(resid + row_off + (size_t)v * N);
        }
      }
      for (int s = 0; s < c.world; ++s) {
        const T* p = my_partial + (size_t)s * src_stride + (size_t)lr * a.H;
        Vec16<T> x[kRB];
#pragma unroll
        for (int b = 0; b < kRB; ++b) {
          const int v = v0 + vstep * b;
          if (v < nvec) x[b] = ldcg16(p + (size_t)v * N);
        }
#pragma unroll
        for (int b = 0; b < kRB; ++b)
          if (v0 + vstep * b < nvec) {
#pragma unroll
            for (int j = 0; j < N; ++j) acc[b][j] += DT<T>::to_f(x[b].v[j]);
          }
      }
#pragma unroll
      for (int b = 0; b < kRB; ++b) {
        const int v = v0 + vstep * b;
        if (v >= nvec) continue;
        Vec16<T> z;
#pragma unroll
        for (int j = 0; j < N; ++j) {
          float f = acc[b][j];
          if (bias) f = rt<T>(rt<T>(f) + DT<T>::to_f(bv[b].v[j]));
          if (resid) f = rt<T>(DT<T>::to_f(rv[b].v[j]) + rt<T>(f));
          z.v[j] = DT<T>::from_f(f);
          const float zf = DT<T>::to_f(z.v[j]);
          ss += zf * zf;
        }
        st16(zrow_local + (size_t)v * N, z);
        if (nw) {
          if (a.resid_copy) st16((T*)a.resid_copy + row_off + (size_t)v * N, z);
          if (a.write_resid_all)
            for (int d = 1; d < c.world; ++d) {
              const int dst = (c.rank + d) % c.world;
              st16((T*)(c.heap[dst] + c.resid_off[a.set]) + row_off + (size_t)v * N, z);
            }
        } else {
          if (a.out_copy) st16((T*)a.out_copy + row_off + (size_t)v * N, z);
          for (int d = 1; d < c.world; ++d) {
            const int dst = (c.rank + d) % c.world;
            st16((T*)(c.heap[dst] + c.out_off[a.set]) + row_off + (size_t)v * N, z);
          }
        }
      }
    }
    if (nw) {
      ss = warp_sum(ss);
      if (tw > 1) {
        if (lane == 0) s_ss[warp] = ss;
        team_barrier(1 + team, 32 * tw);
        ss = 0.f;
        for (int i = 0; i < tw; ++i) ss += s_ss[team * tw + i];
        team_barrier(1 + team, 32 * tw);  // everyone has read before the next row overwrites
      }
      const float inv = rsqrtf(ss / (float)a.H + a.eps);
      __syncwarp();
      // pass 2: y = round(z * inv) * w, to every rank (each lane re-reads the vectors it wrote itself)
      for (int v0 = wt * 32 + lane; v0 < nvec; v0 += vstep * kRB) {
        Vec16<T> z[kRB], w[kRB];
#pragma unroll
        for (int b = 0; b < kRB; ++b) {
          const int v = v0 + vstep * b;
          if (v < nvec) {
            z[b] = ld16(zrow_local + (size_t)v * N);
            w[b] = ld16(nw + (size_t)v * N);
          }
        }
#pragma unroll
        for (int b = 0; b < kRB; ++b) {
          const int v = v0 + vstep * b;
          if (v >= nvec) continue;
          Vec16<T> y;
#pragma unroll
          for (int j = 0; j < N; ++j)
            y.v[j] = DT<T>::from_f(rt<T>(DT<T>::to_f(z[b].v[j]) * inv) * DT<T>::to_f(w[b].v[j]));
          if (a.out_copy) st16((T*)a.out_copy + row_off + (size_t)v * N, y);
          for (int d = 0; d < c.world; ++d) {
            const int dst = (c.rank + d) % c.world;
            st16((T*)(c.heap[dst] + c.out_off[a.set]) + row_off + (size_t)v * N, y);
          }
        }
      }
    }
    // publish the row: every warp of the team makes its stores visible, then the row is counted once on every rank
    fence_scope(sys);
    if (tw > 1) team_barrier(1 + team, 32 * tw); else __syncwarp();
    if (wt == 0 && lane < c.world) red_add_relaxed(comm_counter(c, lane, CC_DONE0 + a.set), 1u, sys);
  }
}

// Wait until every row of this call has landed in this rank's buffers; one thread per CTA waits.
__device__ __forceinline__ bool finish_phase(const CommView& c, const ReduceArgs& a) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const uint32_t target = *(volatile uint32_t*)comm_counter(c, c.rank, CC_DONE_TGT0 + a.set) + a.done_per_call;
    const bool ok = wait_counter(comm_counter(c, c.rank, CC_DONE0 + a.set), target, a.wait_cycles, c.world > 1);
    if (!ok) record_status(c, CS_TIMEOUT_DONE);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// Last step of every collective kernel, called by all threads of every CTA after their phases:
// the last CTA to get here advances the cumulative targets of this call's set.  Every CTA has
// read the old targets by then (it reads them before it can finish), and the next collective on
// this set is a later kernel on the same stream.
__device__ __forceinline__ void advance_targets(const CommView& c, const ReduceArgs& a) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* ticket = comm_counter(c, c.rank, CC_EXIT_TICKET);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *(volatile uint32_t*)comm_counter(c, c.rank, CC_PUSH_TGT0 + a.set) += a.push_per_call;
      *(volatile uint32_t*)comm_counter(c, c.rank, CC_DONE_TGT0 + a.set) += a.done_per_call;
      *(volatile uint32_t*)ticket = 0;
      __threadfence();
    }
  }
}

// Copy rows owned by OTHER ranks from the local heap regions into the caller's tensors.
template <typename T>
__device__ void copy_out_phase(const CommView& c, const ReduceArgs& a, int tid_global, int nthreads_global) {
  constexpr int N = Vec16<T>::N;
  const int nvec = a.H / N;
  const int row0 = c.rank * a.rows_per_rank, row1 = min(a.T, row0 + a.rows_per_rank);
  const size_t total = (size_t)a.T * nvec;
  const T* src_out = (const T*)(c.heap[c.rank] + c.out_off[a.set]);
  const T* src_res = (const T*)(c.heap[c.rank] + c.resid_off[a.set]);
  for (size_t i = tid_global; i < total; i += nthreads_global) {
    const int t = (int)(i / nvec);
    if (t >= row0 && t < row1) continue;  // own rows were written directly by reduce_phase
    if (a.out_copy) st16((T*)a.out_copy + i * N, ld16(src_out + i * N));
    if (a.resid_copy && a.norm_w && a.write_resid_all) st16((T*)a.resid_copy + i * N, ld16(src_res + i * N));
  }
}

}  // namespace sb200
