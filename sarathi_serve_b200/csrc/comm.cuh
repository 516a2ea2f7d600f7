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

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Bounded spin until *p has reached `target` (wrap-safe).  Returns false on timeout.
__device__ __forceinline__ bool wait_counter(const uint32_t* p, uint32_t target, long long limit_cycles) {
  if ((int32_t)(ld_acquire_sys(p) - target) >= 0) return true;
  const long long t0 = clock64();
  while ((int32_t)(ld_acquire_sys(p) - target) < 0) {
    __nanosleep(64);
    if (clock64() - t0 > limit_cycles) return false;
  }
  return true;
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
// One warp per owned row, rows striped over all warps of the grid.
template <typename T>
__device__ void reduce_phase(const CommView& c, const ReduceArgs& a, int warp_global, int num_warps_global) {
  constexpr int N = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int row0 = c.rank * a.rows_per_rank;
  const int nrows = max(0, min(a.rows_per_rank, a.T - row0));
  if (nrows > 0) {
    bool ok = true;
    if (lane == 0) {
      const uint32_t target = *(volatile uint32_t*)comm_counter(c, c.rank, CC_PUSH_TGT0 + a.set) + a.push_per_call;
      ok = wait_counter(comm_counter(c, c.rank, CC_PUSH0 + a.set), target, a.wait_cycles);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) {
      if (lane == 0) record_status(c, CS_TIMEOUT_PUSH);
      return;
    }
  }
  const int nvec = a.H / N;
  const T* bias = (const T*)a.bias;
  const T* resid = (const T*)a.residual;
  const T* nw = (const T*)a.norm_w;
  const char* my_partial = c.heap[c.rank] + c.partial_off[a.set];
  for (int lr = warp_global; lr < nrows; lr += num_warps_global) {
    const int t = row0 + lr;
    float ss = 0.f;
    // pass 1: z = round(sum_src partial + bias + residual); keep z in the local resid/out region
    T* zrow_local = (T*)(c.heap[c.rank] + (nw ? c.resid_off[a.set] : c.out_off[a.set])) + (size_t)t * a.H;
    for (int v = lane; v < nvec; v += 32) {
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = 0.f;
      for (int s = 0; s < c.world; ++s) {
        const T* p = (const T*)my_partial + ((size_t)s * a.rows_per_rank + lr) * a.H + (size_t)v * N;
        const Vec16<T> x = ld16(p);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += DT<T>::to_f(x.v[j]);
      }
      Vec16<T> z;
      if (bias) {
        const Vec16<T> b = ld16(bias + (size_t)v * N);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = rt<T>(rt<T>(acc[j]) + DT<T>::to_f(b.v[j]));
      }
      if (resid) {
        const Vec16<T> r = ld16(resid + (size_t)t * a.H + (size_t)v * N);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] = rt<T>(DT<T>::to_f(r.v[j]) + rt<T>(acc[j]));
      }
#pragma unroll
      for (int j = 0; j < N; ++j) {
        z.v[j] = DT<T>::from_f(acc[j]);
        const float f = DT<T>::to_f(z.v[j]);
        ss += f * f;
      }
      st16(zrow_local + (size_t)v * N, z);
      if (nw) {
        if (a.resid_copy) st16((T*)a.resid_copy + (size_t)t * a.H + (size_t)v * N, z);
        if (a.write_resid_all)
          for (int d = 1; d < c.world; ++d) {
            const int dst = (c.rank + d) % c.world;
            st16((T*)(c.heap[dst] + c.resid_off[a.set]) + (size_t)t * a.H + (size_t)v * N, z);
          }
      } else {
        if (a.out_copy) st16((T*)a.out_copy + (size_t)t * a.H + (size_t)v * N, z);
        for (int d = 1; d < c.world; ++d) {
          const int dst = (c.rank + d) % c.world;
          st16((T*)(c.heap[dst] + c.out_off[a.set]) + (size_t)t * a.H + (size_t)v * N, z);
        }
      }
    }
    if (nw) {
      ss = warp_sum(ss);
      const float inv = rsqrtf(ss / (float)a.H + a.eps);
      __syncwarp();
      // pass 2: y = round(z * inv) * w, to every rank (each lane re-reads the vectors it wrote itself)
      for (int v = lane; v < nvec; v += 32) {
        const Vec16<T> z = ld16(zrow_local + (size_t)v * N);
        const Vec16<T> w = ld16(nw + (size_t)v * N);
        Vec16<T> y;
#pragma unroll
        for (int j = 0; j < N; ++j) y.v[j] = DT<T>::from_f(rt<T>(DT<T>::to_f(z.v[j]) * inv) * DT<T>::to_f(w.v[j]));
        if (a.out_copy) st16((T*)a.out_copy + (size_t)t * a.H + (size_t)v * N, y);
        for (int d = 0; d < c.world; ++d) {
          const int dst = (c.rank + d) % c.world;
          st16((T*)(c.heap[dst] + c.out_off[a.set]) + (size_t)t * a.H + (size_t)v * N, y);
        }
      }
    }
    // publish the row: make the stores visible system-wide, then count it on every rank
    __threadfence_system();
    __syncwarp();
    if (lane < c.world) red_release_sys_add(comm_counter(c, lane, CC_DONE0 + a.set), 1u);
  }
}

// Wait until every row of this call has landed in this rank's buffers; one thread per CTA waits.
__device__ __forceinline__ bool finish_phase(const CommView& c, const ReduceArgs& a) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const uint32_t target = *(volatile uint32_t*)comm_counter(c, c.rank, CC_DONE_TGT0 + a.set) + a.done_per_call;
    const bool ok = wait_counter(comm_counter(c, c.rank, CC_DONE0 + a.set), target, a.wait_cycles);
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
