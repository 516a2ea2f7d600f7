// Device-side view of the tensor-parallel communication context and the
// reduce / gather phases shared by the fused row-parallel GEMM and the
// standalone all-reduce.
//
// Every rank owns one "symmetric heap" with the same layout, mapped into every
// peer (P2P over NVLink/NVSwitch) and, when the heaps are bound to an NVSwitch
// multicast object, reachable as ONE multicast address range as well.
// One collective call runs as:
//   produce : each rank writes its partial [T, H] into its OWN heap and tells
//             the ranks that will read it with a flag (the call's number);
//   reduce  : the owner of a row waits for every rank's flag, sums the row over
//             the ranks in fp32 (+bias, +residual), optionally RMS-normalises,
//             and publishes the finished row;
//   gather  : every rank ends up with all finished rows in its own heap.
// Row t is owned by rank t / rows_per_rank.  Three schemes share the buffers
// and flags:
//   owner-reduce + gather (peer loads only): owners pull the partial rows from
//       the peers' heaps, store finished rows locally, and the peers pull them;
//   one-shot (peer loads only): every rank pulls ALL partial rows and finishes
//       all T rows itself -- one flag hand-off and one trip over the links;
//   multicast (NVLS): the owner sums a row with ONE multimem.ld_reduce per
//       16 bytes (the switch reads the eight heaps and adds in fp32) and
//       publishes the finished row with multimem.st, which the switch copies
//       into every rank's heap; flags are multimem stores too.  The reduce
//       traffic leaves a GPU while the broadcast traffic enters it, so the two
//       halves of the collective overlap on the full-duplex links.
//
// The `partial` buffers and all flags are double buffered by the parity of the
// call number, which lives ON THE DEVICE (CC_CALLS, advanced by the last CTA of
// every collective kernel): two ranks can be at most one call apart -- a rank
// that owns rows cannot finish call n before every rank has produced for call
// n -- so a buffer of one parity is rewritten in call n+2 at the earliest, after
// every reader of call n has been released.  Because no per-call value comes
// from the host, a captured CUDA graph with any number of collectives can be
// replayed any number of times.  The `out` / `resid` regions the results are
// left in are chosen by the host (`ReduceArgs::set`) so that the caller knows
// their addresses when it enqueues the call; a finished row is written there
// only after every rank has entered the call, i.e. after every kernel that the
// ranks enqueued before it -- the readers of an earlier result -- has completed.
// All waits are bounded; a wait that runs out sets the status word and the
// kernel returns.
#pragma once

#include "common.cuh"

namespace sb200 {

constexpr int kMaxRanks = 8;

// control words (uint32) at the start of each heap; groups sit on separate 128-byte lines
enum CommCounter {
  CC_STATUS = 0,        // first error recorded by a kernel on this rank (0 = none)
  CC_EXIT_TICKET = 1,   // CTAs of the running collective kernel that have finished
  CC_CALLS = 2,         // collectives completed on this context: the running call has number CC_CALLS + 1
  CC_LOCAL_DONE = 4,    // local: reduce teams / CTAs of the running call that have finished their rows
  CC_LOCAL_PUSH = 32,   // local: [kMaxRanks] arrivals of this rank's own pushes, per destination owner
  CC_PUSH_FLAG0 = 64,   // [kMaxRanks] written by rank s: "my partial rows (that you own) are stored" (call number), parity 0
  CC_PUSH_FLAG1 = 96,   //   ... parity 1
  CC_DONE_FLAG0 = 128,  // [kMaxRanks] written by rank s: "all rows I own are finished" (call number), parity 0
  CC_DONE_FLAG1 = 160,  //   ... parity 1
  CC_COUNT = 192
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
  char* mc;                // multicast alias of all heaps (same offsets), or null
  size_t partial_off[2];   // byte offsets inside a heap
  size_t out_off[2];
  size_t resid_off[2];
  size_t region_bytes;     // capacity of each of the six regions
};

__device__ __forceinline__ uint32_t* comm_counter(const CommView& c, int r, int which) {
  return reinterpret_cast<uint32_t*>(c.heap[r]) + which;
}
__device__ __forceinline__ uint32_t* comm_counter_mc(const CommView& c, int which) {
  return reinterpret_cast<uint32_t*>(c.mc) + which;
}

// Memory-ordering helpers.  Flags of a multi-rank context are written by peers over NVLink and
// need system scope; a single-rank context (tensor-parallel size 1) stays at GPU scope.
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
__device__ __forceinline__ void st_release(uint32_t* p, uint32_t v, bool sys) {
  if (sys) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
  else asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// Arrival counter increment with release + acquire semantics at GPU scope: publishes what the caller
// (and the threads it has synchronised with through a barrier) stored before, and makes what earlier
// arrivals published visible to the caller.  Returns the old value.
__device__ __forceinline__ uint32_t arrive_acq_rel(uint32_t* p) {
  uint32_t old;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(p) : "memory");
  return old;
}

__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p, bool sys) {
  uint32_t v;
  if (sys) asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ---- NVSwitch multicast (multimem) accesses; `p` is an address inside the multicast alias -------
// One store that the switch delivers to the same offset of every rank's heap.
__device__ __forceinline__ void mc_st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("multimem.st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void mc_st16(void* p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w) : "memory");
}
// 16 bytes of the element-wise sum over all ranks' heaps: the addition happens in the switch, in fp32,
// and the result is rounded to T once.
template <typename T> __device__ __forceinline__ uint4 mc_ld_reduce16(const void* p);
template <> __device__ __forceinline__ uint4 mc_ld_reduce16<__nv_bfloat16>(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 mc_ld_reduce16<__half>(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
template <> __device__ __forceinline__ uint4 mc_ld_reduce16<float>(const void* p) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Bounded spin until the flag word at p has reached call number `epoch` (a flag word only ever grows; a
// waiter can see a later number only if the writer was allowed to run ahead, in which case the data it
// waits for is there as well).  Polls with relaxed loads; the load that ends the wait is an acquire load
// that reads a value the signalling rank stored with release semantics, so what that rank wrote before
// its flag is visible to this thread (and, through a following barrier, to the threads it releases).  A
// system-scope fence costs microseconds on this machine, an acquire load does not, so no fence is used
// on the waiting side.  Returns false on timeout.
__device__ __forceinline__ bool flag_reached(uint32_t v, uint32_t epoch) { return (int32_t)(v - epoch) >= 0; }
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t epoch, long long limit_cycles, bool sys) {
  const long long t0 = clock64();
  while (!flag_reached(ld_relaxed(p, sys), epoch)) {
    __nanosleep(20);
    if (clock64() - t0 > limit_cycles) return false;
  }
  return flag_reached(ld_acquire(p, sys), epoch);
}

__device__ __forceinline__ void record_status(const CommView& c, int code) {
  atomicCAS(comm_counter(c, c.rank, CC_STATUS), 0u, (uint32_t)code);
}

struct ReduceArgs {
  int T, H;               // rows of the whole batch, row length
  int rows_per_rank;      // ownership granule: owner(t) = t / rows_per_rank
  int set;                // which of the two out / resid regions receives the results (chosen by the host)
  int one_shot;           // 1: every rank loads ALL partial rows and finishes all T rows itself (one flag wait and one
                          // trip over the links instead of two; pays off while (world-1)*T*H bytes is small); 0: rows
                          // are reduced by their owners and gathered afterwards
  int use_mc;             // 1 (only with one_shot = 0): owners reduce and publish through the NVSwitch multicast alias
  int mc_pull;            // with use_mc: owners keep their finished rows in their own heap and the peers pull them (peer
                          // loads), instead of multicast stores followed by a system-scope fence in every CTA
  uint32_t push_expected[kMaxRanks];  // arrivals this rank's own kernel reports per destination owner
                                      // (epilogue warp-tiles of the GEMM, or CTAs of the all-reduce); one-shot and
                                      // multicast calls count all arrivals in [0]
  const void* bias;       // [H] or null, added after the sum (reference: layers.py:448-453)
  const void* residual;   // [T, H] local tensor or null: z = sum + residual
  const void* norm_w;     // [H] or null: also produce rms_norm(z) * norm_w
  float eps;
  int write_resid_all;    // store z into every rank's resid region (else only the owner's)
  void* out_copy;         // optional local [T, H] tensor that receives the primary result
  void* resid_copy;       // optional local [T, H] tensor that receives z when norm_w != null
  long long wait_cycles;
#ifdef SB200_TRACE
  unsigned long long* trace;  // [gridDim.x][16] nanosecond time stamps of the phases (profiling builds only)
#endif
};

#ifdef SB200_TRACE
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Thread 0 of every CTA records when it passed phase boundary `slot`.
__device__ __forceinline__ void trace_mark(const ReduceArgs& a, int slot) {
  if (a.trace && threadIdx.x == 0) a.trace[(size_t)blockIdx.x * 16 + slot] = global_ns();
}
#else
__device__ __forceinline__ void trace_mark(const ReduceArgs&, int) {}
#endif

// Number of the running call on this context (1, 2, ...): every CTA reads it before the call's last CTA
// advances it.  Its parity selects the `partial` buffer and the flag words of the call.
__device__ __forceinline__ uint32_t call_number(const CommView& c) {
  return *(volatile uint32_t*)comm_counter(c, c.rank, CC_CALLS) + 1u;
}
__device__ __forceinline__ int push_flag_index(uint32_t n, int src) { return ((n & 1u) ? CC_PUSH_FLAG1 : CC_PUSH_FLAG0) + src; }
__device__ __forceinline__ int done_flag_index(uint32_t n, int src) { return ((n & 1u) ? CC_DONE_FLAG1 : CC_DONE_FLAG0) + src; }
// This rank's partial [T, H] of call n.
__device__ __forceinline__ char* partial_of(const CommView& c, int r, uint32_t n) {
  return c.heap[r] + c.partial_off[n & 1u];
}

// Called by ONE thread after the stores it and its group made to this rank's partial region and a
// barrier (__syncwarp / __syncthreads) of that group: counts the arrival locally with a release
// increment (which covers the group's stores); the arrival that completes this rank's share of
// `owner`'s rows tells the owner with a single remote release store.
__device__ __forceinline__ void signal_push(const CommView& c, const ReduceArgs& a, int owner) {
  const uint32_t cnt = arrive_acq_rel(comm_counter(c, c.rank, CC_LOCAL_PUSH + owner)) + 1u;
  if (cnt == a.push_expected[owner]) {
    const uint32_t n = call_number(c);
    st_release(comm_counter(c, owner, push_flag_index(n, c.rank)), n, c.world > 1);
  }
}
// One-shot and multicast calls: every rank reads all of this rank's rows (or the switch does), so the
// arrivals are counted in one counter (push_expected[0] = all arrivals of this rank's kernel) and the
// last one flags every rank.  Called by ALL lanes of a converged warp after its stores (and, for a
// CTA-wide share, a __syncthreads): lane 0 counts the arrival; when it completes the count, one
// multicast store reaches every rank's flag word, or, without multicast, lanes 0..world-1 store one
// rank's flag each, so the fan-out costs one release, not world of them in a row.
__device__ __forceinline__ void signal_push_all(const CommView& c, const ReduceArgs& a) {
  const int lane = threadIdx.x & 31;
  __syncwarp();
  uint32_t cnt = 0;
  if (lane == 0) cnt = arrive_acq_rel(comm_counter(c, c.rank, CC_LOCAL_PUSH)) + 1u;
  cnt = __shfl_sync(0xffffffffu, cnt, 0);
  __syncwarp();  // a memory-ordering barrier of the warp: lane 0's acquire comes before the other lanes' release stores
  if (cnt != a.push_expected[0]) return;
  const uint32_t n = call_number(c);
  if (a.use_mc) {
    if (lane == 0) mc_st_release_u32(comm_counter_mc(c, push_flag_index(n, c.rank)), n);
  } else if (lane < c.world) {
    st_release(comm_counter(c, lane, push_flag_index(n, c.rank)), n, lane != c.rank);
  }
}

// Primary result = rms_norm(z)*w when norm_w is set, else z, kept in the `out` region; z is
// additionally kept in the `resid` region when a norm is applied (so the caller gets both the
// normalised rows and the new residual).
//
// A row is handled by a team of 1, 2, 4 or 8 warps of one CTA: as many as the grid can spare for
// the rows this rank owns, and at least as many as it takes to hold the row in registers (VPL
// 16-byte vectors per lane).  The loads of a row -- its residual and the partials of up
// to SB source ranks -- are issued together, so a row costs about one memory round trip per SB
// sources; z stays in registers for the normalisation.  The teams' partial sums of squares meet in
// shared memory through named barriers.
constexpr int kReduceWarps = 8;     // warps of a CTA that take part (warps 0..7)
// A row has at most 32 * kReduceWarps * MAXVPL 16-byte vectors: MAXVPL = 4 (16 KiB rows) inside the GEMM
// kernel, whose 320 threads leave 168 registers each, 8 (32 KiB rows) in the standalone all-reduce.
constexpr int kMaxVecPerLaneGemm = 4;
constexpr int kMaxVecPerLaneAllReduce = 8;

template <typename T>
__device__ __forceinline__ Vec16<T> ldcg16(const T* p) {
  Vec16<T> r;
  r.raw = __ldcg(reinterpret_cast<const uint4*>(p));
  return r;
}

__device__ __forceinline__ void team_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// z = round(round(sum + bias) + residual) for one 16-byte vector; returns the vector's sum of squares.
template <typename T>
__device__ __forceinline__ float finish_vec(const float* acc, const Vec16<T>* bias, const Vec16<T>* resid, Vec16<T>* z) {
  constexpr int N = Vec16<T>::N;
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < N; ++j) {
    float f = acc[j];
    if (bias) f = rt<T>(rt<T>(f) + DT<T>::to_f(bias->v[j]));
    if (resid) f = rt<T>(DT<T>::to_f(resid->v[j]) + rt<T>(f));
    z->v[j] = DT<T>::from_f(f);
    const float zf = DT<T>::to_f(z->v[j]);
    ss += zf * zf;
  }
  return ss;
}

template <typename T, int VPL>
__device__ __forceinline__ void reduce_rows(const CommView& c, const ReduceArgs& a, uint32_t n, int gteam, int num_teams,
                                            int tw, int team, int wt, int lane, int warp, int row0, int nrows,
                                            float* s_ss) {
  constexpr int N = Vec16<T>::N;
  constexpr int SB = VPL <= 2 ? 8 : 8 / VPL;  // source ranks whose loads are issued together (8-16 vectors in flight per lane)
  const int nvec = a.H / N;
  const T* bias = (const T*)a.bias;
  const T* resid = (const T*)a.residual;
  const T* nw = (const T*)a.norm_w;
  const int vstep = 32 * tw, vbase = wt * 32 + lane;
  // When all source ranks fit in one batch of loads, the partials of a team's NEXT row are requested
  // while the current row is normalised and stored, so a team with several rows pays the trip over
  // the links once.
  const bool prefetch = c.world <= SB;
  Vec16<T> x[SB][VPL];
  auto load_batch = [&](int s0, size_t row_off) {
#pragma unroll
    for (int i = 0; i < SB; ++i)
      if (s0 + i < c.world) {
        const T* p = (const T*)partial_of(c, s0 + i, n) + row_off;
#pragma unroll
        for (int b = 0; b < VPL; ++b) {
          const int v = vbase + vstep * b;
          if (v < nvec) x[i][b] = ldcg16(p + (size_t)v * N);
        }
      }
  };
  if (prefetch && gteam < nrows) load_batch(0, (size_t)(row0 + gteam) * a.H);
  for (int lr = gteam; lr < nrows; lr += num_teams) {
    const size_t row_off = (size_t)(row0 + lr) * a.H;
    float acc[VPL][N];
    Vec16<T> rv[VPL];
#pragma unroll
    for (int b = 0; b < VPL; ++b) {
#pragma unroll
      for (int j = 0; j < N; ++j) acc[b][j] = 0.f;
      const int v = vbase + vstep * b;
      if (resid && v < nvec) rv[b] = ld16(resid + row_off + (size_t)v * N);
    }
    for (int s0 = 0; s0 < c.world; s0 += SB) {
      if (!prefetch) load_batch(s0, row_off);
#pragma unroll
      for (int i = 0; i < SB; ++i)
        if (s0 + i < c.world) {
#pragma unroll
          for (int b = 0; b < VPL; ++b)
            if (vbase + vstep * b < nvec) {
#pragma unroll
              for (int j = 0; j < N; ++j) acc[b][j] += DT<T>::to_f(x[i][b].v[j]);
            }
        }
    }
    if (prefetch && lr + num_teams < nrows) load_batch(0, (size_t)(row0 + lr + num_teams) * a.H);
    // z = round(round(sum + bias) + residual)
    Vec16<T> z[VPL];
    float ss = 0.f;
    T* zrow = (T*)(c.heap[c.rank] + (nw ? c.resid_off[a.set] : c.out_off[a.set])) + row_off;
    T* zcopy = (T*)(nw ? a.resid_copy : a.out_copy);
#pragma unroll
    for (int b = 0; b < VPL; ++b) {
      const int v = vbase + vstep * b;
      if (v >= nvec) continue;
      Vec16<T> bv;
      if (bias) bv = ld16(bias + (size_t)v * N);
      ss += finish_vec<T>(acc[b], bias ? &bv : nullptr, resid ? &rv[b] : nullptr, &z[b]);
      st16(zrow + (size_t)v * N, z[b]);
      if (zcopy) st16(zcopy + row_off + (size_t)v * N, z[b]);
    }
    if (nw) {
      Vec16<T> w[VPL];
#pragma unroll
      for (int b = 0; b < VPL; ++b) {
        const int v = vbase + vstep * b;
        if (v < nvec) w[b] = ld16(nw + (size_t)v * N);
      }
      ss = warp_sum(ss);
      if (tw > 1) {
        if (lane == 0) s_ss[warp] = ss;
        team_barrier(1 + team, 32 * tw);
        ss = 0.f;
        for (int i = 0; i < tw; ++i) ss += s_ss[team * tw + i];
        team_barrier(1 + team, 32 * tw);  // everyone has read before the next row overwrites
      }
      const float inv = rsqrtf(ss / (float)a.H + a.eps);
      T* yrow = (T*)(c.heap[c.rank] + c.out_off[a.set]) + row_off;
#pragma unroll
      for (int b = 0; b < VPL; ++b) {
        const int v = vbase + vstep * b;
        if (v >= nvec) continue;
        Vec16<T> y;
#pragma unroll
        for (int j = 0; j < N; ++j)
          y.v[j] = DT<T>::from_f(rt<T>(DT<T>::to_f(z[b].v[j]) * inv) * DT<T>::to_f(w[b].v[j]));
        st16(yrow + (size_t)v * N, y);
        if (a.out_copy) st16((T*)a.out_copy + row_off + (size_t)v * N, y);
      }
    }
  }
}

template <typename T, int MAXVPL>
__device__ void reduce_phase(const CommView& c, const ReduceArgs& a, int cta, int num_ctas) {
  constexpr int N = Vec16<T>::N;
  __shared__ float s_ss[kReduceWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (warp >= kReduceWarps) return;
  const bool sys = c.world > 1;
  const int row0 = a.one_shot ? 0 : c.rank * a.rows_per_rank;
  const int nrows = a.one_shot ? a.T : max(0, min(a.rows_per_rank, a.T - row0));
  if (nrows == 0) return;  // owns nothing: nobody waits for this rank's done flag
  const int nvec = a.H / N;
  // team width: what the row needs to fit in registers, then as many warps as the grid can spare
  int tw = 1;
  while (tw < kReduceWarps && nvec > 32 * tw * MAXVPL) tw <<= 1;
  while (tw < kReduceWarps && 32 * tw < nvec && (long long)num_ctas * kReduceWarps >= (long long)nrows * tw * 2) tw <<= 1;
  const int vpl = (nvec + 32 * tw - 1) / (32 * tw);
  const int teams_per_cta = kReduceWarps / tw;
  const int team = warp / tw, wt = warp - team * tw;
  const int gteam = cta * teams_per_cta + team, num_teams = num_ctas * teams_per_cta;
  const uint32_t n = call_number(c);
  const int teams_with_rows = min(num_teams, nrows);
  if (cta * teams_per_cta >= nrows) return;  // no row for any team of this CTA: nothing to wait for either
  {
    // lanes 0..world-1 of warp 0 wait for one source rank each; the other reduce warps wait at a barrier
    trace_mark(a, 2);
    if (warp == 0) {
      bool ok = true;
      if (lane < c.world) ok = wait_flag(comm_counter(c, c.rank, push_flag_index(n, lane)), n, a.wait_cycles, sys);
      ok = __all_sync(0xffffffffu, ok);
      if (lane == 0 && !ok) record_status(c, CS_TIMEOUT_PUSH);
    }
    team_barrier(15, 32 * kReduceWarps);
    trace_mark(a, 3);
    // (after a timeout the warps still walk their rows -- the status word tells the host that the
    //  results are not to be used -- so that every rank keeps counting the same arrivals)
  }
  if (gteam >= nrows) return;
  if (vpl <= 1) reduce_rows<T, 1>(c, a, n, gteam, num_teams, tw, team, wt, lane, warp, row0, nrows, s_ss);
  else if (vpl <= 2) reduce_rows<T, 2>(c, a, n, gteam, num_teams, tw, team, wt, lane, warp, row0, nrows, s_ss);
  else if (vpl <= 4 || MAXVPL <= 4) reduce_rows<T, 4>(c, a, n, gteam, num_teams, tw, team, wt, lane, warp, row0, nrows, s_ss);
  else reduce_rows<T, (MAXVPL > 4 ? 8 : 4)>(c, a, n, gteam, num_teams, tw, team, wt, lane, warp, row0, nrows, s_ss);
  if (a.one_shot) return;  // every rank has finished all rows itself: nothing to tell, nothing to gather
  // publish: the team is counted locally (a release increment after the team's barrier covers the
  // stores of all its warps), and the team that completes the count tells every peer, with one remote
  // release store each, that this rank's rows are done
  if (tw > 1) team_barrier(1 + team, 32 * tw); else __syncwarp();
  if (wt == 0) {
    uint32_t cnt = 0;
    if (lane == 0) cnt = arrive_acq_rel(comm_counter(c, c.rank, CC_LOCAL_DONE)) + 1u;
    cnt = __shfl_sync(0xffffffffu, cnt, 0);
    __syncwarp();  // lane 0's acquire is ordered before the other lanes' release stores
    if (cnt == (uint32_t)teams_with_rows && lane < c.world && lane != c.rank)
      st_release(comm_counter(c, lane, done_flag_index(n, c.rank)), n, sys);
  }
}

// Bring the rows other ranks own into this rank's heap (and the caller's tensors).  The CTAs split
// into one group per peer; a group waits for its peer's done flag only, then copies that peer's rows
// with up to 8 loads in flight per thread.  Called by all threads of every CTA.
template <typename T>
__device__ void gather_phase(const CommView& c, const ReduceArgs& a, int cta, int num_ctas) {
  constexpr int N = Vec16<T>::N;
  constexpr int U = 8;
  __shared__ int s_ok;
  const int others = c.world - 1;
  if (others == 0 || a.one_shot) return;
  const int nvec = a.H / N;
  const uint32_t n = call_number(c);
  const int groups = min(others, num_ctas);
  const int group = cta % groups, rank_in_group = cta / groups;
  const int ctas_in_group = (num_ctas - group + groups - 1) / groups;
  const bool pull_resid = a.norm_w != nullptr && a.write_resid_all;
  for (int j = group; j < others; j += groups) {
    const int o = (c.rank + 1 + j) % c.world;
    const int r0 = o * a.rows_per_rank;
    const int nr = min(a.rows_per_rank, a.T - r0);
    if (nr <= 0) continue;
    if (threadIdx.x == 0) {
      const bool ok = wait_flag(comm_counter(c, c.rank, done_flag_index(n, o)), n, a.wait_cycles, true);
      if (!ok) record_status(c, CS_TIMEOUT_DONE);
      s_ok = ok ? 1 : 0;
    }
    __syncthreads();
    const bool ok = s_ok != 0;
    __syncthreads();  // s_ok may be rewritten for the next peer
    if (!ok) return;
    const size_t base = (size_t)r0 * a.H;
    const T* src_out = (const T*)(c.heap[o] + c.out_off[a.set]) + base;
    const T* src_res = (const T*)(c.heap[o] + c.resid_off[a.set]) + base;
    T* dst_out = (T*)(c.heap[c.rank] + c.out_off[a.set]) + base;
    T* dst_res = (T*)(c.heap[c.rank] + c.resid_off[a.set]) + base;
    T* cp_out = a.out_copy ? (T*)a.out_copy + base : nullptr;
    T* cp_res = (pull_resid && a.resid_copy) ? (T*)a.resid_copy + base : nullptr;
    const size_t total = (size_t)nr * nvec;
    const size_t stride = (size_t)ctas_in_group * blockDim.x;
    for (size_t i0 = (size_t)rank_in_group * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
      Vec16<T> y[U], z[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + stride * u;
        if (i < total) {
          y[u] = ldcg16(src_out + i * N);
          if (pull_resid) z[u] = ldcg16(src_res + i * N);
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const size_t i = i0 + stride * u;
        if (i < total) {
          st16(dst_out + i * N, y[u]);
          if (cp_out) st16(cp_out + i * N, y[u]);
          if (pull_resid) {
            st16(dst_res + i * N, z[u]);
            if (cp_res) st16(cp_res + i * N, z[u]);
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------- multicast (NVLS) scheme
// Rows of one owner, one CTA per row at a time (all kReduceWarps warps share the row).  The
// multimem.ld_reduce of a CTA's NEXT row is in flight while the current one is normalised.
template <typename T, int VPL>
__device__ __forceinline__ void mc_reduce_rows(const CommView& c, const ReduceArgs& a, uint32_t n, int cta, int num_ctas,
                                               int row0, int nrows, float* s_ss) {
  constexpr int N = Vec16<T>::N;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = a.H / N;
  const T* bias = (const T*)a.bias;
  const T* resid = (const T*)a.residual;
  const T* nw = (const T*)a.norm_w;
  const int vbase = warp * 32 + lane, vstep = 32 * kReduceWarps;
  const T* mc_partial = (const T*)(c.mc + c.partial_off[n & 1u]);
  T* mc_out = (T*)(c.mc + c.out_off[a.set]);
  T* mc_res = (T*)(c.mc + c.resid_off[a.set]);
  T* my_res = (T*)(c.heap[c.rank] + c.resid_off[a.set]);
  T* my_out = (T*)(c.heap[c.rank] + c.out_off[a.set]);
  Vec16<T> x[VPL];
  auto load_row = [&](size_t row_off) {
#pragma unroll
    for (int b = 0; b < VPL; ++b) {
      const int v = vbase + vstep * b;
      if (v < nvec) x[b].raw = mc_ld_reduce16<T>(mc_partial + row_off + (size_t)v * N);
    }
  };
  if (cta < nrows) load_row((size_t)(row0 + cta) * a.H);
  int parity = 0;
  for (int lr = cta; lr < nrows; lr += num_ctas, parity ^= 1) {
    const size_t row_off = (size_t)(row0 + lr) * a.H;
    Vec16<T> z[VPL];
    float ss = 0.f;
#pragma unroll
    for (int b = 0; b < VPL; ++b) {
      const int v = vbase + vstep * b;
      if (v >= nvec) continue;
      Vec16<T> rv, bv;
      if (resid) rv = ld16(resid + row_off + (size_t)v * N);
      if (bias) bv = ld16(bias + (size_t)v * N);
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = DT<T>::to_f(x[b].v[j]);
      ss += finish_vec<T>(acc, bias ? &bv : nullptr, resid ? &rv : nullptr, &z[b]);
    }
    trace_mark(a, 7);  // the row's sum has arrived from the switch
    if (lr + num_ctas < nrows) load_row((size_t)(row0 + lr + num_ctas) * a.H);
#pragma unroll
    for (int b = 0; b < VPL; ++b) {
      const int v = vbase + vstep * b;
      if (v >= nvec) continue;
      const size_t e = row_off + (size_t)v * N;
      if (a.mc_pull && (!nw || a.write_resid_all)) {
        st16((nw ? my_res : my_out) + e, z[b]);            // kept here; the peers pull it
        T* zc = (T*)(nw ? a.resid_copy : a.out_copy);
        if (zc) st16(zc + e, z[b]);
      } else if (!nw) {
        mc_st16(mc_out + e, z[b].raw);                     // z is the primary result: every rank gets it
      } else if (a.write_resid_all) {
        mc_st16(mc_res + e, z[b].raw);
      } else {
        st16(my_res + e, z[b]);                            // the new residual stays with the owner of the row
        if (a.resid_copy) st16((T*)a.resid_copy + e, z[b]);
      }
    }
    if (nw) {
      Vec16<T> w[VPL];
#pragma unroll
      for (int b = 0; b < VPL; ++b) {
        const int v = vbase + vstep * b;
        if (v < nvec) w[b] = ld16(nw + (size_t)v * N);
      }
      ss = warp_sum(ss);
      if (lane == 0) s_ss[parity * kReduceWarps + warp] = ss;  // two sets of slots: no second barrier per row
      team_barrier(14, 32 * kReduceWarps);
      ss = 0.f;
#pragma unroll
      for (int i = 0; i < kReduceWarps; ++i) ss += s_ss[parity * kReduceWarps + i];
      const float inv = rsqrtf(ss / (float)a.H + a.eps);
#pragma unroll
      for (int b = 0; b < VPL; ++b) {
        const int v = vbase + vstep * b;
        if (v >= nvec) continue;
        Vec16<T> y;
#pragma unroll
        for (int j = 0; j < N; ++j)
          y.v[j] = DT<T>::from_f(rt<T>(DT<T>::to_f(z[b].v[j]) * inv) * DT<T>::to_f(w[b].v[j]));
        if (a.mc_pull) {
          st16(my_out + row_off + (size_t)v * N, y);
          if (a.out_copy) st16((T*)a.out_copy + row_off + (size_t)v * N, y);
        } else {
          mc_st16(mc_out + row_off + (size_t)v * N, y.raw);
        }
      }
    }
    trace_mark(a, 8);  // the finished row has been issued to the switch
  }
}

// Multicast scheme, last step: every owner's rows have arrived in this rank's heap once its done flag has.
// Then the caller's own tensors are filled, if it asked for copies (the heap regions are the primary
// location).  Called by all threads of every CTA.
template <typename T>
__device__ void mc_wait_all_done(const CommView& c, const ReduceArgs& a, uint32_t n, int cta, int num_ctas) {
  constexpr int N = Vec16<T>::N;
  __shared__ int s_ok;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nvec = a.H / N;
  if (warp == 0) {
    bool ok = true;
    if (lane < c.world && lane * a.rows_per_rank < a.T)
      ok = wait_flag(comm_counter(c, c.rank, done_flag_index(n, lane)), n, a.wait_cycles, true);
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
      if (!ok) record_status(c, CS_TIMEOUT_DONE);
      s_ok = ok ? 1 : 0;
    }
  }
  __syncthreads();
  if (!s_ok) return;
  const bool copy_res = a.resid_copy && a.norm_w && a.write_resid_all;
  if (a.out_copy || copy_res) {
    const T* src_out = (const T*)(c.heap[c.rank] + c.out_off[a.set]);
    const T* src_res = (const T*)(c.heap[c.rank] + c.resid_off[a.set]);
    const size_t total = (size_t)a.T * nvec;
    const size_t stride = (size_t)num_ctas * blockDim.x;
    for (size_t i = (size_t)cta * blockDim.x + threadIdx.x; i < total; i += stride) {
      if (a.out_copy) st16((T*)a.out_copy + i * N, ldcg16(src_out + i * N));
      if (copy_res) st16((T*)a.resid_copy + i * N, ldcg16(src_res + i * N));
    }
  }
}

// Reduce + publish the rows this rank owns through the multicast alias, then wait until every owner
// has published.  Called by all threads of every CTA (warps beyond kReduceWarps only take part in
// the final barrier and copy).
template <typename T, int MAXVPL>
__device__ void mc_reduce_gather_phase(const CommView& c, const ReduceArgs& a, int cta, int num_ctas) {
  constexpr int N = Vec16<T>::N;
  __shared__ float s_ss[2 * kReduceWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint32_t n = call_number(c);
  const int row0 = c.rank * a.rows_per_rank;
  const int nrows = max(0, min(a.rows_per_rank, a.T - row0));
  const int nvec = a.H / N;
  const int ctas_with_rows = min(num_ctas, nrows);
  if (warp < kReduceWarps && cta < nrows) {
    trace_mark(a, 2);
    if (warp == 0) {
      bool ok = true;
      if (lane < c.world) ok = wait_flag(comm_counter(c, c.rank, push_flag_index(n, lane)), n, a.wait_cycles, true);
      ok = __all_sync(0xffffffffu, ok);
      if (lane == 0 && !ok) record_status(c, CS_TIMEOUT_PUSH);
    }
    team_barrier(15, 32 * kReduceWarps);
    trace_mark(a, 3);
    const int vpl = (nvec + 32 * kReduceWarps - 1) / (32 * kReduceWarps);
    if (vpl <= 1) mc_reduce_rows<T, 1>(c, a, n, cta, num_ctas, row0, nrows, s_ss);
    else if (vpl <= 2) mc_reduce_rows<T, 2>(c, a, n, cta, num_ctas, row0, nrows, s_ss);
    else if (vpl <= 4 || MAXVPL <= 4) mc_reduce_rows<T, 4>(c, a, n, cta, num_ctas, row0, nrows, s_ss);
    else mc_reduce_rows<T, (MAXVPL > 4 ? 8 : 4)>(c, a, n, cta, num_ctas, row0, nrows, s_ss);
    // This CTA's multicast stores have to be performed at every rank before the done flag: the CTA's
    // warps meet, one thread fences at system scope (which covers, through the barrier, the stores of
    // the whole CTA) and counts the CTA; the CTA that completes the count publishes the flag with one
    // multicast store.
    team_barrier(15, 32 * kReduceWarps);
    if (threadIdx.x == 0) {
      if (!a.mc_pull) fence_sys();  // (local stores are covered by the flag's release)
      trace_mark(a, 9);  // this CTA's multicast stores are performed
      if (arrive_acq_rel(comm_counter(c, c.rank, CC_LOCAL_DONE)) + 1u == (uint32_t)ctas_with_rows)
        mc_st_release_u32(comm_counter_mc(c, done_flag_index(n, c.rank)), n);
    }
    trace_mark(a, 4);
  }
  if (a.mc_pull) gather_phase<T>(c, a, cta, num_ctas);  // own rows: already in place, with the caller's copies
  else mc_wait_all_done<T>(c, a, n, cta, num_ctas);
}

// The phases after the partial rows have been produced, for whichever scheme the call uses.
template <typename T, int MAXVPL>
__device__ __forceinline__ void collective_tail(const CommView& c, const ReduceArgs& a, int cta, int num_ctas) {
  if (a.use_mc) {
    mc_reduce_gather_phase<T, MAXVPL>(c, a, cta, num_ctas);
  } else {
    reduce_phase<T, MAXVPL>(c, a, cta, num_ctas);
    trace_mark(a, 4);
    gather_phase<T>(c, a, cta, num_ctas);
  }
  trace_mark(a, 5);
}

// Last step of every collective kernel, called by all threads of every CTA after their phases:
// the last CTA to get here closes the call -- it advances the call counter and clears the local
// arrival counters.  Every CTA has read the call number by then (it reads it before it can finish),
// the local counters are only touched by this rank's own kernels, and the next collective on this
// context is a later kernel on the same stream.
__device__ __forceinline__ void advance_targets(const CommView& c, const ReduceArgs& a) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    uint32_t* ticket = comm_counter(c, c.rank, CC_EXIT_TICKET);
    if (atomicAdd(ticket, 1u) == gridDim.x - 1) {
      *(volatile uint32_t*)comm_counter(c, c.rank, CC_CALLS) += 1u;
      for (int i = 0; i < kMaxRanks; ++i) *(volatile uint32_t*)comm_counter(c, c.rank, CC_LOCAL_PUSH + i) = 0u;
      *(volatile uint32_t*)comm_counter(c, c.rank, CC_LOCAL_DONE) = 0u;
      *(volatile uint32_t*)ticket = 0;
      __threadfence();
    }
  }
}

}  // namespace sb200
