// Tensor-parallel communication context (symmetric heaps mapped between the
// ranks of one node), the standalone all-reduce built on the reduce / gather
// phases of comm.cuh, and the row-parallel projection entry point that runs
// the same phases inside the GEMM kernel.
//
// Replaces the all-reduce call site of the reference,
// tensor_parallel/mappings.py:16-26 (torch.distributed.all_reduce over NCCL),
// and the sequence RowParallelLinear.forward -> all_reduce -> (+bias) ->
// residual add -> RMSNorm (tensor_parallel/layers.py:425-454,
// models/llama.py:248-254, csrc/layernorm_kernels.cu:10-35).
#include "gemm_host.cuh"

#include <new>
#include <string.h>

struct sb200_comm {
  int rank, world, device;
  size_t region_bytes, heap_bytes;
  void* heap[sb200::kMaxRanks];
  bool own_heap;
  bool ipc_opened[sb200::kMaxRanks];
  void* mc;          // multicast alias of all ranks' heaps (NVSwitch), or null
  int mc_pull;       // multicast scheme: finished rows are pulled by the peers instead of multicast-stored
  uint64_t seq;
  long long wait_cycles;
  unsigned long long* trace;
  size_t one_shot_bytes;
};

namespace sb200 {

constexpr size_t kCounterBytes = 4096;
constexpr int kRegions = 7;  // partial[2], out[2], resid[2], scratch

static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static CommView make_view(const sb200_comm* c) {
  CommView v = {};
  v.rank = c->rank;
  v.world = c->world;
  for (int i = 0; i < c->world; ++i) v.heap[i] = (char*)c->heap[i];
  v.mc = (char*)c->mc;
  size_t off = kCounterBytes;
  v.partial_off[0] = off; off += c->region_bytes;
  v.partial_off[1] = off; off += c->region_bytes;
  v.out_off[0] = off; off += c->region_bytes;
  v.out_off[1] = off; off += c->region_bytes;
  v.resid_off[0] = off; off += c->region_bytes;
  v.resid_off[1] = off; off += c->region_bytes;
  v.region_bytes = c->region_bytes;
  return v;
}
static size_t scratch_off(const sb200_comm* c) { return kCounterBytes + 6 * c->region_bytes; }

// Standalone all-reduce: copy the rows of a local tensor into the heap, then the shared phases.
template <typename T>
__global__ void __launch_bounds__(256)
all_reduce_kernel(const __grid_constant__ CommView c, const __grid_constant__ ReduceArgs a, const T* __restrict__ in,
                  const int rows_per_token) {
  // `in` is [T, rows_per_token, H]: the rows of a token are summed (fp32, rounded to T) while they are
  // copied -- rows_per_token = 1 for a plain all-reduce, top_k for the per-slot expert outputs of the
  // MoE layer (the reference's torch.sum(dim=1) before its all-reduce, fused_moe.py:539-543).
  constexpr int N = Vec16<T>::N;
  trace_mark(a, 0);
  const int nvec = a.H / N;
  const size_t total = (size_t)a.T * nvec;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  T* const partial = (T*)partial_of(c, c.rank, call_number(c));
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int t = (int)(i / nvec), v = (int)(i - (size_t)t * nvec);
    T* dst = partial + i * N;
    if (rows_per_token == 1) {
      st16(dst, ld16(in + i * N));
    } else {
      float acc[N];
#pragma unroll
      for (int j = 0; j < N; ++j) acc[j] = 0.f;
      for (int s = 0; s < rows_per_token; ++s) {
        const Vec16<T> x = ld16(in + ((size_t)t * rows_per_token + s) * a.H + (size_t)v * N);
#pragma unroll
        for (int j = 0; j < N; ++j) acc[j] += DT<T>::to_f(x.v[j]);
      }
      Vec16<T> o;
#pragma unroll
      for (int j = 0; j < N; ++j) o.v[j] = DT<T>::from_f(acc[j]);
      st16(dst, o);
    }
  }
  trace_mark(a, 1);
  __syncthreads();
  // this CTA's share of the rows is stored: one arrival per owner (or one in all when every rank reads all rows)
  if (a.one_shot || a.use_mc) { if (threadIdx.x < 32) signal_push_all(c, a); }
  else if (threadIdx.x < c.world) signal_push(c, a, threadIdx.x);
  collective_tail<T, kMaxVecPerLaneAllReduce>(c, a, blockIdx.x, gridDim.x);
  advance_targets(c, a);
  trace_mark(a, 6);
}

// All-gather of row blocks: rank r contributes rows [r * rows_per_rank, ...) of a [T, H] tensor (`in` holds just
// those rows); afterwards every rank has all T rows in its `out` region (and in out_copy).  The produce /
// reduce halves of a collective do not exist here: a rank publishes its rows -- one multimem.st per 16 bytes
// when the heaps have a multicast alias, else a local copy that the peers pull -- and flags them done.
template <typename T>
__global__ void __launch_bounds__(256)
all_gather_kernel(const __grid_constant__ CommView c, const __grid_constant__ ReduceArgs a, const T* __restrict__ in) {
  constexpr int N = Vec16<T>::N;
  const int nvec = a.H / N;
  const uint32_t n = call_number(c);
  const int row0 = c.rank * a.rows_per_rank;
  const int nrows = max(0, min(a.rows_per_rank, a.T - row0));
  const size_t total = (size_t)nrows * nvec, base = (size_t)row0 * nvec;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  T* const local_out = (T*)(c.heap[c.rank] + c.out_off[a.set]);
  T* const mc_out = a.use_mc ? (T*)(c.mc + c.out_off[a.set]) : nullptr;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const Vec16<T> v = ld16(in + i * N);
    if (mc_out) mc_st16(mc_out + (base + i) * N, v.raw);
    else st16(local_out + (base + i) * N, v);
    if (!mc_out && a.out_copy) st16((T*)a.out_copy + (base + i) * N, v);
  }
  __syncthreads();
  if (threadIdx.x == 0 && nrows > 0) {
    if (mc_out) fence_sys();  // this CTA's multicast stores are performed everywhere before the flag
    if (arrive_acq_rel(comm_counter(c, c.rank, CC_LOCAL_DONE)) + 1u == gridDim.x) {
      if (mc_out) {
        mc_st_release_u32(comm_counter_mc(c, done_flag_index(n, c.rank)), n);
      } else {
        for (int r = 0; r < c.world; ++r)
          if (r != c.rank) st_release(comm_counter(c, r, done_flag_index(n, c.rank)), n, true);
      }
    }
  }
  if (mc_out) mc_wait_all_done<T>(c, a, n, blockIdx.x, gridDim.x);
  else gather_phase<T>(c, a, blockIdx.x, gridDim.x);
  advance_targets(c, a);
}

static int all_reduce_grid(int64_t T_, int64_t H, int dtype, int rows_per_rank) {
  const int64_t nvec = H / (16 / (int64_t)dtype_size(dtype));
  int64_t g = (T_ * nvec + 1023) / 1024;
  const int64_t by_rows = (rows_per_rank + 7) / 8;
  if (g < by_rows) g = by_rows;
  if (g > sm_count()) g = sm_count();
  if (g < 1) g = 1;
  return (int)g;
}

struct CallPlan {
  ReduceArgs ra;
  CommView cv;
};

// Common argument checks + per-call bookkeeping.
static int plan_call(sb200_comm* c, int64_t T_, int64_t H, int dtype, const void* bias, const void* residual,
                     const void* norm_w, float eps, int write_resid_all, void* out_copy, void* resid_copy,
                     CallPlan* p, int max_vec_per_lane = kMaxVecPerLaneAllReduce) {
  SB_CHECK_ARG(c != nullptr, "null communication context");
  const size_t es = dtype_size(dtype);
  SB_CHECK_ARG(T_ > 0 && H > 0 && T_ <= INT32_MAX && H <= INT32_MAX, "bad shape T=%lld H=%lld", (long long)T_, (long long)H);
  SB_CHECK_ARG((H * es) % 16 == 0, "row length %lld is not a multiple of 16 bytes", (long long)H);
  SB_CHECK_ARG(H * es <= (size_t)16 * 32 * kReduceWarps * max_vec_per_lane, "row length %lld exceeds %d bytes",
               (long long)H, 16 * 32 * kReduceWarps * max_vec_per_lane);
  const int rpr = (int)((T_ + c->world - 1) / c->world);
  SB_CHECK_ARG((size_t)T_ * H * es <= c->region_bytes && (size_t)rpr * c->world * H * es <= c->region_bytes,
               "batch of %lld x %lld elements exceeds the context's region size (%zu bytes)", (long long)T_,
               (long long)H, c->region_bytes);
  SB_CHECK_ARG((!bias || aligned16(bias)) && (!residual || aligned16(residual)) && (!norm_w || aligned16(norm_w)) &&
                   (!out_copy || aligned16(out_copy)) && (!resid_copy || aligned16(resid_copy)),
               "bias / residual / norm weight / output tensors must be 16-byte aligned");
  int dev = -1;
  SB_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev == c->device, "current device %d is not the context's device %d", dev, c->device);
  ReduceArgs& a = p->ra;
  a = ReduceArgs{};
  a.T = (int)T_; a.H = (int)H; a.rows_per_rank = rpr;
  a.set = (int)(c->seq & 1);
  // one-shot while the rows every rank would have to load stay below ~4 MB (always with two ranks,
  // where both schemes move the same bytes); the owner-reduce + gather scheme above that
  a.one_shot = (c->world == 1 || (size_t)(c->world - 1) * T_ * H * es <= c->one_shot_bytes) ? 1 : 0;
  // larger ones go through the NVSwitch multicast alias when the heaps are bound to one
  a.use_mc = (!a.one_shot && c->mc != nullptr) ? 1 : 0;
  a.mc_pull = c->mc_pull;
  a.bias = bias; a.residual = residual; a.norm_w = norm_w; a.eps = eps;
  a.write_resid_all = write_resid_all;
  a.out_copy = out_copy; a.resid_copy = resid_copy;
  a.wait_cycles = c->wait_cycles;
#ifdef SB200_TRACE
  a.trace = c->trace;
#endif
  p->cv = make_view(c);
  return SB200_OK;
}

static void commit_call(sb200_comm* c, CallPlan* p, void** out_ptr, void** resid_ptr) {
  const int set = p->ra.set;
  if (out_ptr) *out_ptr = (char*)c->heap[c->rank] + p->cv.out_off[set];
  if (resid_ptr) *resid_ptr = p->ra.norm_w ? (void*)((char*)c->heap[c->rank] + p->cv.resid_off[set]) : nullptr;
  c->seq++;
}

template <typename T>
static int launch_all_reduce(const CallPlan& p, const void* in, int rows_per_token, int grid, cudaStream_t s) {
  all_reduce_kernel<T><<<grid, 256, 0, s>>>(p.cv, p.ra, (const T*)in, rows_per_token);
  SB_CHECK_LAUNCH("all_reduce_kernel");
  return SB200_OK;
}

static int do_all_reduce(sb200_comm* c, const void* in, int64_t T_, int64_t H, int dtype, const void* bias,
                         const void* residual, const void* norm_w, float eps, int write_resid_all, void* out_copy,
                         void* resid_copy, cudaStream_t s, void** out_ptr, void** resid_ptr, int rows_per_token = 1) {
  CallPlan p;
  int rc = plan_call(c, T_, H, dtype, bias, residual, norm_w, eps, write_resid_all, out_copy, resid_copy, &p);
  if (rc) return rc;
  SB_CHECK_ARG(in && aligned16(in), "all_reduce: input must be a 16-byte aligned device pointer");
  const int grid = all_reduce_grid(T_, H, dtype, p.ra.rows_per_rank);
  for (int o = 0; o < c->world; ++o) p.ra.push_expected[o] = (uint32_t)grid;  // every CTA reports once (per owner)
  commit_call(c, &p, out_ptr, resid_ptr);
  SB_DISPATCH_FLOAT(dtype, return (launch_all_reduce<scalar_t>(p, in, rows_per_token, grid, s)));
  return SB200_OK;
}

}  // namespace sb200

using namespace sb200;

extern "C" int64_t sb200_comm_heap_bytes(int64_t region_bytes) {
  return (int64_t)(kCounterBytes + kRegions * round_up((size_t)region_bytes, 1024));
}

static int comm_new(sb200_comm** out, int rank, int world, int64_t region_bytes) {
  SB_CHECK_ARG(out != nullptr, "comm_create: null output");
  SB_CHECK_ARG(world >= 1 && world <= kMaxRanks && rank >= 0 && rank < world, "comm_create: bad rank %d / world %d (max %d ranks)",
               rank, world, kMaxRanks);
  SB_CHECK_ARG(region_bytes > 0, "comm_create: region_bytes must be positive");
  sb200_comm* c = new (std::nothrow) sb200_comm();
  SB_CHECK_ARG(c != nullptr, "comm_create: out of host memory");
  memset(c, 0, sizeof(*c));
  c->rank = rank; c->world = world;
  c->region_bytes = round_up((size_t)region_bytes, 1024);
  c->heap_bytes = kCounterBytes + kRegions * c->region_bytes;
  c->wait_cycles = 5 * ptx::kWaitLimitCycles;  // ~10 s: ranks of a serving engine can be seconds apart on the host (first steps, GC)
  c->one_shot_bytes = 4u << 20;
  if (const char* e = getenv("SB200_ONE_SHOT_BYTES")) c->one_shot_bytes = (size_t)atoll(e);
  if (const char* e = getenv("SB200_MC_PULL")) c->mc_pull = atoi(e) != 0 ? 1 : 0;
  if (const char* e = getenv("SB200_WAIT_LIMIT_CYCLES")) { const long long v = atoll(e); if (v > 0) c->wait_cycles = v; }
  if (cudaGetDevice(&c->device) != cudaSuccess) { delete c; set_error("comm_create: no current CUDA device"); return SB200_ERR_CUDA; }
  *out = c;
  return SB200_OK;
}

extern "C" int sb200_comm_create(sb200_comm** out, int rank, int world, int64_t region_bytes) {
  int rc = comm_new(out, rank, world, region_bytes);
  if (rc) return rc;
  sb200_comm* c = *out;
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, c->heap_bytes);
  if (e == cudaSuccess) e = cudaMemset(p, 0, c->heap_bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    if (p) cudaFree(p);
    delete c; *out = nullptr;
    return cuda_fail(e, "comm_create: allocating the symmetric heap");
  }
  c->heap[rank] = p;
  c->own_heap = true;
  return SB200_OK;
}

extern "C" int sb200_comm_create_external(sb200_comm** out, int rank, int world, int64_t region_bytes,
                                          void* const* heaps) {
  SB_CHECK_ARG(heaps != nullptr, "comm_create_external: null heap table");
  int rc = comm_new(out, rank, world, region_bytes);
  if (rc) return rc;
  sb200_comm* c = *out;
  for (int i = 0; i < world; ++i) {
    if (!heaps[i] || !aligned16(heaps[i])) { delete c; *out = nullptr; set_error("comm_create_external: heap %d is null or misaligned", i); return SB200_ERR_INVALID_ARGUMENT; }
    c->heap[i] = heaps[i];
  }
  c->own_heap = false;
  return SB200_OK;
}

extern "C" int sb200_comm_ipc_handle(sb200_comm* c, void* handle_out) {
  SB_CHECK_ARG(c && handle_out && c->own_heap, "comm_ipc_handle: context does not own its heap");
  static_assert(sizeof(cudaIpcMemHandle_t) == SB200_IPC_HANDLE_BYTES, "IPC handle size");
  cudaIpcMemHandle_t h;
  SB_CUDA(cudaIpcGetMemHandle(&h, c->heap[c->rank]));
  memcpy(handle_out, &h, sizeof(h));
  return SB200_OK;
}

extern "C" int sb200_comm_open_peers(sb200_comm* c, const void* handles) {
  SB_CHECK_ARG(c && handles && c->own_heap, "comm_open_peers: bad arguments");
  for (int i = 0; i < c->world; ++i) {
    if (i == c->rank || c->heap[i]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, (const char*)handles + (size_t)i * sizeof(h), sizeof(h));
    void* p = nullptr;
    SB_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->heap[i] = p;
    c->ipc_opened[i] = true;
  }
  return SB200_OK;
}

extern "C" int sb200_comm_destroy(sb200_comm* c) {
  if (!c) return SB200_OK;
  for (int i = 0; i < c->world; ++i)
    if (c->ipc_opened[i] && c->heap[i]) cudaIpcCloseMemHandle(c->heap[i]);
  if (c->own_heap && c->heap[c->rank]) cudaFree(c->heap[c->rank]);
  delete c;
  return SB200_OK;
}

extern "C" void* sb200_comm_local_heap(sb200_comm* c) { return c ? c->heap[c->rank] : nullptr; }
extern "C" void* sb200_comm_scratch(sb200_comm* c) { return c ? (char*)c->heap[c->rank] + scratch_off(c) : nullptr; }
extern "C" int64_t sb200_comm_region_bytes(sb200_comm* c) { return c ? (int64_t)c->region_bytes : 0; }

extern "C" int sb200_comm_set_wait_limit(sb200_comm* c, int64_t cycles) {
  SB_CHECK_ARG(c && cycles > 0, "comm_set_wait_limit: bad arguments");
  c->wait_cycles = cycles;
  return SB200_OK;
}

extern "C" int sb200_comm_set_one_shot_bytes(sb200_comm* c, int64_t bytes) {
  SB_CHECK_ARG(c && bytes >= 0, "comm_set_one_shot_bytes: bad arguments");
  c->one_shot_bytes = (size_t)bytes;
  return SB200_OK;
}

extern "C" int sb200_comm_set_multicast(sb200_comm* c, void* multicast_base) {
  SB_CHECK_ARG(c, "comm_set_multicast: null context");
  SB_CHECK_ARG(multicast_base == nullptr || (c->world > 1 && aligned16(multicast_base)),
               "comm_set_multicast: needs a 16-byte aligned address and more than one rank");
  c->mc = multicast_base;
  return SB200_OK;
}

extern "C" int sb200_comm_has_multicast(sb200_comm* c) { return (c && c->mc) ? 1 : 0; }

// Back to the state of a fresh context: control words (call counter, flags, arrival counters, status) and the
// arrival counters of the split-K workspace.  Every rank has to call it, with no collective in flight anywhere
// (host barrier before and after), e.g. after a wait on a peer ran out and left the ranks' counters out of step.
extern "C" int sb200_comm_reset(sb200_comm* c, sb200_stream_t stream) {
  SB_CHECK_ARG(c, "comm_reset: null context");
  cudaStream_t s = (cudaStream_t)stream;
  SB_CUDA(cudaMemsetAsync(c->heap[c->rank], 0, kCounterBytes, s));
  SB_CUDA(cudaMemsetAsync((char*)c->heap[c->rank] + scratch_off(c), 0, kWsCounterBytes, s));
  SB_CUDA(cudaStreamSynchronize(s));
  c->seq = 0;
  return SB200_OK;
}

#ifdef SB200_TRACE
extern "C" int sb200_comm_set_trace(sb200_comm* c, void* device_buffer) {
  SB_CHECK_ARG(c, "comm_set_trace: null context");
  c->trace = (unsigned long long*)device_buffer;
  return SB200_OK;
}
#endif

extern "C" int sb200_comm_status(sb200_comm* c, sb200_stream_t stream, uint32_t* host_status) {
  SB_CHECK_ARG(c && host_status, "comm_status: bad arguments");
  uint32_t* w = reinterpret_cast<uint32_t*>(c->heap[c->rank]) + CC_STATUS;
  SB_CUDA(cudaMemcpyAsync(host_status, w, sizeof(uint32_t), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  SB_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
  if (*host_status != 0) {
    set_error("device-side wait timed out (code %u: %s)", *host_status,
              *host_status == CS_TIMEOUT_MBARRIER ? "GEMM pipeline barrier"
              : *host_status == CS_TIMEOUT_PUSH   ? "partial rows from a peer did not arrive"
                                                  : "finished rows from a peer did not arrive");
    return SB200_ERR_PEER_TIMEOUT;
  }
  return SB200_OK;
}

extern "C" int sb200_comm_clear_status(sb200_comm* c, sb200_stream_t stream) {
  SB_CHECK_ARG(c, "comm_clear_status: null context");
  uint32_t* w = reinterpret_cast<uint32_t*>(c->heap[c->rank]) + CC_STATUS;
  SB_CUDA(cudaMemsetAsync(w, 0, sizeof(uint32_t), (cudaStream_t)stream));
  return SB200_OK;
}

extern "C" int sb200_all_reduce(sb200_comm* comm, const void* in, int64_t T, int64_t H, int dtype, const void* bias,
                                const void* residual, const void* norm_w, float eps, int write_resid_all,
                                void* out_copy, void* resid_copy, sb200_stream_t stream, void** out_ptr,
                                void** resid_ptr) {
  return do_all_reduce(comm, in, T, H, dtype, bias, residual, norm_w, eps, write_resid_all, out_copy, resid_copy,
                       (cudaStream_t)stream, out_ptr, resid_ptr);
}

extern "C" int sb200_all_gather_rows(sb200_comm* comm, const void* in_rows, int64_t T, int64_t H, int dtype,
                                     void* out_copy, sb200_stream_t stream, void** out_ptr) {
  CallPlan p;
  int rc = plan_call(comm, T, H, dtype, nullptr, nullptr, nullptr, 0.f, 0, out_copy, nullptr, &p);
  if (rc) return rc;
  const int rpr = p.ra.rows_per_rank;
  const int64_t own = T - (int64_t)comm->rank * rpr < rpr ? T - (int64_t)comm->rank * rpr : rpr;
  SB_CHECK_ARG(own <= 0 || (in_rows && aligned16(in_rows)), "all_gather_rows: this rank's rows must be a 16-byte aligned device pointer");
  p.ra.one_shot = 0;                       // rows always travel from their owner
  p.ra.use_mc = comm->mc != nullptr ? 1 : 0;
  int64_t g = ((own > 0 ? own : 1) * (H / (16 / (int64_t)dtype_size(dtype))) + 1023) / 1024;
  if (comm->world > 1 && g < comm->world - 1) g = comm->world - 1;  // the pulling scheme wants a CTA group per peer
  if (g > sm_count()) g = sm_count();
  if (g < 1) g = 1;
  commit_call(comm, &p, out_ptr, nullptr);
  cudaStream_t s = (cudaStream_t)stream;
  SB_DISPATCH_FLOAT(dtype, all_gather_kernel<scalar_t><<<(int)g, 256, 0, s>>>(p.cv, p.ra, (const scalar_t*)in_rows));
  SB_CHECK_LAUNCH("all_gather_kernel");
  return SB200_OK;
}

extern "C" int sb200_moe_sum_all_reduce(sb200_comm* comm, const void* in3, const void* residual, int64_t T, int top_k,
                                        int64_t H, int dtype, void* out_copy, sb200_stream_t stream, void** out_ptr) {
  SB_CHECK_ARG(top_k >= 1, "moe_sum_all_reduce: top_k must be positive");
  return do_all_reduce(comm, in3, T, H, dtype, nullptr, residual, nullptr, 0.f, 0, out_copy, nullptr,
                       (cudaStream_t)stream, out_ptr, nullptr, top_k);
}

extern "C" int sb200_gemm_rowpar(sb200_comm* comm, const void* x, int64_t ldx, const void* w, int64_t ldw, int64_t T,
                                 int64_t N, int64_t K, int dtype, const void* bias, const void* residual,
                                 const void* norm_w, float eps, int write_resid_all, void* out_copy, void* resid_copy,
                                 int tile_cfg, sb200_stream_t stream, void** out_ptr, void** resid_ptr) {
  SB_CHECK_ARG(comm && x && w, "gemm_rowpar: null pointer");
  SB_CHECK_ARG(T > 0 && N > 0 && K > 0 && K <= INT32_MAX, "gemm_rowpar: bad shape T=%lld N=%lld K=%lld", (long long)T,
               (long long)N, (long long)K);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == SB200_F32) {
    // fp32: FFMA GEMM into the context's scratch region, then the standalone all-reduce phases.
    // (the first kWsCounterBytes of the scratch region are the split-K counters of the tensor-core path)
    SB_CHECK_ARG((size_t)T * N * 4 + kWsCounterBytes <= comm->region_bytes,
                 "gemm_rowpar: batch exceeds the context's region size");
    float* tmp = (float*)((char*)sb200_comm_scratch(comm) + kWsCounterBytes);
    int rc = run_gemm_f32(tmp, N, (const float*)x, ldx, (const float*)w, ldw, nullptr, (int)T, (int)N, (int)K, s);
    if (rc) return rc;
    return do_all_reduce(comm, tmp, T, N, dtype, bias, residual, norm_w, eps, write_resid_all, out_copy, resid_copy,
                         s, out_ptr, resid_ptr);
  }
  CallPlan p;
  int rc = plan_call(comm, T, N, dtype, bias, residual, norm_w, eps, write_resid_all, out_copy, resid_copy, &p,
                     kMaxVecPerLaneGemm);
  if (rc) return rc;
  SB_CHECK_ARG(N % 8 == 0, "gemm_rowpar: output width must be a multiple of 8");
  // split-K partial tiles live in the context's scratch region (its counters stay zero between launches)
  void* ws = sb200_comm_scratch(comm);
  const GemmPlan plan = plan_gemm(EPI_PUSH, T, N, K, 0, tile_cfg, comm->region_bytes);
  SB_CHECK_ARG(plan.bn != 0, "gemm_rowpar: bad tile configuration %d", tile_cfg);
  // arrivals this rank's kernel reports for each owner's rows (the arrival that completes a count
  // sends that owner its flag)
  const int rpr = p.ra.rows_per_rank;
  for (int o = 0; o < comm->world; ++o) {
    const int64_t lo = (int64_t)o * rpr, hi = (lo + rpr < T ? lo + rpr : T);
    p.ra.push_expected[o] = gemm_push_increments(plan, T, lo, hi);
  }
  if (p.ra.one_shot || p.ra.use_mc) p.ra.push_expected[0] = gemm_push_increments(plan, T, 0, T);  // one arrival per finished (tile, 32-row slot)
  GemmArgs g = {};
  g.M = (int)T; g.N = (int)N; g.K = (int)K;
  g.head_size = 128;
  // validate the operands before touching the epoch bookkeeping (a failed call must not desynchronise ranks)
  CUtensorMap probe;
  rc = make_tmap_2d(&probe, dtype, x, T, K, ldx, 128, kBK);
  if (rc) return rc;
  rc = make_tmap_2d(&probe, dtype, w, N, K, ldw, plan.cta2 ? plan.bn / 2 : plan.bn, kBK);
  if (rc) return rc;
  commit_call(comm, &p, out_ptr, resid_ptr);
  return run_gemm_sm100(dtype, EPI_PUSH, plan, x, ldx, w, ldw, g, ws, p.cv, p.ra, s);
}
