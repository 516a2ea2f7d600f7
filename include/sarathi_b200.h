/* C ABI of libsarathi_b200.so -- the B200 (sm_100a) implementation of the
 * tensor-parallel decoder-layer path of Sarathi-Serve.
 *
 * Conventions
 *   - Every entry point returns 0 (SB200_OK) or a positive status code;
 *     sb200_last_error() returns a human-readable message for the calling
 *     thread's last failure.
 *   - All pointers are DEVICE pointers unless named host_*; the caller owns
 *     every buffer; no entry point allocates device memory unless it says so.
 *   - `stream` is a cudaStream_t passed as void* (0 = the legacy default
 *     stream).  Kernels are launched on it and nothing is synchronised.
 *   - The current CUDA device of the calling thread must be the device that
 *     owns the buffers (the reference's ops install no device guard either).
 *   - dtype ids: SB200_F32 / SB200_F16 / SB200_BF16.
 *   - "reference" citations are paths inside the microsoft/sarathi-serve tree.
 */
#ifndef SARATHI_B200_H_
#define SARATHI_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* sb200_stream_t;

enum sb200_dtype { SB200_F32 = 0, SB200_F16 = 1, SB200_BF16 = 2 };
enum sb200_itype { SB200_I32 = 0, SB200_I64 = 1, SB200_I16 = 2, SB200_I8 = 3, SB200_U8 = 4 };

enum sb200_status {
  SB200_OK = 0,
  SB200_ERR_INVALID_ARGUMENT = 1, /* bad pointer / shape / stride / alignment */
  SB200_ERR_UNSUPPORTED = 2,      /* dtype or shape outside what the kernels cover */
  SB200_ERR_CUDA = 3,             /* a CUDA runtime / driver call failed */
  SB200_ERR_PEER_TIMEOUT = 4,     /* a bounded device-side wait on a peer or barrier ran out */
  SB200_ERR_NOT_INITIALISED = 5
};

/* Message for the last non-zero status returned to this thread. */
const char* sb200_last_error(void);
/* Library version string. */
const char* sb200_version(void);

/* ------------------------------------------------------------------ norms */

/* out[t,:] = ((T)(x[t,:] * rsqrt(mean(x[t,:]^2) + eps))) * w      (statistics in fp32).
 * Replaces: layernorm_ops.rms_norm -- csrc/layernorm.cpp:3-13,
 * csrc/layernorm_kernels.cu:10-62 (called from
 * sarathi/model_executor/layers/layernorm.py:31-40).
 * x, out: [T, H] contiguous rows; w: [H]. */
int sb200_rms_norm(void* out, const void* x, const void* w, float eps,
                   int64_t T, int64_t H, int dtype, sb200_stream_t stream);

/* z = (T)(x + residual); residual_out = z; out = rms_norm(z, w, eps).
 * Replaces the pair "hidden = residual + hidden" + RMSNorm of the decoder layer:
 * sarathi/model_executor/models/llama.py:248-252,254 (torch add, then
 * csrc/layernorm_kernels.cu:10-35).  residual_out may alias residual or x. */
int sb200_fused_add_rms_norm(void* out, void* residual_out, const void* x, const void* residual,
                             const void* w, float eps, int64_t T, int64_t H, int dtype,
                             sb200_stream_t stream);

/* ------------------------------------------------------------ activations */

/* out[t,i] = ((T) silu(in[t,i])) * in[t,d+i]; in: [T, 2d], out: [T, d].
 * Replaces: activation_ops.silu_and_mul -- csrc/activation.cpp:3-5,
 * csrc/activation_kernels.cu:8-48. */
int sb200_silu_and_mul(void* out, const void* in, int64_t T, int64_t d, int dtype,
                       sb200_stream_t stream);
/* Element-wise tanh-approximated GELUs on [T, d].
 * Replace: activation_ops.gelu_new / gelu_fast -- csrc/activation_kernels.cu:53-112. */
int sb200_gelu_new(void* out, const void* in, int64_t T, int64_t d, int dtype, sb200_stream_t stream);
int sb200_gelu_fast(void* out, const void* in, int64_t T, int64_t d, int dtype, sb200_stream_t stream);

/* ------------------------------------------------------------------ rotary */

/* In-place rotary embedding of query [T, nq*head_size] and key [T, nkv*head_size]
 * whose rows are q_stride / k_stride ELEMENTS apart (views into a fused qkv
 * buffer are fine).  cos_sin_cache: [max_pos, rot_dim] = cos(rot_dim/2) | sin(rot_dim/2)
 * in the same dtype; positions: int64 [T].  is_neox != 0 pairs (i, i+rot_dim/2),
 * otherwise (2i, 2i+1).
 * Replaces: pos_encoding_ops.rotary_embedding -- csrc/pos_encoding.cpp:3-15,
 * csrc/pos_encoding_kernels.cu:8-127. */
int sb200_rotary_embedding(const int64_t* positions, void* query, void* key, int64_t T,
                           int num_heads, int num_kv_heads, int head_size, int rot_dim,
                           int64_t q_stride, int64_t k_stride, const void* cos_sin_cache,
                           int is_neox, int dtype, sb200_stream_t stream);

/* -------------------------------------------------------------- MoE routing */

/* Softmax over E experts in fp32, then k rounds of arg-max (ties -> lowest
 * index).  gating: [T, E] in gating_dtype (fp32 reproduces the reference op;
 * fp16/bf16 fold in the reference's `.float()` cast, fused_moe.py:367).
 * topk_weights: fp32 [T,k]; topk_ids, token_expert_indices: int32 [T,k]
 * (token_expert_indices[t,j] = j*T + t; may be NULL).  renormalize != 0 divides
 * each row of weights by its sum (fused_moe.py:371-372).  Any E is accepted
 * (powers of two <= 256 take the warp-level path); no workspace is needed.
 * Replaces: moe_ops.topk_softmax -- csrc/moe.cpp:3-8,
 * csrc/moe_topk_softmax_kernels.cu:50-166,182-380,421-503. */
int sb200_topk_softmax(float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices,
                       const void* gating, int gating_dtype, int64_t T, int E, int k,
                       int renormalize, sb200_stream_t stream);

/* Stable counting sort of the flat (token, k) slots by expert, each expert's
 * segment padded to a multiple of block_size.  sorted_token_ids (capacity
 * sorted_capacity >= numel + min(E,numel)*(block_size-1)) is fully written: slot
 * indices in the defined prefix, `numel` as the pad value everywhere else (the
 * reference pre-fills it in Python, fused_moe.py:191-195).  expert_ids[b] is
 * written for b < num_tokens_post_pad/block_size.  Ids outside [0, E) are
 * skipped.  `scratch` (device, sb200_moe_align_scratch_bytes() bytes) is
 * optional: with it, inputs above 8192 slots are spread over many CTAs;
 * without it one CTA does the whole sort in shared memory.
 * Replaces: moe_ops.moe_align_block_size -- csrc/moe.cpp:10-17,
 * csrc/moe_align_block_size_kernels.cu:23-135. */
int sb200_moe_align_block_size(const void* topk_ids, int ids_itype, int64_t numel, int num_experts,
                               int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                               int32_t* expert_ids, int64_t expert_ids_capacity,
                               int32_t* num_tokens_post_pad, void* scratch, int64_t scratch_bytes,
                               sb200_stream_t stream);
/* Bytes of scratch the multi-CTA path of sb200_moe_align_block_size wants. */
int64_t sb200_moe_align_scratch_bytes(int64_t numel, int num_experts);

/* Same sort and same outputs as sb200_moe_align_block_size, for callers that can neither
 * pass a scratch buffer nor allocate one (a worker whose GPU memory is already committed
 * to its KV cache, code that must not trigger the device-wide synchronisation of
 * cudaMalloc / cudaFree, a plugin boundary that forwards only inputs and outputs).  It calls
 * no allocator: its per-segment counters live in a fixed array inside the library image
 * (about 258 KiB held by every GPU that loads the library, until the process exits).
 * Limits: numel <= SB200_ALIGN_NOALLOC_MAX_SLOTS and num_experts <=
 * SB200_ALIGN_NOALLOC_MAX_EXPERTS, otherwise SB200_ERR_UNSUPPORTED.  All calls on a device
 * share that array: calls that overlap on the GPU race, so keep them on one stream or
 * order them.  The first call on each device resolves the array's device address; make it
 * outside any stream capture.
 * This entry point has no counterpart in the reference. */
#define SB200_ALIGN_NOALLOC_MAX_SLOTS 65536
#define SB200_ALIGN_NOALLOC_MAX_EXPERTS 256
int sb200_moe_align_block_size_noalloc(const void* topk_ids, int ids_itype, int64_t numel, int num_experts,
                                       int block_size, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                       int32_t* expert_ids, int64_t expert_ids_capacity,
                                       int32_t* num_tokens_post_pad, sb200_stream_t stream);

/* ------------------------------------------------- column-parallel projections */

enum sb200_epilogue {
  SB200_EPI_NONE = 0,     /* out = x * w^T (+ bias) */
  SB200_EPI_ROTARY = 1,   /* qkv projection with the rotary embedding of q and k applied in the epilogue */
  SB200_EPI_SILU_MUL = 2  /* gate_up projection with silu(gate) * up applied in the epilogue */
};

typedef struct sb200_rotary_args {
  const int64_t* positions;   /* int64 [T] */
  const void* cos_sin_cache;  /* [max_pos, rot_dim], output dtype */
  int head_size;              /* 64, 128 or 256 */
  int rot_dim;                /* must equal head_size for the fused epilogue */
  int rot_cols;               /* output columns [0, rot_cols) are q and k heads; the rest (v) pass through */
  int is_neox;
  /* Optional: also append this step's keys and values to the paged KV cache from the epilogue (what the
   * reference's attention wrapper does with three .contiguous() copies and flashinfer's
   * append_paged_kv_cache, attention/flashinfer_attention_wrapper.py:253-270).  kv_cache NULL: off. */
  void* kv_cache;             /* [pages, 2, page_size, kv_heads, head_size], output dtype */
  const int64_t* kv_slots;    /* [T] from sb200_kv_cache_slots (-1: token not stored) */
  int kv_page_size;
  int num_kv_heads;           /* k columns are [rot_cols - num_kv_heads * head_size, rot_cols), v columns the next
                                 num_kv_heads * head_size */
} sb200_rotary_args;

/* out[T, N] = x[T, K] * w[N, K]^T: the local matmul of a ColumnParallelLinear /
 * ReplicatedLinear shard (w is the nn.Linear weight [out_features/tp, in_features],
 * row-major, used as is).  ldx / ldw / ldo are row strides in elements.
 * bf16 / fp16 run on tcgen05 tensor cores with fp32 accumulation; fp32 runs a plain
 * FFMA kernel and supports SB200_EPI_NONE only.
 *   SB200_EPI_ROTARY   : additionally applies rotary_embedding to the q / k heads
 *                        (out is the fused qkv buffer [T, N]).
 *   SB200_EPI_SILU_MUL : w holds the gate shard in rows [0, N/2) and the up shard in
 *                        rows [N/2, N); out is [T, N/2].
 * residual / ldr: optional [T, N] tensor (row stride ldr) added to the rounded product in the
 *   epilogue of the plain bf16 / fp16 kernel: out = residual + round(x w^T (+ bias)) -- the
 *   `hidden_states = residual + hidden_states` that follows a row-parallel projection when there is
 *   nothing to reduce (tensor-parallel size 1), models/llama.py:248,254.  NULL: none.
 * status: optional device word that receives a non-zero code if a bounded
 * pipeline wait inside the kernel ran out.
 * tile_cfg: 0 = let the library choose the tile shape, else
 *   BN + 1000*MODE + 100000*S  (BN = tile columns 32..256 step 32; MODE = 1|2: one CTA
 *   with 1|2 accumulators of 128 rows; MODE = 3|4: CTA pairs (tcgen05 cta_group::2) with
 *   1|2 accumulators of 256 rows; S >= 2 spreads the k-blocks of the tiles that do not fill
 *   a last round over about S units per tile, in equal ranges; a bare BN means MODE = 1,
 *   whole tiles per CTA; MODE = 5: CTA pairs, every tile computed by a cluster of S = 2 or 4 pairs
 *   that split its k-blocks and combine their fp32 accumulators through distributed shared memory --
 *   accepted when the problem has at most #SMs / (2 S) tiles and at least S k-blocks (with the
 *   row-parallel epilogue of sb200_gemm_rowpar: S = 2 only, and only as many clusters as the
 *   device reports co-resident, because that kernel's CTAs wait for one another).
 * workspace: optional device buffer (zero-filled once by the caller, at least 64 KiB +
 *   room for the fp32 partial tiles) that allows tiles to be cut along K;
 *   the library leaves its first 64 KiB zero again after every launch.  NULL / 0: whole
 *   tiles per CTA only.
 * Replaces: ColumnParallelLinear.apply_weights / ReplicatedLinear.apply_weights
 * (F.linear -> cuBLAS), sarathi/model_executor/parallel_utils/tensor_parallel/layers.py:278-284,516-518,
 * and, with the fused epilogues, the rotary_embedding call of models/llama.py:176-177
 * and the SiluAndMul call of models/llama.py:101-104. */
int sb200_gemm_colpar(void* out, int64_t ldo, const void* x, int64_t ldx, const void* w, int64_t ldw,
                      const void* bias, const void* residual, int64_t ldr, int64_t T, int64_t N, int64_t K,
                      int dtype, int epilogue,
                      const sb200_rotary_args* rot, uint32_t* status, int tile_cfg, void* workspace,
                      int64_t workspace_bytes, sb200_stream_t stream);

/* Paged KV cache, layout [pages, 2, page_size, kv_heads, head_dim] ("NHD"; the reference's
 * attention/flashinfer_attention_wrapper.py:69-77).  Entry i of a step belongs to request
 * batch_indices[i] and is the token at position positions[i] of that request; its key goes to
 * cache[page, 0, slot], its value to cache[page, 1, slot] with page = kv_indices[kv_indptr[b] + p / page_size],
 * slot = p % page_size -- the semantics of flashinfer's append_paged_kv_cache, which the reference calls at
 * flashinfer_attention_wrapper.py:261-270.
 * sb200_kv_cache_slots: slots[i] = page * 2 * page_size + slot (the row of the cache seen as
 *   [pages * 2 * page_size, kv_heads * head_dim] that receives the key; the value goes page_size rows
 *   further), or -1 when batch_indices[i] < 0.  All arrays on the device, int32 except slots (int64).
 * sb200_kv_cache_append: copies k / v rows ([n, kv_heads * head_dim] with row strides ldk / ldv in
 *   elements: views of the fused qkv buffer are fine, no contiguous copy is needed) to those rows. */
int sb200_kv_cache_slots(int64_t* slots, const int32_t* batch_indices, const int32_t* positions,
                         const int32_t* kv_indices, const int32_t* kv_indptr, int64_t n, int page_size,
                         sb200_stream_t stream);
int sb200_kv_cache_append(void* cache, const void* k, int64_t ldk, const void* v, int64_t ldv, const int64_t* slots,
                          int64_t n, int num_kv_heads, int head_dim, int page_size, int dtype, sb200_stream_t stream);

/* The tile shape and schedule the two GEMM entry points would pick (epilogue 3 = the
 * row-parallel kernel): out[0..11] = cta_pairs, accumulators, BN, scheduling units,
 * tiles handed out whole, S of the configuration, units that share the k-blocks of the
 * remaining tiles (= their number when nothing is cut), pipeline stages, M tiles, N tiles,
 * k-blocks, CTA pairs per tile (> 1: MODE 5, the tile's k-blocks are split inside a cluster).
 * Host-only; no counterpart in the reference. */
int sb200_gemm_plan(int epilogue, int64_t T, int64_t N, int64_t K, int head_size, int tile_cfg,
                    int64_t workspace_bytes, int* out);

/* Diagnostic: clocks the tensor pipe takes for `iters` k-blocks of four tcgen05.mma (bf16, K = 16 each) with
 * M = 128 on one CTA (pair = 0) or M = 256 on a CTA pair (pair = 1) and N columns, both operands resident in
 * shared memory (no loads in the timed loop).  dev_clocks[0] = SM clocks until the last MMA was issued,
 * dev_clocks[1] = until all had completed (-1: the wait ran out).  These are the per-MMA costs the tile
 * planner's model uses; `python -m sarathi_serve_b200.mma_rate` prints the table for the current GPU.
 * No counterpart in the reference. */
int sb200_diag_mma_rate(int pair, int n, int iters, int64_t* dev_clocks, sb200_stream_t stream);

/* Vocabulary-parallel embedding lookup: out[t, :] = weight[ids[t] - vocab_start, :] if
 * vocab_start <= ids[t] < vocab_end, else zeros.  out: [T, H]; ids: [T] int64 (device); weight:
 * this rank's rows [vocab_end - vocab_start, H] of the embedding table.  Followed by
 * sb200_all_reduce over the tensor-parallel ranks it gives the full lookup.
 * Replaces: VocabParallelEmbedding.forward (mask, F.embedding, masked fill),
 * sarathi/model_executor/parallel_utils/tensor_parallel/layers.py:147-168. */
int sb200_vocab_embedding(void* out, const int64_t* ids, const void* weight, int64_t T, int64_t H,
                          int64_t vocab_start, int64_t vocab_end, int dtype, sb200_stream_t stream);

/* Arrivals the row-parallel kernel of one rank counts for the owner of rows [lo, hi) under the
 * schedule sb200_gemm_plan(3, T, N, K, ., tile_cfg, workspace_bytes) reports (-1: no such schedule).
 * Host-only, used by the tests of that bookkeeping; no counterpart in the reference. */
int64_t sb200_gemm_rowpar_arrivals(int64_t T, int64_t N, int64_t K, int tile_cfg, int64_t workspace_bytes,
                                   int64_t lo, int64_t hi);

/* ------------------------------------------- tensor-parallel communication */

/* One context per (process, GPU, TP group).  It owns a "symmetric heap" on the
 * current device; after the handle exchange every rank's kernels can load from
 * every other rank's heap over NVLink (and store one flag word per peer and phase).  All ranks must issue the same
 * sequence of sb200_all_reduce / sb200_gemm_rowpar calls with the same shapes.
 * Replaces the NCCL communicator behind get_tensor_model_parallel_group()
 * (sarathi/model_executor/parallel_utils/parallel_state.py:147-158,235-240) for
 * the all-reduce of tensor_parallel/mappings.py:16-26. */
typedef struct sb200_comm sb200_comm;
#define SB200_IPC_HANDLE_BYTES 64

/* Bytes of device memory a context with the given region size allocates. */
int64_t sb200_comm_heap_bytes(int64_t region_bytes);
/* Allocates (cudaMalloc) and zeroes the heap on the current device.  region_bytes
 * must hold the largest [T, H] batch: T * H * sizeof(dtype), T rounded up to a
 * multiple of `world`. */
int sb200_comm_create(sb200_comm** out, int rank, int world, int64_t region_bytes);
/* Same, over heaps the caller allocated, zeroed and peer-mapped itself
 * (heaps[i] = address of rank i's heap in this process, sb200_comm_heap_bytes() each). */
int sb200_comm_create_external(sb200_comm** out, int rank, int world, int64_t region_bytes, void* const* heaps);
/* CUDA IPC handle (SB200_IPC_HANDLE_BYTES bytes, host memory) of this rank's heap. */
int sb200_comm_ipc_handle(sb200_comm* comm, void* host_handle_out);
/* host_handles: world * SB200_IPC_HANDLE_BYTES bytes, rank-major.  Maps every peer heap.
 * The caller must run a host barrier across the ranks before the first collective. */
int sb200_comm_open_peers(sb200_comm* comm, const void* host_handles);
int sb200_comm_destroy(sb200_comm* comm);
void* sb200_comm_local_heap(sb200_comm* comm);
void* sb200_comm_scratch(sb200_comm* comm);
int64_t sb200_comm_region_bytes(sb200_comm* comm);
/* Limit of every device-side wait on a peer, in SM clock cycles (default 2e10, about 10 s). */
int sb200_comm_set_wait_limit(sb200_comm* comm, int64_t cycles);
/* Collectives whose (world - 1) * T * H * sizeof(dtype) is at most `bytes` run "one-shot": every rank
 * loads all partial rows and finishes all T rows itself (one wait and one trip over the links);
 * larger ones have each row reduced by its owner and gathered afterwards.  Default 4 MiB
 * (environment override SB200_ONE_SHOT_BYTES at creation); 0 = never.  Every rank must use the
 * same value.  No counterpart in the reference (NCCL picks its algorithm internally). */
int sb200_comm_set_one_shot_bytes(sb200_comm* comm, int64_t bytes);
/* Synchronises `stream`, reads the context's device status word into *host_status and returns
 * SB200_ERR_PEER_TIMEOUT if a bounded wait ran out since the last clear. */
int sb200_comm_status(sb200_comm* comm, sb200_stream_t stream, uint32_t* host_status);
int sb200_comm_clear_status(sb200_comm* comm, sb200_stream_t stream);
/* `multicast_base`: address at which ALL ranks' heaps are mapped as one NVSwitch multicast range (same
 * offsets as the heaps themselves: a multimem store there lands in every rank's heap, a multimem
 * ld_reduce returns the element-wise sum over the heaps), e.g. the multicast pointer of a torch
 * symmetric-memory allocation whose per-rank buffers were given to sb200_comm_create_external.  With it,
 * collectives above the one-shot size are reduced and broadcast by the switch (multimem.ld_reduce /
 * multimem.st) instead of by peer loads.  NULL (the default) switches that off.  Every rank must make
 * the same choice.  Replaces what NCCL's NVLS algorithm does behind torch.distributed.all_reduce
 * (tensor_parallel/mappings.py:24). */
int sb200_comm_set_multicast(sb200_comm* comm, void* multicast_base);
int sb200_comm_has_multicast(sb200_comm* comm);
/* Puts the context back into its initial state (call counter, flags, arrival counters, status word).
 * After a device-side wait has run out the ranks' counters are out of step and every later collective
 * would miscount: all ranks call this, with nothing in flight on any of them (host barrier before and
 * after).  Synchronises `stream`.  No counterpart in the reference (a failed NCCL communicator is
 * destroyed and rebuilt). */
int sb200_comm_reset(sb200_comm* comm, sb200_stream_t stream);

/* All-gather of row blocks over the ranks: rank r holds rows [r * ceil(T / world), ...) of a [T, H]
 * tensor (`in_rows` points at just those rows); afterwards every rank has all T rows in a
 * context-owned buffer (*out_ptr, valid until the second-next collective) and, if given, in the local
 * [T, H] tensor `out_copy`.  With a multicast alias each rank publishes its rows with multimem stores,
 * otherwise the peers pull them.  Replaces gather-style plumbing around the layer stack such as the
 * broadcast of a step's hidden states to the tensor-parallel workers; the reference itself has every
 * worker receive the full batch (sarathi/model_executor/model_runner.py:67-117). */
int sb200_all_gather_rows(sb200_comm* comm, const void* in_rows, int64_t T, int64_t H, int dtype, void* out_copy,
                          sb200_stream_t stream, void** out_ptr);

/* Sum `in` [T, H] over the ranks; then, on the summed rows,
 *   z = sum (+ bias) (+ residual);   y = norm_w ? rms_norm(z, norm_w, eps) : z.
 * The primary result (y) lands in a context-owned buffer on EVERY rank
 * (*out_ptr, valid until the second-next collective on this context) and, if
 * out_copy != NULL, in that tensor.  With norm_w, z is also produced: in
 * *resid_ptr / resid_copy (all rows if write_resid_all, else only this rank's rows
 * [rank*ceil(T/world), ...)).  bias / residual / norm_w may be NULL.
 * Replaces: reduce_from_tensor_model_parallel_region ->
 * torch.distributed.all_reduce, tensor_parallel/mappings.py:16-26,270-271, plus the
 * bias add of tensor_parallel/layers.py:448-453, the residual add of
 * models/llama.py:248,254 and rms_norm (csrc/layernorm_kernels.cu:10-35). */
int sb200_all_reduce(sb200_comm* comm, const void* in, int64_t T, int64_t H, int dtype, const void* bias,
                     const void* residual, const void* norm_w, float eps, int write_resid_all,
                     void* out_copy, void* resid_copy, sb200_stream_t stream, void** out_ptr, void** resid_ptr);

/* Row-parallel projection fused with its all-reduce and the element-wise tail:
 *   partial = x[T, K/tp] * w[N, K/tp]^T  (tcgen05; the GEMM epilogue stores the partial
 *   rows into this rank's own heap and flags their owners), then the reduce (owners load
 *   the partial rows of every rank over NVLink) / bias / residual / RMSNorm / gather phases
 *   of sb200_all_reduce in the same kernel.
 * Arguments and results as sb200_all_reduce (H = N; rows of at most 16 KiB here, 32 KiB there).
 * Replaces: RowParallelLinear.forward (F.linear -> cuBLAS, then NCCL all-reduce),
 * tensor_parallel/layers.py:421-454, with the same element-wise tail. */
int sb200_gemm_rowpar(sb200_comm* comm, const void* x, int64_t ldx, const void* w, int64_t ldw, int64_t T,
                      int64_t N, int64_t K, int dtype, const void* bias, const void* residual,
                      const void* norm_w, float eps, int write_resid_all, void* out_copy, void* resid_copy,
                      int tile_cfg, sb200_stream_t stream, void** out_ptr, void** resid_ptr);

/* ---------------------------------------------------- mixture-of-experts GEMMs */

/* The expert GEMMs of a tensor-parallel MoE layer on the tcgen05 kernel.  They work on the
 * expert-sorted, block-padded slot order produced by sb200_moe_align_block_size with
 * block_size = sb200_moe_block_rows() (one tile row block = one expert).  rows_cap = capacity of
 * the sorted order (a multiple of the block); *num_post_pad (device) = rows in use.
 * Replace: fused_experts / invoke_fused_moe_kernel / the Triton fused_moe_kernel,
 * sarathi/model_executor/layers/fused_moe/fused_moe.py:15-148,207-259,411-544. */
int sb200_moe_block_rows(void);
/* xs[r, :] = x[sorted_ids[r] / top_k, :] for r < *num_post_pad (zeros for padding slots). */
int sb200_moe_gather_rows(void* xs, const void* x, const int32_t* sorted_ids, const int32_t* num_post_pad,
                          int64_t rows_cap, int64_t T, int64_t H, int top_k, int dtype, sb200_stream_t stream);
/* act[r, 0:d] = silu(xs[r] . w13[e][0:d]^T) * (xs[r] . w13[e][d:2d]^T), e = expert_ids[r / block];
 * w13: [E, 2d, K] (fused_moe/layer.py:80-90). */
int sb200_moe_gemm1(void* act, const void* xs, const void* w13, const int32_t* expert_ids,
                    const int32_t* num_post_pad, int64_t rows_cap, int E, int64_t two_d, int64_t K, int dtype,
                    uint32_t* status, int tile_cfg, sb200_stream_t stream);
/* out3[sorted_ids[r], :] = (act[r] . w2[e]^T) * topk_weights[sorted_ids[r]]; w2: [E, H, d];
 * out3: [num_slots = T * top_k, H]; padding rows write nothing. */
int sb200_moe_gemm2(void* out3, const void* act, const void* w2, const int32_t* expert_ids,
                    const int32_t* num_post_pad, const int32_t* sorted_ids, const float* topk_weights,
                    int64_t rows_cap, int64_t num_slots, int E, int64_t H, int64_t d, int dtype,
                    uint32_t* status, int tile_cfg, sb200_stream_t stream);
/* out[t, :] = sum_j in3[t * top_k + j, :] (fp32 sum rounded once; fused_moe.py:539-543).  With
 * `residual` [T, H] (may be NULL): out = residual + that sum, the add that follows the MoE block in the
 * decoder layer (models/mixtral.py:257). */
int sb200_moe_sum(void* out, const void* in3, const void* residual, int64_t T, int top_k, int64_t H, int dtype,
                  sb200_stream_t stream);
/* The same sum fused into the copy-in phase of the all-reduce over the tensor-parallel ranks
 * (fused_moe/layer.py:128-132); results as sb200_all_reduce without bias / norm; `residual` [T, H] (may
 * be NULL) is added to the reduced rows. */
int sb200_moe_sum_all_reduce(sb200_comm* comm, const void* in3, const void* residual, int64_t T, int top_k, int64_t H,
                             int dtype,
                             void* out_copy, sb200_stream_t stream, void** out_ptr);

#ifdef __cplusplus
}
#endif
#endif /* SARATHI_B200_H_ */
