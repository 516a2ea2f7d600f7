"""Tensor-parallel mixture-of-experts layer with the function and class names of the
reference (sarathi/model_executor/layers/fused_moe/fused_moe.py and layer.py):
``fused_topk``, ``moe_align_block_size``, ``fused_experts``, ``fused_moe`` and the
``FusedMoE`` module (parameters ``w13_weight [E, 2I/tp, H]``, ``w2_weight [E, H, I/tp]``).

Where the reference runs a cast, the routing kernel, a renormalisation, a Triton
grouped GEMM, ``silu_and_mul``, a second Triton GEMM, ``torch.sum`` and an NCCL
all-reduce, this runs: one routing kernel (cast + softmax/top-k + renormalise),
the block alignment, a row gather, two tcgen05 grouped GEMMs (SiLU*mul fused into
the first, the routed weight and the scatter to (token, k) slots into the
second), and one kernel that sums the k slots while it pushes them into the
all-reduce."""
from __future__ import annotations

import ctypes
from typing import Any, Dict, Optional, Tuple

import torch

from . import _native as N
from . import dense_ops, moe_ops
from . import parallel_state as ps


def block_rows(pairs: bool = False) -> int:
    """Rows per expert block the grouped GEMMs work with (one tile row block = one expert): 128 for single-CTA
    tiles, 256 for CTA-pair tiles."""
    return int(N.lib().sb200_moe_block_rows()) * (2 if pairs else 1)


def use_pair_tiles(num_slots: int, num_experts: int) -> bool:
    """CTA-pair tiles (256-row expert blocks) once an expert sees 128 slots or more on average: a pair loads half of
    the weight tile per SM, and the operand feed is what bounds these GEMMs, which outweighs the extra padding;
    small batches keep 128-row blocks."""
    return num_slots >= 128 * num_experts


def fused_topk(hidden_states: torch.Tensor, gating_output: torch.Tensor, topk: int, renormalize: bool):
    """Softmax + top-k routing (fused_moe.py:346-373): returns (topk_weights f32 [T,k], topk_ids i32 [T,k]).
    The ``.float()`` cast and the renormalisation happen inside the kernel."""
    assert hidden_states.shape[0] == gating_output.shape[0], "Number of tokens mismatch"
    M = hidden_states.shape[0]
    topk_weights = torch.empty(M, topk, dtype=torch.float32, device=hidden_states.device)
    topk_ids = torch.empty(M, topk, dtype=torch.int32, device=hidden_states.device)
    moe_ops.topk_softmax(topk_weights, topk_ids, None, gating_output.contiguous(), renormalize=renormalize)
    return topk_weights, topk_ids


def moe_align_block_size(topk_ids: torch.Tensor, block_size: int, num_experts: int
                         ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Block-aligned expert sort (fused_moe.py:151-204): returns (sorted_token_ids, expert_ids,
    num_tokens_post_padded) with the reference's buffer sizes; the pad value is topk_ids.numel()."""
    max_num_tokens_padded = topk_ids.numel() + num_experts * (block_size - 1)
    sorted_ids = torch.empty((max_num_tokens_padded,), dtype=torch.int32, device=topk_ids.device)
    max_num_m_blocks = (max_num_tokens_padded + block_size - 1) // block_size
    expert_ids = torch.empty((max_num_m_blocks,), dtype=torch.int32, device=topk_ids.device)
    num_tokens_post_pad = torch.empty((1,), dtype=torch.int32, device=topk_ids.device)
    moe_ops.moe_align_block_size(topk_ids, num_experts, block_size, sorted_ids, expert_ids, num_tokens_post_pad)
    return sorted_ids, expert_ids, num_tokens_post_pad


def _expert_slots(hidden_states, w1, w2, topk_weights, topk_ids, ids_in_range: bool = False, pairs: Optional[bool] = None):
    """Common part of fused_experts: returns out3 [T*k, H] (per-slot expert outputs, already scaled by
    the routed weights) for bf16/fp16 inputs.  ``ids_in_range``: the caller guarantees 0 <= id < E for
    every slot (ids produced by ``fused_topk``); otherwise the slots are zeroed first, because a slot whose
    id is out of range is skipped by the alignment and the GEMMs and would keep uninitialised memory."""
    T, H = hidden_states.shape
    E, two_d, K = w1.shape
    k = topk_ids.shape[1]
    if K != H or w2.shape[0] != E or w2.shape[2] * 2 != two_d:
        raise RuntimeError("fused_experts: weight shapes do not match")
    dev, dt = hidden_states.device, hidden_states.dtype
    pairs = use_pair_tiles(T * k, E) if pairs is None else bool(pairs)
    blk = block_rows(pairs)
    cfg = 3256 if pairs else 0
    # capacity of the sorted order, rounded up to whole blocks (the grouped GEMMs address whole row blocks)
    rows_cap = (T * k + E * (blk - 1) + blk - 1) // blk * blk
    sorted_ids = torch.empty(rows_cap, dtype=torch.int32, device=dev)
    expert_ids = torch.empty(rows_cap // blk, dtype=torch.int32, device=dev)
    num_post_pad = torch.empty(1, dtype=torch.int32, device=dev)
    moe_ops.moe_align_block_size(topk_ids, E, blk, sorted_ids, expert_ids, num_post_pad)
    lib = N.lib()
    st = N.ptr(dense_ops.status_word(dev))
    xs = torch.empty(rows_cap, H, dtype=dt, device=dev)
    N.check(lib.sb200_moe_gather_rows(N.ptr(xs), N.ptr(hidden_states), N.ptr(sorted_ids), N.ptr(num_post_pad), rows_cap,
                                      T, H, k, N.dtype_id(hidden_states), N.stream_ptr()), "moe_gather_rows")
    act = torch.empty(rows_cap, two_d // 2, dtype=dt, device=dev)
    N.check(lib.sb200_moe_gemm1(N.ptr(act), N.ptr(xs), N.ptr(w1), N.ptr(expert_ids), N.ptr(num_post_pad), rows_cap, E,
                                two_d, K, N.dtype_id(hidden_states), st, cfg, N.stream_ptr()), "moe_gemm1")
    out3 = (torch.empty if ids_in_range else torch.zeros)(T * k, w2.shape[1], dtype=dt, device=dev)
    N.check(lib.sb200_moe_gemm2(N.ptr(out3), N.ptr(act), N.ptr(w2), N.ptr(expert_ids), N.ptr(num_post_pad),
                                N.ptr(sorted_ids), N.ptr(topk_weights), rows_cap, T * k, E, w2.shape[1], w2.shape[2],
                                N.dtype_id(hidden_states), st, cfg, N.stream_ptr()), "moe_gemm2")
    return out3


def fused_experts(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, topk_weights: torch.Tensor,
                  topk_ids: torch.Tensor, inplace: bool = False, override_config: Optional[Dict[str, Any]] = None,
                  w1_scale=None, w2_scale=None, a1_scale=None, a2_scale=None) -> torch.Tensor:
    """Expert MLPs of the routed tokens (fused_moe.py:411-544); the sum over the k slots included."""
    assert hidden_states.shape[1] == w1.shape[2], "Hidden size mismatch"
    assert topk_weights.shape == topk_ids.shape, "topk shape mismatch"
    assert hidden_states.is_contiguous(), "Hidden_states must be contiguous"
    assert w1.is_contiguous() and w2.is_contiguous(), "Expert weights must be contiguous"
    assert w1_scale is None and w2_scale is None and a1_scale is None and a2_scale is None
    if hidden_states.dtype not in (torch.float16, torch.bfloat16):
        raise RuntimeError("fused_experts: bf16 / fp16 only")
    N.require_cuda(hidden_states, w1, w2, topk_weights, topk_ids)
    T = hidden_states.shape[0]
    out = hidden_states if inplace else torch.empty_like(hidden_states)
    if T == 0:
        return out
    out3 = _expert_slots(hidden_states, w1, w2, topk_weights.contiguous(), topk_ids.contiguous())
    N.check(N.lib().sb200_moe_sum(N.ptr(out), N.ptr(out3), None, T, topk_ids.shape[1], out.shape[1], N.dtype_id(out),
                                  N.stream_ptr()), "moe_sum")
    return out


def fused_moe(hidden_states: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, gating_output: torch.Tensor, topk: int,
              renormalize: bool, inplace: bool = False, override_config: Optional[Dict[str, Any]] = None,
              use_grouped_topk: bool = False, num_expert_group: Optional[int] = None,
              topk_group: Optional[int] = None, **scales) -> torch.Tensor:
    """Routing + expert MLPs (fused_moe.py:547-622)."""
    assert gating_output.shape[1] == w1.shape[0], "Number of experts mismatch"
    if use_grouped_topk:
        raise NotImplementedError("grouped_topk (DeepSeek-V2 routing) is outside this path")
    topk_weights, topk_ids = fused_topk(hidden_states, gating_output, topk, renormalize)
    return fused_experts(hidden_states, w1, w2, topk_weights, topk_ids, inplace=inplace,
                         override_config=override_config, **scales)


class FusedMoE(torch.nn.Module):
    """MoE layer whose experts are sharded along the intermediate dimension over the tensor-parallel
    ranks (fused_moe/layer.py:12-134); same constructor keywords and parameter names."""

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 params_dtype: Optional[torch.dtype] = None, reduce_results: bool = False, renormalize: bool = True,
                 use_grouped_topk: bool = False, num_expert_group: Optional[int] = None,
                 topk_group: Optional[int] = None, linear_metric_name: Optional[str] = None,
                 communication_metric_name: Optional[str] = None, world_size: Optional[int] = None,
                 layer_id: Optional[int] = None):
        super().__init__()
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.params_dtype = params_dtype
        self.tp_size = ps.get_tensor_model_parallel_world_size()
        self.top_k = top_k
        self.num_experts = num_experts
        self.hidden_size = hidden_size
        self.intermediate_size_per_partition = intermediate_size // self.tp_size
        self.reduce_results = reduce_results
        self.renormalize = renormalize
        self.use_grouped_topk = use_grouped_topk
        if self.use_grouped_topk:
            assert num_expert_group is not None and topk_group is not None
        self.num_expert_group = num_expert_group
        self.topk_group = topk_group
        self.world_size = ps.get_tensor_model_parallel_world_size() if world_size is None else world_size
        self.create_weights()

    def create_weights(self):
        dev = torch.cuda.current_device() if torch.cuda.is_available() else "cpu"
        self.w13_weight = torch.nn.Parameter(torch.empty(self.num_experts, 2 * self.intermediate_size_per_partition,
                                                         self.hidden_size, dtype=self.params_dtype, device=dev),
                                             requires_grad=False)
        self.w2_weight = torch.nn.Parameter(torch.empty(self.num_experts, self.hidden_size,
                                                        self.intermediate_size_per_partition, dtype=self.params_dtype,
                                                        device=dev), requires_grad=False)

    def apply_weights(self, x: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        return fused_moe(x, self.w13_weight, self.w2_weight, router_logits, self.top_k, renormalize=self.renormalize,
                         inplace=True, use_grouped_topk=self.use_grouped_topk,
                         num_expert_group=self.num_expert_group, topk_group=self.topk_group)

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        """Overwrites and returns ``hidden_states`` (the reference runs the experts in place too)."""
        if not (self.reduce_results and self.world_size > 1):
            return self.apply_weights(hidden_states, router_logits)
        return self.forward_fused(hidden_states, router_logits, None, out=hidden_states)

    def forward_fused(self, hidden_states: torch.Tensor, router_logits: torch.Tensor,
                      residual: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``residual + experts(hidden_states)`` (just the experts' output when ``residual`` is None) written to
        ``out`` (a new tensor by default; ``hidden_states`` itself is allowed): the sum over the k routed slots,
        the all-reduce over the tensor-parallel ranks and the decoder layer's residual add
        (models/mixtral.py:257) happen in one kernel.  ``hidden_states`` is not modified unless it is ``out``."""
        if self.use_grouped_topk:
            raise NotImplementedError("grouped_topk (DeepSeek-V2 routing) is outside this path")
        T, H = hidden_states.shape
        if out is None:
            out = torch.empty_like(hidden_states)
        if T == 0:
            return out
        topk_weights, topk_ids = fused_topk(hidden_states, router_logits, self.top_k, self.renormalize)
        out3 = _expert_slots(hidden_states, self.w13_weight, self.w2_weight, topk_weights, topk_ids, ids_in_range=True)
        if self.reduce_results and self.world_size > 1:
            comm = ps.get_tensor_model_parallel_comm()
            comm._usable()
            op = ctypes.c_void_p()
            # sum over the k slots fused into the push of the all-reduce
            N.check(N.lib().sb200_moe_sum_all_reduce(comm._h, N.ptr(out3), N.ptr(residual), T, self.top_k, H,
                                                     N.dtype_id(out3), N.ptr(out), N.stream_ptr(), ctypes.byref(op)),
                    "moe_sum_all_reduce")
        else:
            N.check(N.lib().sb200_moe_sum(N.ptr(out), N.ptr(out3), N.ptr(residual), T, self.top_k, H, N.dtype_id(out3),
                                          N.stream_ptr()), "moe_sum")
        return out
