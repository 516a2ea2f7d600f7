"""Tensor-parallel linear layers with the constructor signatures, attributes,
parameter names / shapes and (output, output_bias) return convention of the
reference (sarathi/model_executor/parallel_utils/tensor_parallel/layers.py:
VocabParallelEmbedding :72-177, ColumnParallelLinear :180-308, RowParallelLinear
:311-454, ReplicatedLinear :457-530), so model files and weight loaders work unchanged.

Differences that matter:
  * the local matmul is this library's tcgen05 GEMM, not F.linear;
  * RowParallelLinear does the GEMM, the all-reduce and the bias add in ONE
    kernel (no NCCL call), and offers ``forward_fused`` which also applies the
    residual add and the next RMSNorm in that kernel;
  * ColumnParallelLinear offers ``forward_rotary`` / ``forward_silu_mul`` with the
    rotary embedding / SiLU*mul applied in the GEMM epilogue.
The ``*_metric_name`` / ``layer_id`` keywords are accepted and ignored (the
reference wraps each op in a profiler timer; kernels here are fused, so there
are no separate linear / communication phases to time)."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch.nn.parameter import Parameter

from . import dense_ops
from . import parallel_state as ps
from .mappings import (divide, gather_from_tensor_model_parallel_region, reduce_from_tensor_model_parallel_region,
                       scatter_to_tensor_model_parallel_region)


def _param_device():
    return torch.cuda.current_device() if torch.cuda.is_available() else "cpu"


class VocabParallelEmbedding(torch.nn.Module):
    """Embedding table split along the vocabulary: rank r holds rows [r*V/tp, (r+1)*V/tp).  ``forward`` looks the
    ids of this rank's slice up (zeros for the others) in one kernel and sums over the ranks with this library's
    all-reduce (the reference: mask, F.embedding, masked fill, NCCL all-reduce)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, *, params_dtype: Optional[torch.dtype] = None,
                 use_cpu_initialization: bool = False, perform_initialization: bool = False,
                 linear_metric_name: Optional[str] = None, communication_metric_name: Optional[str] = None,
                 reduce_results: Optional[bool] = True, world_size: Optional[int] = None,
                 rank: Optional[int] = None):
        super().__init__()
        assert not perform_initialization
        assert not use_cpu_initialization
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.tensor_model_parallel_size = ps.get_tensor_model_parallel_world_size() if world_size is None else world_size
        self.rank = ps.get_tensor_model_parallel_rank() if rank is None else rank
        self.reduce_results = reduce_results
        per_partition = divide(num_embeddings, self.tensor_model_parallel_size)
        self.vocab_start_index = self.rank * per_partition
        self.vocab_end_index = self.vocab_start_index + per_partition
        self.num_embeddings_per_partition = per_partition
        self.weight = Parameter(torch.empty(per_partition, embedding_dim, device=_param_device(), dtype=params_dtype),
                                requires_grad=False)

    def forward(self, input_: torch.Tensor) -> torch.Tensor:
        from . import embedding_ops
        ids = input_.reshape(-1).contiguous()
        out = torch.empty(ids.numel(), self.embedding_dim, dtype=self.weight.dtype, device=self.weight.device)
        embedding_ops.vocab_embedding(out, ids, self.weight, self.vocab_start_index, self.vocab_end_index)
        if self.reduce_results and self.tensor_model_parallel_size > 1 and ids.numel() > 0:
            out = reduce_from_tensor_model_parallel_region(out)
        return out.view(*input_.shape, self.embedding_dim)


class ColumnParallelLinear(torch.nn.Module):
    """Y = X A^T + b with A split along its output dimension: rank r holds rows
    [r*N/tp, (r+1)*N/tp) of the [N, K] weight."""

    def __init__(self, input_size, output_size, *, bias=True, gather_output=True, stride=1, skip_bias_add=False,
                 params_dtype=None, use_cpu_initialization=False, perform_initialization=False,
                 linear_metric_name: Optional[str] = None, communication_metric_name: Optional[str] = None,
                 world_size: Optional[int] = None, layer_id: Optional[int] = None):
        super().__init__()
        assert not perform_initialization
        assert not use_cpu_initialization
        self.input_size = input_size
        self.output_size = output_size
        self.gather_output = gather_output
        self.world_size = ps.get_tensor_model_parallel_world_size() if world_size is None else world_size
        self.output_size_per_partition = divide(output_size, self.world_size)
        self.skip_bias_add = skip_bias_add
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.create_weights(params_dtype)
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size_per_partition, device=_param_device(),
                                              dtype=params_dtype), requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def create_weights(self, dtype: torch.dtype) -> None:
        self.weight = Parameter(torch.empty(self.output_size_per_partition, self.input_size,
                                            device=_param_device(), dtype=dtype), requires_grad=False)

    def _cfg(self, kind: str, x: torch.Tensor) -> int:
        return dense_ops.tuned_cfg(kind, x.shape[0] if x.dim() == 2 else x.numel() // x.shape[-1],
                                   self.weight.shape[0], self.weight.shape[1], x.dtype)

    def tune(self, num_tokens: int, kind: str = "store", head_size: int = 128) -> int:
        """Pick the fastest tile configuration for [num_tokens, in] inputs (see dense_ops.autotune)."""
        return dense_ops.autotune(kind, num_tokens, self.weight.shape[0], self.weight.shape[1], self.weight.dtype,
                                  self.weight.device, head_size)

    def apply_weights(self, x: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
        return dense_ops.linear(x, self.weight, bias, tile_n=self._cfg("store", x))

    def forward(self, input_) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        bias = self.bias if not self.skip_bias_add else None
        output_parallel = self.apply_weights(input_, bias)
        output = gather_from_tensor_model_parallel_region(output_parallel) if self.gather_output else output_parallel
        return output, (self.bias if self.skip_bias_add else None)

    # -- fused variants (no bias) ------------------------------------------
    def forward_rotary(self, input_: torch.Tensor, positions: torch.Tensor, rotary_emb, rot_cols: int,
                       kv_append=None, num_kv_heads: int = 0) -> torch.Tensor:
        """qkv projection with ``rotary_emb`` applied to output columns [0, rot_cols).  ``kv_append`` =
        (paged_kv_cache, kv_slots): the k columns (the last ``num_kv_heads`` heads below rot_cols) and the v
        columns are also stored into the paged KV cache."""
        assert self.bias is None and not self.gather_output
        cache, slots = kv_append if kv_append is not None else (None, None)
        if dense_ops.fused_rotary_supported(input_, rotary_emb.head_size, rotary_emb.rotary_dim):
            return dense_ops.linear_rotary(input_, self.weight, positions, rotary_emb.cos_sin_cache,
                                           rotary_emb.head_size, rot_cols, rotary_emb.is_neox_style,
                                           tile_n=self._cfg("rotary", input_), kv_cache=cache, kv_slots=slots,
                                           num_kv_heads=num_kv_heads)
        qkv = dense_ops.linear(input_, self.weight)
        n_rot_heads = rot_cols // rotary_emb.head_size
        # one call over q|k as a single strided "query" view; no separate key tensor
        rotary_emb.rotate_inplace(positions, qkv[:, :rot_cols], n_rot_heads)
        if cache is not None:  # fp32 (or an unsupported head size): the append runs as its own kernel
            from . import kv_cache_ops
            kvc = num_kv_heads * rotary_emb.head_size
            kv_cache_ops.append_rows(cache, qkv[:, rot_cols - kvc:rot_cols], qkv[:, rot_cols:rot_cols + kvc], slots)
        return qkv

    def forward_silu_mul(self, input_: torch.Tensor) -> torch.Tensor:
        """gate_up projection returning silu(gate) * up ([T, N/(2 tp)])."""
        assert self.bias is None and not self.gather_output
        if input_.dtype in (torch.bfloat16, torch.float16):
            return dense_ops.linear_silu_mul(input_, self.weight, tile_n=self._cfg("silu", input_))
        from . import activation_ops
        gate_up = dense_ops.linear(input_, self.weight)
        out = torch.empty(gate_up.shape[0], gate_up.shape[1] // 2, dtype=gate_up.dtype, device=gate_up.device)
        activation_ops.silu_and_mul(out, gate_up)
        return out


class RowParallelLinear(torch.nn.Module):
    """Y = X A^T + b with A split along its input dimension: rank r holds columns
    [r*K/tp, (r+1)*K/tp) of the [N, K] weight and the matching slice of X; the
    partial products are summed over the group."""

    def __init__(self, input_size, output_size, *, bias=True, input_is_parallel=False, skip_bias_add=False,
                 params_dtype=None, use_cpu_initialization=False, perform_initialization=False, reduce_results=True,
                 linear_metric_name: Optional[str] = None, communication_metric_name: Optional[str] = None,
                 world_size: Optional[int] = None, layer_id: Optional[int] = None):
        super().__init__()
        assert not perform_initialization
        assert not use_cpu_initialization
        self.input_size = input_size
        self.output_size = output_size
        self.input_is_parallel = input_is_parallel
        self.reduce_results = reduce_results
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.world_size = ps.get_tensor_model_parallel_world_size() if world_size is None else world_size
        self.input_size_per_partition = divide(input_size, self.world_size)
        self.skip_bias_add = skip_bias_add
        self.create_weights(params_dtype)
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size, device=_param_device(), dtype=params_dtype),
                                  requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def create_weights(self, dtype: torch.dtype) -> None:
        self.weight = Parameter(torch.empty(self.output_size, self.input_size_per_partition,
                                            device=_param_device(), dtype=dtype), requires_grad=False)

    def apply_weights(self, x: torch.Tensor) -> torch.Tensor:
        return dense_ops.linear(x, self.weight)

    def tune(self, num_tokens: int) -> int:
        """Pick the fastest tile configuration of the fused GEMM for [num_tokens, in/tp] inputs; every rank of
        the tensor-parallel group must call this together (rank 0's choice is shared)."""
        group = ps.get_tensor_model_parallel_group() if self.world_size > 1 else None
        if self.world_size == 1:  # forward_fused runs the plain GEMM there
            dense_ops.autotune("store", num_tokens, self.weight.shape[0], self.weight.shape[1], self.weight.dtype,
                               self.weight.device)
        return dense_ops.autotune("push", num_tokens, self.weight.shape[0], self.weight.shape[1], self.weight.dtype,
                                  self.weight.device, group=group)

    def _cfg(self, x: torch.Tensor) -> int:
        return dense_ops.tuned_cfg("push", x.shape[0], self.weight.shape[0], self.weight.shape[1], x.dtype)

    def _comm(self, T: int):
        es = torch.empty((), dtype=self.weight.dtype).element_size()
        rows = -(-T // self.world_size) * self.world_size
        need = rows * self.output_size * es
        comm = ps._TP_COMM
        if comm is None:
            return ps.get_tensor_model_parallel_comm(max(need, ps.default_comm_region_bytes()))
        if need > comm.region_bytes:
            # the context is shared by every layer of the process and sized once, by its first user
            raise RuntimeError(f"a [{rows}, {self.output_size}] batch needs {need} bytes per region of the tensor-parallel "
                               f"context, which was created with {comm.region_bytes}: create it before the first forward "
                               f"with parallel_state.get_tensor_model_parallel_comm(max_num_batched_tokens * hidden_size * "
                               f"itemsize), or set SB200_COMM_REGION_BYTES")
        return comm

    def forward(self, input_) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        input_parallel = input_ if self.input_is_parallel else scatter_to_tensor_model_parallel_region(input_)
        add_bias = self.bias if (self.bias is not None and not self.skip_bias_add) else None
        if self.reduce_results and self.world_size > 1:
            lead = input_parallel.shape[:-1]
            x2 = input_parallel.reshape(-1, input_parallel.shape[-1])
            out = torch.empty(x2.shape[0], self.output_size, dtype=x2.dtype, device=x2.device)
            self._comm(x2.shape[0]).rowpar_linear(x2, self.weight, bias=add_bias, out=out, tile_n=self._cfg(x2))
            output = out.view(*lead, self.output_size)
        else:
            # No reduction: the bias (if any) is added to the local product, as the reference does.
            output = dense_ops.linear(input_parallel, self.weight, add_bias)
        return output, (self.bias if self.skip_bias_add else None)

    def forward_fused(self, input_: torch.Tensor, residual: torch.Tensor, norm_weight: Optional[torch.Tensor],
                      eps: float = 0.0, resid_everywhere: bool = True, out: Optional[torch.Tensor] = None,
                      resid_out: Optional[torch.Tensor] = None):
        """GEMM + all-reduce + (bias) + residual add (+ RMSNorm with ``norm_weight``) in one kernel.

        Returns (y, z): z = residual + sum_over_ranks(x @ W^T) (+ bias) rounded to the
        dtype, y = rms_norm(z) * norm_weight.  Without a norm weight returns (z, None).
        Without ``out`` / ``resid_out`` the results are views into the communication
        context (valid until the second-next collective)."""
        assert self.input_is_parallel and self.reduce_results
        add_bias = self.bias if (self.bias is not None and not self.skip_bias_add) else None
        if self.world_size == 1 and residual is not None:
            # Nothing to exchange: the plain GEMM followed by the one-pass add (+ RMSNorm) kernel is faster
            # than the in-kernel tail, whose rows have to wait for every column tile of the GEMM.
            from . import layernorm_ops
            cfg = dense_ops.tuned_cfg("store", input_.shape[0], self.weight.shape[0], self.weight.shape[1], input_.dtype)
            if norm_weight is None:
                if input_.dtype == torch.float32:
                    return torch.add(residual, dense_ops.linear(input_, self.weight, add_bias), out=out), None
                # the residual add rides in the GEMM epilogue
                return dense_ops.linear(input_, self.weight, add_bias, out=out, tile_n=cfg, residual=residual), None
            prod = dense_ops.linear(input_, self.weight, add_bias, tile_n=cfg)
            y = out if out is not None else torch.empty_like(prod)
            z = resid_out if resid_out is not None else torch.empty_like(prod)
            layernorm_ops.fused_add_rms_norm(y, z, prod, residual, norm_weight, eps)
            return y, z
        return self._comm(input_.shape[0]).rowpar_linear(input_, self.weight, bias=add_bias, residual=residual,
                                                         norm_weight=norm_weight, eps=eps,
                                                         resid_everywhere=resid_everywhere, out=out,
                                                         resid_out=resid_out, tile_n=self._cfg(input_))


class ReplicatedLinear(torch.nn.Module):
    """Unsharded linear layer (the MoE router gate)."""

    def __init__(self, input_size: int, output_size: int, bias: bool = True, skip_bias_add: bool = False,
                 params_dtype: Optional[torch.dtype] = None, metric_name: Optional[str] = None,
                 layer_id: Optional[int] = None):
        super().__init__()
        self.input_size = input_size
        self.output_size = output_size
        self.skip_bias_add = skip_bias_add
        if params_dtype is None:
            params_dtype = torch.get_default_dtype()
        self.params_dtype = params_dtype  # the reference reads this attribute without setting it (layers.py:494)
        self.create_weights(params_dtype)
        if bias:
            self.bias = Parameter(torch.zeros(self.output_size, device=_param_device(), dtype=params_dtype),
                                  requires_grad=False)
        else:
            self.register_parameter("bias", None)

    def create_weights(self, dtype: torch.dtype) -> None:
        self.weight = Parameter(torch.empty(self.output_size, self.input_size, device=_param_device(), dtype=dtype),
                                requires_grad=False)

    def apply_weights(self, x: torch.Tensor) -> torch.Tensor:
        return dense_ops.linear(x, self.weight)

    def forward(self, x: torch.Tensor):
        if not self.skip_bias_add:
            return dense_ops.linear(x, self.weight, self.bias), None
        return dense_ops.linear(x, self.weight), self.bias
