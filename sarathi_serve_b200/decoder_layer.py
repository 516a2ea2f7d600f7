"""The callers of the hot path: Llama-style attention / MLP / decoder-layer
modules with the reference's constructor and forward signatures and parameter
names (sarathi/model_executor/models/llama.py:60-106,109-188,191-255), built on
this package's layers.

``LlamaDecoderLayer.forward`` keeps the reference's contract
(positions, hidden_states, layer_cache_idx, attention_backend_wrapper) ->
hidden_states, and runs five kernels besides attention:
    rms_norm | qkv GEMM + rotary | o_proj GEMM + all-reduce + residual + RMSNorm |
    gate_up GEMM + SiLU*mul | down GEMM + all-reduce + residual.
``forward_carry`` is the variant for a stack of layers: it takes the already
normalised hidden states and the residual, and its last kernel also applies the
NEXT layer's input RMSNorm, so a layer costs four kernels."""
from __future__ import annotations

from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import parallel_state as ps
from .fused_moe import FusedMoE
from .nn_layers import RMSNorm, SiluAndMul, get_rope
from .mappings import gather_from_tensor_model_parallel_region
from .tp_layers import ColumnParallelLinear, ReplicatedLinear, RowParallelLinear, VocabParallelEmbedding


def fused_kv_append(attention_backend_wrapper, layer_cache_idx: int):
    """An attention wrapper that keeps a paged KV cache of layout [pages, 2, page_size, kv_heads, head_dim] can
    have this step's keys and values stored by the qkv GEMM's epilogue instead of appending them itself
    (the reference's wrapper appends inside ``forward``:
    attention/flashinfer_attention_wrapper.py:253-270).  It opts in by defining

        fused_kv_append(layer_cache_idx) -> (paged_kv_cache, kv_slots) | None

    with ``kv_slots`` from ``kv_cache_ops.slots`` (computed once per step in its ``begin_forward``); its
    ``forward`` must then not append again.  Wrappers without that method are used unchanged."""
    hook = getattr(attention_backend_wrapper, "fused_kv_append", None)
    return hook(layer_cache_idx) if hook is not None else None


class LlamaMLP(nn.Module):
    def __init__(self, hidden_size: int, intermediate_size: int, hidden_act: str,
                 layer_id: Optional[int] = None) -> None:
        super().__init__()
        self.gate_up_proj = ColumnParallelLinear(hidden_size, 2 * intermediate_size, bias=False, gather_output=False,
                                                 perform_initialization=False, layer_id=layer_id)
        self.down_proj = RowParallelLinear(intermediate_size, hidden_size, bias=False, input_is_parallel=True,
                                           perform_initialization=False, layer_id=layer_id)
        if hidden_act != "silu":
            raise ValueError(f"Unsupported activation: {hidden_act}. Only silu is supported for now.")
        self.act_fn = SiluAndMul()

    def forward(self, x):
        """Module-by-module path (three kernels + the all-reduce inside down_proj)."""
        gate_up, _ = self.gate_up_proj(x)
        x = self.act_fn(gate_up)
        x, _ = self.down_proj(x)
        return x


class LlamaAttention(nn.Module):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, rope_theta: float = 10000,
                 rope_scaling: Optional[Dict[str, Any]] = None, max_position_embeddings: int = 8192,
                 layer_id: Optional[int] = None) -> None:
        super().__init__()
        self.hidden_size = hidden_size
        tp_size = ps.get_tensor_model_parallel_world_size()
        self.total_num_heads = num_heads
        assert self.total_num_heads % tp_size == 0
        self.num_heads = self.total_num_heads // tp_size
        self.total_num_kv_heads = num_kv_heads
        assert self.total_num_kv_heads % tp_size == 0
        self.num_kv_heads = self.total_num_kv_heads // tp_size
        self.head_dim = hidden_size // self.total_num_heads
        self.q_size = self.num_heads * self.head_dim
        self.kv_size = self.num_kv_heads * self.head_dim
        self.scaling = self.head_dim ** -0.5
        self.rope_theta = rope_theta
        self.max_position_embeddings = max_position_embeddings
        self.layer_id = layer_id
        self.qkv_proj = ColumnParallelLinear(hidden_size,
                                             (self.total_num_heads + 2 * self.total_num_kv_heads) * self.head_dim,
                                             bias=False, gather_output=False, perform_initialization=False,
                                             layer_id=layer_id)
        self.o_proj = RowParallelLinear(self.total_num_heads * self.head_dim, hidden_size, bias=False,
                                        input_is_parallel=True, perform_initialization=False, layer_id=layer_id)
        self.rotary_emb = get_rope(head_size=self.head_dim, rotary_dim=self.head_dim,
                                   max_position=self.max_position_embeddings, base=self.rope_theta,
                                   is_neox_style=True, rope_scaling=rope_scaling)

    def qkv_rotary(self, positions: torch.Tensor, hidden_states: torch.Tensor, kv_append=None):
        """qkv projection with the rotary embedding fused into the GEMM epilogue; returns q, k, v views.
        ``kv_append``: optional (paged_kv_cache, kv_slots) -- the rotated keys and the values are then also
        stored into the paged cache from the same epilogue (see ``fused_kv_append``)."""
        qkv = self.qkv_proj.forward_rotary(hidden_states, positions, self.rotary_emb, self.q_size + self.kv_size,
                                           kv_append=kv_append, num_kv_heads=self.num_kv_heads)
        return qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor, layer_cache_idx: int,
                attention_backend_wrapper) -> torch.Tensor:
        """Module-by-module path, as in the reference (llama.py:168-188)."""
        qkv, _ = self.qkv_proj(hidden_states)
        q, k, v = qkv.split([self.q_size, self.kv_size, self.kv_size], dim=-1)
        q, k = self.rotary_emb(positions, q, k)
        attn_output = attention_backend_wrapper.forward(q, k, v, layer_cache_idx, self.scaling, self.layer_id)
        output, _ = self.o_proj(attn_output)
        return output


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config, layer_id: Optional[int] = None) -> None:
        super().__init__()
        self.hidden_size = config.hidden_size
        rope_theta = getattr(config, "rope_theta", 10000)
        rope_scaling = getattr(config, "rope_scaling", None)
        max_position_embeddings = getattr(config, "max_position_embeddings", 8192)
        self.self_attn = LlamaAttention(hidden_size=self.hidden_size, num_heads=config.num_attention_heads,
                                        num_kv_heads=config.num_key_value_heads, rope_theta=rope_theta,
                                        rope_scaling=rope_scaling, max_position_embeddings=max_position_embeddings,
                                        layer_id=layer_id)
        self.mlp = LlamaMLP(hidden_size=self.hidden_size, intermediate_size=config.intermediate_size,
                            hidden_act=config.hidden_act, layer_id=layer_id)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps, layer_id=layer_id)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps, layer_id=layer_id)

    # ------------------------------------------------------------- unfused
    def forward_unfused(self, positions, hidden_states, layer_cache_idx, attention_backend_wrapper) -> torch.Tensor:
        """Op-for-op the reference's sequence (llama.py:232-255): every module called on its own."""
        residual = hidden_states
        hidden_states = self.input_layernorm(hidden_states)
        hidden_states = self.self_attn(positions=positions, hidden_states=hidden_states,
                                       layer_cache_idx=layer_cache_idx,
                                       attention_backend_wrapper=attention_backend_wrapper)
        hidden_states, residual = self.post_attention_layernorm.forward_add(hidden_states, residual)
        hidden_states = self.mlp(hidden_states)
        return residual + hidden_states

    # --------------------------------------------------------------- fused
    def _attn_mlp(self, positions, normed, residual, layer_cache_idx, attn, next_norm_weight, next_eps, out=None,
                  resid_everywhere=True):
        sa = self.self_attn
        q, k, v = sa.qkv_rotary(positions, normed, fused_kv_append(attn, layer_cache_idx))
        attn_out = attn.forward(q, k, v, layer_cache_idx, sa.scaling, sa.layer_id)
        # the mid-layer residual is only read by the down projection's tail, which touches the rows this
        # rank owns: they need not be gathered on every rank
        h, resid = sa.o_proj.forward_fused(attn_out, residual, self.post_attention_layernorm.weight.data,
                                           self.post_attention_layernorm.variance_epsilon, resid_everywhere=False)
        act = self.mlp.gate_up_proj.forward_silu_mul(h)
        return self.mlp.down_proj.forward_fused(act, resid, next_norm_weight, next_eps, out=out,
                                                resid_everywhere=resid_everywhere)

    def tune(self, num_tokens: int) -> None:
        """Autotune the four projections for batches of ``num_tokens`` tokens (all tensor-parallel ranks together)."""
        sa = self.self_attn
        fused_rot = sa.qkv_proj.weight.dtype in (torch.bfloat16, torch.float16)
        sa.qkv_proj.tune(num_tokens, "rotary" if fused_rot else "store", sa.head_dim)
        sa.o_proj.tune(num_tokens)
        self.mlp.gate_up_proj.tune(num_tokens, "silu" if fused_rot else "store")
        self.mlp.down_proj.tune(num_tokens)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor, layer_cache_idx: int,
                attention_backend_wrapper) -> torch.Tensor:
        normed = self.input_layernorm(hidden_states)
        out = torch.empty_like(hidden_states)  # caller-owned result, like the reference's
        self._attn_mlp(positions, normed, hidden_states, layer_cache_idx, attention_backend_wrapper, None, 0.0,
                       out=out)
        return out

    def forward_carry(self, positions: torch.Tensor, normed: torch.Tensor, residual: torch.Tensor,
                      layer_cache_idx: int, attention_backend_wrapper, next_norm: RMSNorm,
                      shard_residual: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
        """(normed_l, residual_l) -> (normed_{l+1}, residual_{l+1}); ``next_norm`` is the following
        layer's input_layernorm (or the model's final norm).

        ``shard_residual``: the residual stream is only ever read by the tail of the next row-parallel
        projection, which touches the rows this rank owns (rows [rank * ceil(T/tp), ...)); with this flag
        the returned residual is guaranteed for those rows only (the other ranks' rows are not gathered),
        and the ``residual`` passed in needs to be valid for those rows only -- what a stack of layers
        calling each other through ``forward_carry`` needs.  The normed hidden states are always complete."""
        return self._attn_mlp(positions, normed, residual, layer_cache_idx, attention_backend_wrapper,
                              next_norm.weight.data, next_norm.variance_epsilon,
                              resid_everywhere=not shard_residual)


class LlamaModel(nn.Module):
    """Embedding, the stack of decoder layers and the final norm, with the reference's attribute names
    (``embed_tokens``, ``layers``, ``norm``) and forward signature (models/llama.py:258-314; one pipeline stage).

    The layers call each other through ``forward_carry``: the normed hidden states and the residual stream (kept
    sharded by rows) go from layer to layer, every layer is four kernels, and the last one applies ``norm`` --
    the reference's ``norm(hidden_states)`` after the loop -- in its down-projection kernel."""

    def __init__(self, config) -> None:
        super().__init__()
        self.config = config
        self.padding_idx = getattr(config, "pad_token_id", None)
        self.vocab_size = config.vocab_size
        vocab_size = ((config.vocab_size + 63) // 64) * 64
        self.embed_tokens = VocabParallelEmbedding(vocab_size, config.hidden_size, perform_initialization=False)
        self.layers = nn.ModuleList([LlamaDecoderLayer(config, layer_id=i) for i in range(config.num_hidden_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps)

    def forward(self, hidden_states: torch.Tensor, positions: torch.Tensor, attention_backend_wrapper) -> torch.Tensor:
        """``hidden_states``: token ids [T] (looked up in ``embed_tokens``); returns norm(last hidden states) [T, H]."""
        residual = self.embed_tokens(hidden_states)
        normed = self.layers[0].input_layernorm(residual)
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            next_norm = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            normed, residual = layer.forward_carry(positions, normed, residual, i, attention_backend_wrapper, next_norm,
                                                   shard_residual=True)
        return normed


class LlamaForCausalLM(nn.Module):
    """``model`` + ``lm_head`` (vocabulary-sharded ColumnParallelLinear, no bias, output not gathered), as in
    models/llama.py:317-345; ``compute_logits`` is the sampler's projection + gather (layers/sampler.py:89-97)."""

    def __init__(self, config) -> None:
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        vocab_size = ((config.vocab_size + 63) // 64) * 64
        self.lm_head = ColumnParallelLinear(config.hidden_size, vocab_size, bias=False, gather_output=False,
                                            perform_initialization=False)

    def forward(self, hidden_states: torch.Tensor, positions: torch.Tensor, attention_backend_wrapper) -> torch.Tensor:
        return self.model(hidden_states, positions, attention_backend_wrapper)

    def compute_logits(self, hidden_states: torch.Tensor) -> torch.Tensor:
        """[num_rows, H] -> [num_rows, vocab]: this rank's vocabulary slice of the logits, gathered over the ranks
        and cut to the real vocabulary size."""
        logits, _ = self.lm_head(hidden_states)
        logits = gather_from_tensor_model_parallel_region(logits)
        return logits[:, :self.config.vocab_size]


class MixtralMoE(nn.Module):
    """Router + experts of a Mixtral block, every expert sharded over the tensor-parallel ranks
    (sarathi/model_executor/models/mixtral.py:58-108): ``gate`` is a replicated [E, H] linear,
    ``experts`` a FusedMoE that also all-reduces its output."""

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int,
                 params_dtype: Optional[torch.dtype] = None, layer_id: Optional[int] = None):
        super().__init__()
        self.hidden_size = hidden_size
        self.gate = ReplicatedLinear(hidden_size, num_experts, bias=False, params_dtype=params_dtype,
                                     layer_id=layer_id)
        self.experts = FusedMoE(num_experts=num_experts, top_k=top_k, hidden_size=hidden_size,
                                intermediate_size=intermediate_size, params_dtype=params_dtype, reduce_results=True,
                                renormalize=True, layer_id=layer_id)

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        num_tokens, hidden_size = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)
        router_logits, _ = self.gate(hidden_states)
        final_hidden_states = self.experts(hidden_states, router_logits)
        return final_hidden_states.view(num_tokens, hidden_size)

    def forward_fused(self, hidden_states: torch.Tensor, residual: torch.Tensor) -> torch.Tensor:
        """``residual + moe(hidden_states)`` in a new tensor; ``hidden_states`` is left as it is (it may be a
        view into the communication context)."""
        router_logits, _ = self.gate(hidden_states)
        return self.experts.forward_fused(hidden_states, router_logits, residual)


class MixtralDecoderLayer(nn.Module):
    """Mixtral decoder layer (mixtral.py:194-258): Llama-style attention block, MoE feed-forward.
    Attribute / parameter names follow the reference: ``self_attn``, ``block_sparse_moe``,
    ``input_layernorm``, ``post_attention_layernorm``."""

    def __init__(self, config, layer_id: Optional[int] = None) -> None:
        super().__init__()
        self.hidden_size = config.hidden_size
        rope_theta = getattr(config, "rope_theta", 10000)
        self.self_attn = LlamaAttention(hidden_size=self.hidden_size, num_heads=config.num_attention_heads,
                                        num_kv_heads=config.num_key_value_heads, rope_theta=rope_theta,
                                        max_position_embeddings=getattr(config, "max_position_embeddings", 8192),
                                        layer_id=layer_id)
        self.block_sparse_moe = MixtralMoE(num_experts=config.num_local_experts, top_k=config.num_experts_per_tok,
                                           hidden_size=config.hidden_size,
                                           intermediate_size=config.intermediate_size, layer_id=layer_id)
        self.input_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps, layer_id=layer_id)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, eps=config.rms_norm_eps, layer_id=layer_id)

    def forward(self, positions: torch.Tensor, hidden_states: torch.Tensor, layer_cache_idx: int,
                attention_backend_wrapper) -> torch.Tensor:
        sa = self.self_attn
        normed = self.input_layernorm(hidden_states)
        q, k, v = sa.qkv_rotary(positions, normed, fused_kv_append(attention_backend_wrapper, layer_cache_idx))
        attn_out = attention_backend_wrapper.forward(q, k, v, layer_cache_idx, sa.scaling, sa.layer_id)
        # o_proj + all-reduce + residual add + post-attention RMSNorm in one kernel
        h, resid = sa.o_proj.forward_fused(attn_out, hidden_states, self.post_attention_layernorm.weight.data,
                                           self.post_attention_layernorm.variance_epsilon)
        # experts + sum over the routed slots + all-reduce + the layer's residual add, without touching `h`
        return self.block_sparse_moe.forward_fused(h, resid)
