"""Seeded synthetic inputs for the tensor-parallel decoder-layer path.

One CPU ``torch.Generator`` per case draws, in this fixed order, the FULL
(unsharded) fp32 tensors  Wq [nq*hd, H], Wk [nkv*hd, H], Wv, Wo [H, nq*hd],
Wgate [I, H], Wup [I, H], Wdown [H, I]  ~ N(0, 0.02^2), then the hidden states
x [T, H] ~ N(0, 1), then the decode positions.  Every rank draws the same
tensors and slices its shard the way the reference's loaders do
(models/llama.py:395-470: q/k/v row blocks per rank concatenated, gate/up row
blocks concatenated, o/down column blocks), so no broadcast is needed.  These
inputs stand in for the trace-driven workloads of the reference's benchmark
harness: the path is token-wise, only shapes and value distributions matter.
"""
from __future__ import annotations

from dataclasses import dataclass
from types import SimpleNamespace
from typing import Dict

import torch


@dataclass
class LayerCase:
    name: str
    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    intermediate_size: int
    rms_norm_eps: float
    rope_theta: float
    max_position: int
    prefill_tokens: int
    prefill_start: int
    decode_tokens: int
    decode_pos_lo: int
    decode_pos_hi: int
    dtype: torch.dtype
    seed: int = 0
    norm_weight_noise: float = 0.0  # 0 -> ones (as the reference constructs them)

    @property
    def num_tokens(self) -> int:
        return self.prefill_tokens + self.decode_tokens

    def hf_config(self) -> SimpleNamespace:
        """Plain-namespace model config with the attribute names the decoder layer reads."""
        return SimpleNamespace(hidden_size=self.hidden_size, num_attention_heads=self.num_heads,
                               num_key_value_heads=self.num_kv_heads, intermediate_size=self.intermediate_size,
                               rms_norm_eps=self.rms_norm_eps, rope_theta=self.rope_theta, rope_scaling=None,
                               max_position_embeddings=self.max_position, hidden_act="silu", num_hidden_layers=1)


# Named workloads (config1: CPU/gloo fp32 oracle case, config2: Llama-3-8B-shaped bf16 layer, config4_*: 70B-shaped).
CASES: Dict[str, LayerCase] = {
    "config1": LayerCase("config1", 1024, 16, 4, 64, 2816, 1e-5, 10000.0, 2048, 256, 0, 32, 256, 2048, torch.float32),
    "config2": LayerCase("config2", 4096, 32, 8, 128, 14336, 1e-5, 500000.0, 8192, 448, 0, 64, 512, 8192, torch.bfloat16),
    "config2_mid": LayerCase("config2_mid", 4096, 32, 8, 128, 14336, 1e-5, 500000.0, 8192, 448, 1024, 64, 512, 8192,
                             torch.bfloat16),
    "config4_512": LayerCase("config4_512", 8192, 64, 8, 128, 28672, 1e-5, 500000.0, 8192, 448, 0, 64, 512, 8192,
                             torch.bfloat16),
    "config4_2048": LayerCase("config4_2048", 8192, 64, 8, 128, 28672, 1e-5, 500000.0, 8192, 1792, 0, 256, 2048, 8192,
                              torch.bfloat16),
    # small cases for fast parity tests and golden fixtures
    "mini_f32": LayerCase("mini_f32", 256, 4, 2, 64, 512, 1e-5, 10000.0, 512, 20, 0, 4, 20, 512, torch.float32,
                          norm_weight_noise=0.02),
    "mini_bf16": LayerCase("mini_bf16", 512, 4, 2, 128, 1024, 1e-5, 500000.0, 1024, 40, 3, 9, 64, 1024, torch.bfloat16,
                           norm_weight_noise=0.02),
    "mini_f16": LayerCase("mini_f16", 512, 8, 2, 64, 768, 1e-6, 10000.0, 1024, 130, 0, 6, 130, 1024, torch.float16,
                          norm_weight_noise=0.02),
    # eight kv heads: shards over up to 8 tensor-parallel ranks (the reference splits whole kv heads)
    "mini8_bf16": LayerCase("mini8_bf16", 1024, 8, 8, 128, 2048, 1e-5, 500000.0, 1024, 57, 5, 12, 64, 1024, torch.bfloat16,
                            norm_weight_noise=0.02),
}


@dataclass
class LayerTensors:
    case: LayerCase
    wq: torch.Tensor
    wk: torch.Tensor
    wv: torch.Tensor
    wo: torch.Tensor
    wgate: torch.Tensor
    wup: torch.Tensor
    wdown: torch.Tensor
    x: torch.Tensor
    positions: torch.Tensor
    ln1: torch.Tensor
    ln2: torch.Tensor


def generate(case: LayerCase) -> LayerTensors:
    """Full fp32 tensors of a case (cast / shard with ``shard``)."""
    c = case
    g = torch.Generator(device="cpu").manual_seed(c.seed)
    H, I, hd = c.hidden_size, c.intermediate_size, c.head_dim

    def w(rows, cols):
        return torch.randn(rows, cols, generator=g, dtype=torch.float32) * 0.02

    wq, wk, wv = w(c.num_heads * hd, H), w(c.num_kv_heads * hd, H), w(c.num_kv_heads * hd, H)
    wo = w(H, c.num_heads * hd)
    wgate, wup, wdown = w(I, H), w(I, H), w(H, I)
    x = torch.randn(c.num_tokens, H, generator=g, dtype=torch.float32)
    prefill = torch.arange(c.prefill_start, c.prefill_start + c.prefill_tokens, dtype=torch.int64)
    decode = torch.randint(c.decode_pos_lo, c.decode_pos_hi, (c.decode_tokens,), generator=g, dtype=torch.int64)
    positions = torch.cat([prefill, decode])
    if c.norm_weight_noise > 0:
        ln1 = 1.0 + torch.randn(H, generator=g, dtype=torch.float32) * c.norm_weight_noise
        ln2 = 1.0 + torch.randn(H, generator=g, dtype=torch.float32) * c.norm_weight_noise
    else:
        ln1, ln2 = torch.ones(H, dtype=torch.float32), torch.ones(H, dtype=torch.float32)
    return LayerTensors(c, wq, wk, wv, wo, wgate, wup, wdown, x, positions, ln1, ln2)


def shard(t: LayerTensors, rank: int, world: int, dtype: torch.dtype = None) -> Dict[str, torch.Tensor]:
    """This rank's parameters, named like the reference's state dict, in the case dtype."""
    dtype = dtype or t.case.dtype

    def rows(wt):
        return wt.chunk(world, dim=0)[rank]

    def cols(wt):
        return wt.chunk(world, dim=1)[rank]

    return {
        "self_attn.qkv_proj.weight": torch.cat([rows(t.wq), rows(t.wk), rows(t.wv)], 0).to(dtype).contiguous(),
        "self_attn.o_proj.weight": cols(t.wo).to(dtype).contiguous(),
        "mlp.gate_up_proj.weight": torch.cat([rows(t.wgate), rows(t.wup)], 0).to(dtype).contiguous(),
        "mlp.down_proj.weight": cols(t.wdown).to(dtype).contiguous(),
        "input_layernorm.weight": t.ln1.to(dtype).contiguous(),
        "post_attention_layernorm.weight": t.ln2.to(dtype).contiguous(),
    }


def load_layer(layer: torch.nn.Module, params: Dict[str, torch.Tensor]) -> None:
    """Copy a ``shard`` dict into a decoder layer through its state dict (as the reference's loaders do)."""
    sd = layer.state_dict()
    with torch.no_grad():
        for name, value in params.items():
            sd[name].copy_(value.to(sd[name].device))


# ------------------------------------------------------------------ MoE cases
@dataclass
class MoeCase:
    name: str
    hidden_size: int
    num_experts: int
    top_k: int
    intermediate_size: int
    num_tokens: int
    dtype: torch.dtype
    block_size: int = 64
    seed: int = 0


MOE_CASES: Dict[str, MoeCase] = {
    "config5": MoeCase("config5", 4096, 8, 2, 14336, 1024, torch.bfloat16),
    "mini_moe": MoeCase("mini_moe", 256, 8, 2, 512, 77, torch.bfloat16),
}


def generate_moe(case: MoeCase, world: int = 1, rank: int = 0) -> Dict[str, torch.Tensor]:
    """Router logits ~ N(0,1) drawn directly, hidden states ~ N(0,1), expert weights ~ N(0, 0.02^2)
    (w13 [E, 2I, H] = gate rows then up rows, w2 [E, H, I]), sharded along I for ``rank``."""
    c = case
    g = torch.Generator(device="cpu").manual_seed(c.seed)
    logits = torch.randn(c.num_tokens, c.num_experts, generator=g, dtype=torch.float32)
    x = torch.randn(c.num_tokens, c.hidden_size, generator=g, dtype=torch.float32)
    Ish = c.intermediate_size // world
    w13 = torch.empty(c.num_experts, 2 * Ish, c.hidden_size, dtype=torch.float32)
    w2 = torch.empty(c.num_experts, c.hidden_size, Ish, dtype=torch.float32)
    for e in range(c.num_experts):
        # drawn per expert and per rank-shard so that large cases never materialise the full fp32 weights
        for r in range(world):
            gate = torch.randn(Ish, c.hidden_size, generator=g, dtype=torch.float32) * 0.02
            up = torch.randn(Ish, c.hidden_size, generator=g, dtype=torch.float32) * 0.02
            down = torch.randn(c.hidden_size, Ish, generator=g, dtype=torch.float32) * 0.02
            if r == rank:
                w13[e, :Ish], w13[e, Ish:], w2[e] = gate, up, down
    return {"logits": logits, "x": x.to(c.dtype), "w13": w13.to(c.dtype), "w2": w2.to(c.dtype)}
