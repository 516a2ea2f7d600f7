"""Module wrappers with the reference's class names and constructor signatures:
RMSNorm (sarathi/model_executor/layers/layernorm.py:12-40), SiluAndMul / NewGELU
/ FastGELU (layers/activation.py:9-45) and the rotary embedding family with
get_rope (layers/rotary_embedding.py:33-344).  They allocate the output and call
the ops modules of this package."""
from __future__ import annotations

import math
from typing import Any, Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import activation_ops, layernorm_ops, pos_encoding_ops


def _param_device():
    return torch.cuda.current_device() if torch.cuda.is_available() else "cpu"


class RMSNorm(nn.Module):
    """x -> w * x / sqrt(mean(x^2) + eps)."""

    def __init__(self, hidden_size: int, eps: float = 1e-6, norm_name: Optional[str] = None,
                 layer_id: Optional[int] = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden_size, device=_param_device()), requires_grad=False)
        self.variance_epsilon = eps

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        layernorm_ops.rms_norm(out, x, self.weight.data, self.variance_epsilon)
        return out

    def forward_add(self, x: torch.Tensor, residual: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """(rms_norm(x + residual), x + residual) in one pass over the rows."""
        out, z = torch.empty_like(x), torch.empty_like(x)
        layernorm_ops.fused_add_rms_norm(out, z, x, residual, self.weight.data, self.variance_epsilon)
        return out, z


class SiluAndMul(nn.Module):
    """x -> silu(x[:, :d]) * x[:, d:], d = x.shape[1] // 2."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape[0], x.shape[1] // 2, dtype=x.dtype, device=x.device)
        activation_ops.silu_and_mul(out, x)
        return out


class NewGELU(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        activation_ops.gelu_new(out, x)
        return out


class FastGELU(nn.Module):
    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty_like(x)
        activation_ops.gelu_fast(out, x)
        return out


_ACTIVATION_REGISTRY = {"gelu": nn.GELU(), "gelu_fast": FastGELU(), "gelu_new": NewGELU(),
                        "gelu_pytorch_tanh": nn.GELU(approximate="tanh"), "relu": nn.ReLU()}


def get_act_fn(act_fn: str) -> nn.Module:
    act_fn = act_fn.lower()
    if act_fn in _ACTIVATION_REGISTRY:
        return _ACTIVATION_REGISTRY[act_fn]
    raise ValueError(f"Activation function {act_fn!r} is not supported.")


# --------------------------------------------------------------------- rotary
def _inv_freq(base: float, rotary_dim: int, device) -> torch.Tensor:
    exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float, device=device) / rotary_dim
    return 1.0 / (base ** exponents)


def _cache_from(inv_freq: torch.Tensor, positions: torch.Tensor, mscale: float = 1.0) -> torch.Tensor:
    freqs = torch.einsum("i,j -> ij", positions, inv_freq)
    return torch.cat((freqs.cos() * mscale, freqs.sin() * mscale), dim=-1)


class RotaryEmbedding(nn.Module):
    """Rotary position embedding with a precomputed [max_pos, rot_dim] cos|sin table
    in the default dtype (reference: rotary_embedding.py:33-102)."""

    def __init__(self, head_size: int, rotary_dim: int, max_position_embeddings: int, base: int,
                 is_neox_style: bool) -> None:
        super().__init__()
        self.head_size = head_size
        self.rotary_dim = rotary_dim
        self.max_position_embeddings = max_position_embeddings
        self.base = base
        self.is_neox_style = is_neox_style
        cache = self._compute_cos_sin_cache().to(torch.get_default_dtype())
        self.register_buffer("cos_sin_cache", cache, persistent=False)

    def _device(self):
        return _param_device()

    def _compute_cos_sin_cache(self) -> torch.Tensor:
        dev = self._device()
        t = torch.arange(self.max_position_embeddings, dtype=torch.float, device=dev)
        return _cache_from(_inv_freq(self.base, self.rotary_dim, dev), t)

    def forward(self, positions: torch.Tensor, query: torch.Tensor, key: torch.Tensor):
        pos_encoding_ops.rotary_embedding(positions, query, key, self.head_size, self.cos_sin_cache,
                                          self.is_neox_style)
        return query, key

    def rotate_inplace(self, positions: torch.Tensor, heads: torch.Tensor, num_heads: int) -> None:
        """Rotate a single strided [T, num_heads*head_size] view (q and k heads together)."""
        pos_encoding_ops.rotary_embedding(positions, heads, heads[:, :0], self.head_size, self.cos_sin_cache,
                                          self.is_neox_style)


class LinearScalingRotaryEmbedding(RotaryEmbedding):
    """Positions divided by a constant factor; table covers max_pos * factor positions."""

    def __init__(self, head_size, rotary_dim, max_position_embeddings, base, is_neox_style, scaling_factor: float):
        self.scaling_factor = scaling_factor
        super().__init__(head_size, rotary_dim, max_position_embeddings, base, is_neox_style)

    def _compute_cos_sin_cache(self) -> torch.Tensor:
        dev = self._device()
        max_len = self.max_position_embeddings * self.scaling_factor
        t = torch.arange(max_len, dtype=torch.float, device=dev) / self.scaling_factor
        return _cache_from(_inv_freq(self.base, self.rotary_dim, dev), t)


class DynamicNTKScalingRotaryEmbedding(RotaryEmbedding):
    """NTK-aware base rescaling for the extended length max_pos * factor."""

    def __init__(self, head_size, rotary_dim, max_position_embeddings, base, is_neox_style, scaling_factor: float):
        self.scaling_factor = scaling_factor
        super().__init__(head_size, rotary_dim, max_position_embeddings, base, is_neox_style)

    def _compute_cos_sin_cache(self) -> torch.Tensor:
        dev = self._device()
        max_len = self.max_position_embeddings * self.scaling_factor
        ratio = (self.scaling_factor * max_len / self.max_position_embeddings) - (self.scaling_factor - 1)
        base = self.base * ratio ** (self.rotary_dim / (self.rotary_dim - 2))
        t = torch.arange(max_len, dtype=torch.float, device=dev)
        return _cache_from(_inv_freq(base, self.rotary_dim, dev), t)


def _yarn_correction_dim(num_rotations: float, dim: int, base: float, max_pos: int) -> float:
    return (dim * math.log(max_pos / (num_rotations * 2 * math.pi))) / (2 * math.log(base))


def _yarn_correction_range(low_rot, high_rot, dim, base, max_pos):
    low = math.floor(_yarn_correction_dim(low_rot, dim, base, max_pos))
    high = math.ceil(_yarn_correction_dim(high_rot, dim, base, max_pos))
    return max(low, 0), min(high, dim - 1)


def _yarn_mscale(scale: float = 1.0) -> float:
    return 1.0 if scale <= 1 else 0.1 * math.log(scale) + 1.0


class YaRNScalingRotaryEmbedding(RotaryEmbedding):
    """YaRN (Peng et al.): blend of interpolated and extrapolated frequencies with a
    linear ramp between two rotation counts, and a magnitude correction."""

    def __init__(self, head_size, rotary_dim, max_position_embeddings, base, is_neox_style, scaling_factor: float, *,
                 extrapolation_factor: float = 1, attn_factor: float = 1, beta_fast: float = 32,
                 beta_slow: float = 1) -> None:
        self.scaling_factor = scaling_factor
        self.extrapolation_factor = extrapolation_factor
        self.attn_factor = attn_factor
        self.beta_fast = beta_fast
        self.beta_slow = beta_slow
        self.mscale = float(_yarn_mscale(self.scaling_factor) * attn_factor)
        super().__init__(head_size, rotary_dim, max_position_embeddings, base, is_neox_style)

    def _compute_cos_sin_cache(self) -> torch.Tensor:
        dev = self._device()
        pos_freqs = self.base ** (torch.arange(0, self.rotary_dim, 2, dtype=torch.float, device=dev) / self.rotary_dim)
        extrapolation = 1.0 / pos_freqs
        interpolation = 1.0 / (self.scaling_factor * pos_freqs)
        low, high = _yarn_correction_range(self.beta_fast, self.beta_slow, self.rotary_dim, self.base,
                                           self.max_position_embeddings)
        if low == high:
            high += 0.001
        ramp = torch.clamp((torch.arange(self.rotary_dim // 2, dtype=torch.float, device=dev) - low) / (high - low), 0, 1)
        mask = (1 - ramp) * self.extrapolation_factor
        inv_freq = interpolation * (1 - mask) + extrapolation * mask
        t = torch.arange(self.max_position_embeddings * self.scaling_factor, device=dev, dtype=torch.float32)
        return _cache_from(inv_freq, t, self.mscale)


def get_rope(head_size: int, rotary_dim: int, max_position: int, base: int, is_neox_style: bool,
             rope_scaling: Optional[Dict[str, Any]]) -> RotaryEmbedding:
    """Factory with the reference's signature and scaling-type names (rotary_embedding.py:301-344)."""
    if rope_scaling is None:
        return RotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style)
    kind = rope_scaling["type"]
    factor = rope_scaling["factor"]
    if kind == "linear":
        return LinearScalingRotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, factor)
    if kind == "dynamic":
        return DynamicNTKScalingRotaryEmbedding(head_size, rotary_dim, max_position, base, is_neox_style, factor)
    if kind == "yarn":
        original = rope_scaling["original_max_position_embeddings"]
        assert max_position == original * factor
        extra = {k: v for k, v in rope_scaling.items()
                 if k in ("extrapolation_factor", "attn_factor", "beta_fast", "beta_slow")}
        return YaRNScalingRotaryEmbedding(head_size, rotary_dim, original, base, is_neox_style, factor, **extra)
    raise ValueError(f"Unknown RoPE scaling type {kind}")
