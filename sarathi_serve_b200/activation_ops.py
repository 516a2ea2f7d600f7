"""Drop-in for the reference's pybind module ``sarathi.activation_ops``
(csrc/activation.cpp:3-27)."""
import torch

from . import _native as N


def _check(out, input, fn):
    N.require_cuda(out, input)
    if not (out.is_contiguous() and input.is_contiguous()):
        raise RuntimeError(f"{fn}: tensors must be contiguous")
    if out.dtype != input.dtype:
        raise RuntimeError(f"{fn}: dtype mismatch")


def silu_and_mul(out: torch.Tensor, input: torch.Tensor) -> None:
    """out[T,d] <- silu(input[T,:d]) * input[T,d:] (csrc/activation_kernels.cu:29-48)."""
    _check(out, input, "silu_and_mul")
    d = input.shape[-1] // 2
    T = input.numel() // (2 * d) if d else 0
    if out.numel() != T * d:
        raise RuntimeError("silu_and_mul: out must be [num_tokens, d]")
    N.check(N.lib().sb200_silu_and_mul(N.ptr(out), N.ptr(input), T, d, N.dtype_id(input), N.stream_ptr()),
            "silu_and_mul")


def gelu_new(out: torch.Tensor, input: torch.Tensor) -> None:
    """GPT-2 style tanh GELU (csrc/activation_kernels.cu:86-91,104-109)."""
    _check(out, input, "gelu_new")
    d = input.shape[-1]
    T = input.numel() // d if d else 0
    N.check(N.lib().sb200_gelu_new(N.ptr(out), N.ptr(input), T, d, N.dtype_id(input), N.stream_ptr()), "gelu_new")


def gelu_fast(out: torch.Tensor, input: torch.Tensor) -> None:
    """Approximate GELU (csrc/activation_kernels.cu:93-98,111-116)."""
    _check(out, input, "gelu_fast")
    d = input.shape[-1]
    T = input.numel() // d if d else 0
    N.check(N.lib().sb200_gelu_fast(N.ptr(out), N.ptr(input), T, d, N.dtype_id(input), N.stream_ptr()), "gelu_fast")
