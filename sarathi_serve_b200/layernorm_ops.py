"""Drop-in for the reference's pybind module ``sarathi.layernorm_ops``
(csrc/layernorm.cpp:3-13): same function name, argument order and in-place
output convention, backed by the sm_100a kernel behind the C ABI."""
import torch

from . import _native as N


def rms_norm(out: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:
    """out[T,H] <- RMSNorm(input[T,H]) * weight[H] (csrc/layernorm_kernels.cu:39-62)."""
    N.require_cuda(out, input, weight)
    if not (input.is_contiguous() and out.is_contiguous() and weight.is_contiguous()):
        raise RuntimeError("rms_norm: tensors must be contiguous")
    if out.dtype != input.dtype or weight.dtype != input.dtype:
        raise RuntimeError("rms_norm: out, input and weight must share a dtype")
    H = input.shape[-1]
    T = input.numel() // H if H else 0
    N.check(N.lib().sb200_rms_norm(N.ptr(out), N.ptr(input), N.ptr(weight), float(epsilon), T, H,
                                   N.dtype_id(input), N.stream_ptr()), "rms_norm")


def fused_add_rms_norm(out: torch.Tensor, residual_out: torch.Tensor, input: torch.Tensor,
                       residual: torch.Tensor, weight: torch.Tensor, epsilon: float) -> None:
    """residual_out <- input + residual (rounded to the dtype); out <- RMSNorm(residual_out) * weight.

    The reference has no such op: it is the torch add of models/llama.py:248,254
    followed by rms_norm, in one pass over the rows."""
    N.require_cuda(out, residual_out, input, residual, weight)
    for t in (out, residual_out, input, residual, weight):
        if not t.is_contiguous():
            raise RuntimeError("fused_add_rms_norm: tensors must be contiguous")
        if t.dtype != input.dtype:
            raise RuntimeError("fused_add_rms_norm: dtype mismatch")
    H = input.shape[-1]
    T = input.numel() // H if H else 0
    N.check(N.lib().sb200_fused_add_rms_norm(N.ptr(out), N.ptr(residual_out), N.ptr(input), N.ptr(residual),
                                             N.ptr(weight), float(epsilon), T, H, N.dtype_id(input),
                                             N.stream_ptr()), "fused_add_rms_norm")
