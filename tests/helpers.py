"""Shared helpers of the test-suite (fixture loading, tolerances)."""
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Parity bar: max|a-b| / max|ref| per tensor.
TOL = {torch.float32: 1e-4, torch.bfloat16: 2e-2, torch.float16: 2e-2}

_DT = {"torch.float32": torch.float32, "torch.bfloat16": torch.bfloat16, "torch.float16": torch.float16}


def load_golden(case: str, world: int):
    """Returns (tensors: dict name -> torch tensor in the case dtype, sums: dict, row_step)."""
    z = np.load(os.path.join(GOLDEN, f"{case}_tp{world}.npz"))
    dtype = _DT[str(z["__dtype"][0])]
    step = int(z["__row_step"][0])
    tensors, sums = {}, {}
    for k in z.files:
        if k.startswith("__"):
            continue
        if k.endswith("__sum"):
            sums[k[:-5]] = z[k]
            continue
        a = torch.from_numpy(z[k])
        tensors[k] = a.view(dtype) if a.dtype == torch.int16 else a
    return tensors, sums, step, dtype


def rel_err(a: torch.Tensor, ref: torch.Tensor) -> float:
    denom = float(ref.double().abs().max())
    return float((a.double().cpu() - ref.double().cpu()).abs().max()) / (denom if denom > 0 else 1.0)
