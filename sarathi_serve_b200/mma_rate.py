"""``python -m sarathi_serve_b200.mma_rate``: clocks per tcgen05.mma on this GPU, one CTA (M = 128) against a
CTA pair (M = 256), for N = 64 ... 256, operands resident in shared memory.  These are the constants of the tile
planner's cost model (csrc/gemm.cu): a single CTA's MMA occupies the tensor pipe for about the same number of
clocks whatever its N, a pair runs at N/2 clocks per MMA down to a floor."""
from __future__ import annotations

import torch

from . import _native as N


def measure(pair: bool, n: int, iters: int = 512) -> dict:
    out = torch.zeros(2, dtype=torch.int64, device="cuda")
    for _ in range(2):  # the second run is the one reported
        N.check(N.lib().sb200_diag_mma_rate(1 if pair else 0, n, iters, N.ptr(out), N.stream_ptr()), "diag_mma_rate")
        torch.cuda.synchronize()
    issue, done = (int(v) for v in out.tolist())
    return {"pair": pair, "n": n, "clk_per_mma_issue": issue / (4 * iters), "clk_per_mma_complete": done / (4 * iters),
            "nominal_clk_per_mma": n / 2 if pair else n / 2}


def main() -> None:
    print("mode        N   clk/MMA issued   clk/MMA completed   nominal (128 rows x N x 16 per SM at 8192 FLOP/clk)")
    for pair in (False, True):
        for n in (64, 96, 128, 192, 256):
            if pair and n % 32:
                continue
            r = measure(pair, n)
            print(f"{'CTA pair' if pair else 'one CTA ':9s} {n:4d}   {r['clk_per_mma_issue']:10.1f}   {r['clk_per_mma_complete']:14.1f}   {n / 2:10.1f}")


if __name__ == "__main__":
    main()
