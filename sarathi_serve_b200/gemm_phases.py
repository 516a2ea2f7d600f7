"""Where the time of one tcgen05 GEMM launch goes: phase marks of CTA 0, read from a trace build.

The product library carries no trace code.  ``python -m sarathi_serve_b200.build --trace DIR`` compiles the
same sources with ``-DSB200_TRACE`` into ``DIR/libsarathi_b200_trace.so``; in that build CTA 0 of every GEMM
launch stores ``%globaltimer`` at its phase boundaries (prologue done, first load requested / arrived, last MMA
issued, accumulators complete, tile stored, TMEM released ...).  This module replays a CUDA graph of back-to-back
launches of one problem on that library and prints the marks in microseconds from the kernel's entry, plus the
gap between one launch's TMEM release and the next launch's entry.  Every mark costs ~0.1 us itself.

    python -m sarathi_serve_b200.build --trace /tmp/sb200_trace
    python -m sarathi_serve_b200.gemm_phases --library /tmp/sb200_trace/libsarathi_b200_trace.so
"""
from __future__ import annotations

import argparse
import ctypes
import os
import sys

MARKS = ["entry", "prologue done", "first stage requested", "last stage requested", "first stage arrived",
         "last MMA issued", "accumulators complete", "tile stored (warp 2)", "exit barrier passed (thread 0)",
         "TMEM released", "dependency wait done", "stage 0 free", "before TMEM release", "tile stored (warp 9)",
         "producer entered", "first work item known"]
ORDER = (1, 10, 14, 15, 11, 2, 4, 3, 5, 6, 7, 13, 12, 9)
# cluster K-split launches reuse three slots for the exchange
MARKS_SPLIT = dict(enumerate(MARKS))
MARKS_SPLIT.update({6: "all pairs' MMAs complete", 7: "shares handed to the copy engine", 13: "shares received"})


def run(lib, dense_ops, torch, T, N, K, cfg, launches=8):
    dev = torch.device("cuda", torch.cuda.current_device())
    copies = 8
    ws = [torch.randn(N, K, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
    x = torch.randn(T, K, device=dev).to(torch.bfloat16)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        dense_ops.linear(x, ws[0], tile_n=cfg)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for i in range(launches):
                dense_ops.linear(x, ws[i % copies], tile_n=cfg)
        graph.replay()
        graph.replay()
        torch.cuda.synchronize()
    buf = (ctypes.c_ulonglong * (64 * 16))()
    count = ctypes.c_uint(0)
    lib.sb200_debug_gemm_trace(buf, ctypes.byref(count))
    last = count.value
    rows = [[buf[((last - launches + i) % 64) * 16 + j] for j in range(16)] for i in range(launches)]
    acc = [0.0] * 16
    gaps = []
    for i in range(2, launches):  # the first launches of a replay start on an idle GPU
        for j in range(16):
            acc[j] += (rows[i][j] - rows[i][0]) / 1e3
        gaps.append((rows[i][0] - rows[i - 1][9]) / 1e3)
    m = launches - 2
    names = MARKS_SPLIT if (cfg // 1000) % 100 == 5 else dict(enumerate(MARKS))
    print(f"T={T} N={N} K={K} tile_cfg={cfg}: next launch enters {sum(gaps) / len(gaps):.2f} us after this one released its TMEM")
    for j in ORDER:
        if acc[j] > 0:
            print(f"    {names[j]:36s} {acc[j] / m:6.2f} us")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--library", required=True, help="libsarathi_b200_trace.so made by `build --trace DIR`")
    ap.add_argument("--problem", action="append", default=[], help="T,N,K,tile_cfg (repeatable)")
    args = ap.parse_args(argv)
    os.environ["SB200_LIBRARY"] = os.path.abspath(args.library)
    import torch

    from . import _native, dense_ops
    lib = _native.lib()
    if not hasattr(lib, "sb200_debug_gemm_trace"):
        print("this library was not built with --trace", file=sys.stderr)
        return 2
    lib.sb200_debug_gemm_trace.restype = ctypes.c_int
    lib.sb200_debug_gemm_trace.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    torch.cuda.set_device(0)
    problems = [tuple(int(v) for v in p.split(",")) for p in args.problem] or [
        (128, 128, 64, 128), (512, 4096, 512, 101128), (512, 4096, 512, 3256), (512, 4096, 512, 205256),
        (512, 768, 512, 405128)]
    for T, N, K, cfg in problems:
        run(lib, dense_ops, torch, T, N, K, cfg)
    return 0


if __name__ == "__main__":
    sys.exit(main())
