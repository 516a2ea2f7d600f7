"""Where the time of one tcgen05 GEMM launch goes: phase marks of CTA 0, read from a trace build.

The product library carries no trace code.  ``python -m sarathi_serve_b200.build --trace DIR`` compiles the
same sources with ``-DSB200_TRACE`` into ``DIR/libsarathi_b200_trace.so``; in that build CTA 0 of every GEMM
launch stores ``%globaltimer`` at its phase boundaries (prologue done, first load requested / arrived, last MMA
issued, accumulators complete, tile stored, TMEM released ...).  This module replays a CUDA graph of back-to-back
launches of one problem on that library and prints the marks in microseconds from the kernel's entry, plus the
gap between one launch's TMEM release and the next launch's entry.  Every mark costs ~0.1 us itself.

    python -m sarathi_serve_b200.build --trace /tmp/sb200_trace
    python -m sarathi_serve_b200.gemm_phases --library /tmp/sb200_trace/libsarathi_b200_trace.so

``--sweep`` needs no trace build: it times launches of the product library with CUDA events for a range of K
per tile configuration (fixed cost and per-k-block cost of each schedule) and the same problem on cuBLAS.
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


def _time_graph(torch, call, launches=8, reps=5):
    stream = torch.cuda.Stream()
    try:
        with torch.cuda.stream(stream):
            call(0)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(launches):
                    call(i)
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(reps):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (launches * reps)
    except RuntimeError:  # the planner rejects the configuration for this problem
        return float("nan")


def sweep(dense_ops, torch, T=512):
    """Microseconds per launch against K for some tile configurations (weights cycled through more than L2)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    ks = (64, 256, 512, 1024, 2048, 4096)

    def time_cfg(t, n, k, cfg):
        copies = max(2, min(8, int(260e6 // (n * k * 2)) + 1))
        ws = [torch.randn(n, k, device=dev).mul_(0.02).to(torch.bfloat16) for _ in range(copies)]
        x = torch.randn(t, k, device=dev).to(torch.bfloat16)
        return _time_graph(torch, lambda i: dense_ops.linear(x, ws[i % copies], tile_n=cfg))

    for n, cfgs in ((4096, (101128, 3128, 3256, 205256, 203256)), (768, (101128, 3064, 405128, 205128, 205064)),
                    (3584, (3128, 3256, 205256, 203256))):
        print(f"T={T} N={n}: us per launch (graph of 8)")
        print("tile_cfg  " + "".join(f"K={k:<7d}" for k in ks) + " ns per k-block (2048->4096)   intercept us")
        for cfg in cfgs:
            ts = [time_cfg(T, n, k, cfg) for k in ks]
            slope = (ts[5] - ts[4]) / 32 * 1e3
            print(f"{cfg:<9d} " + "".join(f"{t:<9.1f}" for t in ts) + f" {slope:8.0f} {ts[5] - slope * 64 / 1e3:27.1f}")
    print(f"launch floor, T=128 N=128 K=64: {time_cfg(128, 128, 64, 128):.2f} us")
    x = torch.randn(512, 512, device=dev).to(torch.bfloat16)
    ws = [torch.randn(4096, 512, device=dev).to(torch.bfloat16) for _ in range(8)]
    y = torch.empty(512, 4096, device=dev, dtype=torch.bfloat16)
    print(f"cuBLAS (torch.matmul) 512x4096x512: {_time_graph(torch, lambda i: torch.matmul(x, ws[i % 8].t(), out=y)):.2f} us; "
          f"this library, tile_cfg 101128: {time_cfg(512, 4096, 512, 101128):.2f} us")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--library", help="libsarathi_b200_trace.so made by `build --trace DIR`")
    ap.add_argument("--sweep", action="store_true", help="CUDA-event time per launch against K (product library)")
    ap.add_argument("--problem", action="append", default=[], help="T,N,K,tile_cfg (repeatable)")
    args = ap.parse_args(argv)
    if not args.sweep and not args.library:
        ap.error("give --library (phase marks of a trace build) or --sweep")
    if args.library:
        os.environ["SB200_LIBRARY"] = os.path.abspath(args.library)
    import torch

    from . import _native, dense_ops
    torch.cuda.set_device(0)
    if args.sweep:
        sweep(dense_ops, torch)
        return 0
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
