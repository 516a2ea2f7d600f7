"""Tensor-level wrappers of the dense projection entry points of the C ABI
(``sb200_gemm_colpar``): the local matmul of a column-parallel / replicated
linear layer, optionally with the rotary embedding or SiLU*mul applied in the
GEMM epilogue.  bf16/fp16 run on tcgen05 tensor cores, fp32 on an FFMA kernel."""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native as N

EPI_NONE, EPI_ROTARY, EPI_SILU_MUL = 0, 1, 2

_status_words: dict = {}
_workspaces: dict = {}

# Split-K workspace per device: 64 KiB of arrival counters (kept zero by the kernels) + fp32 partial tiles.
WORKSPACE_BYTES = (64 << 10) + (96 << 20)


def workspace(device: torch.device) -> torch.Tensor:
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _workspaces.get(key)
    if w is None:
        w = torch.zeros(WORKSPACE_BYTES, dtype=torch.uint8, device=device)
        _workspaces[key] = w
    return w


def status_word(device: torch.device) -> torch.Tensor:
    """Per-device uint32 word the GEMM kernels write a non-zero code into when a
    bounded pipeline wait runs out (checked by ``check_status``)."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    w = _status_words.get(key)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[key] = w
    return w


def check_status(device: torch.device) -> None:
    """Synchronises and raises if any GEMM on ``device`` reported a timed-out wait."""
    w = status_word(device)
    v = int(w.item())
    if v != 0:
        w.zero_()
        raise RuntimeError(f"sm_100a GEMM pipeline wait timed out (device status code {v})")


_status_host: dict = {}


def enqueue_status_read(device: torch.device) -> None:
    """Asynchronous (graph-capturable) copy of the device's GEMM status word into pinned host memory."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    h = _status_host.get(key)
    if h is None:
        h = _status_host[key] = torch.zeros(1, dtype=torch.int32).pin_memory()
    h.copy_(status_word(device), non_blocking=True)


def raise_if_flagged(device: torch.device) -> None:
    """No synchronisation: raises if the status word last read by ``enqueue_status_read`` was non-zero."""
    key = (device.type, device.index if device.index is not None else torch.cuda.current_device())
    h = _status_host.get(key)
    if h is not None and int(h[0]) != 0:
        code = int(h[0])
        h.zero_()
        status_word(device).zero_()
        raise RuntimeError(f"sm_100a GEMM pipeline wait timed out in an earlier step (device status code {code})")


def _ws(x: torch.Tensor):
    """(pointer, bytes) of the split-K workspace for x's device; fp32 runs the FFMA kernel and needs none."""
    if x.dtype == torch.float32:
        return None, 0
    w = workspace(x.device)
    return N.ptr(w), w.numel()


def _rows_2d(x: torch.Tensor, what: str) -> torch.Tensor:
    if x.dim() != 2:
        x = x.reshape(-1, x.shape[-1])
    if x.stride(1) != 1:
        raise RuntimeError(f"{what}: inner stride must be 1")
    return x


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out: Optional[torch.Tensor] = None, tile_n: int = 0, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """y[T, N] = x[T, K] @ weight[N, K]^T (+ bias): F.linear semantics
    (reference call sites: tensor_parallel/layers.py:284,423,518).  ``residual`` [T, N] (bf16 / fp16 only):
    y = residual + round(x @ weight^T (+ bias)), the add of models/llama.py:248,254 in the GEMM epilogue."""
    N.require_cuda(x, weight, bias, residual)
    lead = x.shape[:-1]
    x2 = _rows_2d(x, "linear input")
    if weight.dim() != 2 or weight.stride(1) != 1 or weight.shape[1] != x2.shape[1]:
        raise RuntimeError(f"linear: weight {tuple(weight.shape)} does not match input {tuple(x.shape)}")
    if weight.dtype != x2.dtype or (bias is not None and bias.dtype != x2.dtype):
        raise RuntimeError("linear: dtype mismatch")
    T, K = x2.shape
    Nn = weight.shape[0]
    if out is None:
        out = torch.empty(T, Nn, dtype=x2.dtype, device=x2.device)
    elif out.shape != (T, Nn) or out.stride(1) != 1 or out.dtype != x2.dtype:
        raise RuntimeError("linear: bad out tensor")
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    ldr = 0
    if residual is not None:
        residual = _rows_2d(residual, "linear residual")
        if residual.shape != (T, Nn) or residual.dtype != x2.dtype:
            raise RuntimeError("linear: residual must be [T, N] of the activation dtype")
        ldr = residual.stride(0)
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), N.ptr(bias), N.ptr(residual), ldr, T, Nn, K, N.dtype_id(x2),
                                      EPI_NONE, None,
                                      N.ptr(status_word(x2.device)), tile_n, *_ws(x2), N.stream_ptr()), "gemm_colpar")
    return out.view(*lead, Nn) if len(lead) != 1 else out


def fused_rotary_supported(x: torch.Tensor, head_size: int, rot_dim: int) -> bool:
    return x.dtype in (torch.bfloat16, torch.float16) and rot_dim == head_size and head_size in (64, 128, 256)


def linear_rotary(x: torch.Tensor, weight: torch.Tensor, positions: torch.Tensor, cos_sin_cache: torch.Tensor,
                  head_size: int, rot_cols: int, is_neox: bool, out: Optional[torch.Tensor] = None,
                  tile_n: int = 0, kv_cache: Optional[torch.Tensor] = None, kv_slots: Optional[torch.Tensor] = None,
                  num_kv_heads: int = 0) -> torch.Tensor:
    """qkv[T, N] = x @ weight^T with rotary_embedding applied to columns [0, rot_cols)
    (the q and k heads) in the GEMM epilogue -- the qkv_proj + rotary_emb pair of
    models/llama.py:175-177 in one kernel.  With ``kv_cache`` ([pages, 2, page_size, num_kv_heads, head_size])
    and ``kv_slots`` (kv_cache_ops.slots(...)) the rotated keys and the values are also appended to the paged
    cache from the epilogue."""
    N.require_cuda(x, weight, positions, cos_sin_cache, kv_cache, kv_slots)
    x2 = _rows_2d(x, "linear_rotary input")
    T, K = x2.shape
    Nn = weight.shape[0]
    if positions.dtype != torch.int64 or positions.numel() != T or not positions.is_contiguous():
        raise RuntimeError("linear_rotary: positions must be contiguous int64 [T]")
    if cos_sin_cache.dtype != x2.dtype or not cos_sin_cache.is_contiguous():
        raise RuntimeError("linear_rotary: cos_sin_cache must be contiguous and share the activation dtype")
    if out is None:
        out = torch.empty(T, Nn, dtype=x2.dtype, device=x2.device)
    page = 0
    if kv_cache is not None:
        if (kv_slots is None or kv_slots.dtype != torch.int64 or kv_slots.numel() != T or not kv_slots.is_contiguous()
                or kv_cache.dim() != 5 or kv_cache.shape[1] != 2 or tuple(kv_cache.shape[3:]) != (num_kv_heads, head_size)
                or kv_cache.dtype != x2.dtype or not kv_cache.is_contiguous()):
            raise RuntimeError("linear_rotary: kv_cache must be a contiguous [pages, 2, page_size, num_kv_heads, head_size] "
                               "tensor of the activation dtype and kv_slots a contiguous int64 [T] tensor")
        page = kv_cache.shape[2]
    rot = N.RotaryArgs(N.ptr(positions), N.ptr(cos_sin_cache), head_size, cos_sin_cache.shape[1], rot_cols,
                       1 if is_neox else 0, N.ptr(kv_cache), N.ptr(kv_slots) if kv_cache is not None else None, page,
                       num_kv_heads)
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), None, None, 0, T, Nn, K, N.dtype_id(x2), EPI_ROTARY,
                                      ctypes.byref(rot), N.ptr(status_word(x2.device)), tile_n, *_ws(x2),
                                      N.stream_ptr()),
            "gemm_colpar[rotary]")
    return out


def linear_silu_mul(x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor] = None,
                    tile_n: int = 0) -> torch.Tensor:
    """act[T, d] = silu(x @ Wgate^T) * (x @ Wup^T) with weight = [Wgate; Wup] ([2d, K]):
    the gate_up_proj + SiluAndMul pair of models/llama.py:101-104 in one kernel."""
    N.require_cuda(x, weight)
    x2 = _rows_2d(x, "linear_silu_mul input")
    T, K = x2.shape
    Nn = weight.shape[0]
    if out is None:
        out = torch.empty(T, Nn // 2, dtype=x2.dtype, device=x2.device)
    N.check(N.lib().sb200_gemm_colpar(N.ptr(out), out.stride(0), N.ptr(x2), x2.stride(0), N.ptr(weight),
                                      weight.stride(0), None, None, 0, T, Nn, K, N.dtype_id(x2), EPI_SILU_MUL, None,
                                      N.ptr(status_word(x2.device)), tile_n, *_ws(x2), N.stream_ptr()),
            "gemm_colpar[silu_mul]")
    return out


def gemm_plan(epilogue: int, T: int, Nn: int, K: int, head_size: int = 128, tile_cfg: int = 0,
              workspace_bytes: int = WORKSPACE_BYTES) -> dict:
    """The tile shape / schedule the library would use for a [T, K] x [Nn, K]^T projection."""
    out = (ctypes.c_int * 12)()
    N.check(N.lib().sb200_gemm_plan(epilogue, T, Nn, K, head_size, tile_cfg, workspace_bytes, out), "gemm_plan")
    keys = ("cta_pairs", "accumulators", "bn", "units", "tiles_full", "k_parts", "rem_units", "stages", "m_tiles",
            "n_tiles", "k_blocks", "cluster_split")
    return dict(zip(keys, out))


# ---------------------------------------------------------------- autotuning
_tuned: dict = {}


def save_tuned(path: str) -> None:
    """Write the tile configurations found so far to a JSON file (see ``load_tuned``)."""
    import json
    rows = [{"kind": k[0], "T": k[1], "N": k[2], "K": k[3], "dtype": str(k[4]).replace("torch.", ""), "cfg": v}
            for k, v in _tuned.items()]
    with open(path, "w") as fh:
        json.dump(rows, fh, indent=1)


def load_tuned(path: str) -> int:
    """Adopt tile configurations saved by ``save_tuned``; ``autotune`` then returns them without timing
    anything.  Returns the number of entries read."""
    import json
    with open(path) as fh:
        rows = json.load(fh)
    for r in rows:
        _tuned[(r["kind"], int(r["T"]), int(r["N"]), int(r["K"]), getattr(torch, r["dtype"]))] = int(r["cfg"])
    return len(rows)


def tuned_cfg(kind: str, T: int, Nn: int, K: int, dtype: torch.dtype) -> int:
    """Tile configuration found by ``autotune`` for this problem, or 0 (library default)."""
    return _tuned.get((kind, T, Nn, K, dtype), 0)


def _candidates(kind: str, T: int, Nn: int, K: int, head_size: int):
    epi = {"store": EPI_NONE, "rotary": EPI_ROTARY, "silu": EPI_SILU_MUL, "push": 3}[kind]
    seen, out = set(), []
    for mode in (1, 3, 4, 5):
        for bn in (64, 96, 128, 160, 192, 224, 256):
            for s in ((2, 4) if mode == 5 else (1, 2, 3, 4, 6, 8)):
                cfg = bn + 1000 * mode + 100000 * s
                try:
                    p = gemm_plan(epi, T, Nn, K, head_size, cfg)
                except RuntimeError:
                    continue
                key = tuple(p.values())
                if key in seen:
                    continue
                seen.add(key)
                # encode what the planner actually accepted, so that the key reproduces the plan
                if p["cluster_split"] > 1:
                    out.append(p["bn"] + 5000 + 100000 * p["cluster_split"])
                    continue
                mode_eff = (2 + p["accumulators"]) if p["cta_pairs"] else p["accumulators"]
                out.append(p["bn"] + 1000 * mode_eff + 100000 * p["k_parts"])
    return sorted(set(out))


def autotune(kind: str, T: int, Nn: int, K: int, dtype: torch.dtype, device: torch.device, head_size: int = 128,
             group=None, launches: int = 6, reps: int = 3) -> int:
    """Time the tile configurations the planner accepts for one projection shape (CUDA-graph
    replay of ``launches`` back-to-back kernels over rotating weight copies) and remember the
    fastest.  ``kind``: "store" | "rotary" | "silu" | "push" (row-parallel: tuned with the plain
    store epilogue, which has the same main loop).  With ``group`` (tensor-parallel ranks) rank 0's
    choice is broadcast so that every rank uses the same schedule."""
    key = (kind, T, Nn, K, dtype)
    if key in _tuned:
        return _tuned[key]
    if dtype == torch.float32:
        _tuned[key] = 0
        return 0
    run_kind = "store" if kind == "push" else kind
    ncopy = max(2, min(8, int(260e6 // (Nn * K * 2)) + 1))
    ws = [torch.randn(Nn, K, device=device, dtype=torch.float32).mul_(0.02).to(dtype) for _ in range(ncopy)]
    x = torch.randn(T, K, device=device, dtype=torch.float32).to(dtype)
    pos = torch.zeros(T, dtype=torch.int64, device=device)
    cache = torch.ones(8, head_size, device=device, dtype=dtype)

    def call(i, cfg):
        if run_kind == "silu":
            return linear_silu_mul(x, ws[i % ncopy], tile_n=cfg)
        if run_kind == "rotary":
            return linear_rotary(x, ws[i % ncopy], pos, cache, head_size, (Nn // head_size // 2) * head_size, True,
                                 tile_n=cfg)
        return linear(x, ws[i % ncopy], tile_n=cfg)

    best, best_us = 0, float("inf")
    stream = torch.cuda.Stream(device=device)
    for cfg in [0] + _candidates(kind, T, Nn, K, head_size):
        try:
            with torch.cuda.stream(stream):
                call(0, cfg)
                torch.cuda.synchronize(device)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(launches):
                        call(i, cfg)
                graph.replay()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                for _ in range(reps):
                    graph.replay()
                e1.record(stream)
                torch.cuda.synchronize(device)
            us = e0.elapsed_time(e1) * 1e3 / (launches * reps)
        except RuntimeError:
            continue
        if us < best_us:
            best, best_us = cfg, us
    if group is not None:
        import torch.distributed as dist
        box = [best]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if hasattr(dist, "get_global_rank") else 0,
                                   group=group)
        best = box[0]
    _tuned[key] = best
    check_status(device)
    return best
