"""Tensor-parallel communication context: symmetric device heaps mapped between
the ranks of one node, and the collectives built on them (all-reduce and the
row-parallel projection fused with its all-reduce, residual add and RMSNorm).

torch.distributed is used only as plumbing: the heaps come from torch's
symmetric-memory allocator when the node's NVSwitch offers multicast (each rank's
buffer is mapped into every peer AND all of them are bound to one multicast
address range, which the kernels use for in-switch reduction and broadcast), or
from cudaMalloc with the 64-byte CUDA IPC handles exchanged once at
construction; either way a host barrier follows.  The data path is this
library's own kernels over NVLink; NCCL is not called on it.

The multicast heaps are the default; ``SB200_NVLS=0`` in the environment (or
``multicast=False``) keeps the heaps on plain peer mappings (so does a node
without NVSwitch multicast, or a start-up self-test of the multicast path that
fails on any rank).  Every rank of a group has to make the same choice."""
from __future__ import annotations

import ctypes
import os
from typing import Optional, Tuple

import torch

from . import _native as N

_STATUS_TEXT = {1: "GEMM pipeline barrier", 2: "partial rows from a peer never arrived",
                3: "finished rows from a peer never arrived"}


class _DeviceMemory:
    """Exposes a raw device range through __cuda_array_interface__ so torch can view it."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False),
                                         "version": 3, "strides": None}


class TPComm:
    """One per (process, GPU, tensor-parallel group).

    ``region_bytes`` bounds the largest [T, H] batch a collective may carry
    (T rounded up to a multiple of the group size)."""

    def __init__(self, rank: int, world: int, region_bytes: int, group=None, device: Optional[torch.device] = None,
                 multicast: Optional[bool] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("TPComm needs a CUDA device (there is no CPU fallback)")
        self.rank, self.world, self.group = rank, world, group
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self._h = ctypes.c_void_p()
        self._symm = None       # (tensor, handle) of the symmetric-memory allocation, when the heaps come from there
        self._poisoned = False
        self._status_host = None
        self.multicast = False
        lib = N.lib()
        if multicast is None:
            multicast = os.environ.get("SB200_NVLS", "1") != "0"
        with torch.cuda.device(self.device):
            if world > 1 and multicast and self._create_on_symmetric_memory(lib, int(region_bytes)):
                pass
            else:
                N.check(lib.sb200_comm_create(ctypes.byref(self._h), rank, world, int(region_bytes)), "comm_create")
                if world > 1:
                    import torch.distributed as dist
                    mine = (ctypes.c_ubyte * 64)()
                    N.check(lib.sb200_comm_ipc_handle(self._h, mine), "comm_ipc_handle")
                    handles = [None] * world
                    dist.all_gather_object(handles, bytes(mine), group=group)
                    blob = b"".join(handles)
                    N.check(lib.sb200_comm_open_peers(self._h, blob), "comm_open_peers")
                    dist.barrier(group=group)
        self.region_bytes = int(lib.sb200_comm_region_bytes(self._h))
        heap_ptr = lib.sb200_comm_local_heap(self._h)
        heap_bytes = int(lib.sb200_comm_heap_bytes(self.region_bytes))
        self._heap = torch.as_tensor(_DeviceMemory(heap_ptr, heap_bytes), device=self.device)
        self._heap_ptr = heap_ptr
        if self.multicast:
            with torch.cuda.device(self.device):
                self._self_test_multicast()

    def _self_test_multicast(self) -> None:
        """One small all-reduce through the switch against the same all-reduce over peer loads, once, at
        construction.  If any rank sees a difference or a wait that ran out, every rank drops the multicast
        alias (the heaps stay, the collectives use peer loads) -- a box whose NVSwitch multicast does not behave
        costs speed, not results."""
        import torch.distributed as dist
        lib = N.lib()
        T, H = 4 * self.world + 3, 512
        x = ((torch.arange(T * H, device=self.device, dtype=torch.float32).view(T, H) % 61) * 0.125
             - 3.0 + 0.25 * self.rank).to(torch.bfloat16)
        default_wait = int(os.environ.get("SB200_WAIT_LIMIT_CYCLES", "0")) or 20_000_000_000
        default_one_shot = int(os.environ.get("SB200_ONE_SHOT_BYTES", str(4 << 20)))
        mc_ptr = ctypes.c_void_p(self._mc_ptr)
        ok = 1
        try:
            self.set_wait_limit_cycles(3_000_000_000)   # about a second and a half
            self.set_one_shot_bytes(0)                  # the owner-reduce schemes, whatever the size
            y_mc = self.all_reduce(x)[0].float().clone()
            N.check(lib.sb200_comm_set_multicast(self._h, None), "comm_set_multicast")
            y_pl = self.all_reduce(x)[0].float().clone()
            N.check(lib.sb200_comm_set_multicast(self._h, mc_ptr), "comm_set_multicast")
            torch.cuda.synchronize(self.device)
            if self.status_code() != 0 or float((y_mc - y_pl).abs().max()) > 0.26:  # sums up to ~40: 2 units in the last place
                ok = 0
        except RuntimeError:
            ok = 0
        verdict = [None] * self.world
        dist.all_gather_object(verdict, ok, group=self.group)
        self.set_wait_limit_cycles(default_wait)
        self.set_one_shot_bytes(default_one_shot)
        if not all(verdict):
            N.check(lib.sb200_comm_set_multicast(self._h, None), "comm_set_multicast")
            self.multicast = False
            self._poisoned = False
            self.reset()

    def _create_on_symmetric_memory(self, lib, region_bytes: int) -> bool:
        """Heaps from torch's symmetric-memory allocator, bound to an NVSwitch multicast range.  Every rank
        reaches the same verdict (the outcome is agreed over the group), so either all ranks use these heaps
        or none does.  Returns False when the allocator, the rendezvous or multicast is not available."""
        import torch.distributed as dist
        heap_bytes = int(lib.sb200_comm_heap_bytes(region_bytes))
        tensor = handle = None
        ok = 0
        try:
            import torch.distributed._symmetric_memory as symm_mem
            grp = self.group if self.group is not None else dist.group.WORLD
            tensor = symm_mem.empty(heap_bytes, dtype=torch.uint8, device=self.device)
            handle = symm_mem.rendezvous(tensor, grp)
            off = int(getattr(handle, "offset", 0))  # of the tensor inside the allocator's block
            ptrs = [int(p) + off for p in handle.buffer_ptrs]
            mc_ptr = int(handle.multicast_ptr) + off if int(handle.multicast_ptr) else 0
            ok = 1 if (mc_ptr != 0 and len(ptrs) == self.world and handle.rank == self.rank
                       and ptrs[self.rank] == tensor.data_ptr()) else 0
        except Exception:  # allocator / rendezvous unavailable: plain peer mappings serve
            ok = 0
        verdict = [None] * self.world
        dist.all_gather_object(verdict, ok, group=self.group)
        if not all(verdict):
            return False
        tensor.zero_()
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)  # every heap is zeroed before anybody's kernels touch it
        table = (ctypes.c_void_p * self.world)(*ptrs)
        N.check(lib.sb200_comm_create_external(ctypes.byref(self._h), self.rank, self.world, region_bytes, table),
                "comm_create_external")
        N.check(lib.sb200_comm_set_multicast(self._h, ctypes.c_void_p(mc_ptr)), "comm_set_multicast")
        self._symm = (tensor, handle)
        self._mc_ptr = mc_ptr
        self.multicast = True
        return True

    # ------------------------------------------------------------------ utils
    def close(self) -> None:
        if self._h:
            torch.cuda.synchronize(self.device)
            N.lib().sb200_comm_destroy(self._h)
            self._h = ctypes.c_void_p()
            self._heap = None
            self._symm = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_wait_limit_cycles(self, cycles: int) -> None:
        N.check(N.lib().sb200_comm_set_wait_limit(self._h, int(cycles)), "comm_set_wait_limit")

    def set_one_shot_bytes(self, nbytes: int) -> None:
        """Collectives with (world - 1) * T * H * itemsize <= nbytes run one-shot (every rank loads all
        partial rows and finishes all rows itself); larger ones reduce rows at their owners and gather
        them.  Every rank must set the same value."""
        N.check(N.lib().sb200_comm_set_one_shot_bytes(self._h, int(nbytes)), "comm_set_one_shot_bytes")

    def check_status(self) -> None:
        """Synchronises the current stream; raises if a device-side wait ran out.  After that the ranks'
        device-side call counters are out of step: every later collective on this context raises until all
        ranks have called ``reset()``."""
        st = ctypes.c_uint32(0)
        rc = N.lib().sb200_comm_status(self._h, N.stream_ptr(), ctypes.byref(st))
        if rc != 0:
            self._poisoned = True
            N.lib().sb200_comm_clear_status(self._h, N.stream_ptr())
            N.check(rc, "tensor-parallel collective")

    def enqueue_status_read(self) -> None:
        """Asynchronous copy of the device status word into pinned host memory on the current stream (it can be
        captured into a CUDA graph); ``raise_if_flagged`` looks at the last value that arrived."""
        if self._status_host is None:
            self._status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._status_host.copy_(self._heap[0:4].view(torch.int32), non_blocking=True)

    def raise_if_flagged(self) -> None:
        """No synchronisation: raises if the last status word read by ``enqueue_status_read`` was non-zero, i.e.
        a device-side wait of an EARLIER step ran out (errors surface at the next launch, like the
        asynchronous device errors of the reference's ops)."""
        if self._status_host is None:
            return
        code = int(self._status_host[0])
        if code != 0:
            self._poisoned = True
            raise RuntimeError(f"tensor-parallel collective: device-side wait timed out in an earlier step "
                               f"(code {code}: {_STATUS_TEXT.get(code, 'unknown')}); call reset() on every rank")

    def reset(self) -> None:
        """Collective over the group: host barrier, control words back to their initial state, host barrier.
        The way back after ``check_status`` raised on any rank."""
        torch.cuda.synchronize(self.device)
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
        N.check(N.lib().sb200_comm_reset(self._h, N.stream_ptr()), "comm_reset")
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier(group=self.group)
        if self._status_host is not None:
            self._status_host.zero_()
        self._poisoned = False

    def _usable(self) -> None:
        if self._poisoned:
            raise RuntimeError("this tensor-parallel context saw a device-side timeout: its ranks are out of step "
                               "until every rank calls reset()")

    def status_code(self) -> int:
        st = ctypes.c_uint32(0)
        N.lib().sb200_comm_status(self._h, N.stream_ptr(), ctypes.byref(st))
        return int(st.value)

    def clear_status(self) -> None:
        N.check(N.lib().sb200_comm_clear_status(self._h, N.stream_ptr()), "comm_clear_status")

    def _view(self, ptr: Optional[int], T: int, H: int, dtype: torch.dtype) -> Optional[torch.Tensor]:
        if not ptr:
            return None
        off = ptr - self._heap_ptr
        nbytes = T * H * torch.empty((), dtype=dtype).element_size()
        return self._heap[off:off + nbytes].view(dtype).view(T, H)

    # ------------------------------------------------------------ collectives
    def _tail_args(self, T, H, x_dtype, bias, residual, norm_weight, out, resid_out):
        for name, t in (("bias", bias), ("norm_weight", norm_weight)):
            if t is not None and (t.dtype != x_dtype or t.numel() != H or not t.is_contiguous()):
                raise RuntimeError(f"{name} must be a contiguous [{H}] tensor of the activation dtype")
        for name, t in (("residual", residual), ("out", out), ("resid_out", resid_out)):
            if t is not None and (t.dtype != x_dtype or tuple(t.shape) != (T, H) or not t.is_contiguous()):
                raise RuntimeError(f"{name} must be a contiguous [{T}, {H}] tensor of the activation dtype")

    def all_reduce(self, x: torch.Tensor, *, bias=None, residual=None, norm_weight=None, eps: float = 0.0,
                   resid_everywhere: bool = True, out=None, resid_out=None) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """Sum x [T, H] over the group, then (+bias) (+residual) and an optional RMSNorm.

        Returns (y, z): y = the primary result on every rank, z = the pre-norm sum
        (only when norm_weight is given).  Without ``out`` / ``resid_out`` the results
        are views into the context's heap, valid until the second-next collective."""
        self._usable()
        N.require_cuda(x, bias, residual, norm_weight, out, resid_out)
        if x.dim() != 2 or not x.is_contiguous():
            raise RuntimeError("all_reduce: input must be a contiguous [T, H] tensor")
        T, H = x.shape
        if T == 0:
            return (x if out is None else out), None
        self._tail_args(T, H, x.dtype, bias, residual, norm_weight, out, resid_out)
        op, rp = ctypes.c_void_p(), ctypes.c_void_p()
        N.check(N.lib().sb200_all_reduce(self._h, N.ptr(x), T, H, N.dtype_id(x), N.ptr(bias), N.ptr(residual),
                                         N.ptr(norm_weight), float(eps), 1 if resid_everywhere else 0, N.ptr(out),
                                         N.ptr(resid_out), N.stream_ptr(), ctypes.byref(op), ctypes.byref(rp)),
                "all_reduce")
        y = out if out is not None else self._view(op.value, T, H, x.dtype)
        z = resid_out if resid_out is not None else self._view(rp.value, T, H, x.dtype)
        return y, (z if norm_weight is not None else None)

    def all_gather_rows(self, rows: torch.Tensor, T: int, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``rows``: this rank's block of a [T, H] tensor -- rows [rank * ceil(T / world), ...), possibly none.
        Returns the full [T, H] tensor (``out``, or a view into the context's heap valid until the
        second-next collective) on every rank."""
        self._usable()
        N.require_cuda(rows, out)
        if rows.dim() != 2 or not rows.is_contiguous():
            raise RuntimeError("all_gather_rows: rows must be a contiguous [n, H] tensor")
        H = rows.shape[1]
        rpr = -(-T // self.world)
        own = max(0, min(rpr, T - self.rank * rpr))
        if rows.shape[0] != own:
            raise RuntimeError(f"all_gather_rows: rank {self.rank} of {self.world} holds {own} of {T} rows, got {rows.shape[0]}")
        if out is not None and (out.dtype != rows.dtype or tuple(out.shape) != (T, H) or not out.is_contiguous()):
            raise RuntimeError(f"out must be a contiguous [{T}, {H}] tensor of the rows' dtype")
        op = ctypes.c_void_p()
        N.check(N.lib().sb200_all_gather_rows(self._h, N.ptr(rows) if own else None, T, H, N.dtype_id(rows), N.ptr(out),
                                              N.stream_ptr(), ctypes.byref(op)), "all_gather_rows")
        return out if out is not None else self._view(op.value, T, H, rows.dtype)

    def rowpar_linear(self, x: torch.Tensor, weight: torch.Tensor, *, bias=None, residual=None, norm_weight=None,
                      eps: float = 0.0, resid_everywhere: bool = True, out=None, resid_out=None,
                      tile_n: int = 0) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """(x[T, K/tp] @ weight[N, K/tp]^T) summed over the group, with the same tail
        and result conventions as ``all_reduce`` -- one kernel for bf16/fp16."""
        self._usable()
        N.require_cuda(x, weight, bias, residual, norm_weight, out, resid_out)
        if x.dim() != 2 or x.stride(1) != 1 or weight.dim() != 2 or weight.stride(1) != 1:
            raise RuntimeError("rowpar_linear: x and weight must be 2-D with unit inner stride")
        if weight.shape[1] != x.shape[1] or weight.dtype != x.dtype:
            raise RuntimeError("rowpar_linear: weight does not match the input")
        T, K = x.shape
        H = weight.shape[0]
        if T == 0:
            return torch.empty(0, H, dtype=x.dtype, device=x.device), None
        self._tail_args(T, H, x.dtype, bias, residual, norm_weight, out, resid_out)
        op, rp = ctypes.c_void_p(), ctypes.c_void_p()
        N.check(N.lib().sb200_gemm_rowpar(self._h, N.ptr(x), x.stride(0), N.ptr(weight), weight.stride(0), T, H, K,
                                          N.dtype_id(x), N.ptr(bias), N.ptr(residual), N.ptr(norm_weight),
                                          float(eps), 1 if resid_everywhere else 0, N.ptr(out), N.ptr(resid_out),
                                          tile_n, N.stream_ptr(), ctypes.byref(op), ctypes.byref(rp)),
                "gemm_rowpar")
        y = out if out is not None else self._view(op.value, T, H, x.dtype)
        z = resid_out if resid_out is not None else self._view(rp.value, T, H, x.dtype)
        return y, (z if norm_weight is not None else None)
