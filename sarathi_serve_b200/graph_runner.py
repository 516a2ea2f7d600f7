"""CUDA-graph replay of a decoder layer for a fixed batch shape.

The kernels of this path take a few microseconds to a few tens of microseconds each, so a step
launched op by op from Python is bound by the host.  ``LayerGraph`` captures one call of a layer
(``layer(positions, hidden_states, layer_cache_idx, attention_backend_wrapper)``, the signature of
the reference's ``LlamaDecoderLayer.forward``, models/llama.py:232-255) into a CUDA graph over
static input / output buffers and replays it: a step then costs two copies into the static buffers
and one graph launch.  The collectives of the tensor-parallel path keep their call counters on the
device, so a captured layer can be replayed on every rank any number of times; every rank of the
group has to build and replay its graph in the same order.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import dense_ops
from . import parallel_state as ps


class LayerGraph:
    """Graph of ``layer.forward`` for ``num_tokens`` tokens.

    ``__call__(positions, hidden_states)`` accepts device or (pinned) host tensors, copies them into
    the graph's static inputs, replays, and returns the static output tensor (overwritten by the
    next call).  Shapes other than the captured one are rejected.

    With ``host_io=True`` the graph also owns pinned host buffers (``host_positions``,
    ``host_hidden_states``, ``host_output``) and the copies between them and the device are nodes of
    the graph: a step is then ONE graph launch -- fill the host inputs, ``replay_host_io()``,
    synchronise, read ``host_output`` -- which matters when several ranks have to stay in step.

    ``shard_host_io=True`` (with ``host_io``, tensor-parallel size > 1): the hidden states cross PCIe once
    per node instead of once per rank.  Rank r's host buffers hold only the token rows
    [r * ceil(T/tp), (r+1) * ceil(T/tp)) -- ``row_range`` -- of the input and of the output; the graph
    uploads those rows, assembles the full [T, H] input on every rank with an all-gather over NVLink
    (``TPComm.all_gather_rows``), runs the layer and downloads this rank's rows of the result.  (The
    reference hands every worker the full batch: model_runner.py:67-117.)

    ``copies_in_graph=False`` (with ``host_io``): the graph holds the layer only; ``upload()`` and ``download()``
    enqueue the host copies on whatever stream is current, so that ``HostPipeline`` can run them on copy
    streams of their own, under the layer of a neighbouring step.  The rows to download are first copied, inside
    the graph, out of the layer's output into a buffer of this graph when the output lives in the communication
    heap (tensor-parallel size > 1), where a later collective would overwrite it.

    ``poll_status`` (default on): every replay also copies the device status words (bounded waits that ran
    out in a collective or in a GEMM pipeline) to pinned host memory, and the NEXT call raises if they were
    set -- errors surface one step late and without a synchronisation, like the asynchronous device errors
    of the reference's ops."""

    def __init__(self, layer: torch.nn.Module, num_tokens: int, attention_backend_wrapper, *, layer_cache_idx: int = 0,
                 dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None, warmup: int = 2,
                 host_io: bool = False, shard_host_io: bool = False, poll_status: bool = True,
                 copies_in_graph: bool = True):
        p = next(layer.parameters())
        self.device = device or p.device
        self.dtype = dtype or p.dtype
        if self.device.type != "cuda":
            raise RuntimeError("LayerGraph: the layer must live on a CUDA device")
        self.layer = layer
        self.num_tokens = int(num_tokens)
        hidden = layer.hidden_size
        self.positions = torch.zeros(self.num_tokens, dtype=torch.int64, device=self.device)
        self.hidden_states = torch.zeros(self.num_tokens, hidden, dtype=self.dtype, device=self.device)
        self.host_io = bool(host_io)
        self.copies_in_graph = bool(copies_in_graph) or not self.host_io
        self.poll_status = bool(poll_status)
        world = ps.get_tensor_model_parallel_world_size()
        self.shard_host_io = bool(shard_host_io) and self.host_io and world > 1
        self.row_range = (0, self.num_tokens)
        if self.shard_host_io:
            rpr = -(-self.num_tokens // world)
            lo = min(self.num_tokens, ps.get_tensor_model_parallel_rank() * rpr)
            self.row_range = (lo, min(self.num_tokens, lo + rpr))
        lo, hi = self.row_range
        if self.host_io:
            self.host_positions = torch.zeros(self.num_tokens, dtype=torch.int64).pin_memory()
            self.host_hidden_states = torch.zeros(hi - lo, hidden, dtype=self.dtype).pin_memory()
            self.host_output = torch.zeros(hi - lo, hidden, dtype=self.dtype).pin_memory()
        if self.shard_host_io:
            self._rows = torch.zeros(hi - lo, hidden, dtype=self.dtype, device=self.device)
            self._comm_io = ps.get_tensor_model_parallel_comm()
        self.in_rows = self._rows if self.shard_host_io else self.hidden_states  # what the host rows are uploaded into
        private_out = self.host_io and not self.copies_in_graph and world > 1
        self.out_rows = torch.zeros(hi - lo, hidden, dtype=self.dtype, device=self.device) if private_out else None
        self.stream = torch.cuda.Stream(device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream), torch.inference_mode():
            for _ in range(max(1, warmup)):  # first calls create the communication context, tile plans, caches
                layer(self.positions, self._gathered() if self.shard_host_io else self.hidden_states,
                      layer_cache_idx, attention_backend_wrapper)
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                if self.host_io and self.copies_in_graph:
                    self.positions.copy_(self.host_positions, non_blocking=True)
                    self.in_rows.copy_(self.host_hidden_states, non_blocking=True)
                hidden = self._gathered() if self.shard_host_io else self.hidden_states
                self.output = layer(self.positions, hidden, layer_cache_idx, attention_backend_wrapper)
                if self.host_io and self.copies_in_graph:
                    self.host_output.copy_(self.output[lo:hi], non_blocking=True)
                elif private_out:
                    self.out_rows.copy_(self.output[lo:hi])
                # the device status words (bounded waits that ran out) travel to pinned host memory with every
                # replay; the NEXT call looks at them before it launches, without a synchronisation
                self._comm = ps._TP_COMM if poll_status else None
                if self._comm is not None:
                    self._comm.enqueue_status_read()
                if poll_status:
                    dense_ops.enqueue_status_read(self.device)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        if self.host_io and self.out_rows is None:
            self.out_rows = self.output[lo:hi]

    def upload(self) -> None:
        """Enqueue the copies host inputs -> static device inputs on the current stream."""
        self.positions.copy_(self.host_positions, non_blocking=True)
        self.in_rows.copy_(self.host_hidden_states, non_blocking=True)

    def download(self) -> None:
        """Enqueue the copy of this rank's output rows -> ``host_output`` on the current stream."""
        self.host_output.copy_(self.out_rows, non_blocking=True)

    def _gathered(self) -> torch.Tensor:
        """Full [T, H] hidden states assembled from every rank's rows (a view into the communication heap)."""
        return self._comm_io.all_gather_rows(self._rows, self.num_tokens)

    def _raise_if_an_earlier_step_failed(self) -> None:
        if not self.poll_status:
            return
        if self._comm is not None:
            self._comm.raise_if_flagged()
        dense_ops.raise_if_flagged(self.device)

    def replay_host_io(self) -> torch.Tensor:
        """One launch: host inputs -> device, the layer, output -> ``host_output`` (valid after the
        current stream has been synchronised)."""
        if not self.host_io:
            raise RuntimeError("LayerGraph: built without host_io=True")
        self._raise_if_an_earlier_step_failed()
        if self.copies_in_graph:
            self.graph.replay()
        else:
            self.upload()
            self.graph.replay()
            self.download()
        return self.host_output

    def __call__(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        if self.host_io:
            raise RuntimeError("LayerGraph: built with host_io=True -- fill host_positions / host_hidden_states and "
                               "call replay_host_io()")
        if hidden_states.shape != self.hidden_states.shape or positions.shape != self.positions.shape:
            raise RuntimeError(f"LayerGraph: captured for {tuple(self.hidden_states.shape)} hidden states, "
                               f"got {tuple(hidden_states.shape)}")
        self._raise_if_an_earlier_step_failed()
        self.positions.copy_(positions, non_blocking=True)
        self.hidden_states.copy_(hidden_states, non_blocking=True)
        self.graph.replay()
        return self.output


class HostPipeline:
    """Steps fed from host buffers with the copies of neighbouring steps under the layer of the current one.

    ``slots``: two or more ``LayerGraph``s built with ``host_io=True, copies_in_graph=False`` (of one layer, or of
    consecutive layers -- each has its own static buffers).  ``submit()`` takes the next slot in turn and enqueues
    its upload on one copy stream, its graph on the compute stream and its download on a second copy stream,
    chained by events; ``collect()`` waits for the oldest outstanding step's download and returns that slot's
    ``host_output``.  With three steps in flight the upload of step i+1 and the download of step i-1 run while the
    kernels of step i do, so a step costs max(layer, upload, download) instead of their sum; every step's input
    still crosses PCIe and every result is read by the host.  All kernels stay on ONE stream (the collectives of
    a communication context must not overlap one another), and every rank of a tensor-parallel group has to
    submit in the same order.  A slot's host buffers may be refilled once its step has been collected."""

    def __init__(self, slots):
        slots = list(slots)
        if len(slots) < 2:
            raise RuntimeError("HostPipeline: needs at least two slots")
        for g in slots:
            if not g.host_io or g.copies_in_graph:
                raise RuntimeError("HostPipeline: build the LayerGraphs with host_io=True, copies_in_graph=False")
        self.slots = slots
        dev = slots[0].device
        self.device = dev
        self.compute = torch.cuda.Stream(device=dev)
        self.up = torch.cuda.Stream(device=dev)
        self.down = torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream(dev)
        for st in (self.compute, self.up, self.down):
            st.wait_stream(cur)
        n = len(slots)
        self._uploaded = [torch.cuda.Event() for _ in range(n)]
        self._computed = [torch.cuda.Event() for _ in range(n)]
        self._downloaded = [torch.cuda.Event() for _ in range(n)]
        self.submitted = 0
        self.collected = 0

    @property
    def in_flight(self) -> int:
        return self.submitted - self.collected

    def next_slot(self) -> "LayerGraph":
        """The slot the next ``submit()`` uses (fill its ``host_positions`` / ``host_hidden_states`` first)."""
        return self.slots[self.submitted % len(self.slots)]

    def submit(self) -> None:
        if self.in_flight >= len(self.slots):
            raise RuntimeError("HostPipeline: every slot is in flight -- collect() a result first")
        s = self.submitted % len(self.slots)
        g = self.slots[s]
        g._raise_if_an_earlier_step_failed()
        with torch.cuda.stream(self.up):
            g.upload()
            self._uploaded[s].record(self.up)
        with torch.cuda.stream(self.compute):
            self.compute.wait_event(self._uploaded[s])
            g.graph.replay()
            self._computed[s].record(self.compute)
        with torch.cuda.stream(self.down):
            self.down.wait_event(self._computed[s])
            g.download()
            self._downloaded[s].record(self.down)
        self.submitted += 1

    def collect(self) -> torch.Tensor:
        if self.collected == self.submitted:
            raise RuntimeError("HostPipeline: nothing in flight")
        s = self.collected % len(self.slots)
        self._downloaded[s].synchronize()
        self.collected += 1
        return self.slots[s].host_output

    def drain(self) -> None:
        while self.collected < self.submitted:
            self.collect()
