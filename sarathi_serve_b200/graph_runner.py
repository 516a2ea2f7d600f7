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


class LayerGraph:
    """Graph of ``layer.forward`` for ``num_tokens`` tokens.

    ``__call__(positions, hidden_states)`` accepts device or (pinned) host tensors, copies them into
    the graph's static inputs, replays, and returns the static output tensor (overwritten by the
    next call).  Shapes other than the captured one are rejected."""

    def __init__(self, layer: torch.nn.Module, num_tokens: int, attention_backend_wrapper, *, layer_cache_idx: int = 0,
                 dtype: Optional[torch.dtype] = None, device: Optional[torch.device] = None, warmup: int = 2):
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
        self.stream = torch.cuda.Stream(device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream), torch.inference_mode():
            for _ in range(max(1, warmup)):  # first calls create the communication context, tile plans, caches
                layer(self.positions, self.hidden_states, layer_cache_idx, attention_backend_wrapper)
            self.stream.synchronize()
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, stream=self.stream):
                self.output = layer(self.positions, self.hidden_states, layer_cache_idx, attention_backend_wrapper)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)

    def __call__(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        if hidden_states.shape != self.hidden_states.shape or positions.shape != self.positions.shape:
            raise RuntimeError(f"LayerGraph: captured for {tuple(self.hidden_states.shape)} hidden states, "
                               f"got {tuple(hidden_states.shape)}")
        self.positions.copy_(positions, non_blocking=True)
        self.hidden_states.copy_(hidden_states, non_blocking=True)
        self.graph.replay()
        return self.output
