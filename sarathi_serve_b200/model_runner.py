"""Host side of a model step: flattening a Sarathi batch into padded token / position tensors and replaying the
WHOLE layer stack from CUDA graphs captured per padded batch size.

Mirrors the two pieces of the reference's ``ModelRunner`` that sit around the decoder-layer path
(sarathi/model_executor/model_runner.py): ``_prepare_inputs`` (:67-117 -- prefill chunks first, then one token
per decoding request, padded to a multiple of 8) and the model call of ``run`` (:225-256).  The reference
launches every op of every layer from Python each step; once a layer takes tens of microseconds that host
work dominates, so here the stack is captured once per batch-size bucket and a step is: copy the token ids and
positions into the bucket's static buffers, one graph launch, a view of the static output.
Scheduling, sampling and the attention metadata stay with the caller.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import dense_ops
from . import parallel_state as ps


def pad_to_alignment(x: List[int], multiple_of: int) -> List[int]:
    """Zero-pad to a multiple (reference: sarathi/model_executor/utils.py, used at model_runner.py:108-109)."""
    return x + [0] * ((-len(x)) % multiple_of)


def prepare_inputs(prompt_chunks: Sequence[Tuple[Sequence[int], int]], decodes: Sequence[Tuple[int, int]],
                   device, multiple_of: int = 8) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """``prompt_chunks``: (token ids of the chunk, tokens of that prompt processed before it) per prefill request
    of the batch, in batch order; ``decodes``: (last token id, context length) per decoding request.  Returns
    (tokens int64 [n_padded], positions int64 [n_padded], n) laid out as the reference lays them out: all prompt
    chunks, then the decode tokens at position context_len - 1, then zeros up to a multiple of ``multiple_of``."""
    tokens: List[int] = []
    positions: List[int] = []
    for chunk, processed in prompt_chunks:
        tokens.extend(int(t) for t in chunk)
        positions.extend(range(processed, processed + len(chunk)))
    for token, context_len in decodes:
        tokens.append(int(token))
        positions.append(int(context_len) - 1)
    n = len(tokens)
    tokens = pad_to_alignment(tokens, multiple_of)
    positions = pad_to_alignment(positions, multiple_of)
    return (torch.tensor(tokens, dtype=torch.long, device=device),
            torch.tensor(positions, dtype=torch.long, device=device), n)


class ModelGraphRunner:
    """Replays ``model(hidden_states=token_ids, positions=positions, attention_backend_wrapper=...)`` -- the call
    of model_runner.py:239-243 -- from CUDA graphs.

    One graph per bucket of padded batch sizes (``buckets``: ascending multiples of 8; the scheduler's chunk
    size bounds the largest).  A batch is padded with zeros to the smallest bucket that holds it (padding rows
    are computed and discarded, as the reference computes its own padding rows).  Graphs are captured lazily,
    on first use of a bucket; with tensor parallelism every rank sees the same batch sizes in the same order,
    so all ranks capture and replay in step.  The attention wrapper is called inside the captured region: it
    must be capturable for a fixed batch size (static metadata buffers), which the stand-in wrappers of the
    tests are.  ``run`` returns a view of the bucket's static output, valid until that bucket is used again."""

    def __init__(self, model: torch.nn.Module, attention_backend_wrapper, buckets: Sequence[int] = (8, 16, 32, 64, 128,
                 256, 512, 1024, 2048), device: Optional[torch.device] = None, warmup: int = 2):
        self.model = model
        self.attn = attention_backend_wrapper
        self.buckets = sorted(int(b) for b in buckets)
        if any(b % 8 for b in self.buckets):
            raise ValueError("bucket sizes must be multiples of 8 (the reference pads batches to a multiple of 8)")
        self.device = device or next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("ModelGraphRunner: the model must live on a CUDA device")
        self.warmup = max(1, int(warmup))
        self._graphs: Dict[int, dict] = {}
        self.stream = torch.cuda.Stream(device=self.device)

    def bucket_for(self, n: int) -> int:
        for b in self.buckets:
            if n <= b:
                return b
        raise RuntimeError(f"batch of {n} tokens exceeds the largest bucket ({self.buckets[-1]})")

    def _capture(self, size: int) -> dict:
        tokens = torch.zeros(size, dtype=torch.long, device=self.device)
        positions = torch.zeros(size, dtype=torch.long, device=self.device)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.stream), torch.inference_mode():
            for _ in range(self.warmup):
                self.model(hidden_states=tokens, positions=positions, attention_backend_wrapper=self.attn)
            self.stream.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=self.stream):
                out = self.model(hidden_states=tokens, positions=positions, attention_backend_wrapper=self.attn)
                comm = ps._TP_COMM
                if comm is not None:
                    comm.enqueue_status_read()
                dense_ops.enqueue_status_read(self.device)
        torch.cuda.current_stream(self.device).wait_stream(self.stream)
        entry = {"graph": graph, "tokens": tokens, "positions": positions, "out": out, "comm": ps._TP_COMM}
        self._graphs[size] = entry
        return entry

    def run(self, tokens: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """``tokens`` / ``positions``: int64 [n] (device or pinned host), e.g. from ``prepare_inputs``.  Returns
        the model output for those n rows."""
        n = tokens.numel()
        if positions.numel() != n:
            raise RuntimeError("tokens and positions differ in length")
        size = self.bucket_for(n)
        g = self._graphs.get(size) or self._capture(size)
        if g["comm"] is not None:
            g["comm"].raise_if_flagged()   # a bounded device-side wait of an earlier step ran out
        dense_ops.raise_if_flagged(self.device)
        if n < size:
            g["tokens"][n:].zero_()
            g["positions"][n:].zero_()
        g["tokens"][:n].copy_(tokens, non_blocking=True)
        g["positions"][:n].copy_(positions, non_blocking=True)
        g["graph"].replay()
        return g["out"][:n]
