"""Pipelined inference over a stream of host batches.

``Latticeformer.forward`` on one batch is a chain host -> device copy, ~40 kernel launches, device -> host copy; run
batch after batch with a synchronisation in between, the GPU idles while the host issues the next batch's launches
and the host idles while the GPU computes.  ``PipelinedPredictor`` keeps ``depth`` batches in flight instead: the
inputs of batch t+1 are copied on a second stream while batch t computes, results land in a ring of pinned host
buffers, and the caller only waits when it asks for a result (or when the ring is full).

    runner = PipelinedPredictor(model, depth=3)
    tickets = [runner.submit(batch) for batch in host_batches]      # batch: x, pos, trans_vec, sizes on the host
    outputs = [runner.result(t) for t in tickets]                   # (num_crystals, n_targets) host tensors

Host batches should be pinned (``tensor.pin_memory()``) for the copies to be asynchronous.  Results must be collected
in submission order.  The model must be in eval mode with its ``gauss_scale`` buffers set (a trained model, or one
calibrating training-mode forward); outputs are identical to ``model(batch)``.
"""
from __future__ import annotations

import types
from collections import deque
from typing import Deque, Optional, Tuple

import torch


class PipelinedPredictor:
    def __init__(self, model: torch.nn.Module, depth: int = 3, device: Optional[torch.device] = None, post=None,
                 gather=None):
        """``post``: optional callable applied to the model output on the device before it is copied to the host
        (e.g. an all-gather of the ranks' outputs).  ``gather``: a ``sharding.PeerGather`` handed to the model, which
        then returns the outputs of every rank's crystals."""
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.model = model
        self.device = device if device is not None else next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("PipelinedPredictor needs a CUDA model: crystalformer_b200 has no CPU path")
        self.depth = depth
        self.post = post
        self.gather = gather
        self.copy_stream = torch.cuda.Stream(self.device)
        self._inflight: Deque[Tuple[int, torch.cuda.Event, torch.Tensor, int]] = deque()
        self._out_ring = [None] * depth
        self._next = 0

    def submit(self, batch) -> int:
        """Queues one host batch (attributes x (N,98), pos (N,3), trans_vec (B,3,3), sizes (B) int64); returns a ticket."""
        if len(self._inflight) >= self.depth:
            raise RuntimeError("the pipeline is full: collect a result before submitting more")
        sizes_host = batch.sizes
        counts = sizes_host.tolist()  # host memory: no device synchronisation
        n_atoms, n_edges, max_atoms = sum(counts), sum(n * n for n in counts), max(counts) if counts else 1
        compute = torch.cuda.current_stream(self.device)
        with torch.cuda.stream(self.copy_stream):
            dev = types.SimpleNamespace(
                x=batch.x.to(self.device, non_blocking=True), pos=batch.pos.to(self.device, non_blocking=True),
                trans_vec=batch.trans_vec.to(self.device, non_blocking=True),
                sizes=sizes_host.to(self.device, non_blocking=True))
            copied = torch.cuda.Event()
            copied.record(self.copy_stream)
        compute.wait_event(copied)
        for t in vars(dev).values():
            t.record_stream(compute)  # allocated on the copy stream, consumed on the compute stream
        with torch.no_grad():
            extra = {} if self.gather is None else {"gather": self.gather}
            y = self.model(dev, counts=(n_atoms, n_edges, max_atoms), **extra)
            if self.post is not None:
                y = self.post(y)
        slot = self._next % self.depth
        out = self._out_ring[slot]
        if out is None or out.shape != y.shape:
            out = self._out_ring[slot] = torch.empty(y.shape, dtype=y.dtype).pin_memory()
        out.copy_(y, non_blocking=True)
        done = torch.cuda.Event()
        done.record(compute)
        ticket = self._next
        self._inflight.append((ticket, done, out, len(counts)))
        self._next += 1
        return ticket

    def result(self, ticket: int) -> torch.Tensor:
        """Waits for the oldest batch in flight (``ticket`` must be its ticket) and returns its output on the host.
        The returned tensor is a view of a ring buffer that is reused ``depth`` submissions later: copy it to keep it."""
        if not self._inflight or self._inflight[0][0] != ticket:
            raise RuntimeError("results must be collected in submission order")
        _, done, out, _ = self._inflight.popleft()
        done.synchronize()
        return out

    def pending(self) -> int:
        return len(self._inflight)
