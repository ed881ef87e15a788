"""Pipelined inference over a stream of host batches.

``Latticeformer.forward`` on one batch is a chain host -> device copy, a dozen kernel launches, device -> host copy; run
batch after batch with a synchronisation in between, the GPU idles while the host issues the next batch's launches
and the host idles while the GPU computes.  ``PipelinedPredictor`` keeps ``depth`` batches in flight instead: the
inputs of batch t+1 are copied on a second stream while batch t computes, its preparation (geometry, term lists)
starts as soon as the copy is done, results land in a ring of pinned host buffers, and the caller only waits when it
asks for a result (or when the ring is full).

    runner = PipelinedPredictor(model, depth=3)
    tickets = [runner.submit(batch) for batch in host_batches]      # batch: x, pos, trans_vec, sizes on the host
    outputs = [runner.result(t) for t in tickets]                   # (num_crystals, n_targets) host tensors

Host batches should be pinned (``tensor.pin_memory()``) for the copies to be asynchronous.  Results must be collected
in submission order.  The model must be in eval mode with its ``gauss_scale`` buffers set (a trained model, or one
calibrating training-mode forward); outputs are identical to ``model(batch)``.  The model's weights are read when the
predictor is built (and again after ``refresh()``): change them, then call ``refresh()``.
"""
from __future__ import annotations

import ctypes
import types
from collections import deque
from typing import Deque, Optional, Tuple

import numpy as np
import torch

from . import _lib


class PipelinedPredictor:
    def __init__(self, model: torch.nn.Module, depth: int = 3, device: Optional[torch.device] = None, post=None,
                 gather=None, streams: int = 1, dense_tile_rows: Optional[int] = None):
        """``post``: optional callable applied to the model output on the device before it is copied to the host
        (e.g. an all-gather of the ranks' outputs).  ``gather``: a ``sharding.PeerGather`` handed to the model, which
        then returns the outputs of every rank's crystals.  ``streams``: compute streams the batches alternate between
        (1 = the stream current at ``submit``).  With two, the kernels of consecutive, independent batches run side by
        side and fill each other's idle issue slots (they are latency-bound), at the price of a longer latency per
        batch; with a ``gather`` only if it overlaps its collects (its steps must otherwise run in one order on every
        rank's one stream).  ``dense_tile_rows`` (16, 32 or 0 = chosen per launch; default 32 with several streams, else
        0): the row tile of the fused dense blocks when batches are submitted through the library's one-call path:
        32-row tiles take a little longer per forward and less SM time in total, which pays once streams overlap."""
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.model = model
        self.device = device if device is not None else next(model.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("PipelinedPredictor needs a CUDA model: crystalformer_b200 has no CPU path")
        self.depth = depth
        self.dense_tile_rows = (32 if streams > 1 else 0) if dense_tile_rows is None else int(dense_tile_rows)
        self.post = post
        self.gather = gather
        if streams < 1 or (streams > 1 and gather is not None and not getattr(gather, "overlap", False)):
            raise ValueError("streams must be at least 1, and 1 with a peer gather that does not overlap its collects")
        self.copy_stream = torch.cuda.Stream(self.device)
        self.compute_streams = [torch.cuda.Stream(self.device) for _ in range(streams)] if streams > 1 else None
        self._inflight: Deque[Tuple[int, torch.cuda.Event, torch.Tensor, Optional[torch.Tensor]]] = deque()
        # per slot of the ring: device input buffers, an event "the forward that read them has run", the pinned output
        # buffer and (with a peer gather) a pinned copy of the gather's status word
        self._in_ring = [None] * depth
        self._in_free = [None] * depth
        self._copied = [torch.cuda.Event() for _ in range(depth)]
        self._done = [torch.cuda.Event() for _ in range(depth)]
        self._out_ring = [None] * depth
        self._status_ring = [None] * depth
        self._native = [None] * depth  # per slot: the buffers, events and cf_serve_slot of the one-call submit
        self._next = 0
        self._plan = None
        self.refresh()

    def refresh(self) -> None:
        """Re-reads the model's weights (call after changing them)."""
        native = getattr(self.model, "_native_ok", None)
        self._plan = self.model.native_plan(self.device) if (native is not None and not self.model.training
                                                             and native_ok_without_grad(self.model)) else None
        if self._plan is not None and "desc" in self._plan:
            self._plan["desc"].dense_tile_rows = self.dense_tile_rows

    def _device_inputs(self, slot: int, batch):
        """Device tensors of the slot with the batch's shapes (allocated once per shape, not per batch)."""
        bufs = self._in_ring[slot]
        shapes = (tuple(batch.x.shape), tuple(batch.pos.shape), tuple(batch.trans_vec.shape), tuple(batch.sizes.shape))
        if bufs is None or bufs[0] != shapes:
            dev = self.device
            ns = types.SimpleNamespace(
                x=torch.empty(shapes[0], dtype=batch.x.dtype, device=dev), pos=torch.empty(shapes[1], dtype=batch.pos.dtype, device=dev),
                trans_vec=torch.empty(shapes[2], dtype=batch.trans_vec.dtype, device=dev),
                sizes=torch.empty(shapes[3], dtype=torch.int64, device=dev))
            bufs = self._in_ring[slot] = (shapes, ns)
        return bufs[1]

    def _native_slot(self, slot: int, n_atoms: int, n_crystals: int, n_edges: int, compute):
        """The slot's state for ``cf_serve_submit``: device inputs, workspace and outputs sized for the largest batch seen
        (with a quarter of headroom, so that batches of similar size do not reallocate), a pinned host output, the three
        events, and the C structure that names them."""
        st = self._native[slot]
        if st is not None and n_atoms <= st["c"].max_atoms_total and n_crystals <= st["c"].max_crystals \
                and n_edges <= st["c"].max_edges:
            st["c"].compute_stream = compute.cuda_stream
            return st
        plan, dev = self._plan, self.device
        grow = lambda have, need: max(need + need // 4, have)
        old = st["c"] if st is not None else None
        N = grow(old.max_atoms_total if old else 0, n_atoms)
        B = grow(old.max_crystals if old else 0, n_crystals)
        E = grow(old.max_edges if old else 0, n_edges)
        nbytes = int(_lib.load().cf_model_workspace_bytes(N, B, E, plan["w"]["ff"]))
        t = dict(x=torch.empty((N, plan["emb"].shape[1]), dtype=torch.float32, device=dev),
                 species=torch.empty(N, dtype=torch.int64, device=dev),
                 pos=torch.empty((N, 3), dtype=torch.float32, device=dev), trans=torch.empty((B, 3, 3), dtype=torch.float32, device=dev),
                 sizes=torch.empty(B, dtype=torch.int64, device=dev), work=torch.empty(nbytes, dtype=torch.uint8, device=dev),
                 y=torch.empty((B, plan["targets"]), dtype=torch.float32, device=dev),
                 y_host=torch.empty((B, plan["targets"]), dtype=torch.float32).pin_memory())
        events = [torch.cuda.Event() for _ in range(3)]
        for e in events:
            e.record(compute)  # an event has a handle once it has been recorded
        c = _lib.ServeSlot(copy_stream=self.copy_stream.cuda_stream, compute_stream=compute.cuda_stream,
                           copied=events[0].cuda_event, inputs_free=events[1].cuda_event, done=events[2].cuda_event,
                           x=t["x"].data_ptr(), pos=t["pos"].data_ptr(), trans=t["trans"].data_ptr(), sizes=t["sizes"].data_ptr(),
                           workspace=t["work"].data_ptr(), y=t["y"].data_ptr(), y_host=t["y_host"].data_ptr(),
                           max_atoms_total=N, max_crystals=B, max_edges=E, species=t["species"].data_ptr())
        if self.gather is not None:
            g = self.gather
            t["y_all"] = torch.empty((g.total_rows, g.targets), dtype=torch.float32, device=dev)
            t["y_all_host"] = torch.empty((g.total_rows, g.targets), dtype=torch.float32).pin_memory()
            t["status_host"] = torch.zeros(1, dtype=torch.int32).pin_memory()
            stored = torch.cuda.Event()
            stored.record(compute)
            events.append(stored)
        st = self._native[slot] = dict(c=c, tensors=t, events=events, used=False)
        return st

    def _native_applies(self, batch) -> bool:
        """One C call per batch (``cf_serve_submit``) when the model runs its one-call forward with the embedding folded
        into the first block, nothing but a peer gather is applied to the outputs on the device, and the inputs are
        host tensors of the types the kernels read."""
        plan = self._plan
        if plan is None or "desc" not in plan or self.post is not None:
            return False
        if getattr(self.model.encoder, "attention_event_log", None) is not None:
            return False  # (per-layer timing events are handed over by the framework-level path)
        ok = lambda t, dt: t.device.type == "cpu" and t.dtype == dt and t.is_contiguous()
        if getattr(batch, "x", None) is not None:
            species_ok = ok(batch.x, torch.float32) and batch.x.shape[1] == plan["emb"].shape[1]
        else:
            species_ok = ok(batch.z, torch.int64)
        return species_ok and ok(batch.pos, torch.float32) and ok(batch.trans_vec, torch.float32) and ok(batch.sizes, torch.int64)

    def submit(self, batch) -> int:
        """Queues one host batch (attributes x (N,98), pos (N,3), trans_vec (B,3,3), sizes (B) int64); returns a ticket.
        Instead of the one-hot species rows ``x`` a batch may carry ``z`` (N) int64, the position of the 1 in every row
        (only on the one-call path: 8 bytes per atom go to the device instead of 392; same outputs)."""
        if len(self._inflight) >= self.depth:
            raise RuntimeError("the pipeline is full: collect a result before submitting more")
        sizes_np = batch.sizes.numpy()  # host memory: no device synchronisation
        n_atoms, n_edges = int(sizes_np.sum()), int(np.dot(sizes_np, sizes_np))
        max_atoms = int(sizes_np.max()) if sizes_np.size else 1
        slot = self._next % self.depth
        caller = torch.cuda.current_stream(self.device)
        compute = caller if self.compute_streams is None else self.compute_streams[self._next % len(self.compute_streams)]
        if n_atoms > 0 and self._native_applies(batch):
            n_crystals = int(sizes_np.size)
            st = self._native_slot(slot, n_atoms, n_crystals, n_edges, compute)
            t = st["tensors"]
            gather = None
            if self.gather is not None:
                if n_crystals != self.gather.local_rows:
                    raise ValueError(f"the peer gather expects {self.gather.local_rows} crystals per batch of this rank")
                gather = self.gather.serve_step(compute, t["y_all"], t["y_all_host"], t["status_host"], st["events"][3])
            with torch.cuda.device(self.device):
                x = getattr(batch, "x", None)
                _lib.call("cf_serve_submit", ctypes.byref(self._plan["desc"]), ctypes.byref(st["c"]),
                          None if x is None else x.data_ptr(), batch.pos.data_ptr(), batch.trans_vec.data_ptr(),
                          batch.sizes.data_ptr(), n_atoms, n_crystals, n_edges, max_atoms, 1 if st["used"] else 0,
                          None if gather is None else ctypes.byref(gather), None if x is not None else batch.z.data_ptr())
            st["used"] = True
            st["batch"] = batch  # the copies read the host tensors after this call returns
            ticket = self._next
            if gather is None:
                self._inflight.append((ticket, st["events"][2], t["y_host"][:n_crystals], None))
            else:
                self._inflight.append((ticket, st["events"][2], t["y_all_host"], t["status_host"]))
            self._next += 1
            return ticket
        if getattr(batch, "x", None) is None:
            raise ValueError("species indices `z` are taken by the one-call path only (an inference model with packed "
                             "weights, host tensors, no `post`): pass the one-hot rows `x`")
        dev = self._device_inputs(slot, batch)
        with torch.cuda.stream(self.copy_stream):
            if self._in_free[slot] is not None:
                self.copy_stream.wait_event(self._in_free[slot])  # the forward that last read these buffers has run
            dev.x.copy_(batch.x, non_blocking=True)
            dev.pos.copy_(batch.pos, non_blocking=True)
            dev.trans_vec.copy_(batch.trans_vec, non_blocking=True)
            dev.sizes.copy_(batch.sizes, non_blocking=True)
            self._copied[slot].record(self.copy_stream)
        compute.wait_event(self._copied[slot])
        with torch.no_grad(), torch.cuda.stream(compute):
            counts = (n_atoms, n_edges, max_atoms)
            if self._plan is not None:
                y = self.model._forward_native(dev, counts, self.gather, self._plan, inputs_ready=self._copied[slot])
            else:
                extra = {} if self.gather is None else {"gather": self.gather}
                y = self.model(dev, counts=counts, **extra)
            if self.post is not None:
                y = self.post(y)
        if self._in_free[slot] is None:
            self._in_free[slot] = torch.cuda.Event()
        self._in_free[slot].record(compute)
        out = self._out_ring[slot]
        if out is None or out.shape != y.shape:
            out = self._out_ring[slot] = torch.empty(y.shape, dtype=y.dtype).pin_memory()
        status = None
        # the outputs go to the host from the stream they become valid on: the compute stream, or the stream of an
        # overlapping peer gather's collects
        last = compute if (self.gather is None or not self.gather.overlap) else self.gather.collect_stream
        with torch.cuda.stream(last):
            out.copy_(y, non_blocking=True)
            if self.gather is not None:
                status = self._status_ring[slot]
                if status is None:
                    status = self._status_ring[slot] = torch.zeros(1, dtype=torch.int32).pin_memory()
                status.copy_(self.gather.status, non_blocking=True)
        done = self._done[slot]
        done.record(last)
        ticket = self._next
        self._inflight.append((ticket, done, out, status))
        self._next += 1
        return ticket

    def result(self, ticket: int) -> torch.Tensor:
        """Waits for the oldest batch in flight (``ticket`` must be its ticket) and returns its output on the host.
        The returned tensor is a view of a ring buffer that is reused ``depth`` submissions later: copy it to keep it.
        Raises if the batch's peer gather gave up waiting for a rank (its rows would be NaN)."""
        if not self._inflight or self._inflight[0][0] != ticket:
            raise RuntimeError("results must be collected in submission order")
        _, done, out, status = self._inflight.popleft()
        done.synchronize()
        if status is not None and int(status[0]) != 0:
            raise RuntimeError(f"peer gather: gave up waiting for the outputs of rank {int(status[0]) - 1}")
        return out

    def pending(self) -> int:
        return len(self._inflight)


def native_ok_without_grad(model) -> bool:
    """Whether the model's one-call inference path applies (its check reads the autograd mode)."""
    with torch.no_grad():
        return bool(model._native_ok())
