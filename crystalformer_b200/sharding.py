"""Data-parallel sharding of independent crystals: one process per GPU, no collective on the data path except the
final gather of per-crystal outputs.

The reference splits a batch inside one process (models/latticeformer.py:228-289): it replicates the encoder onto
every GPU on each forward, assigns crystals greedily to the device with the smallest sum of n^2 (:244-252), runs one
Python thread per GPU and gathers the (N,128) atom features back.  Here every rank holds a model replica for good,
the same greedy rule picks each rank's crystals, and only the (B_local, n_targets) outputs travel: one all-gather of
a few KB per forward.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from . import _lib


def lpt_assign(sizes: Sequence[int], num_shards: int, weights: Optional[Sequence[float]] = None) -> List[List[int]]:
    """Greedy longest-processing-time assignment: crystals in descending weight, each to the shard with the smallest
    total so far.  The default weight is the edge count n^2, which makes this the reference's rule
    (models/latticeformer.py:244-252, including its tie-breaking start value); ``crystal_cost`` gives a weight that
    also knows the cell volume."""
    w = np.asarray(sizes, dtype=np.int64) ** 2 if weights is None else np.asarray(weights, dtype=np.float64)
    order = np.argsort(-w, kind="stable")
    totals = np.zeros(num_shards, w.dtype)
    totals[0] = 1
    shards: List[List[int]] = [[] for _ in range(num_shards)]
    for item in order:
        dev = int(np.argmin(totals))
        totals[dev] += w[item]
        shards[dev].append(int(item))
    return shards


def crystal_cost(sizes: Sequence[int], trans_vec: np.ndarray, reach: float = 15.0) -> np.ndarray:
    """Weight of every crystal for splitting a batch over GPUs: n (450 + n (1 + (4 pi / 3) reach^3 / |det trans|)).
    The second term is about the number of (key, translation) pairs within ``reach`` Angstrom, which is what the
    lattice sums cost: two crystals with the same n^2 differ by the ratio of their cell volumes, which n^2 alone does
    not see.  The first is the atoms' share of the dense layers, with the constant measured on a B200 (one step of the
    4-layer model on 128 crystals of 1-30 atoms: 81 ns per atom in the dense blocks, 0.11 ns per lattice-sum term and
    layer in the attention)."""
    n = np.asarray(sizes, dtype=np.float64)
    vol = np.abs(np.linalg.det(np.asarray(trans_vec, dtype=np.float64)))
    return n * (450.0 + n * (1.0 + (4.0 * np.pi / 3.0) * reach ** 3 / np.maximum(vol, 1e-6)))


def shard_balance(sizes: Sequence[int], shards: List[List[int]], weights: Optional[Sequence[float]] = None) -> dict:
    """max/mean of the per-shard edge counts (sum n^2), atom counts (sum n) and, given per-crystal weights, of the
    weights; 1.0 is perfect balance."""
    sizes = np.asarray(sizes, dtype=np.int64)
    e = np.array([int((sizes[s] ** 2).sum()) for s in shards], dtype=np.float64)
    a = np.array([int(sizes[s].sum()) for s in shards], dtype=np.float64)
    out = {"edges_max_over_mean": float(e.max() / max(e.mean(), 1.0)),
           "atoms_max_over_mean": float(a.max() / max(a.mean(), 1.0))}
    if weights is not None:
        w = np.asarray(weights, dtype=np.float64)
        c = np.array([float(w[s].sum()) for s in shards])
        out["cost_max_over_mean"] = float(c.max() / max(c.mean(), 1e-30))
    return out


_GATHER_INDEX: dict = {}


def _gather_index(shards: List[List[int]], longest: int, device) -> torch.Tensor:
    """Row of the gathered (world * longest, T) buffer that holds crystal g of the unsharded batch, for every g.
    Built once per (sharding, device): a host list turned into a device tensor is a synchronous copy, which must not
    sit on the per-step path."""
    key = (tuple(tuple(s) for s in shards), longest, str(device))
    hit = _GATHER_INDEX.get(key)
    if hit is None:
        total = sum(len(s) for s in shards)
        src = np.zeros(total, dtype=np.int64)
        for r, s in enumerate(shards):
            src[np.asarray(s, dtype=np.int64)] = r * longest + np.arange(len(s), dtype=np.int64)
        hit = torch.from_numpy(src).to(device)
        if len(_GATHER_INDEX) > 8:
            _GATHER_INDEX.clear()
        _GATHER_INDEX[key] = hit
    return hit


def gather_outputs(local: torch.Tensor, shards: List[List[int]], group=None) -> torch.Tensor:
    """All-gathers the per-crystal outputs of every rank and puts them back in the order of the unsharded batch.

    ``local`` is (len(shards[rank]), T) on this rank's device (CPU tensors with the gloo backend).  Shards are padded
    to the largest one so that a single fixed-size all-gather suffices."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    longest = max(len(s) for s in shards)
    index = _gather_index(shards, longest, local.device)
    if world == 1:
        return local.index_select(0, index)
    T = local.shape[1]
    if local.shape[0] == longest:
        padded = local.contiguous()
    else:
        padded = local.new_zeros((longest, T))
        padded[: local.shape[0]] = local
    gathered = local.new_empty((world * longest, T))
    dist.all_gather_into_tensor(gathered, padded, group=group)
    return gathered.index_select(0, index)


def peer_descriptor(world: int, rank: int, rows_per_rank: int, step: int,
                    cell_ptrs: Sequence[int]) -> _lib.PeerGatherDescriptor:
    """A ``cf_peer_gather`` for one step: ``cell_ptrs[r]`` is the address, in this process, of the step's slot inside
    rank r's gather buffer."""
    d = _lib.PeerGatherDescriptor()
    d.world, d.rank, d.rows_per_rank, d.step, d.reserved = world, rank, rows_per_rank, step & 0xFFFFFFFF, 0
    for r in range(world):
        d.cells[r] = cell_ptrs[r]
    return d


class PeerGather:
    """The gather of every rank's per-crystal outputs by stores into the peers' memory (one process per GPU of one
    machine), instead of a library all-gather: see ``cf_peer_gather`` in include/crystalformer_b200.h.

        gather = PeerGather(shards, n_targets, device)            # collective: every rank of the group calls it
        y_all = model(batch_of_this_rank, counts=..., gather=gather)   # (all crystals, n_targets), unsharded order

    ``model`` stores its outputs straight from the pooling + head kernel into every rank's buffer; ``store`` does the
    same for outputs that exist already.  Every rank must run the same sequence of gathers.  ``check()`` (a device
    synchronisation) raises if a collect gave up waiting for a rank.

    ``overlap=True``: the collect of a step - the only place where a rank waits for the others - runs on a stream of
    its own instead of the stream of the forward, so a rank that is ahead starts its next batches while the last rows
    of the step arrive.  ``collect()`` then returns a tensor that is valid on ``collect_stream`` once ``ready`` has
    fired: consume it there, or call ``wait_ready()`` to make the current stream wait.  A rank runs at most
    ``slots // 2`` steps ahead of its own collects (the store of step t waits for the collect of step t - slots // 2),
    which is what keeps a slot from being overwritten before every rank has read it.
    """

    def __init__(self, shards: List[List[int]], targets: int, device, group=None, slots: int = 4,
                 timeout_s: float = 5.0, overlap: bool = False):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        if len(shards) != self.world or self.world > _lib.MAX_PEERS:
            raise ValueError(f"{len(shards)} shards for {self.world} ranks (at most {_lib.MAX_PEERS})")
        if slots < 2:
            raise ValueError("a peer gather needs at least two slots")
        self.device = torch.device(device)
        self.targets, self.slots, self.timeout_s = int(targets), int(slots), float(timeout_s)
        self.rows_per_rank = max(len(s) for s in shards)
        self.local_rows = len(shards[self.rank])
        self.total_rows = sum(len(s) for s in shards)
        self.index = _gather_index(shards, self.rows_per_rank, self.device)
        self._slot_bytes = (self.world * self.rows_per_rank * self.targets * 8 + 255) // 256 * 256
        own, handle = ctypes.c_void_p(), (ctypes.c_ubyte * _lib.PEER_HANDLE_BYTES)()
        with torch.cuda.device(self.device):
            _lib.call("cf_peer_alloc", self._slot_bytes * self.slots, ctypes.byref(own), handle)
            self._own = own.value
            handles: List[Optional[bytes]] = [bytes(handle)] * self.world
            if self.world > 1:
                dist.all_gather_object(handles, bytes(handle), group=group)
            self._bases: List[int] = []
            for r in range(self.world):
                if r == self.rank:
                    self._bases.append(self._own)
                else:
                    mapped = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * _lib.PEER_HANDLE_BYTES).from_buffer_copy(handles[r])
                    _lib.call("cf_peer_open", buf, ctypes.byref(mapped))
                    self._bases.append(mapped.value)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.step = 0
        self.overlap = bool(overlap)
        self.collect_stream = torch.cuda.Stream(self.device) if self.overlap else None
        self.ready: Optional[torch.cuda.Event] = None
        self._collected = [None] * self.slots  # per slot: the event after the collect that last read it
        self._lag = max(1, self.slots // 2)
        if self.world > 1:
            dist.barrier(group=group)  # every buffer is mapped everywhere before the first store

    def next_descriptor(self) -> _lib.PeerGatherDescriptor:
        """Advances to the next step and returns its descriptor (for ``cf_model_forward`` / ``store``).  With
        ``overlap`` the current stream is first made to wait for the collect of step - slots // 2."""
        self.step += 1
        if self.overlap and self.step > self._lag:
            done = self._collected[(self.step - self._lag) % self.slots]
            if done is not None:
                torch.cuda.current_stream(self.device).wait_event(done)
        at = (self.step % self.slots) * self._slot_bytes
        return peer_descriptor(self.world, self.rank, self.rows_per_rank, self.step, [b + at for b in self._bases])

    def serve_step(self, compute_stream, y_all: torch.Tensor, y_all_host: torch.Tensor, status_host: torch.Tensor,
                   stored: torch.cuda.Event) -> _lib.ServeGather:
        """Advances to the next step and describes it for ``cf_serve_submit``, which then issues what
        ``next_descriptor`` (the wait for the collect of step - slots // 2), the model's stores and ``collect`` issue:
        the collect on ``collect_stream`` (``overlap``) or on ``compute_stream``, its outputs in ``y_all`` and, with
        the status word, in the two pinned host tensors.  ``stored``: an event of the caller's, recorded by the call."""
        self.step += 1
        after = None
        if self.overlap and self.step > self._lag:
            after = self._collected[(self.step - self._lag) % self.slots]
        slot = self.step % self.slots
        at = slot * self._slot_bytes
        self._serve_desc = peer_descriptor(self.world, self.rank, self.rows_per_rank, self.step, [b + at for b in self._bases])
        collect_stream = self.collect_stream if self.overlap else compute_stream
        done = self._collected[slot]
        if done is None:
            done = self._collected[slot] = torch.cuda.Event()
            done.record(collect_stream)  # (an event has a handle once it has been recorded)
        if self.overlap:
            self.ready = done
        return _lib.ServeGather(
            store=ctypes.addressof(self._serve_desc), collect_stream=collect_stream.cuda_stream,
            store_after=None if after is None else after.cuda_event, stored=stored.cuda_event, collected=done.cuda_event,
            own_cells=self._own + at, index=self.index.data_ptr(), total_rows=self.total_rows, y_all=y_all.data_ptr(),
            y_all_host=y_all_host.data_ptr(), status=self.status.data_ptr(), status_host=status_host.data_ptr(),
            timeout_s=self.timeout_s)

    def store(self, y: torch.Tensor) -> None:
        """Opens the next step with outputs that exist already: (local crystals, targets) on this rank's device."""
        y = y.detach().float().contiguous()
        if y.shape != (self.local_rows, self.targets):
            raise ValueError(f"expected {(self.local_rows, self.targets)} outputs, got {tuple(y.shape)}")
        d = self.next_descriptor()
        with torch.cuda.device(self.device):
            _lib.call("cf_peer_gather_store", y.data_ptr(), y.shape[0], self.targets, ctypes.byref(d),
                      torch.cuda.current_stream(self.device).cuda_stream)

    def collect(self) -> torch.Tensor:
        """Waits, on the device, for every rank's rows of the current step; returns (all crystals, targets) in the
        order of the unsharded batch."""
        if self.step == 0:
            raise RuntimeError("collect() before the first store")
        at = self._own + (self.step % self.slots) * self._slot_bytes
        if not self.overlap:
            out = torch.empty((self.total_rows, self.targets), dtype=torch.float32, device=self.device)
            with torch.cuda.device(self.device):
                _lib.call("cf_peer_gather_collect", at, self.step & 0xFFFFFFFF, self.index.data_ptr(), self.total_rows,
                          self.targets, self.rows_per_rank, out.data_ptr(), self.status.data_ptr(), self.timeout_s,
                          torch.cuda.current_stream(self.device).cuda_stream)
            return out
        slot = self.step % self.slots
        stored = torch.cuda.Event()
        stored.record(torch.cuda.current_stream(self.device))  # this rank's stores of the step have been issued
        with torch.cuda.device(self.device), torch.cuda.stream(self.collect_stream):
            self.collect_stream.wait_event(stored)
            out = torch.empty((self.total_rows, self.targets), dtype=torch.float32, device=self.device)
            _lib.call("cf_peer_gather_collect", at, self.step & 0xFFFFFFFF, self.index.data_ptr(), self.total_rows,
                      self.targets, self.rows_per_rank, out.data_ptr(), self.status.data_ptr(), self.timeout_s,
                      self.collect_stream.cuda_stream)
            done = self._collected[slot]
            if done is None:
                done = self._collected[slot] = torch.cuda.Event()
            done.record(self.collect_stream)
        self.ready = done
        return out

    def wait_ready(self) -> None:
        """``overlap``: makes the current stream wait for the most recent collect."""
        if self.ready is not None:
            torch.cuda.current_stream(self.device).wait_event(self.ready)

    def check(self) -> None:
        code = int(self.status.item())
        if code != 0:
            raise RuntimeError(f"peer gather: rank {self.rank} gave up waiting for the outputs of rank {code - 1}")

    def close(self) -> None:
        """Collective: unmaps the peers' buffers, then frees the own one."""
        if self._own is None:
            return
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            for r, base in enumerate(self._bases):
                if r != self.rank:
                    _lib.call("cf_peer_close", base)
            if self.world > 1:
                dist.barrier(group=self.group)  # nobody has the buffer mapped any more
            _lib.call("cf_peer_free", self._own)
        self._own, self._bases = None, []
