"""Data-parallel sharding of independent crystals: one process per GPU, no collective on the data path except the
final gather of per-crystal outputs.

The reference splits a batch inside one process (models/latticeformer.py:228-289): it replicates the encoder onto
every GPU on each forward, assigns crystals greedily to the device with the smallest sum of n^2 (:244-252), runs one
Python thread per GPU and gathers the (N,128) atom features back.  Here every rank holds a model replica for good,
the same greedy rule picks each rank's crystals, and only the (B_local, n_targets) outputs travel: one all-gather of
a few KB per forward.
"""
from __future__ import annotations

from typing import List, Sequence

import numpy as np
import torch
import torch.distributed as dist


def lpt_assign(sizes: Sequence[int], num_shards: int) -> List[List[int]]:
    """Greedy longest-processing-time assignment on the edge count n^2: crystals in descending n^2, each to the
    shard with the smallest total so far (models/latticeformer.py:244-252, including its tie-breaking start value)."""
    size2 = np.asarray(sizes, dtype=np.int64) ** 2
    order = np.argsort(-size2, kind="stable")
    totals = np.zeros(num_shards, np.int64)
    totals[0] = 1
    shards: List[List[int]] = [[] for _ in range(num_shards)]
    for item in order:
        dev = int(np.argmin(totals))
        totals[dev] += size2[item]
        shards[dev].append(int(item))
    return shards


def shard_balance(sizes: Sequence[int], shards: List[List[int]]) -> dict:
    """max/mean of the per-shard edge counts (sum n^2) and atom counts (sum n); 1.0 is perfect balance."""
    sizes = np.asarray(sizes, dtype=np.int64)
    e = np.array([int((sizes[s] ** 2).sum()) for s in shards], dtype=np.float64)
    a = np.array([int(sizes[s].sum()) for s in shards], dtype=np.float64)
    return {"edges_max_over_mean": float(e.max() / max(e.mean(), 1.0)),
            "atoms_max_over_mean": float(a.max() / max(a.mean(), 1.0))}


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
