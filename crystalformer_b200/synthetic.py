"""Seeded synthetic crystals that stand in for the JARVIS / MEGNet structures.

The reference feeds its model PyG ``Data`` objects holding ``x (N,98)`` one-hot
atomic numbers, ``pos (N,3)`` Cartesian positions, ``trans_vec (B,3,3)`` lattice
rows, ``sizes (B)`` atoms per cell and ``batch (N)`` (dataloaders/dataset_latticeformer.py:11-38).
The datasets themselves are external downloads, so every test and benchmark here
draws crystals with the same layout from a seeded ``numpy`` generator instead.

Everything is numpy on the host; callers move the arrays to a device themselves.
"""
from __future__ import annotations

import dataclasses
from typing import Callable, Optional

import numpy as np

ATOM_FEAT_DIM = 98  # width of the one-hot species vector (models/latticeformer.py:137)


@dataclasses.dataclass
class CrystalBatch:
    """A flat batch of crystals in the reference's ``Data`` layout (numpy, host)."""

    x: np.ndarray          # (N, 98) float32 one-hot species
    pos: np.ndarray        # (N, 3)  float32 Cartesian positions
    trans_vec: np.ndarray  # (B, 3, 3) float32 lattice vectors as rows
    sizes: np.ndarray      # (B,) int64 atoms per cell
    batch: np.ndarray      # (N,) int64 crystal id of each atom
    z: np.ndarray          # (N,) int64 atomic numbers 1..94

    @property
    def num_crystals(self) -> int:
        return int(self.sizes.shape[0])

    @property
    def num_atoms(self) -> int:
        return int(self.pos.shape[0])

    @property
    def num_edges(self) -> int:
        return int((self.sizes.astype(np.int64) ** 2).sum())

    def select(self, crystal_ids) -> "CrystalBatch":
        """Sub-batch holding the given crystals, in the given order."""
        crystal_ids = np.asarray(crystal_ids, dtype=np.int64)
        starts = np.concatenate([[0], np.cumsum(self.sizes)])
        if crystal_ids.size:
            rows = np.concatenate([np.arange(starts[c], starts[c + 1]) for c in crystal_ids])
        else:
            rows = np.zeros((0,), dtype=np.int64)
        sizes = self.sizes[crystal_ids]
        return CrystalBatch(
            x=self.x[rows], pos=self.pos[rows], trans_vec=self.trans_vec[crystal_ids],
            sizes=sizes, batch=np.repeat(np.arange(len(crystal_ids), dtype=np.int64), sizes),
            z=self.z[rows])


def lattice_from_lengths_angles(lengths: np.ndarray, angles_deg: np.ndarray) -> np.ndarray:
    """Rows t1,t2,t3 of the cell from (a,b,c) and (alpha,beta,gamma) in degrees.

    t1 = (a,0,0), t2 = (b cos g, b sin g, 0), t3 = (c cos b, c (cos a - cos b cos g)/sin g, c sqrt(1-cx^2-cy^2)).
    Every angle triple in [60,120]^3 gives a positive volume.
    """
    a, b, c = lengths[:, 0], lengths[:, 1], lengths[:, 2]
    al, be, ga = (np.deg2rad(angles_deg[:, i]) for i in range(3))
    cx = np.cos(be)
    cy = (np.cos(al) - np.cos(be) * np.cos(ga)) / np.sin(ga)
    cz = np.sqrt(np.maximum(1.0 - cx * cx - cy * cy, 1e-12))
    t = np.zeros((lengths.shape[0], 3, 3), dtype=np.float64)
    t[:, 0, 0] = a
    t[:, 1, 0] = b * np.cos(ga)
    t[:, 1, 1] = b * np.sin(ga)
    t[:, 2, 0] = c * cx
    t[:, 2, 1] = c * cy
    t[:, 2, 2] = c * cz
    return t


def make_crystals(
    seed: int,
    num_crystals: int,
    atoms: Callable[[np.random.Generator, int], np.ndarray],
    length_range=(3.0, 15.0),
    angle_range=(60.0, 120.0),
) -> CrystalBatch:
    """Draw ``num_crystals`` cells. Draw order: sizes, lengths, angles, species, fractional coordinates."""
    rng = np.random.Generator(np.random.PCG64(seed))
    sizes = np.asarray(atoms(rng, num_crystals), dtype=np.int64)
    lengths = rng.uniform(length_range[0], length_range[1], size=(num_crystals, 3))
    angles = rng.uniform(angle_range[0], angle_range[1], size=(num_crystals, 3))
    n_atoms = int(sizes.sum())
    z = rng.integers(1, 95, size=n_atoms, dtype=np.int64)
    frac = rng.random(size=(n_atoms, 3))
    trans = lattice_from_lengths_angles(lengths, angles)
    batch = np.repeat(np.arange(num_crystals, dtype=np.int64), sizes)
    pos = np.einsum("nd,nde->ne", frac, trans[batch])
    x = np.zeros((n_atoms, ATOM_FEAT_DIM), dtype=np.float32)
    x[np.arange(n_atoms), z - 1] = 1.0
    return CrystalBatch(x=x, pos=pos.astype(np.float32), trans_vec=trans.astype(np.float32),
                        sizes=sizes, batch=batch, z=z)


def uniform_atoms(lo: int, hi: int):
    return lambda rng, b: rng.integers(lo, hi + 1, size=b)


def lognormal_atoms(median: float, shape: float, lo: int, hi: int):
    return lambda rng, b: np.clip(np.rint(np.exp(rng.normal(np.log(median), shape, size=b))), lo, hi).astype(np.int64)


# The five benchmark configurations, as (seed, crystals, size law, lattice lengths).
CONFIGS = {
    "cfg0": dict(seed=0, num_crystals=128, atoms=uniform_atoms(1, 30), length_range=(3.0, 15.0)),
    "cfg1": dict(seed=1, num_crystals=4096, atoms=uniform_atoms(1, 64), length_range=(3.0, 15.0)),
    "cfg2": dict(seed=2, num_crystals=256, atoms=lognormal_atoms(8.0, 0.75, 1, 60), length_range=(3.0, 15.0)),
    "cfg3": dict(seed=3, num_crystals=256, atoms=uniform_atoms(1, 40), length_range=(3.0, 15.0)),
    "cfg4": dict(seed=4, num_crystals=64, atoms=uniform_atoms(100, 200), length_range=(10.0, 25.0)),
}


def make_config(name: str, seed: Optional[int] = None, num_crystals: Optional[int] = None) -> CrystalBatch:
    """Crystals of one named configuration; ``seed`` / ``num_crystals`` override the defaults."""
    cfg = dict(CONFIGS[name])
    if seed is not None:
        cfg["seed"] = seed
    if num_crystals is not None:
        cfg["num_crystals"] = num_crystals
    return make_crystals(**cfg)


def all_pairs_edges(sizes: np.ndarray) -> np.ndarray:
    """Host restatement of the all-pairs edge list (models/indexed_latticeformer_encoder.py:15-32).

    For a crystal whose atoms are [c, c+n): row 0 repeats each i n times, row 1 cycles j; crystals are concatenated.
    """
    ei, ej = [], []
    c = 0
    for n in np.asarray(sizes, dtype=np.int64):
        idx = np.arange(c, c + n, dtype=np.int64)
        ei.append(np.repeat(idx, n))
        ej.append(np.tile(idx, n))
        c += n
    if not ei:
        return np.zeros((2, 0), dtype=np.int64)
    return np.stack([np.concatenate(ei), np.concatenate(ej)])


def microbench_edges(seed: int = 1, num_pairs: int = 250_000, heads: int = 8):
    """The lattice-sum microbenchmark input: ``num_pairs`` (i,j) pairs drawn without replacement from the
    all-pairs list of the 4096-crystal batch, with one Gaussian width per (pair, head): sigma = 1.4 (0.5 + U(0,1)),
    a = -0.5 / sigma^2. Returns (batch, edges (2,P) int64, pos_ij (P,3) f32, a (P,heads) f32)."""
    cb = make_config("cfg1", seed=seed)
    edges_all = all_pairs_edges(cb.sizes)
    rng = np.random.Generator(np.random.PCG64(seed + 1000))
    pick = np.sort(rng.choice(edges_all.shape[1], size=min(num_pairs, edges_all.shape[1]), replace=False))
    edges = np.ascontiguousarray(edges_all[:, pick])
    sigma = 1.4 * (0.5 + rng.random(size=(edges.shape[1], heads)))
    a = (-0.5 / (sigma * sigma)).astype(np.float32)
    pos_ij = (cb.pos[edges[1]] - cb.pos[edges[0]]).astype(np.float32)
    return cb, edges, pos_ij, a
