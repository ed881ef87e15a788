// Peer gather: the per-crystal outputs of every rank, delivered by plain stores over NVLink.
//
// Crystals are independent, so the only exchange of a data-parallel forward is the gather of the (crystals, targets)
// outputs - a few KB.  The reference gathers the (atoms, 128) features of every GPU inside one process
// (models/latticeformer.py:278-289).  A library all-gather costs more than the bytes: padding the shard, the
// collective's launch and its rendezvous, and a reordering pass.  Here every rank owns a gather buffer that its peers
// have mapped (CUDA IPC); the kernel that produces a crystal's outputs stores them into EVERY rank's buffer, and one
// small kernel per rank waits for all rows and puts them into the order of the unsharded batch.  No multicast, no loads
// from peer memory.
//
// A value travels as one aligned 8-byte cell { float bits, step }: an 8-byte store is indivisible, so a reader that
// sees the step it waits for has the value too - no fence, no separate flag, no count of finished blocks; the latency
// of a gather is one store across NVLink plus the reader's poll.
//
// A gather buffer is `slots` x (world * rows_per_rank * targets) cells; step s (1, 2, ...) uses slot s % slots.  Two
// slots suffice: a rank can produce step s + 2 only after its collect of step s + 1 has seen every peer's rows of
// step s + 1, which a peer stores after its own collect of step s.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace cf {

__device__ __forceinline__ unsigned long long global_timer_ns()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Stores one output value of local crystal c into every rank's buffer.
__device__ __forceinline__ void peer_store(const cf_peer_gather &g, long long c, int targets, int t, float v)
{
    const long long at = ((long long)g.rank * g.rows_per_rank + c) * targets + t;
    const unsigned long long cell = ((unsigned long long)g.step << 32) | __float_as_uint(v);
    for (int r = 0; r < g.world; ++r) *reinterpret_cast<volatile unsigned long long *>(g.cells[r] + at) = cell;
}

}  // namespace cf
