// Row lists: for every atom row i, ALL (key, translation) terms of the row that can matter to any layer, sorted by
// distance - the data structure behind the tensor-core row kernel for batches of small crystals
// (infinite_attn_sorted.cu).
//
// The per-edge term lists (term_list.cuh) keep an edge's terms together, which suits per-edge sums.  The fused
// attention of a row, however, is a sum over all terms of the row,
//     out_i = sum_{j,n} exp(q_i.k_j + a_i d2_jn - lse_i) (v_j + W g(d_jn)),
// and two things become possible when the row's terms are ordered by distance instead:
//   * a layer stops at the first chunk whose terms are all below the weight floor for its Gaussian widths (weights
//     fall monotonically with distance for a fixed key offset bound), so narrow layers read a fraction of the list;
//   * consecutive terms hit neighbouring radial-basis bins, so a chunk of eight terms touches one or two 16-bin tiles
//     of the 64 bins, which is what makes the histogram a short sequence of tensor-core products.
//
// Storage (one workspace of row_list_workspace_bytes(N, E) bytes, carved by row_list_carve):
//   rowdir  [N][2] int4, indexed by PROCESSING SLOT (the position in row_order):
//           { atom i, first atom of its crystal, keys n, crystal c }, { first entry or -1, chunks of 8 entries, first
//           edge e0, 0 } - everything a warp needs to start a row comes with one 32-byte read
//   dmin    [E] float: smallest listed squared distance of every edge
//   sched   [ROW_SCHED_SLOTS][4] unsigned: per attention call { ticket of the shared rows, rows left over, ticket of
//           the left-over launch, ticket of the one-warp rows }; zeroed by the build
//   leftover[N] int: atoms whose row the sorted kernel could not process (no list, or a head whose box misses the list)
//   tasks   [2][N] int + two counters: the slots of the rows with long lists (shared by the four warps of a block) and
//           of all other rows (one warp each), in the order in which the build finished them
//   pool    entries (d2, key) with key = j | |n1| << 8 | |n2| << 16 | |n3| << 24; a row's entries are contiguous,
//           ascending in d2, padded to a multiple of eight with copies of the last d2 whose key (0x7f7f7f00) lies
//           outside every box
// Rows that do not fit (more than ROW_LIST_CAP entries, or the pool is full) get first entry -1 and are processed by
// the enumerating row kernel; results therefore never depend on the capacities.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace cf {

constexpr int ROW_LIST_MAX_KEYS = 64;   // crystals of at most this many atoms
constexpr int ROW_LIST_CAP = 4096;      // entries of one row (sorted in shared memory by the build)
constexpr int ROW_SCHED_SLOTS = 16;     // attention calls per build that find a zeroed scheduling block
constexpr int ROW_PAD_KEY = 0x7f7f7f00; // |n| bytes of 127: outside every box (CF_MAX_RANGE = 32)

struct RowListView {
    int4 *rowdir;
    float *dmin;
    unsigned *sched;
    int *leftover;
    int *tasks;            // [2][N]
    unsigned *task_count;  // [2]: rows with long lists, other rows
    unsigned long long *cursor;
    float2 *pool;
    long long capacity;  // entries
};

constexpr int ROW_COOP_CHUNKS = 64;  // rows listing more chunks than this are shared by the warps of a block

struct RowListBuild {
    const float *pos_ij, *tvecs, *rvlen;
    const int64_t *batch, *edges, *row_start;
    const int32_t *row_order;
    long long N, E;
    BoxRule rule;
    float a_widest;  // the a (< 0) closest to zero that any layer can produce
    float window;    // entries satisfy d2 <= (nearest image of the edge) + window
    int coop_chunks; // rows with more chunks go to the first task list
    RowListView out;
};

size_t row_list_workspace_bytes(long long N, long long E);
RowListView row_list_carve(void *workspace, long long N, long long E);
int launch_row_list_build(const RowListBuild &b, cudaStream_t s);

// True if `key`'s |n1|,|n2|,|n3| bytes are all within the box whose bytes are R1,R2,R3 (boxor = box | 0x808080):
// byte-wise 128 + R - |n| keeps its top bit exactly when |n| <= R, and never borrows for |n| < 128.
__device__ __forceinline__ bool row_key_in_box(int key, unsigned boxor)
{
    return ((boxor - ((unsigned)key >> 8)) & 0x808080u) == 0x808080u;
}

// The sorted row kernel of one attention call (infinite_attn_sorted.cu).  `sched` = the call's scheduling block
// (4 words, zero on entry).  Rows it cannot process are appended to view.leftover / sched[1].
struct SortedRowLaunch {
    const float *q, *k, *v, *a, *rvlen, *W;
    RowListView view;
    unsigned *sched;
    float *out, *lse;
    long long N;
    int max_atoms;
    int K;         // 64: with the radial basis and its projection W; 0: without
    BoxRule rule;
    double dist_max, wscale;
    bool chained;  // launch as a chained kernel (common.cuh)
};
int launch_sorted_rows(const SortedRowLaunch &p, cudaStream_t s);

}  // namespace cf
