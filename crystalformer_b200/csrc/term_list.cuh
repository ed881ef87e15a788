// Term lists: the (key, translation) pairs of a batch that can matter to ANY layer, found once per batch.
//
// The squared distances |pos_j - pos_i + n.T|^2 of a batch depend on the geometry only, while the Gaussian widths a
// change from layer to layer.  Every layer of the encoder used to enumerate its translation boxes again - in the phi
// kernel and in the candidate scan of the row kernel.  A term list stores, per edge (i,j), the translations n whose
// squared distance is within D of the edge's nearest image, D chosen for the WIDEST Gaussian any layer can have
// (a >= a_widest = lower bound of the positive function x -0.5/scale^2): a term outside the list has a weight below the
// floor for every admissible a.  Layers then read the lists: phi is a sum over an edge's entries, the row kernel's
// candidates come from a row's entries.  Entries keep |n1|,|n2|,|n3|, so that every (atom, head) still applies its own
// box of the reference's cut-off rule.
//
// Storage: per edge e the entries pool[start[e] .. start[e] + count[e]) (the entries of a row are contiguous, keys
// ascending); an entry is (d2, key | |n1| << 11 | |n2| << 17 | |n3| << 23).  Rows take their space from the pool with
// one atomic add; a row that does not fit (start < 0 for its edges) is processed by enumeration as before.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace cf {

struct TermList {
    const float2 *pool;    // entries
    const int *start;      // (E): first entry of every edge; < 0: the edge's row has no list
    const int *count;      // (E): entries of every edge
    const float *dmin;     // (E): smallest squared distance among the edge's entries
    float window;          // D: entries satisfy d2 <= (nearest image of the edge) + D
};

struct TermListBuild {
    // geometry
    const float *pos_ij, *tvecs, *rvlen;
    const int64_t *batch, *edges, *row_start;
    const int32_t *row_order;
    long long N, E;
    int max_atoms;
    BoxRule rule;
    float a_widest;        // the a (< 0) closest to zero that any layer can produce
    float window;          // D
    // outputs
    float2 *pool;
    long long capacity;    // entries
    int *start, *count;    // (E) each
    float *dmin;           // (E)
    unsigned long long *cursor;  // pool allocation cursor, zeroed by the build itself
};

size_t term_pool_entries(long long N, long long E);   // capacity the one-call forwards reserve
int launch_term_list_build(const TermListBuild &b, cudaStream_t s);

// Layout of a term-list workspace of term_list_workspace_bytes(N, E) bytes: directory (3 E words), cursor, pool.
size_t term_list_workspace_bytes(long long N, long long E);
void term_list_carve(void *workspace, long long N, long long E, int **start, int **count, float **dmin,
                     unsigned long long **cursor, float2 **pool);
// D for a floor of 2^floor_log2 and the widest Gaussian a_widest < 0
inline float term_window(float floor_log2, float a_widest) { return -floor_log2 / (-a_widest * LOG2E); }

struct PhiListArgs {
    TermList list;
    const float *a, *pos_ij, *tvecs, *rvlen;
    const int64_t *batch, *edges;
    long long E;
    BoxRule rule;
    float floor_log2;
    float *z;              // (E,8)
    unsigned *zero_word;   // optional word to zero (row ticket of the following kernel)
};
int launch_phi_from_list(const PhiListArgs &p, cudaStream_t s);

}  // namespace cf
