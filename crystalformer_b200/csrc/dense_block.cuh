// Arguments of the fused dense block of an encoder layer boundary (dense_block.cu).
#pragma once
#include <cuda_runtime.h>
#include "crystalformer_b200.h"

namespace cf {

// Packed weights (DensePacked order): a Linear weight W (out x in, row-major) is stored as float4 fragments
//   P[(nt * (in/8) + ks) * 32 + lane] = { hi(W[n][k]), hi(W[n][k+4]), c(W[n][k]), c(W[n][k+4]) },
//   n = 8 nt + lane/4,  k = 8 ks + lane%4,  hi(w) = w rounded to TF32 (10-bit mantissa, ties away),
//   c(w) = the 32-bit word { lower half: bfloat16(hi(w)), upper half: bfloat16(w - hi(w)) },
// i.e. the B fragment of mma.m16n8k8 (TF32) for column tile nt and k step ks, and the B fragment of the 16-deep
// bfloat16 correction product of the same k step (whose A operand interleaves the activations' (lo, hi) halves).
struct DenseArgs {
    long long N;
    int tail, head, ff;
    int chained;                    // launch as a chained kernel (common.cuh): set by the one-call forwards
    // tail: weights of the layer that just ran its attention
    const float *attn;              // (N,128) attention output
    const float4 *Wo, *W1, *W2;     // packed
    const float *bo, *b1, *b2;
    // head: weights of the layer whose attention comes next
    const float4 *Wqkv;             // packed (384 x 128)
    const float *bqkv, *w_pos;
    float gauss_scale, gauss_shift, a_factor, elu_beta, lower_bound;
    // embedding (optional, only without a tail): x = features W_embed^T, written and carried into the head
    const float *features;          // (N, feature_dim), feature_dim <= 128; or null with
    const int64_t *species;         // (N) indices: feature row i = the one-hot row of species[i]
    int feature_dim;
    const float4 *Wembed;           // packed (128 x 128, input columns beyond feature_dim zero)
    // activations
    float *x;                       // (N,128), updated in place by the tail
    float *q, *k, *v, *a;           // outputs of the head: (N,128) x 3 and (N,8)
};

int launch_dense_block(const DenseArgs &p, cudaStream_t s);

// True if an encoder of these layers runs through the dense block: every layer brings packed weights (slot 10 of its
// 11 weight pointers) and the feed-forward width is a multiple of 128.
// cf_model_forward with the atoms' species as feature rows or as indices (model_forward.cu)
int model_forward_impl(void *cublas_handle, const float *features, const int64_t *species, int64_t feature_dim, const float *pos,
                       const float *trans, const int64_t *sizes, int64_t N, int64_t B, int64_t E, int64_t max_atoms,
                       const float *W_embed, const float *W_embed_packed, int num_layers, const float *const *weights,
                       const double *scalars, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius, int lattice_range,
                       int minimum_range, const float *W1, const float *b1, int64_t hidden, const float *W2, const float *b2,
                       int64_t targets, double order_reach, void *workspace, float *y, void *const *attn_events,
                       const cf_peer_gather *gather, void *inputs_ready, void *slot_free, void *stream);

inline bool dense_path_available(int num_layers, const float *const *weights, long long ff_dim)
{
    bool ok = ff_dim > 0 && ff_dim % 128 == 0;
    for (int l = 0; l < num_layers; ++l) ok = ok && weights[11 * l + 10] != nullptr;
    return ok;
}

// Embedding to run inside the first dense block of an encoder (x is then an output of the encoder call).
struct EmbedStage {
    const float *features;   // (N, feature_dim), or null with
    const int64_t *species;  // (N) indices below feature_dim (feature row i = one-hot of species[i])
    int feature_dim;         // <= 128
    const float4 *packed;    // W_embed packed as a 128 x 128 weight (input columns beyond feature_dim zero)
};

}  // namespace cf
