// Arguments of the fused dense block of an encoder layer boundary (dense_block.cu).
#pragma once
#include <cuda_runtime.h>

namespace cf {

// Packed weights (DensePacked order): a Linear weight W (out x in, row-major) is stored as float4 fragments
//   P[(nt * (in/8) + ks) * 32 + lane] = { hi(W[n][k]), hi(W[n][k+4]), lo(W[n][k]), lo(W[n][k+4]) },
//   n = 8 nt + lane/4,  k = 8 ks + lane%4,  hi(w) = w rounded to TF32 (10-bit mantissa, ties away), lo(w) = hi(w - hi(w)),
// i.e. the B fragment of mma.m16n8k8 (and its low-order correction) for column tile nt and k step ks.
struct DenseArgs {
    long long N;
    int tail, head, ff;
    // tail: weights of the layer that just ran its attention
    const float *attn;              // (N,128) attention output
    const float4 *Wo, *W1, *W2;     // packed
    const float *bo, *b1, *b2;
    // head: weights of the layer whose attention comes next
    const float4 *Wqkv;             // packed (384 x 128)
    const float *bqkv, *w_pos;
    float gauss_scale, gauss_shift, a_factor, elu_beta, lower_bound;
    // activations
    float *x;                       // (N,128), updated in place by the tail
    float *q, *k, *v, *a;           // outputs of the head: (N,128) x 3 and (N,8)
};

int launch_dense_block(const DenseArgs &p, cudaStream_t s);

}  // namespace cf
