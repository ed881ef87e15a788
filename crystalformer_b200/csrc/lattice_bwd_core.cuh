// Pieces shared by the two backward kernels (per-edge operator and fused attention).
//
// The backward of the radial-basis expansion needs, for every (edge, translation) term and head,
//     c_h(d) = sum_k u_h[k] g_k(d),    g_k(d) = exp(-((k+1) mu0 - d)^2 / (2 (wscale mu0)^2)),
// the upstream gradient u (8 x 64, fixed per edge or per atom) contracted with the basis at distance d.  With lanes
// mapped to terms each lane evaluates the 64 basis values of its own term once (64 ex2) and contracts them with u,
// which is read from shared memory with warp-uniform addresses (broadcast, no bank conflicts); no cross-lane
// reduction is needed per term.
#pragma once
#include "lattice_core.cuh"

namespace cf {

constexpr int U_STRIDE = 64;                  // floats per head row of the u tile
constexpr int BWD_ENTRY_FLOATS = 12;          // x, d2, key index, pad, p0..7
constexpr int BWD_STAGE_FLOATS = 32 * BWD_ENTRY_FLOATS;

// c[h] = sum_k u[h][k] 2^(-((k+1) step - x)^2); u in shared memory, [8][U_STRIDE].
template <int K>
__device__ __forceinline__ void basis_dot(const float *__restrict__ u, float x, float bin_step, float (&c)[8])
{
#pragma unroll
    for (int h = 0; h < 8; ++h) c[h] = 0.f;
    float t = bin_step - x;
#pragma unroll 2
    for (int k = 0; k < K; k += 4) {
        const float t1 = t + bin_step, t2 = t1 + bin_step, t3 = t2 + bin_step;
        const float g0 = ex2(-t * t), g1 = ex2(-t1 * t1), g2 = ex2(-t2 * t2), g3 = ex2(-t3 * t3);
        t = t3 + bin_step;
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float4 uv = *reinterpret_cast<const float4 *>(u + h * U_STRIDE + k);
            c[h] = fmaf(uv.x, g0, c[h]);
            c[h] = fmaf(uv.y, g1, c[h]);
            c[h] = fmaf(uv.z, g2, c[h]);
            c[h] = fmaf(uv.w, g3, c[h]);
        }
    }
}

// The same for a basis of one bin width (BasisParams::windowed): a value more than 8 bins from the term's centre
// xi = x / step - 1 is below 2^-40, so only the 20 bins k0 .. k0 + 19 are evaluated, k0 the multiple of 4 with
// k0 <= floor(xi) - 8 < k0 + 4 (clamped to the table).  The rows of u are then read at lane-dependent offsets.
__device__ __forceinline__ void basis_dot_window(const float *__restrict__ u, float x, float bin_step, float (&c)[8])
{
#pragma unroll
    for (int h = 0; h < 8; ++h) c[h] = 0.f;
    int k0 = (__float2int_rd(__fdividef(x, bin_step)) - 9) & ~3;
    k0 = max(0, min(k0, 44));
    float t = (float)(k0 + 1) * bin_step - x;
    const float *uw = u + k0;
#pragma unroll
    for (int k = 0; k < 20; k += 4) {
        const float t1 = t + bin_step, t2 = t1 + bin_step, t3 = t2 + bin_step;
        const float g0 = ex2(-t * t), g1 = ex2(-t1 * t1), g2 = ex2(-t2 * t2), g3 = ex2(-t3 * t3);
        t = t3 + bin_step;
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float4 uv = *reinterpret_cast<const float4 *>(uw + h * U_STRIDE + k);
            c[h] = fmaf(uv.x, g0, c[h]);
            c[h] = fmaf(uv.y, g1, c[h]);
            c[h] = fmaf(uv.z, g2, c[h]);
            c[h] = fmaf(uv.w, g3, c[h]);
        }
    }
}

// Compacts the lanes' surviving terms into the warp's staging area; returns how many were staged.
__device__ __forceinline__ int stage_terms(float *stage, int lane, bool keep, float x, float d2, int key,
                                           const float (&p)[8])
{
    const unsigned mask = __ballot_sync(FULL, keep);
    if (keep) {
        const int slot = __popc(mask & ((1u << lane) - 1u));
        float4 *row = reinterpret_cast<float4 *>(stage + BWD_ENTRY_FLOATS * slot);
        row[0] = make_float4(x, d2, __int_as_float(key), 0.f);
        row[1] = make_float4(p[0], p[1], p[2], p[3]);
        row[2] = make_float4(p[4], p[5], p[6], p[7]);
    }
    __syncwarp();
    return __popc(mask);
}

}  // namespace cf
