// Shared device helpers of the crystalformer_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "crystalformer_b200.h"

namespace cf {

constexpr int HEADS = 8;          // heads handled by the compiled kernels
constexpr int HEAD_DIM = 16;      // key / value head width
constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// ---- host-side error plumbing (api.cu) --------------------------------------------------------------------
int fail(int code, const char *fmt, ...);
int launch_status(const char *what);
float weight_floor_log2();  // log2 of the weight below which a term is left out of the basis accumulation

#define CF_REQUIRE(cond, code, ...) \
    do {                            \
        if (!(cond)) return ::cf::fail(code, __VA_ARGS__); \
    } while (0)

// ---- fast transcendental wrappers ---------------------------------------------------------------------------
// One MUFU.EX2 each; arguments here are <= 0 and results below 2^-126 flush to zero, which is what the callers want
// (such weights contribute nothing at float precision).
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rsqrt_fast(float x)
{
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- translation box ---------------------------------------------------------------------------------------
// The reference's cut-off rule (models/kernels/real_enc_fwd.cu:63-85), in the same mixed float/double arithmetic so
// that the integers agree exactly:  R = ceil( (double)((radius + 0.01f) * rvlen) / (2.0 * (double)pi_f) ).
struct BoxRule {
    float cutoff;       // 0: fixed box; <0: |cutoff| sigmas of each head's Gaussian; >0: radius in Angstrom
    int lattice_range;  // half-width of the fixed box
    int minimum_range;  // floor applied to adaptive half-widths (0 = none)
};

__device__ __forceinline__ void box_half_widths(const BoxRule &rule, float a, const float *__restrict__ rvlen3,
                                                int &R1, int &R2, int &R3)
{
    R1 = R2 = R3 = rule.lattice_range;
    if (rule.cutoff != 0.0f && rvlen3 != nullptr) {
        float radius = rule.cutoff;
        if (radius < 0.0f) radius = __fmul_rn(__fsqrt_rn(__fdiv_rn(-0.5f, a)), -radius);
        const double two_pi = 2.0 * (double)3.141592654f;
        const float reach = __fadd_rn(radius, 0.01f);
        R1 = (int)ceil((double)__fmul_rn(reach, rvlen3[0]) / two_pi);
        R2 = (int)ceil((double)__fmul_rn(reach, rvlen3[1]) / two_pi);
        R3 = (int)ceil((double)__fmul_rn(reach, rvlen3[2]) / two_pi);
        if (rule.minimum_range > 0) {
            R1 = max(R1, rule.minimum_range);
            R2 = max(R2, rule.minimum_range);
            R3 = max(R3, rule.minimum_range);
        }
    }
    R1 = min(max(R1, 0), CF_MAX_RANGE);
    R2 = min(max(R2, 0), CF_MAX_RANGE);
    R3 = min(max(R3, 0), CF_MAX_RANGE);
}

// Maps a flat term index t in [0, S1*S2*S3) to the translation (n1,n2,n3), n1 slowest, as the reference's loops run.
// Division by multiplication with a rounded reciprocal is exact here: t < 2^19 and the quotient is < 2^7.
struct TermGrid {
    int R1, R2, R3, S3, S23, count;
    float inv_S3, inv_S23;
    __device__ __forceinline__ void set(int r1, int r2, int r3)
    {
        R1 = r1; R2 = r2; R3 = r3;
        S3 = 2 * r3 + 1;
        S23 = (2 * r2 + 1) * S3;
        count = (2 * r1 + 1) * S23;
        inv_S3 = __frcp_rn((float)S3);
        inv_S23 = __frcp_rn((float)S23);
    }
    __device__ __forceinline__ void decode(int t, int &n1, int &n2, int &n3) const
    {
        const int q1 = __float2int_rd(((float)t + 0.5f) * inv_S23);
        const int r = t - q1 * S23;
        const int q2 = __float2int_rd(((float)r + 0.5f) * inv_S3);
        n1 = q1 - R1;
        n2 = q2 - R2;
        n3 = r - q2 * S3 - R3;
    }
};

// Lattice rows and the squared length of r + n.T, contracted the way nvcc contracts the reference's expression
// r + t1*n1 + t2*n2 + t3*n3 (three dependent FMAs per component).
struct Cell {
    float t1x, t1y, t1z, t2x, t2y, t2z, t3x, t3y, t3z;
    __device__ __forceinline__ void load(const float *__restrict__ t)
    {
        t1x = t[0]; t1y = t[1]; t1z = t[2];
        t2x = t[3]; t2y = t[4]; t2z = t[5];
        t3x = t[6]; t3y = t[7]; t3z = t[8];
    }
    __device__ __forceinline__ float dist2(float rx, float ry, float rz, int n1, int n2, int n3) const
    {
        const float f1 = (float)n1, f2 = (float)n2, f3 = (float)n3;
        const float dx = fmaf(t3x, f3, fmaf(t2x, f2, fmaf(t1x, f1, rx)));
        const float dy = fmaf(t3y, f3, fmaf(t2y, f2, fmaf(t1y, f1, ry)));
        const float dz = fmaf(t3z, f3, fmaf(t2z, f2, fmaf(t1z, f1, rz)));
        return fmaf(dz, dz, fmaf(dy, dy, dx * dx));
    }
};

__device__ __forceinline__ float warp_min(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ int warp_max_int(int v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
// Sum over the warp in a fixed butterfly order: every lane ends with the same bits, run to run.
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}

// Picks x[idx] from eight registers without dynamic indexing.
__device__ __forceinline__ float pick8(const float (&x)[8], int idx)
{
    float r = x[0];
#pragma unroll
    for (int h = 1; h < 8; ++h) r = (idx == h) ? x[h] : r;
    return r;
}

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
int sm_count();

}  // namespace cf
