// Building blocks shared by the lattice-sum kernels.
//
// Two mappings of the (edge, translation) terms onto threads are used:
//
//   thread <-> edge   (edge_phi)            every thread walks the whole translation box of its own edge with three
//                                           nested float counters and keeps eight running sums, one per head.  No
//                                           shuffles, no shared memory, no integer->float conversions in the loop.
//                                           Used for the log-sum-exp phi, which is MUFU-bound (8 ex2 per term).
//   lane <-> term, then lane <-> bins       (TermWalker + BinAccumulator)  a warp takes 32 consecutive terms, one per
//                                           lane, evaluates the eight exponents, drops the terms whose weights cannot
//                                           matter, compacts the survivors into shared memory and then turns around:
//                                           each lane owns bins (lane, lane+32) of all heads, i.e. 16 accumulators in
//                                           registers, and per surviving term does 2 ex2 + 16 FMA.  The radial basis is
//                                           thus evaluated once per term and shared by the eight heads.
#pragma once
#include "common.cuh"

namespace cf {

// ---- translation box, division-free -------------------------------------------------------------------------
// R = ceil((double)x / two_pi) with two_pi = 2.0 * (double)3.141592654f, the reference's expression
// (models/kernels/real_enc_fwd.cu:76).  Because x is a float and two_pi has a 24-bit significand, R * two_pi is exact
// in double for R < 2^29, and the rounded quotient lies on the same side of every integer as the exact one; hence R is
// the smallest integer with R * two_pi >= x, which needs two double multiplies instead of a double division.
__device__ __forceinline__ int ceil_div_two_pi(float x)
{
    const double two_pi = 2.0 * (double)3.141592654f;
    if (!(x > 0.0f)) return 0;  // also NaN
    int r = (int)ceilf(x * 0.15915494f);
    r = min(r, 1 << 20);
    while ((double)r * two_pi < (double)x) ++r;
    while (r > 0 && (double)(r - 1) * two_pi >= (double)x) --r;
    return r;
}

// Half-widths of the box of one (atom, head); same rule and rounding as box_half_widths in common.cuh.
__device__ __forceinline__ int packed_box(const BoxRule &rule, float a, const float *__restrict__ rvlen3)
{
    int R1 = rule.lattice_range, R2 = R1, R3 = R1;
    if (rule.cutoff != 0.0f && rvlen3 != nullptr) {
        float radius = rule.cutoff;
        if (radius < 0.0f) radius = __fmul_rn(__fsqrt_rn(__fdiv_rn(-0.5f, a)), -radius);
        const float reach = __fadd_rn(radius, 0.01f);
        R1 = ceil_div_two_pi(__fmul_rn(reach, rvlen3[0]));
        R2 = ceil_div_two_pi(__fmul_rn(reach, rvlen3[1]));
        R3 = ceil_div_two_pi(__fmul_rn(reach, rvlen3[2]));
        if (rule.minimum_range > 0) {
            R1 = max(R1, rule.minimum_range);
            R2 = max(R2, rule.minimum_range);
            R3 = max(R3, rule.minimum_range);
        }
    }
    R1 = min(max(R1, 0), CF_MAX_RANGE);
    R2 = min(max(R2, 0), CF_MAX_RANGE);
    R3 = min(max(R3, 0), CF_MAX_RANGE);
    return R1 | (R2 << 8) | (R3 << 16);
}
__device__ __forceinline__ int box_r1(int pk) { return pk & 0xff; }
__device__ __forceinline__ int box_r2(int pk) { return (pk >> 8) & 0xff; }
__device__ __forceinline__ int box_r3(int pk) { return (pk >> 16) & 0xff; }
// component-wise maximum of two packed boxes (each component < 128, so the bytes never carry)
__device__ __forceinline__ int box_union(int x, int y) { return (int)__vmaxu4((unsigned)x, (unsigned)y); }

// ---- thread <-> edge: phi of one edge, all heads ----------------------------------------------------------------
// z[h] = log sum_{n in box_h} exp(a_h d2_n), evaluated as log sum_n exp(a_h (d2_n - m)) + a_h m with m the smallest
// squared distance in the union box (the reference subtracts each head's own minimum, models/kernels/
// real_enc_fwd.cu:87-143; the value of m does not change the result as long as no sum underflows).  Heads whose own
// box is smaller than the union mask the translations outside it; the masks cost FP32-pipe work only, while the
// loop is bound by the eight ex2 per term, so every thread runs the same code whatever its boxes are.
// Should a head's sum underflow (its box would have to miss the nearest image by hundreds of square Angstrom) it is
// redone with that head's own minimum.
static __device__ __noinline__ float head_phi_own_min(const Cell &cell, float rx, float ry, float rz, float a, int pk)
{
    const float F1 = (float)box_r1(pk), F2 = (float)box_r2(pk), F3 = (float)box_r3(pk);
    float m = 1e10f;
    for (float f1 = -F1; f1 <= F1; f1 += 1.0f)
        for (float f2 = -F2; f2 <= F2; f2 += 1.0f)
            for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
                const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx)));
                const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry)));
                const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz)));
                m = fminf(m, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
            }
    float sum = 0.f;
    const float a2 = a * LOG2E;
    for (float f1 = -F1; f1 <= F1; f1 += 1.0f)
        for (float f2 = -F2; f2 <= F2; f2 += 1.0f)
            for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
                const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx)));
                const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry)));
                const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz)));
                sum += ex2(a2 * (fmaf(dz, dz, fmaf(dy, dy, dx * dx)) - m));
            }
    return fmaf(m, a, logf(sum));
}

__device__ __forceinline__ void edge_phi(const BoxRule &rule, const float (&a)[8], const float *__restrict__ rvlen3,
                                         const Cell &cell, float rx, float ry, float rz, float (&z)[8])
{
    int pk[8];
    float a2[8], r1[8], r2[8], r3[8];
    int uni = 0;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        pk[h] = packed_box(rule, a[h], rvlen3);
        a2[h] = a[h] * LOG2E;
        uni = box_union(uni, pk[h]);
        r1[h] = (float)box_r1(pk[h]);
        r2[h] = (float)box_r2(pk[h]);
        r3[h] = (float)box_r3(pk[h]);
    }
    const float F1 = (float)box_r1(uni), F2 = (float)box_r2(uni), F3 = (float)box_r3(uni);
    float m = 1e10f;
    for (float f1 = -F1; f1 <= F1; f1 += 1.0f) {
        const float ax = fmaf(cell.t1x, f1, rx), ay = fmaf(cell.t1y, f1, ry), az = fmaf(cell.t1z, f1, rz);
        for (float f2 = -F2; f2 <= F2; f2 += 1.0f) {
            const float bx = fmaf(cell.t2x, f2, ax), by = fmaf(cell.t2y, f2, ay), bz = fmaf(cell.t2z, f2, az);
            for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
                const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
                m = fminf(m, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
            }
        }
    }
    float sum[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) sum[h] = 0.f;
    for (float f1 = -F1; f1 <= F1; f1 += 1.0f) {
        const float ax = fmaf(cell.t1x, f1, rx), ay = fmaf(cell.t1y, f1, ry), az = fmaf(cell.t1z, f1, rz);
        for (float f2 = -F2; f2 <= F2; f2 += 1.0f) {
            const float bx = fmaf(cell.t2x, f2, ax), by = fmaf(cell.t2y, f2, ay), bz = fmaf(cell.t2z, f2, az);
            float lim[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) lim[h] = (fabsf(f1) <= r1[h] && fabsf(f2) <= r2[h]) ? r3[h] : -1.0f;
            for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
                const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
                const float rel = fmaf(dz, dz, fmaf(dy, dy, dx * dx)) - m;
                const float af3 = fabsf(f3);
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float w = ex2(a2[h] * rel);
                    if (af3 <= lim[h]) sum[h] += w;
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        z[h] = fmaf(m, a[h], logf(sum[h]));
        if (!(sum[h] > 1e-30f)) z[h] = head_phi_own_min(cell, rx, ry, rz, a[h], pk[h]);
    }
}

// ---- lane <-> term ------------------------------------------------------------------------------------------------
// Walks flat term indices t, t+32, t+64, ... of a (rows x S1 x S2 x S3) mixed-radix space, S3 fastest, keeping the
// digits as small exact floats so that stepping costs a handful of FP32 adds and selects (no division, no conversion).
struct TermWalker {
    float u1, u2, u3;  // digits in [0,S1), [0,S2), [0,S3)
    int row;           // leading digit: which edge of the row (0 when a warp owns a single edge)
    float S1, S2, S3, d1, d2, d3;
    int drow;

    // start < 2^31: a row holds at most (atoms per crystal) x 65^3 terms
    __device__ __forceinline__ void init(int R1, int R2, int R3, unsigned start)
    {
        const unsigned s1 = 2 * R1 + 1, s2 = 2 * R2 + 1, s3 = 2 * R3 + 1;
        S1 = (float)s1; S2 = (float)s2; S3 = (float)s3;
        // digits of the stride 32
        unsigned q = 32u;
        d3 = (float)(q % s3); q /= s3;
        d2 = (float)(q % s2); q /= s2;
        d1 = (float)(q % s1); q /= s1;
        drow = (int)q;
        unsigned t = start;
        u3 = (float)(t % s3); t /= s3;
        u2 = (float)(t % s2); t /= s2;
        u1 = (float)(t % s1); t /= s1;
        row = (int)t;
    }
    __device__ __forceinline__ void step()
    {
        u3 += d3;
        const bool c3 = u3 >= S3;
        u3 -= c3 ? S3 : 0.f;
        u2 += d2 + (c3 ? 1.f : 0.f);
        const bool c2 = u2 >= S2;
        u2 -= c2 ? S2 : 0.f;
        u1 += d1 + (c2 ? 1.f : 0.f);
        const bool c1 = u1 >= S1;
        u1 -= c1 ? S1 : 0.f;
        row += drow + (c1 ? 1 : 0);
    }
};

// ---- lane <-> bins ------------------------------------------------------------------------------------------------
struct BasisParams {
    float bin_step;    // spacing of bin centres in basis units: sqrt(log2 e) / (sqrt2 wscale)
    float bin_scale;   // bin_step / mu0: distance -> basis units
    float d2_cut;      // squared distance beyond which every basis value underflows
    float floor_log2;  // terms whose largest log2-weight is below this are not accumulated
};

constexpr int STAGE_FLOATS = 32 * 12;  // per warp: 32 entries x (x, pad[3], w0..7); 16-byte aligned rows

// Accumulates sum_n w_h(n) g_k(d_n) for one warp.  Protocol per batch of 32 terms:
//   push(keep, x, w[8])    every lane offers its term; survivors are compacted into shared memory with a ballot,
//                          then all lanes sweep the staged entries (lanes <-> bins)
template <int K>
struct BinAccumulator {
    float acc[8][2];
    float c0, c1;
    float *stage;  // STAGE_FLOATS floats of this warp
    int lane;

    __device__ __forceinline__ void init(float *stage_, int lane_, const BasisParams &bp)
    {
        stage = stage_;
        lane = lane_;
        c0 = (float)(lane + 1) * bp.bin_step;
        c1 = (float)(lane + 33) * bp.bin_step;
#pragma unroll
        for (int h = 0; h < 8; ++h) acc[h][0] = acc[h][1] = 0.f;
    }
    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int h = 0; h < 8; ++h) acc[h][0] = acc[h][1] = 0.f;
    }

    // x = basis coordinate of the lane's term, w = its eight weights
    __device__ __forceinline__ void push(bool keep, float x, const float (&w)[8])
    {
        const unsigned mask = __ballot_sync(FULL, keep);
        if (mask == 0u) return;
        if (keep) {
            const int slot = __popc(mask & ((1u << lane) - 1u));
            float4 *row = reinterpret_cast<float4 *>(stage + 12 * slot);
            row[0] = make_float4(x, 0.f, 0.f, 0.f);
            row[1] = make_float4(w[0], w[1], w[2], w[3]);
            row[2] = make_float4(w[4], w[5], w[6], w[7]);
        }
        __syncwarp();
        const int cnt = __popc(mask);
#pragma unroll 2
        for (int m = 0; m < cnt; ++m) {
            const float4 *row = reinterpret_cast<const float4 *>(stage + 12 * m);
            const float x = row[0].x;
            const float4 wa = row[1], wb = row[2];
            const float t0 = c0 - x, t1 = c1 - x;
            const float g0 = ex2(-t0 * t0), g1 = ex2(-t1 * t1);
            acc[0][0] = fmaf(wa.x, g0, acc[0][0]); acc[0][1] = fmaf(wa.x, g1, acc[0][1]);
            acc[1][0] = fmaf(wa.y, g0, acc[1][0]); acc[1][1] = fmaf(wa.y, g1, acc[1][1]);
            acc[2][0] = fmaf(wa.z, g0, acc[2][0]); acc[2][1] = fmaf(wa.z, g1, acc[2][1]);
            acc[3][0] = fmaf(wa.w, g0, acc[3][0]); acc[3][1] = fmaf(wa.w, g1, acc[3][1]);
            acc[4][0] = fmaf(wb.x, g0, acc[4][0]); acc[4][1] = fmaf(wb.x, g1, acc[4][1]);
            acc[5][0] = fmaf(wb.y, g0, acc[5][0]); acc[5][1] = fmaf(wb.y, g1, acc[5][1]);
            acc[6][0] = fmaf(wb.z, g0, acc[6][0]); acc[6][1] = fmaf(wb.z, g1, acc[6][1]);
            acc[7][0] = fmaf(wb.w, g0, acc[7][0]); acc[7][1] = fmaf(wb.w, g1, acc[7][1]);
        }
        __syncwarp();
    }
};

// ---- phi kernel, shared by the per-edge operator and the fused attention (defined in lattice_sum_fwd.cu) -----------
struct PhiArgs {
    const float *a;          // (N,H), or (E,H) when a_per_edge
    const float *pos_ij;     // (E,3) relative positions, or NULL to take pos[j] - pos[i]
    const float *pos;        // (N,3), used when pos_ij is NULL
    const float *tvecs;      // (B,3,3)
    const int64_t *batch;    // (N)
    const int64_t *edges;    // (2,E)
    const float *rvlen;      // (B,3) or NULL
    float *z;                // (E,H) out
    long long E;
    BoxRule rule;
    int a_per_edge;
};
int launch_lattice_phi(const PhiArgs &p, cudaStream_t stream);

// Host-side derivation of the basis constants from the reference's parameters: bins k = 0..K-1 have centres
// (k+1) mu0 and width wscale mu0 with mu0 = dist_max / K (models/kernels/real_enc_fwd.cu:54-55,124-132).
inline BasisParams make_basis_params(long long K, double dist_max, double wscale, float floor_log2)
{
    BasisParams bp{};
    if (K > 0) {
        const double step = sqrt(1.4426950408889634) / (sqrt(2.0) * (double)(float)wscale);
        const double mu0 = (double)(float)dist_max / (double)K;
        bp.bin_step = (float)step;
        bp.bin_scale = (float)(step / mu0);
        const double x_cut = (double)K * step + 11.3;  // (x - K step)^2 > 126  =>  every basis value < 2^-126
        bp.d2_cut = (float)((x_cut / (step / mu0)) * (x_cut / (step / mu0)));
    }
    bp.floor_log2 = floor_log2;
    return bp;
}

}  // namespace cf
