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
    const float t = x * 0.15915494f;  // x / two_pi to within a few ulp
    int r = (int)ceilf(t);
    r = min(r, 1 << 20);
    // unless t is within 1e-4 (relative) of an integer the estimate is already the exact ceiling
    if ((float)r - t > 1e-4f * t + 1e-6f && t - (float)(r - 1) > 1e-4f * t + 1e-6f) return r;
    while ((double)r * two_pi < (double)x) ++r;
    while (r > 0 && (double)(r - 1) * two_pi >= (double)x) --r;
    return r;
}

// Half-widths of the box of one (atom, head), packed as R1 | R2 << 8 | R3 << 16.
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

// TPE threads (a power of two, consecutive lanes) share one edge: thread `sub` takes the (n1,n2) columns
// sub, sub + TPE, ... of the box and the partial minimum / sums are combined with shuffles.  More threads per edge
// give small batches enough warps to hide the latency of the per-term dependency chain.
// Inner loops over n3 for one (n1,n2) column; R3 = 2 (the usual minimum box) is fully unrolled.
template <bool UNROLL5>
__device__ __forceinline__ float column_min(const Cell &cell, float bx, float by, float bz, float F3, float m)
{
    if (UNROLL5) {
#pragma unroll
        for (int t = -2; t <= 2; ++t) {
            const float f3 = (float)t;
            const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
            m = fminf(m, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
        }
    } else {
        for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
            const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
            m = fminf(m, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
        }
    }
    return m;
}

__device__ __forceinline__ void term_sums(const float (&a2)[8], const float (&lim)[8], float a2max, float rel, float af3,
                                          float floor_log2, float (&sum)[8])
{
    // the term with d2 = m contributes 1 to every sum it belongs to, so a term whose largest weight is below the
    // floor (2^-30 by default) changes no sum by more than that fraction: skip its eight ex2
    if (a2max * rel > floor_log2) {
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float w = ex2(a2[h] * rel);
            if (af3 <= lim[h]) sum[h] += w;
        }
    }
}

// TPE threads (a power of two, consecutive lanes) share one edge: thread `sub` takes the (n1,n2) columns
// sub, sub + TPE, ... of the box and the partial minimum / sums are combined with shuffles.  More threads per edge
// give small batches enough warps to hide the latency of the per-term dependency chain.
template <int TPE>
__device__ __forceinline__ void edge_phi(const BoxRule &rule, const float (&a)[8], const float *__restrict__ rvlen3,
                                         const Cell &cell, float rx, float ry, float rz, float floor_log2, int sub,
                                         float (&z)[8])
{
    int pk[8];
    float a2[8];
    int uni = 0;
    float a2max = -INFINITY;  // the widest Gaussian of the eight: bounds every head's weight from above
    // the TPE threads of an edge split the eight box computations and exchange the results
    constexpr int PER = 8 / TPE;
    int mine[PER];
#pragma unroll
    for (int t = 0; t < PER; ++t) mine[t] = packed_box(rule, pick8(a, sub * PER + t), rvlen3);
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        pk[h] = TPE == 1 ? mine[h % PER] : __shfl_sync(FULL, mine[h % PER], h / PER, TPE);
        a2[h] = a[h] * LOG2E;
        a2max = fmaxf(a2max, a2[h]);
        uni = box_union(uni, pk[h]);
    }
    const float F1 = (float)box_r1(uni), F2 = (float)box_r2(uni), F3 = (float)box_r3(uni);
    const bool five = box_r3(uni) == 2;
    const float S2 = 2.0f * F2 + 1.0f;
    // column walk: (f1, f2) advances by TPE columns per step, f2 fastest
    float start1 = -F1, start2 = -F2 + (float)sub, step1 = 0.f, step2 = (float)TPE;
    while (start2 > F2) { start2 -= S2; start1 += 1.0f; }
    while (step2 >= S2) { step2 -= S2; step1 += 1.0f; }

    // A column (n1,n2) is the line b + n3 t3; no point of it is closer to the origin than the line itself, whose
    // squared distance is |b|^2 - (b.t3)^2 / |t3|^2.  Columns that cannot hold the minimum (pass 0) or a weight above
    // the floor (pass 1) are skipped as a whole.  The bound is shaved by 1e-4 relative + 1e-6 so that rounding can
    // only make it skip less.
    const float inv_t3sq = __frcp_rn(fmaf(cell.t3z, cell.t3z, fmaf(cell.t3y, cell.t3y, cell.t3x * cell.t3x)));
    float m = fmaf(rz, rz, fmaf(ry, ry, rx * rx));  // the n = 0 image belongs to every box
    for (float f1 = start1, f2 = start2; f1 <= F1;) {
        const float bx = fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx));
        const float by = fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry));
        const float bz = fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz));
        const float bt = fmaf(bz, cell.t3z, fmaf(by, cell.t3y, bx * cell.t3x));
        const float line2 = fmaf(bz, bz, fmaf(by, by, bx * bx)) - bt * bt * inv_t3sq;
        if (line2 * 0.9999f - 1e-6f <= m)
            m = five ? column_min<true>(cell, bx, by, bz, F3, m) : column_min<false>(cell, bx, by, bz, F3, m);
        f2 += step2; f1 += step1;
        if (f2 > F2) { f2 -= S2; f1 += 1.0f; }
    }
#pragma unroll
    for (int o = TPE / 2; o > 0; o >>= 1) m = fminf(m, __shfl_xor_sync(FULL, m, o));

    float sum[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) sum[h] = 0.f;
    for (float f1 = start1, f2 = start2; f1 <= F1;) {
        const float bx = fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx));
        const float by = fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry));
        const float bz = fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz));
        const float bt = fmaf(bz, cell.t3z, fmaf(by, cell.t3y, bx * cell.t3x));
        const float line2 = fmaf(bz, bz, fmaf(by, by, bx * bx)) - bt * bt * inv_t3sq;
        if (a2max * (line2 * 0.9999f - 1e-6f - m) <= floor_log2) {  // every term of the column is below the floor
            f2 += step2; f1 += step1;
            if (f2 > F2) { f2 -= S2; f1 += 1.0f; }
            continue;
        }
        const int i1 = abs(__float2int_rn(f1)), i2 = abs(__float2int_rn(f2));
        float lim[8];  // head h takes |n3| <= lim[h] in this column (-1: the column is outside its box)
#pragma unroll
        for (int h = 0; h < 8; ++h) lim[h] = (i1 <= box_r1(pk[h]) && i2 <= box_r2(pk[h])) ? (float)box_r3(pk[h]) : -1.0f;
        if (five) {
#pragma unroll
            for (int t = -2; t <= 2; ++t) {
                const float f3 = (float)t;
                const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
                term_sums(a2, lim, a2max, fmaf(dz, dz, fmaf(dy, dy, dx * dx)) - m, fabsf(f3), floor_log2, sum);
            }
        } else {
            for (float f3 = -F3; f3 <= F3; f3 += 1.0f) {
                const float dx = fmaf(cell.t3x, f3, bx), dy = fmaf(cell.t3y, f3, by), dz = fmaf(cell.t3z, f3, bz);
                term_sums(a2, lim, a2max, fmaf(dz, dz, fmaf(dy, dy, dx * dx)) - m, fabsf(f3), floor_log2, sum);
            }
        }
        f2 += step2; f1 += step1;
        if (f2 > F2) { f2 -= S2; f1 += 1.0f; }
    }
#pragma unroll
    for (int h = 0; h < 8; ++h) {
#pragma unroll
        for (int o = TPE / 2; o > 0; o >>= 1) sum[h] += __shfl_xor_sync(FULL, sum[h], o);
        z[h] = fmaf(m, a[h], logf(sum[h]));
        if (!(sum[h] > 1e-30f)) z[h] = head_phi_own_min(cell, rx, ry, rz, a[h], pk[h]);
    }
}

// d = sqrt(d2) by one rsqrt and one multiply (2 ulp), exact zero for d2 = 0.
__device__ __forceinline__ float fast_sqrt(float d2) { return d2 * rsqrt_fast(fmaxf(d2, 1e-35f)); }

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
        // digits of the stride 32 (same reciprocal trick: exact for these small integers)
        const unsigned q3s = (unsigned)__float2int_rd(32.5f * __frcp_rn(S3));
        d3 = (float)(32u - q3s * s3);
        const unsigned q2s = (unsigned)__float2int_rd(((float)q3s + 0.5f) * __frcp_rn(S2));
        d2 = (float)(q3s - q2s * s2);
        const unsigned q1s = (unsigned)__float2int_rd(((float)q2s + 0.5f) * __frcp_rn(S1));
        d1 = (float)(q2s - q1s * s1);
        drow = (int)q1s;
        if (start < 32u) {  // a lane index: at most two quotient digits are non-zero and they are tiny
            unsigned t = start;
            const unsigned q3 = (unsigned)__float2int_rd(((float)t + 0.5f) * __frcp_rn(S3));
            u3 = (float)(t - q3 * s3);
            const unsigned q2 = (unsigned)__float2int_rd(((float)q3 + 0.5f) * __frcp_rn(S2));
            u2 = (float)(q3 - q2 * s2);
            const unsigned q1 = (unsigned)__float2int_rd(((float)q2 + 0.5f) * __frcp_rn(S1));
            u1 = (float)(q2 - q1 * s1);
            row = (int)q1;
        } else {
            unsigned t = start;
            u3 = (float)(t % s3); t /= s3;
            u2 = (float)(t % s2); t /= s2;
            u1 = (float)(t % s1); t /= s1;
            row = (int)t;
        }
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

// ---- candidate ring ------------------------------------------------------------------------------------------------
// Most (edge, translation) terms of a large cell are far beyond the reach of every head's Gaussian.  A cheap upper
// bound on the largest log2-weight of a term (one FMA with the widest Gaussian and the key's largest offset) weeds
// them out BEFORE the eight per-head exponentials are spent: lanes <-> keys only computes d2 and the bound for FOUR
// translations at a time (independent dependency chains), survivors (d2, key) are appended to a 256-entry ring in
// shared memory, and the per-head work runs on full warps of 32 candidates taken from the ring.  `key` carries the
// key index in bits 0..10 and, when heads have different boxes, |n1|, |n2|, |n3| in bits 11..16, 17..22, 23..28.
constexpr int RING_ENTRIES = 256;  // >= 31 left over + 4 x 32 offered + slack, power of two
constexpr int RING_FLOATS = 2 * RING_ENTRIES;

__device__ __forceinline__ int pack_key(int j, int i1, int i2, int i3) { return j | (i1 << 11) | (i2 << 17) | (i3 << 23); }
__device__ __forceinline__ bool key_in_box(int key, int pk)
{
    return ((key >> 11) & 63) <= box_r1(pk) && ((key >> 17) & 63) <= box_r2(pk) && ((key >> 23) & 63) <= box_r3(pk);
}

struct CandidateRing {
    float2 *buf;
    int head, count, lane;
    __device__ __forceinline__ void init(float *storage, int lane_)
    {
        buf = reinterpret_cast<float2 *>(storage);
        head = count = 0;
        lane = lane_;
    }
    // Appends the lanes' candidates of four translations (in translation order, lanes ascending within each).
    // The caller keeps count < 32 before the call, so the ring cannot overflow.
    __device__ __forceinline__ void offer4(const bool (&cand)[4], const float (&d2)[4], const int (&key)[4])
    {
        unsigned m[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) m[u] = __ballot_sync(FULL, cand[u]);
        if ((m[0] | m[1] | m[2] | m[3]) == 0u) return;  // the common case for large cells: nobody in reach
        const unsigned lt = (1u << lane) - 1u;
        int at = head + count;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (cand[u]) buf[(at + __popc(m[u] & lt)) & (RING_ENTRIES - 1)] = make_float2(d2[u], __int_as_float(key[u]));
            at += __popc(m[u]);
        }
        count = at - head;
        __syncwarp();
    }
    // Appends the lanes' candidates of one step (lanes ascending).
    __device__ __forceinline__ void offer(bool cand, float d2, int key)
    {
        const unsigned mask = __ballot_sync(FULL, cand);
        if (mask == 0u) return;
        if (cand) buf[(head + count + __popc(mask & ((1u << lane) - 1u))) & (RING_ENTRIES - 1)] = make_float2(d2, __int_as_float(key));
        count += __popc(mask);
        __syncwarp();
    }
    __device__ __forceinline__ bool ready() const { return count >= 32; }
    // Hands one entry to each of the first min(count, 32) lanes; returns whether this lane got one.
    __device__ __forceinline__ bool take(float &d2, int &key)
    {
        const int n = min(count, 32);
        const float2 e = buf[(head + lane) & (RING_ENTRIES - 1)];
        d2 = e.x;
        key = __float_as_int(e.y);
        head = (head + n) & (RING_ENTRIES - 1);
        count -= n;
        __syncwarp();
        return lane < n;
    }
};

// ---- lane <-> bins ------------------------------------------------------------------------------------------------
struct BasisParams {
    float bin_step;    // spacing of bin centres in basis units: sqrt(log2 e) / (sqrt2 wscale)
    float bin_scale;   // bin_step / mu0: distance -> basis units
    float d2_cut;      // squared distance beyond which every basis value underflows
    float floor_log2;  // terms whose largest log2-weight is below this are not accumulated
    int windowed;      // 1: basis narrow enough for the three-window accumulation (see BinAccumulator)
};

constexpr int STAGE_FLOATS = 32 * 12;  // per warp: 32 entries x (x, pad[3], w0..7); 16-byte aligned rows

// Packed FP32 pair arithmetic of sm_100 (fma.rn.f32x2): one issue slot for two FMAs.
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }

// Accumulates sum_n w_h(n) g_k(d_n) for one warp.  Per batch of 32 terms, push(keep, x, w[8]): every lane offers its
// term; survivors are compacted into shared memory with ballots; then all lanes sweep the staged entries, each lane
// evaluating the basis at ITS bins and updating ITS accumulators for all eight heads (heads paired in f32x2 FMAs).
//
// Two bin layouts:
//   dense     lane owns bins (lane, lane+32): per entry 2 ex2 + 8 packed FMAs.
//   windowed  the basis is a Gaussian of one bin width, so at 8 bins from its centre it is below 2^-46.  The 64 bins
//             are covered by three overlapping 32-bin windows [0,32), [16,48), [32,64); an entry centred at bin xi
//             goes to the window that contains [xi-8, xi+8] (always one of the three), and a lane owns bin
//             16 w + lane in window w: per entry 1 ex2 + 4 packed FMAs, with 12 packed accumulators per lane.
//             Used when (8 bin_step)^2 >= 40, i.e. value_pe_width_scale <= 1.07; otherwise the dense layout.
// flush() adds the accumulators into a per-warp shared-memory tile [8][stride] of per-bin totals.
template <int K>
struct BinAccumulator {
    float2 acc[12];  // dense: [hp][bin slot] = acc[2 hp + slot]; windowed: [window][hp] = acc[4 window + hp]
    float c0, c1, c2;
    float *stage;    // STAGE_FLOATS floats of this warp
    int lane;
    bool windowed;
    float inv_step;

    __device__ __forceinline__ void init(float *stage_, int lane_, const BasisParams &bp)
    {
        stage = stage_;
        lane = lane_;
        windowed = bp.windowed != 0;
        inv_step = __frcp_rn(bp.bin_step);
        if (windowed) {
            c0 = (float)(lane + 1) * bp.bin_step;
            c1 = (float)(lane + 17) * bp.bin_step;
            c2 = (float)(lane + 33) * bp.bin_step;
        } else {
            c0 = (float)(lane + 1) * bp.bin_step;
            c1 = (float)(lane + 33) * bp.bin_step;
            c2 = 0.f;
        }
        clear();
    }
    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int t = 0; t < 12; ++t) acc[t] = make_float2(0.f, 0.f);
    }

    // x = basis coordinate of the lane's term, w = its eight weights
    __device__ __forceinline__ void push(bool keep, float x, const float (&w)[8])
    {
        const unsigned lt = (1u << lane) - 1u;
        if (windowed) {
            // window of the term: bin coordinate xi = x / step - 1; [xi-8, xi+8] lies in window 0 below 24, 1 below 40
            const float xi = fmaf(x, inv_step, -1.0f);
            const int win = (xi >= 24.0f) + (xi >= 40.0f);
            const unsigned m0 = __ballot_sync(FULL, keep && win == 0);
            const unsigned m1 = __ballot_sync(FULL, keep && win == 1);
            const unsigned m2 = __ballot_sync(FULL, keep && win == 2);
            if ((m0 | m1 | m2) == 0u) return;
            const int n0 = __popc(m0), n1 = __popc(m1), n2 = __popc(m2);
            if (keep) {
                const int slot = win == 0 ? __popc(m0 & lt) : (win == 1 ? n0 + __popc(m1 & lt) : n0 + n1 + __popc(m2 & lt));
                float4 *row = reinterpret_cast<float4 *>(stage + 12 * slot);
                row[0] = make_float4(x, 0.f, 0.f, 0.f);
                row[1] = make_float4(w[0], w[1], w[2], w[3]);
                row[2] = make_float4(w[4], w[5], w[6], w[7]);
            }
            __syncwarp();
            sweep_window(0, n0, c0, 0);
            sweep_window(n0, n0 + n1, c1, 4);
            sweep_window(n0 + n1, n0 + n1 + n2, c2, 8);
            __syncwarp();
        } else {
            const unsigned mask = __ballot_sync(FULL, keep);
            if (mask == 0u) return;
            if (keep) {
                const int slot = __popc(mask & lt);
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
                const float x_m = row[0].x;
                const float4 wa = row[1], wb = row[2];
                const float t0 = c0 - x_m, t1 = c1 - x_m;
                const float g0 = ex2(-t0 * t0), g1 = ex2(-t1 * t1);
                const float2 G0 = make_float2(g0, g0), G1 = make_float2(g1, g1);
                acc[0] = fma2(make_float2(wa.x, wa.y), G0, acc[0]); acc[1] = fma2(make_float2(wa.x, wa.y), G1, acc[1]);
                acc[2] = fma2(make_float2(wa.z, wa.w), G0, acc[2]); acc[3] = fma2(make_float2(wa.z, wa.w), G1, acc[3]);
                acc[4] = fma2(make_float2(wb.x, wb.y), G0, acc[4]); acc[5] = fma2(make_float2(wb.x, wb.y), G1, acc[5]);
                acc[6] = fma2(make_float2(wb.z, wb.w), G0, acc[6]); acc[7] = fma2(make_float2(wb.z, wb.w), G1, acc[7]);
            }
            __syncwarp();
        }
    }

    __device__ __forceinline__ void sweep_window(int begin, int end, float centre, int base)
    {
#pragma unroll 2
        for (int m = begin; m < end; ++m) {
            const float4 *row = reinterpret_cast<const float4 *>(stage + 12 * m);
            const float t = centre - row[0].x;
            const float4 wa = row[1], wb = row[2];
            const float g = ex2(-t * t);
            const float2 G = make_float2(g, g);
            acc[base + 0] = fma2(make_float2(wa.x, wa.y), G, acc[base + 0]);
            acc[base + 1] = fma2(make_float2(wa.z, wa.w), G, acc[base + 1]);
            acc[base + 2] = fma2(make_float2(wb.x, wb.y), G, acc[base + 2]);
            acc[base + 3] = fma2(make_float2(wb.z, wb.w), G, acc[base + 3]);
        }
    }

    // Writes the per-bin totals of this warp into tile[h * stride + k] (shared memory, overwritten).
    __device__ __forceinline__ void flush(float *tile, int stride)
    {
        if (windowed) {
#pragma unroll
            for (int hp = 0; hp < 4; ++hp) {
                tile[(2 * hp) * stride + lane] = acc[hp].x;
                tile[(2 * hp + 1) * stride + lane] = acc[hp].y;
                tile[(2 * hp) * stride + lane + 32] = acc[8 + hp].x;
                tile[(2 * hp + 1) * stride + lane + 32] = acc[8 + hp].y;
            }
            __syncwarp();
#pragma unroll
            for (int hp = 0; hp < 4; ++hp) {
                tile[(2 * hp) * stride + lane + 16] += acc[4 + hp].x;
                tile[(2 * hp + 1) * stride + lane + 16] += acc[4 + hp].y;
            }
        } else {
#pragma unroll
            for (int hp = 0; hp < 4; ++hp) {
                tile[(2 * hp) * stride + lane] = acc[2 * hp].x;
                tile[(2 * hp + 1) * stride + lane] = acc[2 * hp].y;
                tile[(2 * hp) * stride + lane + 32] = acc[2 * hp + 1].x;
                tile[(2 * hp + 1) * stride + lane + 32] = acc[2 * hp + 1].y;
            }
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
    float floor_log2;        // weights below 2^floor_log2 of the nearest image's are not summed
    int a_per_edge;
    unsigned *zero_word;  // optional: a word this launch sets to zero (the row ticket of the kernel that follows)
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
        bp.windowed = (K == 64 && (8.0 * step) * (8.0 * step) >= 40.0) ? 1 : 0;
    }
    bp.floor_log2 = floor_log2;
    return bp;
}

}  // namespace cf
