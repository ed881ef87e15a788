// Fused infinitely connected attention, forward, for batches of small crystals (at most 64 atoms per cell): one warp
// per atom row (the four warps of a block share a row whose list is long), the row's terms read from its
// distance-sorted row list (row_list.cuh), every sum over terms done as tensor-core products.
//
// For row i (head h, Gaussian parameter a_h < 0) over its listed terms t = (key j_t, squared distance d2_t):
//     e_th   = exp2( a_h log2e d2_t + s_h[j_t] - M_h )          s_h[j] = q_i.k_j log2e,  M_h = max_j (s_h[j] + a_h log2e dmin_j)
//     P_h[j] = sum_{t : j_t = j} e_th                           (un-normalised p_ij)
//     Psi_h[k] = sum_t e_th g_k(d_t)                            (un-normalised radial-basis histogram)
//     out_i  = ( sum_j P_h[j] v_j + W_h Psi_h ) / sum_j P_h[j],   lse_ih = (M_h + log2 sum_j P_h[j]) ln 2
// M_h bounds every exponent from above (a < 0, d2 >= dmin), so no weight overflows and no separate pass for the
// soft-max statistics is needed: phi, the soft-max and the histogram come out of ONE sweep over the row's entries.
//
// A chunk of eight consecutive entries is one k-step of mma.m16n8k8 (TF32 operands, FP32 accumulators in registers):
//     Psi^T tile [16 bins x 8 heads] += G [16 bins x 8 terms] . E [8 terms x 8 heads]
//     P^T tile   [16 keys x 8 heads] += 1[j_t = key] [16 keys x 8 terms] . E
// Every lane computes its fragment elements directly in registers: lane (g = lane / 4, t = lane % 4) owns the terms
// t and t + 4 of the chunk for head g (two exponentials: the B fragment) and bins g, g + 8 of a tile for the same two
// terms (four exponentials: the A fragment).  FP32-level accuracy from TF32 products by splitting both operands into a
// rounded high part and the exact remainder (three products; the one-hot operand of P is exact, two products).
// Because the entries are sorted by distance a chunk touches only the one or two bin tiles around its distances, and
// the sweep ends at the first chunk whose entries are below the weight floor for every head.
//
// Rows without a list, rows of more than 16 NT keys and rows where a head's sum comes out empty are appended to the
// left-over list and processed by the enumerating row kernel (infinite_attn_fwd.cu) afterwards.  Without a radial
// basis (K = 0: PSI = false) the histogram, its tiles and the projection W drop out; the rest is the same (the
// one-call forwards do not use that variant: there the enumerating kernel with term lists is faster).
#include "lattice_core.cuh"
#include "row_list.cuh"

namespace cf {
namespace {

constexpr int SR_THREADS = 128;
constexpr int SR_WARPS = SR_THREADS / 32;
constexpr int PSI_LD = 68;    // leading dimension of the histogram tile (heads x 64 bins): 4-bank shift per head
constexpr int RING_SLOTS = 3; // groups of eight chunks staged per warp
constexpr int CHANNELS = HEADS * HEAD_DIM;

struct SortedRowArgs {
    const float *q, *k, *v, *a, *rvlen, *W;
    const int4 *rowdir;
    const float *dmin;
    const float2 *pool;
    const int *tasks;              // [2][N]: slots of the shared rows, of the one-warp rows
    const unsigned *task_count;    // [2]
    unsigned *sched;               // { ticket of the shared rows, rows left over, -, ticket of the one-warp rows }
    int *leftover;
    float *out, *lse;
    long long N;
    BoxRule rule;
    float bin_step;      // spacing of bin centres in basis units
    float bin_scale;     // distance -> basis units
    float inv_bin_step;
    float tile_reach;    // bins beyond which a basis value is below the floor
    float floor_log2;
    unsigned long long *stats;  // optional: { chunks swept, (chunk, bin tile) pairs computed, rows } are added here
};

__device__ __forceinline__ void mma_tf32(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1)
{
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x = hi + lo with hi = x cut to the TF32 grid (10 mantissa bits) and lo the exact remainder (0 <= lo < 2^-10 x for the
// non-negative values split here); products of such pairs, hi.hi + lo.hi + hi.lo, are within 2^-19 of x.y
__device__ __forceinline__ void split_tf32(float x, unsigned &hi, unsigned &lo)
{
    hi = __float_as_uint(x) & 0xffffe000u;
    lo = __float_as_uint(x - __uint_as_float(hi));
}

// max over the warp of eight per-lane values, one per head, with nine shuffles: the lanes trade halves of their value
// sets across lane bits 4, 3, 2 (keeping the heads whose index bits match their own), then finish over bits 1, 0.
// Lane l ends with the maximum of head l / 4.
__device__ __forceinline__ float warp_max_heads(const float (&v)[8], int lane)
{
    const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0, b2 = (lane & 4) != 0;
    float w4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
        const float keep = b4 ? v[4 + u] : v[u], send = b4 ? v[u] : v[4 + u];
        w4[u] = fmaxf(keep, __shfl_xor_sync(FULL, send, 16));
    }
    float w2[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
        const float keep = b3 ? w4[2 + u] : w4[u], send = b3 ? w4[u] : w4[2 + u];
        w2[u] = fmaxf(keep, __shfl_xor_sync(FULL, send, 8));
    }
    const float keep = b2 ? w2[1] : w2[0], send = b2 ? w2[0] : w2[1];
    float r = fmaxf(keep, __shfl_xor_sync(FULL, send, 4));
    r = fmaxf(r, __shfl_xor_sync(FULL, r, 2));
    r = fmaxf(r, __shfl_xor_sync(FULL, r, 1));
    return r;
}

// Shared memory of one thread block (NT key tiles of 16; PSI: with the radial basis).
template <int NT, bool PSI>
struct SortedSmem {
    static constexpr int CJ_LD = 16 * NT + 1;  // leading dimension of the per-(head, key) tables (odd: no bank conflicts)
    float wt[PSI ? 64 * CHANNELS : 4];    // W transposed: wt[k][channel], staged once per block
    float cj[SR_WARPS][8 * CJ_LD];        // s_h[j] per (head, key); a block working on one row uses table 0
    float pj[SR_WARPS][8 * CJ_LD];        // P_h[j]
    float psi[SR_WARPS][PSI ? 8 * PSI_LD : 4];  // Psi_h[k]
    float2 ring[SR_WARPS][RING_SLOTS][64];  // list entries, 8 chunks (512 bytes) per slot
    long long next_task;
};

// One row.  COOP = false: the calling warp processes the whole row on its own (only warp-level synchronisation).
// COOP = true: the four warps of the block share the row - the keys of the q.k table, then the row's chunks dealt
// round-robin, every warp with its own accumulators; the partial histograms meet in shared memory and every thread
// finishes one output channel.  Returns false if the row must be left over.
template <int NT, bool COOP, bool PSI>
__device__ __forceinline__ bool sorted_row(const SortedRowArgs &p, SortedSmem<NT, PSI> &sm, const int4 r0, const int4 r1, int warp, int lane)
{
    constexpr int CJ_LD = SortedSmem<NT, PSI>::CJ_LD;
    const int g = lane >> 2, t = lane & 3;
    auto sync = [&]() {
        if (COOP) __syncthreads(); else __syncwarp();
    };
    const int i = r0.x, a0 = r0.y, n = r0.z, c = r0.w;
    const int start = r1.x, chunks = r1.y, e0 = r1.z;
    if (start < 0 || n < 1 || n > 16 * NT) return false;
    float *cj = sm.cj[COOP ? 0 : warp], *pj = sm.pj[warp], *psi = sm.psi[warp];
    float2 (*ring)[64] = sm.ring[warp];

    // ---- the entries stream into shared memory ahead of their use, eight chunks (64 entries, 512 bytes) per group:
    //      a lane copies 16 bytes, four lanes a chunk.  A warp on its own takes consecutive chunks; a warp that shares
    //      the row takes the chunks warp, warp + 4, ...  RING_SLOTS - 1 groups are in flight while one is processed.
    const int my_chunks = COOP ? (chunks - warp + SR_WARPS - 1) / SR_WARPS : chunks;  // (<= 0: none)
    const int groups = (my_chunks + 7) >> 3;
    const float2 *ent = p.pool + start;
    auto fetch = [&](int grp, int ring_slot) {
        const int mine = 8 * grp + (lane >> 2);  // which of this warp's chunks the lane copies a quarter of
        if (grp < groups && mine < my_chunks) {
            const int chunk = COOP ? mine * SR_WARPS + warp : mine;
            const unsigned dst = (unsigned)__cvta_generic_to_shared(&ring[ring_slot][2 * lane]);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(ent + 8 * chunk + 2 * (lane & 3)));
        }
        asm volatile("cp.async.commit_group;");
    };
#pragma unroll
    for (int u = 0; u < RING_SLOTS - 1; ++u) fetch(u, u);

    // ---- the row's constants
    const float4 a_lo = __ldg(reinterpret_cast<const float4 *>(p.a + (size_t)i * HEADS));
    const float4 a_hi = __ldg(reinterpret_cast<const float4 *>(p.a + (size_t)i * HEADS) + 1);
    const float4 q4 = __ldg(reinterpret_cast<const float4 *>(p.q + (size_t)i * CHANNELS) + lane);
    const float dm = lane < n ? __ldg(p.dmin + e0 + lane) : 0.f;
    const float dm2 = (NT > 2 && lane + 32 < n) ? __ldg(p.dmin + e0 + lane + 32) : 0.f;  // keys 32 .. 63
    float rvl[3] = {0.f, 0.f, 0.f};
    if (p.rvlen) { rvl[0] = __ldg(p.rvlen + 3 * c); rvl[1] = __ldg(p.rvlen + 3 * c + 1); rvl[2] = __ldg(p.rvlen + 3 * c + 2); }

    // ---- s_h[j] = q.k_j log2e: a key's 512-byte row is one coalesced read of the warp (lane l: channels
    //      4 l .. 4 l + 3, i.e. head l / 4 = g); the four lanes of a head add their partial dot products.  The rows of
    //      the next four keys are requested before the current four are used.
    {
        const float4 *kp = reinterpret_cast<const float4 *>(p.k + (size_t)a0 * CHANNELS) + lane;
        constexpr int JSTEP = COOP ? 4 * SR_WARPS : 4;
        int j0 = COOP ? 4 * warp : 0;
        float4 cur[4], nxt[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) cur[u] = j0 < n ? __ldg(kp + (size_t)min(j0 + u, n - 1) * 32) : make_float4(0.f, 0.f, 0.f, 0.f);
        while (j0 < n) {
            const int jn = j0 + JSTEP;
#pragma unroll
            for (int u = 0; u < 4; ++u) nxt[u] = jn < n ? __ldg(kp + (size_t)min(jn + u, n - 1) * 32) : cur[u];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float s = fmaf(q4.w, cur[u].w, fmaf(q4.z, cur[u].z, fmaf(q4.y, cur[u].y, q4.x * cur[u].x)));
                s += __shfl_xor_sync(FULL, s, 1);
                s += __shfl_xor_sync(FULL, s, 2);
                if (t == 0 && j0 + u < n) cj[g * CJ_LD + j0 + u] = s * LOG2E;
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) cur[u] = nxt[u];
            j0 = jn;
        }
    }
    const float a8[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
    const float a_g = pick8(a8, g);
    const float a2g = a_g * LOG2E;
    const unsigned boxor = (unsigned)packed_box(p.rule, a_g, p.rvlen ? rvl : nullptr) | 0x808080u;
    sync();
    // ---- M_h and the slack max_j s_h[j] - M_h (how far above its bound a term of distance d2 can be)
    float M_g, slack_g;
    {
        float m8[8], s8[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float s = lane < n ? cj[h * CJ_LD + lane] : -INFINITY;
            s8[h] = s;
            m8[h] = fmaf(a8[h] * LOG2E, dm, s);
            if (NT > 2) {  // (a lane looks after keys lane and lane + 32)
                const float s2 = lane + 32 < n ? cj[h * CJ_LD + lane + 32] : -INFINITY;
                s8[h] = fmaxf(s8[h], s2);
                m8[h] = fmaxf(m8[h], fmaf(a8[h] * LOG2E, dm2, s2));
            }
        }
        M_g = warp_max_heads(m8, lane);
        slack_g = warp_max_heads(s8, lane) - M_g;
    }

    // ---- the sweep: two chunks per step (their instruction streams are independent up to the accumulators)
    float accP[NT][4], accPsi[4][4];
#pragma unroll
    for (int u = 0; u < NT; ++u) accP[u][0] = accP[u][1] = accP[u][2] = accP[u][3] = 0.f;
#pragma unroll
    for (int m = 0; m < 4; ++m) accPsi[m][0] = accPsi[m][1] = accPsi[m][2] = accPsi[m][3] = 0.f;
    const float *cjg = cj + g * CJ_LD;
    const float ucg = (float)(g + 1) * p.bin_step;          // centre of bin g in basis units
    const float step16 = 16.0f * p.bin_step, step8 = 8.0f * p.bin_step;
    bool more = true;
    int ring_slot = 0;
    int swept = 0, tiles_done = 0;  // diagnostics (p.stats)
    for (int grp = 0; grp < groups && more; ++grp) {
        int ahead = ring_slot + RING_SLOTS - 1;
        if (ahead >= RING_SLOTS) ahead -= RING_SLOTS;
        fetch(grp + RING_SLOTS - 1, ahead);
        asm volatile("cp.async.wait_group %0;" ::"n"(RING_SLOTS - 1) : "memory");
        __syncwarp();
        const float2 *stage = ring[ring_slot];
        const int in_group = min(8, my_chunks - 8 * grp);
        for (int ch = 0; ch < in_group; ch += 2) {
            const bool two = ch + 1 < in_group;
            const float2 e0a = stage[8 * ch + t], e0b = stage[8 * ch + t + 4];
            const float2 e1a = stage[8 * (ch + (two ? 1 : 0)) + t], e1b = stage[8 * (ch + (two ? 1 : 0)) + t + 4];
            // entries ascend in d2: once a chunk's first entry is below the floor for every head, all that follow are
            const float d2_first = __shfl_sync(FULL, e0a.x, 0);
            if (__all_sync(FULL, fmaf(a2g, d2_first, slack_g) < p.floor_log2)) { more = false; break; }
            const float d2v[4] = {e0a.x, e0b.x, e1a.x, e1b.x};
            const int keyv[4] = {__float_as_int(e0a.y), __float_as_int(e0b.y), __float_as_int(e1a.y), __float_as_int(e1b.y)};
            // B fragments: the weights of terms t, t + 4 of either chunk for head g
            unsigned w_hi[4], w_lo[4];
            int dj[4];
            float x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int j = keyv[u] & 255;
                float w = ex2(fmaf(a2g, d2v[u], cjg[j]) - M_g);
                w = (row_key_in_box(keyv[u], boxor) && (u < 2 || two)) ? w : 0.f;
                split_tf32(w, w_hi[u], w_lo[u]);
                dj[u] = j - g;
                if (PSI) x[u] = d2v[u] * rsqrt_fast(fmaxf(d2v[u], 1e-35f)) * p.bin_scale;  // basis coordinate of the term
            }
            // P^T tiles: one-hot of the terms' keys (rows g, g + 8 of tile u are keys 16 u + g, 16 u + g + 8)
#pragma unroll
            for (int u = 0; u < NT; ++u) {
                unsigned o[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    o[2 * e] = dj[e] == 16 * u ? 0x3f800000u : 0u;
                    o[2 * e + 1] = dj[e] == 16 * u + 8 ? 0x3f800000u : 0u;
                }
                mma_tf32(accP[u], o[0], o[1], o[2], o[3], w_hi[0], w_hi[1]);
                mma_tf32(accP[u], o[0], o[1], o[2], o[3], w_lo[0], w_lo[1]);
                mma_tf32(accP[u], o[4], o[5], o[6], o[7], w_hi[2], w_hi[3]);
                mma_tf32(accP[u], o[4], o[5], o[6], o[7], w_lo[2], w_lo[3]);
            }
            swept += two ? 2 : 1;
            if (PSI) {
            // the bin tiles the two chunks can reach
            const float x_first = __shfl_sync(FULL, x[0], 0), x_last = __shfl_sync(FULL, x[3], 3);
            const float b_lo = fmaf(x_first, p.inv_bin_step, -1.0f - p.tile_reach);
            const float b_hi = fmaf(x_last, p.inv_bin_step, -1.0f + p.tile_reach);
            const int m_lo = max(0, __float2int_rd(b_lo * 0.0625f));
            const int m_hi = b_hi < 0.0f ? -1 : min(3, __float2int_rd(b_hi * 0.0625f));  // (beyond the last bin: only phi needs the terms)
            const float uu[4] = {x[0] - ucg, x[1] - ucg, x[2] - ucg, x[3] - ucg};
            tiles_done += max(m_hi - m_lo + 1, 0) * (two ? 2 : 1);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                if (m < m_lo || m > m_hi) continue;  // (the same for every lane)
                // A fragments: g_k(d) = exp2(-(c_k - x)^2) at bins 16 m + g, 16 m + g + 8 for the four terms
                unsigned hi[8], lo[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v0 = fmaf(-(float)m, step16, uu[e]), v1 = v0 - step8;
                    split_tf32(ex2(-v0 * v0), hi[2 * e], lo[2 * e]);
                    split_tf32(ex2(-v1 * v1), hi[2 * e + 1], lo[2 * e + 1]);
                }
                mma_tf32(accPsi[m], hi[0], hi[1], hi[2], hi[3], w_hi[0], w_hi[1]);
                mma_tf32(accPsi[m], lo[0], lo[1], lo[2], lo[3], w_hi[0], w_hi[1]);
                mma_tf32(accPsi[m], hi[0], hi[1], hi[2], hi[3], w_lo[0], w_lo[1]);
                mma_tf32(accPsi[m], hi[4], hi[5], hi[6], hi[7], w_hi[2], w_hi[3]);
                mma_tf32(accPsi[m], lo[4], lo[5], lo[6], lo[7], w_hi[2], w_hi[3]);
                mma_tf32(accPsi[m], hi[4], hi[5], hi[6], hi[7], w_lo[2], w_lo[3]);
            }
            }
        }
        __syncwarp();  // every lane is done with the slot before a later fetch overwrites it
        if (++ring_slot == RING_SLOTS) ring_slot = 0;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");  // fetches still in flight after an early end
    if (p.stats != nullptr && lane == 0) {
        atomicAdd(p.stats, (unsigned long long)swept);
        atomicAdd(p.stats + 1, (unsigned long long)tiles_done);
        if (!COOP || warp == 0) atomicAdd(p.stats + 2, 1ull);
    }

    // ---- accumulators -> shared memory (C fragment: rows g, g + 8; columns = heads 2 t, 2 t + 1)
    __syncwarp();
#pragma unroll
    for (int m = 0; m < (PSI ? 4 : 0); ++m) {
        psi[(2 * t) * PSI_LD + 16 * m + g] = accPsi[m][0];
        psi[(2 * t + 1) * PSI_LD + 16 * m + g] = accPsi[m][1];
        psi[(2 * t) * PSI_LD + 16 * m + g + 8] = accPsi[m][2];
        psi[(2 * t + 1) * PSI_LD + 16 * m + g + 8] = accPsi[m][3];
    }
#pragma unroll
    for (int u = 0; u < NT; ++u) {
        pj[(2 * t) * CJ_LD + 16 * u + g] = accP[u][0];
        pj[(2 * t + 1) * CJ_LD + 16 * u + g] = accP[u][1];
        pj[(2 * t) * CJ_LD + 16 * u + g + 8] = accP[u][2];
        pj[(2 * t + 1) * CJ_LD + 16 * u + g + 8] = accP[u][3];
    }
    sync();
    if (COOP) {
        // ---- the four partial tables are added in a fixed order; one output channel per thread
        const int tid = 32 * warp + lane;
        for (int idx = tid; idx < (PSI ? 8 * PSI_LD : 0); idx += SR_THREADS)
            sm.psi[0][idx] = (sm.psi[0][idx] + sm.psi[1][idx]) + (sm.psi[2][idx] + sm.psi[3][idx]);
        for (int idx = tid; idx < 8 * CJ_LD; idx += SR_THREADS)
            sm.pj[0][idx] = (sm.pj[0][idx] + sm.pj[1][idx]) + (sm.pj[2][idx] + sm.pj[3][idx]);
        __syncthreads();
        const int h = tid >> 4;
        const float *pg = sm.pj[0] + h * CJ_LD;
        const float *vp = p.v + (size_t)a0 * CHANNELS + tid;
        float acc = 0.f, S = 0.f;
        for (int j0 = 0; j0 < n; j0 += 8) {
            float vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) vv[u] = __ldg(vp + (size_t)min(j0 + u, n - 1) * CHANNELS);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float pw = j0 + u < n ? pg[j0 + u] : 0.f;
                acc = fmaf(pw, vv[u], acc);
                S += pw;
            }
        }
        const bool failed = __syncthreads_or(!(S > 1e-30f));  // a head without a single listed term inside its box
        if (failed) return false;
        const float *ps = sm.psi[0] + h * PSI_LD;
        float o0 = 0.f, o1 = 0.f;
#pragma unroll 8
        for (int k4 = 0; k4 < (PSI ? 64 : 0); k4 += 4) {
            const float4 pv = *reinterpret_cast<const float4 *>(ps + k4);
            o0 = fmaf(sm.wt[(k4 + 0) * CHANNELS + tid], pv.x, o0);
            o1 = fmaf(sm.wt[(k4 + 1) * CHANNELS + tid], pv.y, o1);
            o0 = fmaf(sm.wt[(k4 + 2) * CHANNELS + tid], pv.z, o0);
            o1 = fmaf(sm.wt[(k4 + 3) * CHANNELS + tid], pv.w, o1);
        }
        p.out[(size_t)i * CHANNELS + tid] = (acc + (o0 + o1)) * __frcp_rn(S);
        const float M_h = __shfl_sync(FULL, M_g, 4 * (h & 7));  // (every warp holds the same bounds: head g in lanes 4 g ..)
        if ((tid & 15) == 0) p.lse[(size_t)i * HEADS + h] = (M_h + log2f(S)) * LN2;
        return true;
    } else {
        // ---- sum_j P_g[j] v_j and S_g = sum_j P_g[j]: lane l owns channels 4 l .. 4 l + 3 (head g)
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float S = 0.f;
        const float4 *vp = reinterpret_cast<const float4 *>(p.v + (size_t)a0 * CHANNELS) + lane;
        const float *pg = pj + g * CJ_LD;
        for (int j0 = 0; j0 < n; j0 += 8) {
            float4 vv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) vv[u] = __ldg(vp + (size_t)min(j0 + u, n - 1) * 32);
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float pw = j0 + u < n ? pg[j0 + u] : 0.f;
                acc.x = fmaf(pw, vv[u].x, acc.x); acc.y = fmaf(pw, vv[u].y, acc.y);
                acc.z = fmaf(pw, vv[u].z, acc.z); acc.w = fmaf(pw, vv[u].w, acc.w);
                S += pw;
            }
        }
        if (__any_sync(FULL, !(S > 1e-30f))) return false;  // a head without a single listed term inside its box
        // ---- W_g Psi_g for the lane's four channels 4 l .. 4 l + 3 (head g): W transposed in shared memory, so a
        //      warp reads 512 consecutive bytes per bin
        const float4 *wt4 = reinterpret_cast<const float4 *>(sm.wt) + lane;
        const float *ps = psi + g * PSI_LD;
        float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
        for (int k4 = 0; k4 < (PSI ? 64 : 0); k4 += 4) {
            const float4 pv = *reinterpret_cast<const float4 *>(ps + k4);
            const float pk[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const float4 wv = wt4[(k4 + u) * (CHANNELS / 4)];
                o.x = fmaf(wv.x, pk[u], o.x); o.y = fmaf(wv.y, pk[u], o.y); o.z = fmaf(wv.z, pk[u], o.z); o.w = fmaf(wv.w, pk[u], o.w);
            }
        }
        const float inv = __frcp_rn(S);
        reinterpret_cast<float4 *>(p.out + (size_t)i * CHANNELS)[lane] =
            make_float4((acc.x + o.x) * inv, (acc.y + o.y) * inv, (acc.z + o.z) * inv, (acc.w + o.w) * inv);
        if (t == 0) p.lse[(size_t)i * HEADS + g] = (M_g + log2f(S)) * LN2;
        __syncwarp();
        return true;
    }
}

// The build sorts the rows into two task lists.  Rows with long lists are processed first, one at a time by a whole
// block (block b starts with task b, further tasks come through an atomic ticket); when they are used up every warp
// takes rows of the second list on its own, again the first by position and the rest through a ticket.  Which warps
// compute a row has no influence on which terms are summed, and the choice between the two organisations depends on
// the row's list alone, so results are repeatable bit for bit.
template <int NT, bool PSI>
__global__ void __launch_bounds__(SR_THREADS, NT > 2 ? 3 : 4) infinite_attn_sorted_rows_kernel(const SortedRowArgs p)
{
    extern __shared__ __align__(16) unsigned char sorted_smem_raw[];
    SortedSmem<NT, PSI> &sm = *reinterpret_cast<SortedSmem<NT, PSI> *>(sorted_smem_raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_launch_dependents();
    // W (8,16,64) -> wt[k][channel]: thread = channel, 256 contiguous bytes read, 64 conflict-free stores (W is a
    // constant: in a chained launch this runs while the kernel before this one drains)
    if (PSI) {
        const float4 *src = reinterpret_cast<const float4 *>(p.W + (size_t)tid * 64);
#pragma unroll 4
        for (int k4 = 0; k4 < 16; ++k4) {
            const float4 w = __ldg(src + k4);
            sm.wt[(4 * k4 + 0) * CHANNELS + tid] = w.x;
            sm.wt[(4 * k4 + 1) * CHANNELS + tid] = w.y;
            sm.wt[(4 * k4 + 2) * CHANNELS + tid] = w.z;
            sm.wt[(4 * k4 + 3) * CHANNELS + tid] = w.w;
        }
    }
    grid_dependency_wait();  // q, k, v, a of the dense block before this kernel; its reads of `out` are over
    const long long n_shared = __ldg(p.task_count), n_single = __ldg(p.task_count + 1);
    // ---- rows shared by the block
    long long task = blockIdx.x;
    while (task < n_shared) {
        __syncthreads();  // W is staged; the previous row's readers are done with the tables and with next_task
        unsigned drawn = 0;
        if (tid == 0) drawn = atomicAdd(p.sched, 1u);  // (needed only after the row)
        const int slot = __ldg(p.tasks + task);
        const int4 r0 = __ldg(p.rowdir + 2 * (long long)slot), r1 = __ldg(p.rowdir + 2 * (long long)slot + 1);
        if (!sorted_row<NT, true, PSI>(p, sm, r0, r1, warp, lane) && tid == 0) p.leftover[atomicAdd(p.sched + 1, 1u)] = r0.x;
        if (tid == 0) sm.next_task = (long long)gridDim.x + drawn;
        __syncthreads();
        task = sm.next_task;
    }
    __syncthreads();
    // ---- rows of one warp each
    task = (long long)blockIdx.x * SR_WARPS + warp;
    const long long first_wave = (long long)gridDim.x * SR_WARPS;
    while (task < n_single) {
        unsigned drawn = 0;
        if (lane == 0) drawn = atomicAdd(p.sched + 3, 1u);
        const int slot = __ldg(p.tasks + p.N + task);
        const int4 r0 = __ldg(p.rowdir + 2 * (long long)slot), r1 = __ldg(p.rowdir + 2 * (long long)slot + 1);
        if (!sorted_row<NT, false, PSI>(p, sm, r0, r1, warp, lane) && lane == 0) p.leftover[atomicAdd(p.sched + 1, 1u)] = r0.x;
        task = first_wave + __shfl_sync(FULL, drawn, 0);
    }
}

}  // namespace

int launch_sorted_rows(const SortedRowLaunch &l, cudaStream_t s)
{
    if (l.N == 0) return CF_OK;
    SortedRowArgs p{};
    p.q = l.q; p.k = l.k; p.v = l.v; p.a = l.a; p.rvlen = l.rvlen; p.W = l.W;
    p.rowdir = l.view.rowdir; p.dmin = l.view.dmin; p.pool = l.view.pool;
    p.tasks = l.view.tasks; p.task_count = l.view.task_count;
    p.sched = l.sched; p.leftover = l.view.leftover;
    p.out = l.out; p.lse = l.lse; p.N = l.N; p.rule = l.rule;
    const BasisParams bp = make_basis_params(64, l.dist_max > 0 ? l.dist_max : 1.0, l.wscale > 0 ? l.wscale : 1.0, weight_floor_log2());
    p.bin_step = bp.bin_step; p.bin_scale = bp.bin_scale; p.inv_bin_step = 1.0f / bp.bin_step;
    // a basis value exp2(-(step * bins)^2) is below the weight floor beyond sqrt(-floor) / step bins (floor clipped to
    // [2^-126, 2^-24]: with the floor switched off the whole float range is kept)
    const float fl = fminf(fmaxf(-weight_floor_log2(), 24.0f), 126.0f);
    p.tile_reach = sqrtf(fl) / bp.bin_step;
    p.floor_log2 = weight_floor_log2();
    p.stats = row_stats_words();
    // key tiles: 1, 2 or 4 (16, 32, 64 keys); with or without the radial basis
    const int variant = (l.max_atoms <= 16 ? 0 : l.max_atoms <= 32 ? 1 : 2) + (l.K > 0 ? 0 : 3);
    void (*kernel)(const SortedRowArgs) = nullptr;
    size_t smem = 0;
    switch (variant) {
    case 0: kernel = infinite_attn_sorted_rows_kernel<1, true>; smem = sizeof(SortedSmem<1, true>); break;
    case 1: kernel = infinite_attn_sorted_rows_kernel<2, true>; smem = sizeof(SortedSmem<2, true>); break;
    case 2: kernel = infinite_attn_sorted_rows_kernel<4, true>; smem = sizeof(SortedSmem<4, true>); break;
    case 3: kernel = infinite_attn_sorted_rows_kernel<1, false>; smem = sizeof(SortedSmem<1, false>); break;
    case 4: kernel = infinite_attn_sorted_rows_kernel<2, false>; smem = sizeof(SortedSmem<2, false>); break;
    default: kernel = infinite_attn_sorted_rows_kernel<4, false>; smem = sizeof(SortedSmem<4, false>); break;
    }
    static thread_local bool configured[64][6] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    bool &done = configured[dev & 63][variant];
    if (!done) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return fail(CF_ERR_CUDA, "sorted row kernel: %zu bytes of shared memory not available", smem);
        }
        done = true;
    }
    const long long cap = (long long)sm_count() * (l.max_atoms > 32 ? 3 : 4);
    const unsigned blocks = (unsigned)(l.N < cap ? l.N : cap);
    launch_chained(kernel, dim3(blocks), dim3(SR_THREADS), smem, s, l.chained, p);
    return launch_status("infinite_attn_sorted_rows_kernel");
}

}  // namespace cf

namespace cf {
int launch_leftover_rows(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                         const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                         const int64_t *row_start, int64_t N, int64_t E, int64_t max_atoms, double dist_max,
                         double wscale, const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                         float *out, float *lse, const int *rows, const unsigned *count, unsigned *ticket, int64_t K,
                         cudaStream_t s);

// One attention call over a batch's row lists: the sorted row kernel, then the enumerating row kernel for whatever it
// left over (normally nothing: that launch then finds a zero count and returns).  sched_slot: which of the
// ROW_SCHED_SLOTS scheduling blocks to use; `zeroed`: the block is still zero from the build (each block serves one
// call per build), otherwise it is cleared here first.
int sorted_attn_impl(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                     const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                     const int64_t *row_start, int64_t N, int64_t E, int64_t max_atoms, double dist_max, double wscale,
                     const float *W, double cutoff_radius, int lattice_range, int minimum_range, float *out, float *lse,
                     const RowListView &view, int sched_slot, bool zeroed, int64_t K, cudaStream_t s)
{
    // (chained launches only when no memset sits between this call's kernels and the one before them)
    unsigned *sched = view.sched + 4 * sched_slot;
    if (!zeroed && cudaMemsetAsync(sched, 0, 4 * sizeof(unsigned), s) != cudaSuccess) return launch_status("row scheduling block");
    SortedRowLaunch l{};
    l.q = q; l.k = k; l.v = v; l.a = a; l.rvlen = cutoff_radius != 0.0 ? rvlen : nullptr; l.W = W;
    l.view = view; l.sched = sched; l.out = out; l.lse = lse; l.N = N; l.max_atoms = (int)max_atoms; l.K = (int)K;
    l.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    l.dist_max = dist_max; l.wscale = wscale;
    l.chained = zeroed;
    int rc = launch_sorted_rows(l, s);
    if (rc != CF_OK) return rc;
    return launch_leftover_rows(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, N, E, max_atoms, dist_max, wscale,
                                W, cutoff_radius, lattice_range, minimum_range, out, lse, view.leftover, sched + 1, sched + 2, K, s);
}
}  // namespace cf

extern "C" int cf_infinite_attn_fwd_sorted(const float *q, const float *k, const float *v, const float *a,
                                           const float *pos_ij, const float *tvecs, const float *rvlen,
                                           const int64_t *batch, const int64_t *edges, const int64_t *row_start,
                                           int64_t N, int64_t B, int64_t H, int64_t D, int64_t E, int64_t K,
                                           int64_t max_atoms, double dist_max, double wscale, const float *W,
                                           double cutoff_radius, int lattice_range, int minimum_range, float *out,
                                           float *lse, void *row_lists, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0 && B >= 0, CF_ERR_INVALID, "cf_infinite_attn_fwd_sorted: negative size");
    CF_REQUIRE(H == HEADS && D == HEAD_DIM && (K == 64 || K == 0), CF_ERR_UNSUPPORTED,
               "cf_infinite_attn_fwd_sorted: H=%lld D=%lld K=%lld, only H=8 D=16 K in {0, 64} is compiled", (long long)H, (long long)D, (long long)K);
    CF_REQUIRE(max_atoms >= 1 && max_atoms <= ROW_LIST_MAX_KEYS, CF_ERR_RANGE,
               "cf_infinite_attn_fwd_sorted: max_atoms=%lld outside [1,%d]", (long long)max_atoms, ROW_LIST_MAX_KEYS);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_infinite_attn_fwd_sorted: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (N == 0) return CF_OK;
    CF_REQUIRE(q && k && v && a && pos_ij && tvecs && batch && edges && row_start && (W || K == 0) && out && lse && row_lists,
               CF_ERR_INVALID, "cf_infinite_attn_fwd_sorted: null pointer");
    CF_REQUIRE(K == 0 || (dist_max > 0 && wscale > 0), CF_ERR_INVALID, "cf_infinite_attn_fwd_sorted: dist_max and wscale must be positive");
    const RowListView view = row_list_carve(row_lists, N, E);
    return sorted_attn_impl(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, N, E, max_atoms, dist_max, wscale, W,
                            cutoff_radius, lattice_range, minimum_range, out, lse, view, ROW_SCHED_SLOTS - 1, false, K,
                            as_stream(stream));
}
