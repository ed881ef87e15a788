// Fused infinitely connected attention, forward:
//     out_i = sum_j softmax_j(q_i.k_j + phi_ij) (v_j + W psi_ij)
// with phi and psi computed from the geometry on the fly.  No per-edge tensor other than the logits exists.
//
// Because W is shared by every edge, sum_j p_ij W psi_ij = W (sum_j p_ij psi_ij): the 8 x 64 radial-basis histogram
// of a row is accumulated over ALL its (key, translation) terms with the final joint weight
//     p_ij p(n | ij) = exp(q_i.k_j - lse_i + a_i d2_ijn)
// and projected once per atom instead of once per edge.
//
// Launch sequence (one stream, no host synchronisation):
//   lattice_phi_kernel        thread per edge : phi_ij for all heads (lattice_core.cuh), written into `logit`
//   infinite_attn_rows_kernel CTA per atom i  : logits q.k + phi (one key per thread, all heads), their log-sum-exp and
//                             p_ij; then the row's (32-key chunk, translation column) work units are dealt round-robin
//                             to the four warps; each warp scans its units with lanes over keys, four translations
//                             at a time, keeps the candidates in a ring and accumulates them with the lane<->bins
//                             turn-around of BinAccumulator; the four partial histograms are added in a fixed order
//                             (deterministic), projected with W and added to sum_j p_ij v_j.
#include <atomic>

#include "lattice_core.cuh"
#include "term_list.cuh"

// Row tickets: each launch of the row kernel gets one zeroed counter out of a small pool, so that launches in flight
// on different streams of a device do not share one.
__device__ unsigned g_row_tickets[64 + 8 * 16];

namespace cf {
namespace {

unsigned *next_ticket()
{
    static std::atomic<unsigned> turn{0};
    void *base = nullptr;
    if (cudaGetSymbolAddress(&base, g_row_tickets) != cudaSuccess) return nullptr;
    return static_cast<unsigned *>(base) + (turn.fetch_add(1) & 63u);
}

// `count` (<= 16) consecutive tickets out of the same pool, in its second half so that a block never wraps.
unsigned *next_ticket_block(int count)
{
    static std::atomic<unsigned> turn{0};
    void *base = nullptr;
    if (count < 1 || count > 16 || cudaGetSymbolAddress(&base, g_row_tickets) != cudaSuccess) return nullptr;
    return static_cast<unsigned *>(base) + 64 + 16 * (turn.fetch_add(1) & 7u);
}

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int KBINS = 64;
constexpr int KV_LD = 132;  // row stride (floats) of the k / v tile: 528 bytes, 16-byte aligned and off the bank period

struct RowArgs {
    const float *q, *k, *v, *a, *pos, *pos_ij, *tvecs, *rvlen, *W;
    const int64_t *batch, *edges, *row_start;
    const int32_t *row_order;  // optional: atoms in the order they are to be processed (heaviest first)
    const unsigned *rows_on_device;  // optional: the number of rows to process (entries of row_order), read on the device
    unsigned *ticket;          // zeroed before the launch: rows beyond the first wave are handed out through it
    TermList list;             // optional (pool == NULL: none): the rows' candidate terms, found once per batch
    long long E;
    float *out, *logit, *lse, *psi_row;
    long long N;
    int max_atoms;
    int keep_logit;  // 0: inference, the logits are not written back
    int phi_in_row;  // 1: no phi kernel ran; rows of at most 32 keys with a basis sum phi from their term lists
                     // themselves, all others (left-over rows of the sorted path) enumerate it edge by edge
    BoxRule rule;
    BasisParams basis;
};

// Shared-memory floats of ONE row group (the ROW_WARPS warps that work on one atom).
__host__ __device__ inline size_t row_group_floats(int max_atoms, bool with_basis, int row_warps)
{
    const size_t ld = ((max_atoms + 31) & ~31) + 1;
    return (size_t)max_atoms * 4 + ((16 * ld + 3) & ~(size_t)3) +
           (with_basis ? row_warps * (STAGE_FLOATS + HEADS * KBINS + RING_FLOATS) : 0) + row_warps * 128 +
           (max_atoms <= 32 ? 32 * KV_LD + 128 : 0);  // batches of small crystals: a tile for the row's k, then v, rows
                                                      // and the row's query
}

// phi of one edge by enumeration, for the rare edge whose row has no term list or whose listed terms miss a head's
// box when the row kernel computes phi itself; kept out of line so that the row kernel's registers do not pay for it.
__device__ __noinline__ void edge_phi_enumerated(const BoxRule rule, const float *a_row, const float *rvlen3,
                                                 const float *tvecs9, const float *pos3, float floor_log2, float *z_out)
{
    float a[8], z[8];
#pragma unroll
    for (int h = 0; h < 8; ++h) a[h] = a_row[h];
    Cell cell;
    cell.load(tvecs9);
    edge_phi<1>(rule, a, rvlen3, cell, pos3[0], pos3[1], pos3[2], floor_log2, 0, z);
#pragma unroll
    for (int h = 0; h < 8; ++h) z_out[h] = z[h];
}

// ROW_WARPS = 4: one thread block per atom (large crystals: the four warps split the translations).
// ROW_WARPS = 1: one warp per atom, four atoms per thread block (small crystals: a row is a few thousand terms and
//                its cost is dominated by the latency of its phases, so four rows progress independently per block
//                and only warp-level synchronisation is needed).
// ENUM_PHI: the kernel for left-over rows of the sorted path that neither a phi kernel nor term lists serve (no basis,
// or more than 32 keys): phi of every edge is enumerated inside the row (a variant of its own, so that the ordinary
// instantiations carry none of its code or registers).
template <int K, int ROW_WARPS, bool ENUM_PHI = false>
__global__ void __launch_bounds__(THREADS, ENUM_PHI ? 2 : (K == 0 ? 6 : (ROW_WARPS == 1 ? 3 : 4))) infinite_attn_rows_kernel(const RowArgs p)
{
    extern __shared__ __align__(16) float smem_all[];
    constexpr int GROUPS = WARPS / ROW_WARPS;        // row groups per block
    constexpr int RT = 32 * ROW_WARPS;               // threads per row group
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int group = warp / ROW_WARPS, wr = warp % ROW_WARPS, rt = tid % RT;
    // barrier of one row group: a warp barrier, or a named block barrier (one id per group) for its 32 ROW_WARPS threads
    auto row_sync = [&]() {
        if (ROW_WARPS == 1)
            __syncwarp();
        else if (ROW_WARPS == WARPS)
            __syncthreads();
        else if (group == 0)
            asm volatile("bar.sync 1, %0;" ::"n"(32 * ROW_WARPS) : "memory");
        else
            asm volatile("bar.sync 2, %0;" ::"n"(32 * ROW_WARPS) : "memory");
    };
    float *smem = smem_all + (size_t)group * row_group_floats(p.max_atoms, K > 0, ROW_WARPS);
    float4 *rel = reinterpret_cast<float4 *>(smem);                    // [max_atoms]
    // per-key tables are head-major with a leading dimension = 1 (mod 32): lanes over keys and lanes over heads both
    // fall into distinct banks
    const int ld = ((p.max_atoms + 31) & ~31) + 1;
    float *cj = smem + (size_t)p.max_atoms * 4;                        // [8][ld] (q.k - lse) log2e
    float *pj = cj + (size_t)8 * ld;                                   // [8][ld] p_ij
    float *stage = cj + (((size_t)16 * ld + 3) & ~(size_t)3);          // [ROW_WARPS][STAGE_FLOATS]
    float *part = stage + (K > 0 ? ROW_WARPS * STAGE_FLOATS : 0);      // [ROW_WARPS][8][64]
    float *rings = part + (K > 0 ? ROW_WARPS * HEADS * KBINS : 0);     // [ROW_WARPS][RING_FLOATS]
    float *vsum = rings + (K > 0 ? ROW_WARPS * RING_FLOATS : 0);       // [ROW_WARPS][128] partial sum_j p v
    float *kv = vsum + ROW_WARPS * 128;                                // [32][KV_LD] when max_atoms <= 32
    float *qrow = kv + 32 * KV_LD;                                     // [128] the row's query (same condition)
    const bool tiled = p.max_atoms <= 32;
    bool prefetched = false;  // the k tile and query of the current row were requested during the previous row
    // all threads of the group copy `rows` 512-byte rows starting at src into the tile, asynchronously
    auto tile_fetch = [&](const float *src, int rows, const float *query) {
        for (int idx = rt; idx < rows * 32; idx += RT) {
            const unsigned dst = (unsigned)__cvta_generic_to_shared(kv + (idx >> 5) * KV_LD + (idx & 31) * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src + (size_t)idx * 4));
        }
        if (query != nullptr && rt < 32) {
            const unsigned dst = (unsigned)__cvta_generic_to_shared(qrow + rt * 4);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(query + rt * 4));
        }
        asm volatile("cp.async.commit_group;");
    };

    BinAccumulator<KBINS> bins;
    CandidateRing ring;
    if (K > 0) {
        bins.init(stage + wr * STAGE_FLOATS, lane, p.basis);
        ring.init(rings + wr * RING_FLOATS, lane);
    }
    const float *__restrict__ kmat = p.k;
    float *__restrict__ logit_io = p.logit;

    // Rows are handed out in the order of p.row_order: the first wave by block index, the rest through an atomic
    // ticket, so that a block that drew a heavy row simply draws fewer rows (longest-processing-time-first).  Which
    // block computes a row has no influence on the row's result.  The ticket and the row's indices (atom, crystal,
    // edge range, first key) are fetched one row ahead, in stages placed where their latency is hidden.
    __shared__ long long next_slot_sh[GROUPS];
    grid_launch_dependents();
    grid_dependency_wait();  // (chained launches: the kernel before this one wrote q, k, v, a, phi or the row count)
    const long long first_wave = (long long)gridDim.x * GROUPS;
    long long slot = (long long)blockIdx.x * GROUPS + group;
    const long long rows = p.rows_on_device ? (long long)*p.rows_on_device : p.N;
    if (slot >= rows) return;
    long long i = p.row_order ? p.row_order[slot] : slot;
    long long c = p.batch[i];
    long long e0 = p.row_start[i];
    int n_raw = (int)(p.row_start[i + 1] - e0);  // keys of the row = atoms of the crystal
    long long a0 = n_raw > 0 ? p.edges[p.E + e0] : 0;  // first atom of the crystal
    long long nslot = slot + first_wave;  // without a ticket: rows dealt round-robin
    if (p.ticket) {
        if (rt == 0) next_slot_sh[group] = first_wave + atomicAdd(p.ticket, 1u);
        row_sync();
        nslot = next_slot_sh[group];
    }

    while (true) {
        // stage 0 of the look-ahead: the next row's atom; thread 0 draws the ticket of the row after it
        const bool has_next = nslot < rows;
        const long long i_n = has_next ? (p.row_order ? (long long)p.row_order[nslot] : nslot) : 0;
        unsigned drawn = 0;
        if (p.ticket && rt == 0) drawn = atomicAdd(p.ticket, 1u);
        // the caller understated max_atoms: the row is poisoned instead of overrunning shared memory
        const bool bad = n_raw > p.max_atoms;
        const int n = bad ? 0 : n_raw;
        // constants of the row's atom and crystal, needed after the soft-max: loaded here so that they arrive meanwhile
        float a_own = 0.f;
        Cell cell;
        float rvl[3] = {0.f, 0.f, 0.f};
        if (K > 0) {
            a_own = p.a[i * HEADS + (lane & 7)];
            cell.load(p.tvecs + 9 * c);
            if (p.rvlen) { rvl[0] = p.rvlen[3 * c]; rvl[1] = p.rvlen[3 * c + 1]; rvl[2] = p.rvlen[3 * c + 2]; }
        }

        // phi of key jk of this row from the edge's term list, by the ROW_WARPS lanes rt % ROW_WARPS of the key: they
        // read its entries sub, sub + ROW_WARPS, ... and combine by a fixed butterfly; lane 0 of the key stores the eight
        // values at dst.  Every thread of the group calls it (keys beyond the row just take part in the shuffles).  The
        // rare edge without a list, or whose listed terms miss a head's box, is enumerated out of line.
        const bool phi_here = K > 0 && p.phi_in_row != 0;
        auto phi_from_lists = [&](int jk, float *dst) {
            float a8[8], a2p[8];
            int pkp[8];
            float a2mx = -INFINITY;
            const int pk_mine = packed_box(p.rule, a_own, p.rvlen ? rvl : nullptr);
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                a8[h] = __shfl_sync(FULL, a_own, h);
                pkp[h] = __shfl_sync(FULL, pk_mine, h);
                a2p[h] = a8[h] * LOG2E;
                a2mx = fmaxf(a2mx, a2p[h]);
            }
            const int sub = rt % ROW_WARPS;
            const bool mine = jk < n;
            const long long e = e0 + (mine ? jk : 0);
            const int first = (mine && p.list.start != nullptr) ? p.list.start[e] : -1;
            const int cnt = first >= 0 ? p.list.count[e] : 0;
            const float m = first >= 0 ? p.list.dmin[e] : 0.f;
            const float2 *ent = p.list.pool + (first >= 0 ? first : 0);
            float s8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float2 n0 = make_float2(0.f, 0.f), n1 = n0;  // entries are requested two steps ahead of their use
            if (sub < cnt) n0 = __ldg(ent + sub);
            if (sub + ROW_WARPS < cnt) n1 = __ldg(ent + sub + ROW_WARPS);
            for (int t = sub; t < cnt; t += ROW_WARPS) {
                const float2 en = n0;
                n0 = n1;
                if (t + 2 * ROW_WARPS < cnt) n1 = __ldg(ent + t + 2 * ROW_WARPS);
                const float d = en.x - m;
                if (a2mx * d < p.basis.floor_log2) continue;  // below the floor for every head
                const int key = __float_as_int(en.y);
#pragma unroll
                for (int h = 0; h < 8; ++h)
                    if (key_in_box(key, pkp[h])) s8[h] += ex2(a2p[h] * d);
            }
            bool done = cnt > 0;
            float z8[8];
#pragma unroll
            for (int h = 0; h < 8; ++h) {  // (all lanes take part in the shuffles, listed or not)
                float t = s8[h];
#pragma unroll
                for (int o = 1; o < ROW_WARPS; o <<= 1) t += __shfl_xor_sync(FULL, t, o);
                z8[h] = fmaf(m, a8[h], logf(t));
                done = done && t > 1e-30f;  // a head whose box misses the listed terms: enumerate instead
            }
            if (mine && sub == 0) {
                if (!done) {
                    edge_phi_enumerated(p.rule, p.a + i * HEADS, p.rvlen ? p.rvlen + 3 * c : nullptr, p.tvecs + 9 * c,
                                        p.pos_ij + 3 * e, p.basis.floor_log2, dst);
                } else {
                    reinterpret_cast<float4 *>(dst)[0] = make_float4(z8[0], z8[1], z8[2], z8[3]);
                    reinterpret_cast<float4 *>(dst)[1] = make_float4(z8[4], z8[5], z8[6], z8[7]);
                }
            }
        };

        if (n <= 32) {
            // ---- up to 32 keys: the soft-max in registers, one key per lane, the heads split over the warps of the group
            //      (logits, statistics by shuffles).
            //      In batches of small crystals all threads first bring the keys' k rows (contiguous: the crystal's
            //      atoms) and the query into shared memory in one round trip; read by one lane per key straight from
            //      global memory, the 32 loads of a 512-byte row go out a few at a time.
            if (tiled && !prefetched) tile_fetch(kmat + a0 * HEADS * HEAD_DIM, n, p.q + i * HEADS * HEAD_DIM);
            if (K > 0 && phi_here) {
                // ---- phi of the row's edges from their term lists, ROW_WARPS lanes per key (key = rt / ROW_WARPS)
                phi_from_lists(rt / ROW_WARPS, part + 8 * (rt / ROW_WARPS));
                row_sync();
            }
            // The warps of the row split the heads (HPW each), one key per lane: a warp's chain of shuffle reductions
            // is then HPW heads long instead of eight.
            constexpr int HPW = HEADS / ROW_WARPS;
            const int h0 = wr * HPW;
            float rx = 0.f, ry = 0.f, rz = 0.f;
            float phi[HPW];
#pragma unroll
            for (int u = 0; u < HPW; ++u) phi[u] = 0.f;
            if (lane < n) {  // this lane's key: position and phi, requested before waiting for the tile
                if (wr == 0) {
                    if (p.pos_ij) {
                        const float *pp = p.pos_ij + 3 * (e0 + lane);
                        rx = pp[0]; ry = pp[1]; rz = pp[2];
                    } else {
                        const float *pp = p.pos + 3 * (a0 + lane), *pi = p.pos + 3 * i;
                        rx = __fsub_rn(pp[0], pi[0]); ry = __fsub_rn(pp[1], pi[1]); rz = __fsub_rn(pp[2], pi[2]);
                    }
                }
                // phi: left in shared memory by the phase above, or in the logit array by the phi kernel, or - a left-over
                // row without a basis, for which neither ran - enumerated here
                __align__(16) float enumerated[8];
                const bool phi_enum = ENUM_PHI && p.phi_in_row != 0 && !phi_here;
                if (phi_enum)
                    edge_phi_enumerated(p.rule, p.a + i * HEADS, p.rvlen ? p.rvlen + 3 * c : nullptr, p.tvecs + 9 * c,
                                        p.pos_ij + 3 * (e0 + lane), p.basis.floor_log2, enumerated);
                const float *src = (phi_enum ? enumerated : phi_here ? part + 8 * lane : logit_io + (e0 + lane) * HEADS) + h0;
                if (HPW == 8) {
                    const float4 v0 = reinterpret_cast<const float4 *>(src)[0], v1 = reinterpret_cast<const float4 *>(src)[1];
                    phi[0] = v0.x; phi[1] = v0.y; phi[2] = v0.z; phi[3] = v0.w;
                    phi[4 % HPW] = v1.x; phi[5 % HPW] = v1.y; phi[6 % HPW] = v1.z; phi[7 % HPW] = v1.w;
                } else if (HPW == 4) {
                    const float4 v0 = reinterpret_cast<const float4 *>(src)[0];
                    phi[0] = v0.x; phi[1] = v0.y; phi[2 % HPW] = v0.z; phi[3 % HPW] = v0.w;
                } else {
                    const float2 v0 = reinterpret_cast<const float2 *>(src)[0];
                    phi[0] = v0.x; phi[1] = v0.y;
                }
            }
            if (tiled) {
                asm volatile("cp.async.wait_all;" ::: "memory");
                row_sync();
            }
            {
                const bool live = lane < n;
                const int j = live ? lane : 0;
                // k row and query from the tile, or (batches with larger crystals) from global memory
                const float4 *qp = tiled ? reinterpret_cast<const float4 *>(qrow)
                                         : reinterpret_cast<const float4 *>(p.q + i * HEADS * HEAD_DIM);
                const float4 *kp = tiled ? reinterpret_cast<const float4 *>(kv + j * KV_LD)
                                         : reinterpret_cast<const float4 *>(kmat + (a0 + j) * HEADS * HEAD_DIM);
                float sc[HPW], lg[HPW];
#pragma unroll
                for (int u = 0; u < HPW; ++u) {
                    const int h = h0 + u;
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int t = 0; t < 4; t += 2) {
                        const float4 k0 = kp[4 * h + t], k1 = kp[4 * h + t + 1];
                        const float4 q0 = qp[4 * h + t], q1 = qp[4 * h + t + 1];
                        s0 = fmaf(q0.x, k0.x, s0); s0 = fmaf(q0.y, k0.y, s0); s0 = fmaf(q0.z, k0.z, s0); s0 = fmaf(q0.w, k0.w, s0);
                        s1 = fmaf(q1.x, k1.x, s1); s1 = fmaf(q1.y, k1.y, s1); s1 = fmaf(q1.z, k1.z, s1); s1 = fmaf(q1.w, k1.w, s1);
                    }
                    sc[u] = s0 + s1;
                    lg[u] = live ? sc[u] + phi[u] : -INFINITY;
                }
                if (p.keep_logit && live) {
                    float *lp = logit_io + (e0 + j) * HEADS + h0;
#pragma unroll
                    for (int u = 0; u < HPW; ++u) lp[u] = lg[u];
                }
                float mxo = -INFINITY, lse_mine = 0.f;
#pragma unroll
                for (int u = 0; u < HPW; ++u) {
                    const int h = h0 + u;
                    const float mx = warp_max(lg[u]);
                    const float den = warp_sum(ex2((lg[u] - mx) * LOG2E));
                    const float lse = mx + logf(den);
                    if (lane == u) lse_mine = lse;
                    const float off = (sc[u] - lse) * LOG2E;
                    if (live) {
                        cj[h * ld + j] = off;
                        pj[h * ld + j] = ex2((lg[u] - lse) * LOG2E);
                    }
                    mxo = fmaxf(mxo, off);
                }
                if (lane < HPW) p.lse[i * HEADS + h0 + lane] = lse_mine;
                if (ROW_WARPS == 1) {
                    if (live) rel[j] = make_float4(rx, ry, rz, mxo);  // .w: the key's largest offset
                } else if (live) {
                    vsum[wr * 32 + lane] = mxo;  // this warp's heads only; combined below
                }
            }
            row_sync();
            // the k rows are no longer needed: the tile is refilled with the keys' v rows while the histogram is built
            if (tiled) tile_fetch(p.v + a0 * HEADS * HEAD_DIM, n, nullptr);
            if (ROW_WARPS > 1) {
                if (wr == 0 && lane < n) {
                    float mxo = vsum[lane];
#pragma unroll
                    for (int w = 1; w < ROW_WARPS; ++w) mxo = fmaxf(mxo, vsum[w * 32 + lane]);
                    rel[lane] = make_float4(rx, ry, rz, mxo);  // .w: the key's largest offset
                }
                row_sync();
            }
        } else {
            // ---- relative positions of the keys
            if (p.pos_ij) {
                for (int j = rt; j < n; j += RT) {
                    const float *pp = p.pos_ij + 3 * (e0 + j);
                    rel[j] = make_float4(pp[0], pp[1], pp[2], 0.f);
                }
            } else {
                const float pix = p.pos[3 * i], piy = p.pos[3 * i + 1], piz = p.pos[3 * i + 2];
                for (int j = rt; j < n; j += RT) {
                    const float *pp = p.pos + 3 * (a0 + j);
                    rel[j] = make_float4(__fsub_rn(pp[0], pix), __fsub_rn(pp[1], piy), __fsub_rn(pp[2], piz), 0.f);
                }
            }
            // ---- the row's query, read back as shared-memory broadcasts (the buffer is reused for sum_j p v later)
            float4 *qs = reinterpret_cast<float4 *>(vsum);
            for (int idx = rt; idx < HEADS * HEAD_DIM / 4; idx += RT)
                qs[idx] = __ldg(reinterpret_cast<const float4 *>(p.q + i * HEADS * HEAD_DIM) + idx);
            row_sync();
            // ---- logits: one key per thread, all eight heads; the key's 512-byte row is 32 independent 16-byte loads
            for (int j = rt; j < n; j += RT) {
                const float4 *kp = reinterpret_cast<const float4 *>(kmat + (a0 + j) * HEADS * HEAD_DIM);
                float4 *lp = reinterpret_cast<float4 *>(logit_io + (e0 + j) * HEADS);  // phi was left here by the phi kernel
                float phi[8];
                if (ENUM_PHI && p.phi_in_row != 0) {  // (a left-over row: no phi kernel ran)
                    edge_phi_enumerated(p.rule, p.a + i * HEADS, p.rvlen ? p.rvlen + 3 * c : nullptr, p.tvecs + 9 * c,
                                        p.pos_ij + 3 * (e0 + j), p.basis.floor_log2, phi);
                } else {
                    const float4 ph0 = lp[0], ph1 = lp[1];
                    phi[0] = ph0.x; phi[1] = ph0.y; phi[2] = ph0.z; phi[3] = ph0.w;
                    phi[4] = ph1.x; phi[5] = ph1.y; phi[6] = ph1.z; phi[7] = ph1.w;
                }
                float lg[8];
#pragma unroll
                for (int h = 0; h < HEADS; ++h) {
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll
                    for (int t = 0; t < 4; t += 2) {
                        const float4 k0 = __ldg(kp + 4 * h + t), k1 = __ldg(kp + 4 * h + t + 1);
                        const float4 q0 = qs[4 * h + t], q1 = qs[4 * h + t + 1];
                        s0 = fmaf(q0.x, k0.x, s0); s0 = fmaf(q0.y, k0.y, s0); s0 = fmaf(q0.z, k0.z, s0); s0 = fmaf(q0.w, k0.w, s0);
                        s1 = fmaf(q1.x, k1.x, s1); s1 = fmaf(q1.y, k1.y, s1); s1 = fmaf(q1.z, k1.z, s1); s1 = fmaf(q1.w, k1.w, s1);
                    }
                    const float sc = s0 + s1;
                    lg[h] = sc + phi[h];
                    cj[h * ld + j] = sc;
                    pj[h * ld + j] = lg[h];
                }
                if (p.keep_logit) {
                    lp[0] = make_float4(lg[0], lg[1], lg[2], lg[3]);
                    lp[1] = make_float4(lg[4], lg[5], lg[6], lg[7]);
                }
            }
            row_sync();
            // ---- soft-max statistics: warp wr of the group owns heads wr, wr + ROW_WARPS, ...
#pragma unroll
            for (int h = wr; h < HEADS; h += ROW_WARPS) {
                float mx = -INFINITY;
                for (int j = lane; j < n; j += 32) mx = fmaxf(mx, pj[h * ld + j]);
                mx = warp_max(mx);
                float den = 0.f;
                for (int j = lane; j < n; j += 32) den += ex2((pj[h * ld + j] - mx) * LOG2E);
                den = warp_sum(den);
                const float lse = mx + logf(den);
                if (lane == 0) p.lse[i * HEADS + h] = lse;
                for (int j = lane; j < n; j += 32) {
                    cj[h * ld + j] = (cj[h * ld + j] - lse) * LOG2E;
                    pj[h * ld + j] = ex2((pj[h * ld + j] - lse) * LOG2E);
                }
            }
            row_sync();

            if (K > 0) {
                // ---- per key: the largest of the eight offsets, kept in the spare component of rel
                for (int j = rt; j < n; j += RT) {
                    float mxo = cj[j];
#pragma unroll
                    for (int h = 1; h < 8; ++h) mxo = fmaxf(mxo, cj[h * ld + j]);
                    rel[j].w = mxo;
                }
                row_sync();
            }
        }
        // stage 1 of the look-ahead: the next row's crystal and edge range
        const long long c_n = p.batch[i_n], e0_n = p.row_start[i_n];
        const int n_n = (int)(p.row_start[i_n + 1] - e0_n);

        if (K > 0) {
            // ---- boxes of the row's heads (they depend on the atom and the head, not on the key)
            const int pk_own = packed_box(p.rule, a_own, p.rvlen ? rvl : nullptr);
            int uni = pk_own;
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) uni = box_union(uni, __shfl_xor_sync(FULL, uni, o));
            const bool masked = !__all_sync(FULL, pk_own == uni);
            float a2[8];
            int pk[8];
            float a2max = -INFINITY;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                a2[h] = __shfl_sync(FULL, a_own, h) * LOG2E;
                pk[h] = __shfl_sync(FULL, pk_own, h);
                a2max = fmaxf(a2max, a2[h]);
            }
            const int R1 = box_r1(uni), R2 = box_r2(uni), R3 = box_r3(uni);
            const int S2 = 2 * R2 + 1;
            const int columns = (2 * R1 + 1) * S2;  // a column = the translations (n1, n2, *)
            const int chunks = (n + 31) >> 5;       // a chunk = 32 keys, one per lane
            const float t3sq = fmaf(cell.t3z, cell.t3z, fmaf(cell.t3y, cell.t3y, cell.t3x * cell.t3x));
            const bool prune = t3sq > 1e-12f;
            const float inv_t3sq = prune ? __frcp_rn(t3sq) : 0.f;
            bins.clear();
            // candidates of the ring -> eight weights each -> accumulation
            auto consume = [&]() {
                float d2;
                int key;
                const bool got = ring.take(d2, key);
                const int j = got ? (key & 2047) : 0;
                float w[8];
                float emax = -INFINITY;
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    float eh = fmaf(a2[h], d2, cj[h * ld + j]);
                    if (!got || (masked && !key_in_box(key, pk[h]))) eh = -INFINITY;
                    w[h] = ex2(eh);
                    emax = fmaxf(emax, eh);
                }
                bins.push(emax > p.basis.floor_log2, fast_sqrt(d2) * p.basis.bin_scale, w);
            };
            const int list_first = (p.list.pool != nullptr && n > 0) ? p.list.start[e0] : -1;
            if (list_first >= 0) {
                // ---- candidates from the row's term list: its entries are contiguous, the warps of the group take
                //      equal shares, 32 entries per step; the one-FMA bound weeds out what this layer's widths do not reach
                const int list_end = p.list.start[e0 + n - 1] + p.list.count[e0 + n - 1];
                const int span = list_end - list_first, share = (span + ROW_WARPS - 1) / ROW_WARPS;
                const int w_lo = list_first + min(wr * share, span), w_hi = list_first + min((wr + 1) * share, span);
                // (the entries of the next step are requested before this step's are processed)
                float2 ahead = make_float2(0.f, 0.f);
                if (w_lo + lane < w_hi) ahead = __ldg(p.list.pool + w_lo + lane);
                for (int at = w_lo; at < w_hi; at += 32) {
                    const bool live = at + lane < w_hi;
                    const float2 en = ahead;
                    if (at + 32 + lane < w_hi) ahead = __ldg(p.list.pool + at + 32 + lane);
                    const int key = __float_as_int(en.y);
                    const int j = key & 2047;
                    // (the lists are built for a box that contains every head's: terms outside this row's boxes drop out here)
                    const bool cand = live && key_in_box(key, uni) && fmaf(a2max, en.x, rel[live ? j : 0].w) > p.basis.floor_log2 &&
                                      en.x < p.basis.d2_cut;
                    ring.offer(cand, en.x, masked ? key : j);
                    while (ring.ready()) consume();
                }
            } else {
                // Work units are (chunk, column) pairs dealt round-robin to the warps of the group (rotated by one warp per
                // chunk), so that the few dense columns around the origin are spread over all of them whatever the number
                // of keys.  Lanes run over the keys of the chunk: a translation is warp-uniform and a lane's key stays
                // in registers.
                for (int ch = 0; ch < chunks; ++ch) {
                    const int j = 32 * ch + lane;
                    const bool live = j < n;
                    const float4 r = rel[live ? j : 0];  // r.w: the key's largest offset
                    // reach of this chunk of keys: no key farther than `far` from the origin, no candidate beyond `reach`
                    // from its key; a translation longer than reach + far cannot produce a candidate (triangle inequality)
                    const float far2 = warp_max(live ? fmaf(r.z, r.z, fmaf(r.y, r.y, r.x * r.x)) : 0.f);
                    const float cmax = warp_max(live ? r.w : -INFINITY);
                    const float reach2 = fminf(__fdividef(p.basis.floor_log2 - cmax, a2max), p.basis.d2_cut);
                    const float bound = sqrtf(fmaxf(reach2, 0.f)) + sqrtf(far2);
                    const float tau2_max = bound * bound * 1.0001f + 1e-4f;
                    // this warp's columns of the chunk: col = (wr - ch) mod ROW_WARPS, then every ROW_WARPS-th
                    int col = (wr - ch) & (ROW_WARPS - 1);
                    int n1 = -R1, n2 = col - R2;
                    while (n2 > R2) { n2 -= S2; ++n1; }
                    for (; col < columns; col += ROW_WARPS) {
                        {
                            const float f1 = (float)n1, f2 = (float)n2;
                            // the n3 of this column whose translation n1 t1 + n2 t2 + n3 t3 is no longer than the bound
                            const float bx = fmaf(cell.t2x, f2, cell.t1x * f1), by = fmaf(cell.t2y, f2, cell.t1y * f1);
                            const float bz = fmaf(cell.t2z, f2, cell.t1z * f1);
                            const float bb = fmaf(bz, bz, fmaf(by, by, bx * bx));
                            const float bt = fmaf(bz, cell.t3z, fmaf(by, cell.t3y, bx * cell.t3x));
                            const float room = fmaf(bb, 1e-5f, tau2_max) - fmaf(-bt * bt, inv_t3sq, bb);  // slack for rounding
                            int lo = -R3, hi = R3;
                            if (prune) {
                                const float half = sqrtf(fmaxf(room, 0.f) * inv_t3sq) + 1e-3f, mid = -bt * inv_t3sq;
                                lo = max(lo, __float2int_ru(mid - half));
                                hi = min(hi, __float2int_rd(mid + half));
                                if (room < 0.f) hi = lo - 1;
                            }
                            // r + n1 t1 + n2 t2, contracted like the reference's expression
                            const float ex = fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, r.x));
                            const float ey = fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, r.y));
                            const float ez = fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, r.z));
                            for (int n3 = lo; n3 <= hi; n3 += 4) {
                                const float f3 = (float)n3;
                                bool cand[4];
                                float d2v[4];
                                int key[4];
    #pragma unroll
                                for (int u = 0; u < 4; ++u) {
                                    const float fu = f3 + (float)u;
                                    const float dx = fmaf(cell.t3x, fu, ex), dy = fmaf(cell.t3y, fu, ey), dz = fmaf(cell.t3z, fu, ez);
                                    d2v[u] = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                                    cand[u] = live && n3 + u <= hi && fmaf(a2max, d2v[u], r.w) > p.basis.floor_log2 &&
                                              d2v[u] < p.basis.d2_cut;
                                    key[u] = masked ? pack_key(j, abs(n1), abs(n2), abs(n3 + u)) : j;
                                }
                                ring.offer4(cand, d2v, key);
                                while (ring.ready()) consume();
                            }
                        }
                        n2 += ROW_WARPS;
                        while (n2 > R2) { n2 -= S2; ++n1; }
                    }
                }
            }
            while (ring.count > 0) consume();
            // ---- partial histograms -> shared memory, fixed-order sum over the warps of the group
            bins.flush(part + wr * HEADS * KBINS, KBINS);
            asm volatile("cp.async.wait_all;" ::: "memory");  // this thread's part of the v tile (published by the barrier)
            row_sync();
            for (int idx = rt; idx < HEADS * KBINS; idx += RT) {
                float s = part[idx];
                if (ROW_WARPS == 2) s = part[idx] + part[HEADS * KBINS + idx];
                if (ROW_WARPS == 4)
                    s = (part[idx] + part[HEADS * KBINS + idx]) + (part[2 * HEADS * KBINS + idx] + part[3 * HEADS * KBINS + idx]);
                part[idx] = s;
                if (p.psi_row) p.psi_row[i * HEADS * KBINS + idx] = s;
            }
            row_sync();
        }

        // stage 2 of the look-ahead: the next row's first key; thread 0 publishes the ticket it drew
        const long long a0_n = (has_next && n_n > 0) ? p.edges[p.E + e0_n] : 0;
        if (p.ticket && rt == 0) next_slot_sh[group] = first_wave + drawn;

        // ---- sum_j p_ij v_j: warp wr takes keys wr, wr + ROW_WARPS, ...; a lane owns four consecutive channels (one
        //      float4 load per key); the partial rows of the group meet in shared memory
        if (K == 0 && tiled && n <= 32) {  // no histogram phase in between: wait for the v tile here
            asm volatile("cp.async.wait_all;" ::: "memory");
            row_sync();
        }
        if (tiled && n <= 32) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const int hh = lane >> 2;
            const float *pr = pj + hh * ld;
            for (int j = wr; j < n; j += ROW_WARPS) {
                const float4 v0 = reinterpret_cast<const float4 *>(kv + j * KV_LD)[lane];
                const float p0 = pr[j];
                acc.x = fmaf(p0, v0.x, acc.x); acc.y = fmaf(p0, v0.y, acc.y); acc.z = fmaf(p0, v0.z, acc.z); acc.w = fmaf(p0, v0.w, acc.w);
            }
            reinterpret_cast<float4 *>(vsum)[wr * 32 + lane] = acc;
        } else {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            const int hh = lane >> 2;  // head of the lane's channels 4 lane .. 4 lane + 3
            const float4 *vp = reinterpret_cast<const float4 *>(p.v + a0 * HEADS * HEAD_DIM) + lane;
            int j = wr;
            for (; j + 3 * ROW_WARPS < n; j += 4 * ROW_WARPS) {
                const float4 v0 = __ldg(vp + (size_t)(j) * 32), v1 = __ldg(vp + (size_t)(j + ROW_WARPS) * 32);
                const float4 v2 = __ldg(vp + (size_t)(j + 2 * ROW_WARPS) * 32), v3 = __ldg(vp + (size_t)(j + 3 * ROW_WARPS) * 32);
                const float *pr = pj + hh * ld + j;
                const float p0 = pr[0], p1 = pr[ROW_WARPS], p2 = pr[2 * ROW_WARPS], p3 = pr[3 * ROW_WARPS];
                acc.x = fmaf(p0, v0.x, acc.x); acc.y = fmaf(p0, v0.y, acc.y); acc.z = fmaf(p0, v0.z, acc.z); acc.w = fmaf(p0, v0.w, acc.w);
                acc.x = fmaf(p1, v1.x, acc.x); acc.y = fmaf(p1, v1.y, acc.y); acc.z = fmaf(p1, v1.z, acc.z); acc.w = fmaf(p1, v1.w, acc.w);
                acc.x = fmaf(p2, v2.x, acc.x); acc.y = fmaf(p2, v2.y, acc.y); acc.z = fmaf(p2, v2.z, acc.z); acc.w = fmaf(p2, v2.w, acc.w);
                acc.x = fmaf(p3, v3.x, acc.x); acc.y = fmaf(p3, v3.y, acc.y); acc.z = fmaf(p3, v3.z, acc.z); acc.w = fmaf(p3, v3.w, acc.w);
            }
            for (; j < n; j += ROW_WARPS) {
                const float4 v0 = __ldg(vp + (size_t)j * 32);
                const float p0 = pj[hh * ld + j];
                acc.x = fmaf(p0, v0.x, acc.x); acc.y = fmaf(p0, v0.y, acc.y); acc.z = fmaf(p0, v0.z, acc.z); acc.w = fmaf(p0, v0.w, acc.w);
            }
            reinterpret_cast<float4 *>(vsum)[wr * 32 + lane] = acc;
        }
        row_sync();
        // the v tile has been consumed: the next row's k rows and query are requested now and arrive while this row is
        // projected and written
        prefetched = tiled && has_next && n_n <= 32;
        if (prefetched) tile_fetch(kmat + a0_n * HEADS * HEAD_DIM, n_n, p.q + i_n * HEADS * HEAD_DIM);
        // ---- out[h][m] = (sum over the partial rows) + sum_k W[h][m][k] Psi[h][k]; one output (h, m) per thread and turn
        for (int idx = rt; idx < HEADS * HEAD_DIM; idx += RT) {
            const int h = idx >> 4;
            float acc = vsum[idx];
            if (ROW_WARPS == 2) acc = vsum[idx] + vsum[128 + idx];
            if (ROW_WARPS == 4) acc = (vsum[idx] + vsum[128 + idx]) + (vsum[256 + idx] + vsum[384 + idx]);
            if (K > 0) {
                const float4 *wp = reinterpret_cast<const float4 *>(p.W + (size_t)idx * KBINS);
                const float4 *pp = reinterpret_cast<const float4 *>(part + h * KBINS);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll 4
                for (int k4 = 0; k4 < KBINS / 4; ++k4) {
                    const float4 wv = __ldg(wp + k4), ps = pp[k4];
                    o0 = fmaf(wv.x, ps.x, o0); o1 = fmaf(wv.y, ps.y, o1); o2 = fmaf(wv.z, ps.z, o2); o3 = fmaf(wv.w, ps.w, o3);
                }
                acc += (o0 + o1) + (o2 + o3);
            }
            p.out[i * HEADS * HEAD_DIM + idx] = bad ? __int_as_float(0x7fc00000) : acc;
        }
        row_sync();
        if (!has_next) break;
        i = i_n; c = c_n; e0 = e0_n; n_raw = n_n; a0 = a0_n;
        nslot = p.ticket ? next_slot_sh[group] : nslot + first_wave;
    }
}

}  // namespace
}  // namespace cf

namespace cf {
// cf_infinite_attn_fwd with an optional term list (see term_list.cuh) in place of the enumeration of translations.
int infinite_attn_fwd_impl(const float *q, const float *k, const float *v, const float *a, const float *pos,
                           const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                           const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D,
                           int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                           double cutoff_radius, int lattice_range, int minimum_range, float *out, float *logit,
                           float *lse, float *psi_row, const int32_t *row_order, const TermList *list, unsigned *ticket_ready,
                           void *stream, bool chained);
unsigned *row_ticket_block(int count);
int launch_rows(const RowArgs &p, int64_t K, long long grid_rows, cudaStream_t s, bool chained);
}

extern "C" int cf_infinite_attn_fwd(const float *q, const float *k, const float *v, const float *a, const float *pos,
                                    const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                                    const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                                    int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                                    const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                                    float *out, float *logit, float *lse, float *psi_row, const int32_t *row_order,
                                    void *stream)
{
    return cf::infinite_attn_fwd_impl(q, k, v, a, pos, pos_ij, tvecs, rvlen, batch, edges, row_start, N, B, H, D, E, K,
                                      max_atoms, dist_max, wscale, W, cutoff_radius, lattice_range, minimum_range, out,
                                      logit, lse, psi_row, row_order, nullptr, nullptr, stream, false);
}

extern "C" int cf_infinite_attn_fwd_listed(const float *q, const float *k, const float *v, const float *a,
                                           const float *pos_ij, const float *tvecs, const float *rvlen,
                                           const int64_t *batch, const int64_t *edges, const int64_t *row_start,
                                           int64_t N, int64_t B, int64_t H, int64_t D, int64_t E, int64_t K,
                                           int64_t max_atoms, double dist_max, double wscale, const float *W,
                                           double cutoff_radius, int lattice_range, int minimum_range, float *out,
                                           float *logit, float *lse, float *psi_row, const int32_t *row_order,
                                           void *term_lists, double a_widest, void *stream)
{
    using namespace cf;
    CF_REQUIRE(term_lists != nullptr && pos_ij != nullptr && a_widest < 0, CF_ERR_INVALID,
               "cf_infinite_attn_fwd_listed: needs term lists, pos_ij and a negative a_widest");
    TermList list{};
    int *start, *count;
    float *dmin;
    unsigned long long *cursor;
    float2 *pool;
    term_list_carve(term_lists, N, E, &start, &count, &dmin, &cursor, &pool);
    list.pool = pool; list.start = start; list.count = count; list.dmin = dmin;
    list.window = term_window(weight_floor_log2(), (float)a_widest);
    return infinite_attn_fwd_impl(q, k, v, a, nullptr, pos_ij, tvecs, rvlen, batch, edges, row_start, N, B, H, D, E, K,
                                  max_atoms, dist_max, wscale, W, cutoff_radius, lattice_range, minimum_range, out, logit,
                                  lse, psi_row, row_order, &list, nullptr, stream, false);
}

int cf::infinite_attn_fwd_impl(const float *q, const float *k, const float *v, const float *a, const float *pos,
                               const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                               const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                               int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                               const float *W, double cutoff_radius, int lattice_range, int minimum_range, float *out,
                               float *logit, float *lse, float *psi_row, const int32_t *row_order,
                               const TermList *list, unsigned *ticket_ready, void *stream, bool chained)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0 && B >= 0, CF_ERR_INVALID, "cf_infinite_attn_fwd: negative size");
    CF_REQUIRE(H == HEADS && D == HEAD_DIM, CF_ERR_UNSUPPORTED, "cf_infinite_attn_fwd: H=%lld D=%lld, only H=8 D=16 is compiled",
               (long long)H, (long long)D);
    CF_REQUIRE(K == 0 || K == 64, CF_ERR_UNSUPPORTED, "cf_infinite_attn_fwd: K=%lld, only K in {0,64} is compiled", (long long)K);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_infinite_attn_fwd: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    CF_REQUIRE(max_atoms >= 1 && max_atoms <= 2048, CF_ERR_RANGE, "cf_infinite_attn_fwd: max_atoms=%lld outside [1,2048]",
               (long long)max_atoms);
    if (N == 0) return CF_OK;
    CF_REQUIRE(q && k && v && a && (pos || pos_ij) && tvecs && batch && edges && row_start && out && logit && lse,
               CF_ERR_INVALID, "cf_infinite_attn_fwd: null pointer");
    CF_REQUIRE(K == 0 || (W != nullptr && dist_max > 0 && wscale > 0), CF_ERR_INVALID,
               "cf_infinite_attn_fwd: K > 0 needs W and positive dist_max, wscale");
    cudaStream_t s = as_stream(stream);
    PhiArgs phi{};
    phi.a = a; phi.pos = pos; phi.pos_ij = pos_ij; phi.tvecs = tvecs; phi.batch = batch; phi.edges = edges; phi.rvlen = rvlen; phi.z = logit;
    phi.E = E; phi.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    phi.floor_log2 = weight_floor_log2();
    // rows with a basis expansion differ widely in cost and are drawn through a ticket, which the phi launch zeroes;
    // without one (K = 0) rows are cheap and uniform and are dealt round-robin
    // (ticket_ready: a ticket that an earlier operation on this stream has zeroed already)
    unsigned *ticket = K > 0 ? (ticket_ready != nullptr ? ticket_ready : next_ticket()) : nullptr;
    CF_REQUIRE(K == 0 || ticket != nullptr, CF_ERR_CUDA, "cf_infinite_attn_fwd: the row ticket could not be set up");
    phi.zero_word = ticket;
    // With term lists and rows of at most 32 keys the row kernel sums phi from the lists itself (one launch less per
    // layer, and the lists are read while they are needed).  Rows of more keys keep the phi kernel: with four lanes per
    // key and one block per row the same sums took longer inside the row kernel (64 crystals of 100-200 atoms: 663
    // against 621 us per call).
    const bool phi_in_row = list != nullptr && pos_ij != nullptr && K > 0 && max_atoms <= 32;
    int rc = CF_OK;
    if (phi_in_row) {
        if (ticket_ready == nullptr && cudaMemsetAsync(ticket, 0, sizeof(unsigned), s) != cudaSuccess)
            rc = launch_status("row ticket");
    } else if (list != nullptr && pos_ij != nullptr) {
        PhiListArgs pl{};
        pl.list = *list;
        pl.a = a; pl.pos_ij = pos_ij; pl.tvecs = tvecs; pl.rvlen = rvlen; pl.batch = batch; pl.edges = edges; pl.E = E;
        pl.rule = phi.rule; pl.floor_log2 = phi.floor_log2; pl.z = logit; pl.zero_word = ticket;
        rc = launch_phi_from_list(pl, s);
    } else {
        rc = launch_lattice_phi(phi, s);
    }
    if (rc != CF_OK) return rc;

    RowArgs p{};
    p.q = q; p.k = k; p.v = v; p.a = a; p.pos = pos; p.pos_ij = pos_ij; p.tvecs = tvecs; p.rvlen = rvlen; p.W = W;
    p.batch = batch; p.edges = edges; p.row_start = row_start; p.row_order = row_order; p.E = E;
    p.out = out; p.logit = logit; p.lse = lse; p.psi_row = psi_row; p.N = N; p.max_atoms = (int)max_atoms;
    p.keep_logit = 1;
    p.phi_in_row = phi_in_row ? 1 : 0;
    p.ticket = ticket;
    if (list != nullptr && pos_ij != nullptr && K > 0) p.list = *list;
    p.rule = phi.rule;
    p.basis = make_basis_params(K, dist_max, wscale, weight_floor_log2());
    return launch_rows(p, K, N, s, chained);
}

namespace cf {
// Launches the row kernel for `grid_rows` rows (the grid is sized for them; the kernel itself processes p.N rows, or
// *p.rows_on_device).  Warps per atom row: 1 for crystals of up to 12 atoms, else 4 (fewer warps per row keep more
// rows in flight but stretch the heaviest rows, which bound the kernel).
int launch_rows(const RowArgs &p, int64_t K, long long grid_rows, cudaStream_t s, bool chained)
{
    const int max_atoms = p.max_atoms;
    const int row_warps = max_atoms <= 12 ? 1 : WARPS;
    const int groups = WARPS / row_warps;
    const size_t smem = sizeof(float) * groups * row_group_floats(max_atoms, K > 0, row_warps);
    void (*kernel)(const RowArgs);
    // left-over rows of the sorted path without a basis, or of more than 32 keys: phi enumerated inside the row
    const bool enum_phi = p.phi_in_row != 0 && (K == 0 || max_atoms > 32);
    if (enum_phi)
        kernel = K > 0 ? infinite_attn_rows_kernel<64, 4, true>
                       : (row_warps == 1 ? infinite_attn_rows_kernel<0, 1, true> : infinite_attn_rows_kernel<0, 4, true>);
    else if (K > 0)
        kernel = row_warps == 1 ? infinite_attn_rows_kernel<64, 1> : infinite_attn_rows_kernel<64, 4>;
    else
        kernel = row_warps == 1 ? infinite_attn_rows_kernel<0, 1> : infinite_attn_rows_kernel<0, 4>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return fail(CF_ERR_RANGE, "cf_infinite_attn_fwd: %zu bytes of shared memory for max_atoms=%d not available",
                        smem, max_atoms);
        }
    }
    static thread_local size_t cached_smem[8] = {};
    static thread_local int cached_occ[8] = {};
    const int slot = (K > 0 ? 2 : 0) + (row_warps == 1 ? 0 : 1) + (enum_phi ? 4 : 0);
    if (cached_occ[slot] == 0 || cached_smem[slot] != smem) {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, THREADS, smem) != cudaSuccess || occ <= 0) occ = 1;
        cached_occ[slot] = occ;
        cached_smem[slot] = smem;
    }
    const long long want = (grid_rows + groups - 1) / groups;
    const long long cap = (long long)sm_count() * cached_occ[slot];
    const int blocks = (int)(want < cap ? want : cap);
    launch_chained(kernel, dim3(blocks), dim3(THREADS), smem, s, chained, p);
    return launch_status("cf_infinite_attn_fwd");
}

// The rows that the sorted row kernel (infinite_attn_sorted.cu) left over: atoms rows[0 .. *count), processed by the
// row kernel above without lists (phi and the candidates by enumeration).  `ticket` must be zero on entry.
int launch_leftover_rows(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                         const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                         const int64_t *row_start, int64_t N, int64_t E, int64_t max_atoms, double dist_max,
                         double wscale, const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                         float *out, float *lse, const int *rows, const unsigned *count, unsigned *ticket, int64_t K,
                         cudaStream_t s)
{
    RowArgs p{};
    p.q = q; p.k = k; p.v = v; p.a = a; p.pos_ij = pos_ij; p.tvecs = tvecs; p.rvlen = rvlen; p.W = W;
    p.batch = batch; p.edges = edges; p.row_start = row_start; p.row_order = rows; p.rows_on_device = count; p.E = E;
    p.out = out; p.logit = nullptr; p.lse = lse; p.psi_row = nullptr; p.N = N; p.max_atoms = (int)max_atoms;
    p.keep_logit = 0;
    p.phi_in_row = 1;  // no list: every edge's phi is enumerated inside the row kernel
    p.ticket = ticket;
    p.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    p.basis = make_basis_params(K, dist_max, wscale, weight_floor_log2());
    // left-over rows are rare: a grid of one block per SM draws them through the ticket
    return launch_rows(p, K, (long long)sm_count() * (max_atoms <= 12 ? WARPS : 1), s, true);
}
}  // namespace cf

unsigned *cf::row_ticket_block(int count) { return next_ticket_block(count); }
