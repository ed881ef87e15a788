// Term lists (see term_list.cuh): the build kernel and phi from a list.
#include "lattice_core.cuh"
#include "term_list.cuh"

namespace cf {
namespace {

// Threads per row of the build: 128 for batches of small crystals (many rows, short walks), 256 when crystals have
// more than 32 atoms (the warps split a row's columns, so a long row finishes sooner).

// Enumerates the terms of one 32-key chunk of a row that belong to warp `wr` (columns dealt round-robin, rotated by
// the chunk as in the row kernel) and calls visit(d2, n1, n2, n3) for every term of this lane's key with d2 <= thr.
template <int TL_WARPS, class Visit>
__device__ __forceinline__ void walk_chunk(const Cell &cell, int R1, int R2, int R3, float4 r, float thr, bool live,
                                           int ch, int wr, Visit &&visit)
{
    const int S2 = 2 * R2 + 1, columns = (2 * R1 + 1) * S2;
    const float t3sq = fmaf(cell.t3z, cell.t3z, fmaf(cell.t3y, cell.t3y, cell.t3x * cell.t3x));
    const bool prune = t3sq > 1e-12f;
    const float inv_t3sq = prune ? __frcp_rn(t3sq) : 0.f;
    // no key of the chunk farther than `far` from the origin, no listed term farther than sqrt(thr) from its key
    const float far2 = warp_max(live ? fmaf(r.z, r.z, fmaf(r.y, r.y, r.x * r.x)) : 0.f);
    const float reach2 = warp_max(live ? thr : 0.f);
    const float bound = sqrtf(fmaxf(reach2, 0.f)) + sqrtf(far2);
    const float tau2_max = bound * bound * 1.0001f + 1e-4f;
    int col = (wr - ch) & (TL_WARPS - 1);
    int n1 = -R1, n2 = col - R2;
    while (n2 > R2) { n2 -= S2; ++n1; }
    for (; col < columns; col += TL_WARPS) {
        const float f1 = (float)n1, f2 = (float)n2;
        const float bx = fmaf(cell.t2x, f2, cell.t1x * f1), by = fmaf(cell.t2y, f2, cell.t1y * f1);
        const float bz = fmaf(cell.t2z, f2, cell.t1z * f1);
        const float bb = fmaf(bz, bz, fmaf(by, by, bx * bx));
        const float bt = fmaf(bz, cell.t3z, fmaf(by, cell.t3y, bx * cell.t3x));
        const float room = fmaf(bb, 1e-5f, tau2_max) - fmaf(-bt * bt, inv_t3sq, bb);
        int lo = -R3, hi = R3;
        if (prune) {
            const float half = sqrtf(fmaxf(room, 0.f) * inv_t3sq) + 1e-3f, mid = -bt * inv_t3sq;
            lo = max(lo, __float2int_ru(mid - half));
            hi = min(hi, __float2int_rd(mid + half));
            if (room < 0.f) hi = lo - 1;
        }
        // r + n1 t1 + n2 t2 + n3 t3, contracted like the reference's expression
        const float ex = fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, r.x));
        const float ey = fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, r.y));
        const float ez = fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, r.z));
        for (int n3 = lo; n3 <= hi; ++n3) {
            const float f3 = (float)n3;
            const float dx = fmaf(cell.t3x, f3, ex), dy = fmaf(cell.t3y, f3, ey), dz = fmaf(cell.t3z, f3, ez);
            const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
            if (live && d2 <= thr) visit(d2, n1, n2, n3);
        }
        n2 += TL_WARPS;
        while (n2 > R2) { n2 -= S2; ++n1; }
    }
}

template <int TL_THREADS>
__global__ void __launch_bounds__(TL_THREADS) term_list_build_kernel(const TermListBuild p)
{
    constexpr int TL_WARPS = TL_THREADS / 32;
    extern __shared__ int smem_i[];
    int *cntw = smem_i;                                      // [4][max_atoms] entries per (warp, key)
    float *thr = reinterpret_cast<float *>(cntw + TL_WARPS * p.max_atoms);  // [max_atoms] d2 threshold per key
    float *minw = thr + p.max_atoms;                         // [4][max_atoms] smallest listed d2 per (warp, key)
    __shared__ long long base_sh;
    __shared__ int scan_sh[TL_THREADS];
    const int tid = threadIdx.x, lane = tid & 31, wr = tid >> 5;

    for (long long slot = blockIdx.x; slot < p.N; slot += gridDim.x) {
        const long long i = p.row_order ? p.row_order[slot] : slot;
        const long long c = p.batch[i];
        const long long e0 = p.row_start[i];
        const int n = (int)(p.row_start[i + 1] - e0);
        if (n > p.max_atoms) {  // the caller understated max_atoms: no list, the row kernel poisons the row
            for (int j = tid; j < n; j += TL_THREADS) p.start[e0 + j] = -1;
            continue;
        }
        Cell cell;
        cell.load(p.tvecs + 9 * c);
        float rvl[3] = {0.f, 0.f, 0.f};
        if (p.rvlen) { rvl[0] = p.rvlen[3 * c]; rvl[1] = p.rvlen[3 * c + 1]; rvl[2] = p.rvlen[3 * c + 2]; }
        const int pk = packed_box(p.rule, p.a_widest, p.rvlen ? rvl : nullptr);  // contains every head's box
        const int R1 = box_r1(pk), R2 = box_r2(pk), R3 = box_r3(pk);
        // ---- threshold per key: (an upper bound of the smallest squared distance ANY head's box can contain) + D.
        //      Boxes of half-width >= 1 contain the 27 nearest translations; otherwise only n = 0 is certain.
        const bool near27 = p.rule.cutoff == 0.0f ? true : p.rule.minimum_range >= 1;
        __syncthreads();  // the previous row's readers are done with the tables
        for (int j = tid; j < n; j += TL_THREADS) {
            const float *pp = p.pos_ij + 3 * (e0 + j);
            const float rx = pp[0], ry = pp[1], rz = pp[2];
            float m = fmaf(rz, rz, fmaf(ry, ry, rx * rx));
            if (near27) {
                const int q1 = min(R1, 1), q2 = min(R2, 1), q3 = min(R3, 1);
                for (int n1 = -q1; n1 <= q1; ++n1)
                    for (int n2 = -q2; n2 <= q2; ++n2)
                        for (int n3 = -q3; n3 <= q3; ++n3) {
                            const float f1 = (float)n1, f2 = (float)n2, f3 = (float)n3;
                            const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx)));
                            const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry)));
                            const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz)));
                            m = fminf(m, fmaf(dz, dz, fmaf(dy, dy, dx * dx)));
                        }
            }
            thr[j] = m + p.window;
        }
        __syncthreads();
        const int chunks = (n + 31) >> 5;
        // ---- pass A: entries per (warp, key)
        for (int ch = 0; ch < chunks; ++ch) {
            const int j = 32 * ch + lane;
            const bool live = j < n;
            const float *pp = p.pos_ij + 3 * (e0 + (live ? j : 0));
            const float4 r = make_float4(pp[0], pp[1], pp[2], 0.f);
            int cnt = 0;
            float dm = INFINITY;
            walk_chunk<TL_WARPS>(cell, R1, R2, R3, r, live ? thr[j] : 0.f, live, ch, wr, [&](float d2, int, int, int) {
                ++cnt;
                dm = fminf(dm, d2);
            });
            if (live) {
                cntw[wr * p.max_atoms + j] = cnt;
                minw[wr * p.max_atoms + j] = dm;
            }
        }
        __syncthreads();
        // ---- exclusive scan in (key, warp) order: thread t owns a contiguous range of keys
        const int per = (n + TL_THREADS - 1) / TL_THREADS;
        const int j_lo = min(tid * per, n), j_hi = min(j_lo + per, n);
        int mine = 0;
        for (int j = j_lo; j < j_hi; ++j)
            for (int w = 0; w < TL_WARPS; ++w) mine += cntw[w * p.max_atoms + j];
        int incl = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(FULL, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) scan_sh[wr] = incl;
        __syncthreads();
        int before = 0, total = 0;
        for (int w = 0; w < TL_WARPS; ++w) {
            if (w < wr) before += scan_sh[w];
            total += scan_sh[w];
        }
        if (tid == 0) {
            const unsigned long long at = atomicAdd(p.cursor, (unsigned long long)total);
            base_sh = (at + (unsigned long long)total <= (unsigned long long)p.capacity) ? (long long)at : -1;
        }
        __syncthreads();
        const long long base = base_sh;
        if (base < 0 || base + total >= (1ll << 31)) {  // the pool is full: this row is processed by enumeration
            for (int j = tid; j < n; j += TL_THREADS) p.start[e0 + j] = -1;
            continue;
        }
        // counts -> offsets (in place), and the per-edge directory
        int run = before + incl - mine;
        for (int j = j_lo; j < j_hi; ++j) {
            p.start[e0 + j] = (int)base + run;
            int edge_total = 0;
            for (int w = 0; w < TL_WARPS; ++w) {
                const int v = cntw[w * p.max_atoms + j];
                cntw[w * p.max_atoms + j] = run;
                run += v;
                edge_total += v;
            }
            p.count[e0 + j] = edge_total;
            float dm = minw[j];
            for (int w = 1; w < TL_WARPS; ++w) dm = fminf(dm, minw[w * p.max_atoms + j]);
            p.dmin[e0 + j] = dm;
        }
        __syncthreads();
        // ---- pass B: the same walk, writing
        for (int ch = 0; ch < chunks; ++ch) {
            const int j = 32 * ch + lane;
            const bool live = j < n;
            const float *pp = p.pos_ij + 3 * (e0 + (live ? j : 0));
            const float4 r = make_float4(pp[0], pp[1], pp[2], 0.f);
            float2 *out = p.pool + base + (live ? cntw[wr * p.max_atoms + j] : 0);
            walk_chunk<TL_WARPS>(cell, R1, R2, R3, r, live ? thr[j] : 0.f, live, ch, wr, [&](float d2, int n1, int n2, int n3) {
                *out++ = make_float2(d2, __int_as_float(pack_key(j, abs(n1), abs(n2), abs(n3))));
            });
        }
    }
}

// TPE (1, 2, 4 or 8) lanes per edge: phi of all heads from the edge's entries (boxes applied per head).  The lanes of
// a group split the eight box computations, read the entries sub, sub + TPE, ... (the group's loads are contiguous)
// and keep partial sums for all heads, combined by a fixed butterfly.  Few lanes per edge for batches of many edges
// with short lists (large cells), eight for few edges with long lists (small cells).  Rows without a list, and edges
// where a head's box misses every listed term, take the enumerating code.
template <int TPE>
__global__ void __launch_bounds__(128) phi_from_list_kernel(const PhiListArgs p)
{
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gtid == 0 && p.zero_word) *p.zero_word = 0u;
    const long long e_raw = gtid / TPE;
    const int sub = (int)(gtid % TPE);
    const bool live = e_raw < p.E;
    const long long e = live ? e_raw : p.E - 1;  // idle tail lanes shadow the last edge so that shuffles stay full
    const long long i = p.edges[e];
    const long long c = p.batch[i];
    float rvl[3] = {0.f, 0.f, 0.f};
    if (p.rvlen) { rvl[0] = p.rvlen[3 * c]; rvl[1] = p.rvlen[3 * c + 1]; rvl[2] = p.rvlen[3 * c + 2]; }
    constexpr int PER = 8 / TPE;  // heads whose box this lane computes
    const int lane = threadIdx.x & 31, group0 = lane & ~(TPE - 1);
    float a_mine[PER];
    int pk_mine[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
        a_mine[u] = p.a[i * HEADS + sub * PER + u];
        pk_mine[u] = packed_box(p.rule, a_mine[u], p.rvlen ? rvl : nullptr);
    }
    float a[8], a2[8];
    int pk[8];
    float a2max = -INFINITY;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        a[h] = __shfl_sync(FULL, a_mine[h % PER], group0 + h / PER);
        pk[h] = __shfl_sync(FULL, pk_mine[h % PER], group0 + h / PER);
        a2[h] = a[h] * LOG2E;
        a2max = fmaxf(a2max, a2[h]);
    }
    float z[8];
    const int first = p.list.start[e];
    const int cnt = first >= 0 ? p.list.count[e] : 0;
    const float m = first >= 0 ? p.list.dmin[e] : 0.f;
    const float2 *ent = p.list.pool + (first >= 0 ? first : 0);
    float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // entries are requested two steps ahead of their use: the lists stream from memory, and a step is short
    float2 n0 = make_float2(0.f, 0.f), n1 = n0;
    if (sub < cnt) n0 = __ldg(ent + sub);
    if (sub + TPE < cnt) n1 = __ldg(ent + sub + TPE);
    for (int t = sub; t < cnt; t += TPE) {
        const float2 en = n0;
        n0 = n1;
        if (t + 2 * TPE < cnt) n1 = __ldg(ent + t + 2 * TPE);
        const float rel = en.x - m;
        if (a2max * rel < p.floor_log2) continue;  // below the floor for every head
        const int key = __float_as_int(en.y);
#pragma unroll
        for (int h = 0; h < 8; ++h)
            if (key_in_box(key, pk[h])) s[h] += ex2(a2[h] * rel);
    }
    bool done = cnt > 0;
#pragma unroll
    for (int h = 0; h < 8; ++h) {  // (all lanes of the warp take part in the shuffles, listed or not)
        float t = s[h];
#pragma unroll
        for (int o = 1; o < TPE; o <<= 1) t += __shfl_xor_sync(FULL, t, o);
        z[h] = fmaf(m, a[h], logf(t));
        done = done && t > 1e-30f;  // a head whose box misses the listed terms: enumerate instead
    }
    if (!done && sub == 0) {
        Cell cell;
        cell.load(p.tvecs + 9 * c);
        edge_phi<1>(p.rule, a, p.rvlen ? p.rvlen + 3 * c : nullptr, cell, p.pos_ij[3 * e], p.pos_ij[3 * e + 1],
                    p.pos_ij[3 * e + 2], p.floor_log2, 0, z);
    }
    if (live && sub == 0) {
        float4 *zo = reinterpret_cast<float4 *>(p.z + e * HEADS);
        zo[0] = make_float4(z[0], z[1], z[2], z[3]);
        zo[1] = make_float4(z[4], z[5], z[6], z[7]);
    }
}

}  // namespace

// About 25 entries per edge are needed for cells of 3-15 Angstrom edges at the default widths (sphere of the window
// over the cell volume), 3 for cells of 10-25 Angstrom; rows that do not fit are enumerated instead.
size_t term_pool_entries(long long N, long long E) { return (size_t)(32 * E + 64 * N + (1ll << 20)); }

size_t term_list_workspace_bytes(long long N, long long E)
{
    return sizeof(int) * (3 * (size_t)E + 32) + sizeof(float2) * term_pool_entries(N, E);
}

void term_list_carve(void *workspace, long long N, long long E, int **start, int **count, float **dmin,
                     unsigned long long **cursor, float2 **pool)
{
    (void)N;
    auto align = [](const void *ptr, uintptr_t to) { return (reinterpret_cast<uintptr_t>(ptr) + to - 1) & ~(to - 1); };
    int *dir = static_cast<int *>(workspace);
    *start = dir;
    *count = dir + E;
    *dmin = reinterpret_cast<float *>(dir + 2 * E);
    *cursor = reinterpret_cast<unsigned long long *>(align(dir + 3 * E, 8));
    *pool = reinterpret_cast<float2 *>(align(dir + 3 * E + 8, 16));
}

int launch_term_list_build(const TermListBuild &b, cudaStream_t s)
{
    if (b.N == 0) return CF_OK;
    if (cudaMemsetAsync(b.cursor, 0, sizeof(unsigned long long), s) != cudaSuccess) return launch_status("term list cursor");
    const int threads = b.max_atoms <= 32 ? 128 : 256;
    const size_t smem = sizeof(int) * (2 * (threads / 32) + 1) * (size_t)b.max_atoms;
    auto kernel = threads == 128 ? term_list_build_kernel<128> : term_list_build_kernel<256>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return fail(CF_ERR_RANGE, "term list: %zu bytes of shared memory for max_atoms=%d not available", smem, b.max_atoms);
        }
    }
    const long long cap = (long long)sm_count() * 8;
    kernel<<<(unsigned)(b.N < cap ? b.N : cap), threads, smem, s>>>(b);
    return launch_status("term_list_build_kernel");
}

int launch_phi_from_list(const PhiListArgs &p, cudaStream_t s)
{
    if (p.E == 0) return CF_OK;
    // lanes per edge: as many as keep the grid at a few waves of the SMs
    const long long per_wave = (long long)sm_count() * 2048;
    const int tpe = p.E * 8 <= 4 * per_wave ? 8 : (p.E * 4 <= 4 * per_wave ? 4 : (p.E * 2 <= 4 * per_wave ? 2 : 1));
    const unsigned blocks = (unsigned)((p.E * tpe + 127) / 128);
    switch (tpe) {
        case 8: phi_from_list_kernel<8><<<blocks, 128, 0, s>>>(p); break;
        case 4: phi_from_list_kernel<4><<<blocks, 128, 0, s>>>(p); break;
        case 2: phi_from_list_kernel<2><<<blocks, 128, 0, s>>>(p); break;
        default: phi_from_list_kernel<1><<<blocks, 128, 0, s>>>(p); break;
    }
    return launch_status("phi_from_list_kernel");
}

}  // namespace cf

extern "C" int64_t cf_term_list_workspace_bytes(int64_t N, int64_t E)
{
    return (int64_t)cf::term_list_workspace_bytes(N, E);
}

extern "C" int cf_term_list_build(const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                                  const int64_t *edges, const int64_t *row_start, const int32_t *row_order, int64_t N,
                                  int64_t E, int64_t max_atoms, double cutoff_radius, int lattice_range,
                                  int minimum_range, double a_widest, void *workspace, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_term_list_build: negative size");
    CF_REQUIRE(a_widest < 0, CF_ERR_INVALID, "cf_term_list_build: a_widest must be negative");
    CF_REQUIRE(max_atoms >= 1 && max_atoms <= 2048, CF_ERR_RANGE, "cf_term_list_build: max_atoms=%lld outside [1,2048]",
               (long long)max_atoms);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_term_list_build: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (N == 0) return CF_OK;
    CF_REQUIRE(pos_ij && tvecs && batch && edges && row_start && workspace, CF_ERR_INVALID, "cf_term_list_build: null pointer");
    TermListBuild tb{};
    tb.pos_ij = pos_ij; tb.tvecs = tvecs; tb.rvlen = cutoff_radius != 0.0 ? rvlen : nullptr;
    tb.batch = batch; tb.edges = edges; tb.row_start = row_start; tb.row_order = row_order;
    tb.N = N; tb.E = E; tb.max_atoms = (int)max_atoms;
    tb.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    tb.a_widest = (float)a_widest;
    tb.window = term_window(weight_floor_log2(), (float)a_widest);
    term_list_carve(workspace, N, E, &tb.start, &tb.count, &tb.dmin, &tb.cursor, &tb.pool);
    tb.capacity = (long long)term_pool_entries(N, E);
    return launch_term_list_build(tb, as_stream(stream));
}
