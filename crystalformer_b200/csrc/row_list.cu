// Row lists (see row_list.cuh): the build kernel.
#include "lattice_core.cuh"
#include "row_list.cuh"
#include "term_list.cuh"

namespace cf {
namespace {

constexpr int RL_THREADS = 256;
constexpr int RL_WARPS = RL_THREADS / 32;
constexpr int RL_BUCKETS = 2 * RL_THREADS;  // (the scan below takes two buckets per thread)
constexpr int RL_MAX_TRANSLATIONS = 4096;  // boxes beyond this are not listed
constexpr size_t RL_SMEM = sizeof(unsigned long long) * 2 * ROW_LIST_CAP + sizeof(int) * (2 * RL_BUCKETS + 8);

// One thread block per row.  Every key's candidate translations (a bounding box of the ball that holds its listed
// terms) are walked by a warp, one per lane and step; terms within `window` of their edge's nearest image are appended to a
// shared-memory buffer (one atomic per warp and step) as 64-bit items (d2 bits << 32 | key).  The items are then
// sorted: distributed over RL_BUCKETS buckets that are equally spaced in d^3 (terms are about uniform in volume, so
// buckets hold a handful of items each), and placed inside their bucket by counting the smaller items of the same
// bucket.  The 64-bit items are distinct except for exact duplicates, so the result does not depend on the order in
// which the atomics arrived.  Four warps per row: most of a row's cost is per thread (set-up, scans, barriers), not
// per item.
__global__ void __launch_bounds__(RL_THREADS) row_list_build_kernel(const RowListBuild p)
{
    extern __shared__ __align__(16) unsigned long long rl_smem[];
    unsigned long long *ent = rl_smem, *ent2 = rl_smem + ROW_LIST_CAP;
    int *hist = reinterpret_cast<int *>(ent2 + ROW_LIST_CAP);  // [RL_BUCKETS] counts, then running cursors
    int *offs = hist + RL_BUCKETS;                             // [RL_BUCKETS] first position of every bucket
    int *wsum = offs + RL_BUCKETS;                             // [RL_WARPS]
    __shared__ int dmin_s[ROW_LIST_MAX_KEYS];
    __shared__ float4 key_s[ROW_LIST_MAX_KEYS];                // relative position of every key, .w = its threshold
    __shared__ int cnt_s;
    __shared__ int4 kbox_s[ROW_LIST_MAX_KEYS];                 // first translation of every key's box, its widths w3 | w2 << 8
    __shared__ int kcnt_s[ROW_LIST_MAX_KEYS];                  // translations in every key's box
    __shared__ float d2max_s[ROW_LIST_MAX_KEYS / 32];          // largest threshold among every 32 keys
    __shared__ long long base_s;
    const int tid = threadIdx.x, lane = tid & 31, wr = tid >> 5;
    const unsigned lt = (1u << lane) - 1u;

    for (long long slot = blockIdx.x; slot < p.N; slot += gridDim.x) {
        const long long i = p.row_order ? p.row_order[slot] : slot;
        const long long c = p.batch[i];
        const long long e0 = p.row_start[i];
        const int n = (int)(p.row_start[i + 1] - e0);
        const long long a0 = n > 0 ? p.edges[p.E + e0] : i;
        __syncthreads();  // the previous row's readers are done with the shared buffers
        if (tid == 0) cnt_s = 0;
        if (tid < ROW_LIST_MAX_KEYS) dmin_s[tid] = 0x7f800000;  // +inf
        for (int b = tid; b < RL_BUCKETS; b += RL_THREADS) hist[b] = 0;
        Cell cell;
        cell.load(p.tvecs + 9 * c);
        float rvl[3] = {0.f, 0.f, 0.f};
        if (p.rvlen) { rvl[0] = p.rvlen[3 * c]; rvl[1] = p.rvlen[3 * c + 1]; rvl[2] = p.rvlen[3 * c + 2]; }
        const int pk = packed_box(p.rule, p.a_widest, p.rvlen ? rvl : nullptr);  // contains every head's box
        const int R1 = box_r1(pk), R2 = box_r2(pk), R3 = box_r3(pk);
        const int S2 = 2 * R2 + 1, S3 = 2 * R3 + 1, T = (2 * R1 + 1) * S2 * S3;
        // boxes of more than RL_MAX_TRANSLATIONS translations (tiny or nearly flat cells) are left to the enumerating
        // kernel, which prunes its walk
        const bool fits = n >= 1 && n <= ROW_LIST_MAX_KEYS && T <= RL_MAX_TRANSLATIONS;
        if (fits) {
            // ---- threshold of every key: (an upper bound of the smallest squared distance ANY head's box can contain)
            //      + window.  Boxes of half-width >= 1 contain the 27 nearest translations (one per lane); otherwise
            //      only n = 0 is certain.
            const bool near27 = p.rule.cutoff == 0.0f ? true : p.rule.minimum_range >= 1;
            const int q1 = min(R1, 1), q2 = min(R2, 1), q3 = min(R3, 1);
            const float g1 = (float)(lane / 9 - 1), g2 = (float)((lane / 3) % 3 - 1), g3 = (float)(lane % 3 - 1);
            const bool probe = lane < 27 && near27 && fabsf(g1) <= (float)q1 && fabsf(g2) <= (float)q2 && fabsf(g3) <= (float)q3;
            for (int j = wr; j < n; j += RL_WARPS) {
                const float *pp = p.pos_ij + 3 * (e0 + j);
                const float rx = pp[0], ry = pp[1], rz = pp[2];
                float m = fmaf(rz, rz, fmaf(ry, ry, rx * rx));
                if (probe) {
                    const float dx = fmaf(cell.t3x, g3, fmaf(cell.t2x, g2, fmaf(cell.t1x, g1, rx)));
                    const float dy = fmaf(cell.t3y, g3, fmaf(cell.t2y, g2, fmaf(cell.t1y, g1, ry)));
                    const float dz = fmaf(cell.t3z, g3, fmaf(cell.t2z, g2, fmaf(cell.t1z, g1, rz)));
                    m = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                }
                m = warp_min(m);
                if (lane == 0) key_s[j] = make_float4(rx, ry, rz, m + p.window);
            }
        }
        __syncthreads();
        // ---- the walk.  A key's listed terms lie in the ball |r + n1 t1 + n2 t2 + n3 t3|^2 <= threshold, a small part of
        //      the box of the cut-off rule: with b_i the reciprocal rows (b_i . t_j = delta_ij), (r + n T) . b_i =
        //      s_i + n_i and |x . b_i| <= |x| |b_i| bound every digit,
        //          | n_i + s_i | <= rho |b_i|,      s_i = r . b_i,  rho = sqrt(threshold).
        //      The first warps compute every key's bounding box, clipped to the rule's box (one key per lane; the
        //      bounds are widened a little beyond any rounding, the test on d2 below decides membership, so the listed
        //      set is that of a walk of the whole box); then the warps take the keys in turn, lanes over the
        //      translations of a key's box.
        if (fits && wr < ROW_LIST_MAX_KEYS / 32) {
            const int key = 32 * wr + lane;
            const float c1x = cell.t2y * cell.t3z - cell.t2z * cell.t3y, c1y = cell.t2z * cell.t3x - cell.t2x * cell.t3z,
                        c1z = cell.t2x * cell.t3y - cell.t2y * cell.t3x;
            const float c2x = cell.t3y * cell.t1z - cell.t3z * cell.t1y, c2y = cell.t3z * cell.t1x - cell.t3x * cell.t1z,
                        c2z = cell.t3x * cell.t1y - cell.t3y * cell.t1x;
            const float c3x = cell.t1y * cell.t2z - cell.t1z * cell.t2y, c3y = cell.t1z * cell.t2x - cell.t1x * cell.t2z,
                        c3z = cell.t1x * cell.t2y - cell.t1y * cell.t2x;
            const float det = cell.t1x * c1x + cell.t1y * c1y + cell.t1z * c1z;
            const bool prune = fabsf(det) > 1e-12f;  // (a flat cell keeps the whole box)
            const float idet = prune ? 1.0f / det : 0.0f;
            int lo1 = -R1, hi1 = R1, lo2 = -R2, hi2 = R2, lo3 = -R3, hi3 = R3;
            const float4 r = key < n ? key_s[key] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (prune) {
                const float rho = sqrtf(fmaxf(r.w, 0.f)) * 1.0001f;
                const float m1 = rho * sqrtf(c1x * c1x + c1y * c1y + c1z * c1z) * fabsf(idet) + 1e-3f;
                const float m2 = rho * sqrtf(c2x * c2x + c2y * c2y + c2z * c2z) * fabsf(idet) + 1e-3f;
                const float m3 = rho * sqrtf(c3x * c3x + c3y * c3y + c3z * c3z) * fabsf(idet) + 1e-3f;
                const float s1 = (r.x * c1x + r.y * c1y + r.z * c1z) * idet, s2 = (r.x * c2x + r.y * c2y + r.z * c2z) * idet,
                            s3 = (r.x * c3x + r.y * c3y + r.z * c3z) * idet;
                // (clamped as floats first: the conversions then see small values only)
                lo1 = (int)ceilf(fmaxf(-m1 - s1, (float)-R1)); hi1 = (int)floorf(fminf(m1 - s1, (float)R1));
                lo2 = (int)ceilf(fmaxf(-m2 - s2, (float)-R2)); hi2 = (int)floorf(fminf(m2 - s2, (float)R2));
                lo3 = (int)ceilf(fmaxf(-m3 - s3, (float)-R3)); hi3 = (int)floorf(fminf(m3 - s3, (float)R3));
            }
            const int w1 = max(hi1 - lo1 + 1, 0), w2 = max(hi2 - lo2 + 1, 0), w3 = max(hi3 - lo3 + 1, 0);
            kcnt_s[key] = key < n ? w1 * w2 * w3 : 0;
            kbox_s[key] = make_int4(lo1, lo2, lo3, max(w3, 1) | (max(w2, 1) << 8));
            const float top = warp_max(key < n ? r.w : 1.0f);
            if (lane == 0) d2max_s[wr] = fmaxf(top, 1.0f);
        }
        __syncthreads();
        float d2_max = 1.0f;  // no listed term is farther (the same value in every thread)
        if (fits) {
#pragma unroll
            for (int u = 0; u < ROW_LIST_MAX_KEYS / 32; ++u) d2_max = fmaxf(d2_max, d2max_s[u]);
        }
        if (fits) {
            // a warp takes a key at a time, its lanes the translations of the key's box (32 per pass)
            for (int j = wr; j < n; j += RL_WARPS) {
                const int4 kb = kbox_s[j];
                const float4 r = key_s[j];
                const int count = kcnt_s[j];
                const int w3 = kb.w & 255, w2 = kb.w >> 8;
                const float inv_w3 = __frcp_rn((float)w3), inv_w2 = __frcp_rn((float)w2);
                for (int tr0 = 0; tr0 < count; tr0 += 32) {  // (warp-uniform bounds: the ballots below are safe)
                    const int tr = tr0 + lane;
                    // digits of tr in the mixed radix (w1, w2, w3): quotients by a rounded-down product with the
                    // reciprocal (exact for these small integers: tr < 2^13, w <= 65)
                    const int i12 = __float2int_rd(((float)tr + 0.5f) * inv_w3), i3 = tr - i12 * w3;
                    const int i1 = __float2int_rd(((float)i12 + 0.5f) * inv_w2), i2 = i12 - i1 * w2;
                    const int n1 = kb.x + i1, n2 = kb.y + i2, n3 = kb.z + i3;
                    const float f1 = (float)n1, f2 = (float)n2, f3 = (float)n3;
                    // r + n1 t1 + n2 t2 + n3 t3, contracted like the reference's expression
                    const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, r.x)));
                    const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, r.y)));
                    const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, r.z)));
                    const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                    const bool keep = tr < count && d2 <= r.w;
                    const unsigned mask = __ballot_sync(FULL, keep);
                    if (mask == 0u) continue;
                    int base = 0;
                    if (lane == 0) base = atomicAdd(&cnt_s, __popc(mask));
                    base = __shfl_sync(FULL, base, 0);
                    if (keep) {
                        const int at = base + __popc(mask & lt);
                        const int key123 = (abs(n1) << 8) | (abs(n2) << 16) | (abs(n3) << 24);
                        if (at < ROW_LIST_CAP) ent[at] = ((unsigned long long)__float_as_uint(d2) << 32) | (unsigned)(key123 | j);
                    }
                }
            }
        }
        __syncthreads();
        const int total = cnt_s;
        const bool sortable = fits && total >= 1 && total <= ROW_LIST_CAP;
        const int chunks = (total + 7) >> 3, out_total = chunks << 3;
        if (sortable) {
            // ---- bucket of an item: about floor(RL_BUCKETS (d / d_max)^3) - terms are roughly uniform in volume, so such
            //      buckets fill evenly - with x^1.5 replaced by x (0.35 + 0.65 x), x = d2 / d2_max: within a few
            //      percent of it on [0, 1] and, evaluated as below, non-decreasing in d2 float by float (products and
            //      fused multiply-adds of non-negative non-decreasing factors round monotonically), which is all the
            //      sort needs: the final order is that of the items themselves whatever the partition into buckets
            const float inv_d2max = 1.0f / d2_max;
            auto bucket_of = [&](unsigned long long item) {
                const float x = __uint_as_float((unsigned)(item >> 32)) * inv_d2max;
                return min(RL_BUCKETS - 1, (int)(x * fmaf(0.65f, x, 0.35f) * ((float)RL_BUCKETS * 0.999f)));
            };
            for (int t = tid; t < total; t += RL_THREADS) atomicAdd(&hist[bucket_of(ent[t])], 1);
            __syncthreads();
            // exclusive scan of the counts (two buckets per thread)
            {
                const int v0 = hist[2 * tid], v1 = hist[2 * tid + 1];
                int incl = v0 + v1;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const int up = __shfl_up_sync(FULL, incl, o);
                    if (lane >= o) incl += up;
                }
                if (lane == 31) wsum[wr] = incl;
                __syncthreads();
                int before = 0;
                for (int w = 0; w < wr; ++w) before += wsum[w];
                const int excl = before + incl - (v0 + v1);
                offs[2 * tid] = excl; offs[2 * tid + 1] = excl + v0;
                hist[2 * tid] = excl; hist[2 * tid + 1] = excl + v0;  // running cursors of the scatter
            }
            __syncthreads();
            for (int t = tid; t < total; t += RL_THREADS) {
                const unsigned long long item = ent[t];
                ent2[atomicAdd(&hist[bucket_of(item)], 1)] = item;
            }
            __syncthreads();
            // an item's place inside its bucket = the number of smaller items there (equal items: by position)
            for (int t = tid; t < total; t += RL_THREADS) {
                const unsigned long long item = ent2[t];
                const int b = bucket_of(item);
                const int lo = offs[b], hi = hist[b];  // (after the scatter the cursor of a bucket is its end)
                int rank = 0;
                for (int u = lo; u < hi; ++u) {
                    const unsigned long long other = ent2[u];
                    rank += (other < item || (other == item && u < t)) ? 1 : 0;
                }
                ent[lo + rank] = item;
                // smallest listed d2 of the item's key (d2 >= 0: the bit patterns order like the values)
                atomicMin(&dmin_s[(int)(item & 255u)], (int)(item >> 32));
            }
            if (tid == 0) {
                const unsigned long long at = atomicAdd(p.out.cursor, (unsigned long long)out_total);
                base_s = (at + (unsigned long long)out_total <= (unsigned long long)p.out.capacity &&
                          at + (unsigned long long)out_total < (1ull << 31)) ? (long long)at : -1;
            }
            __syncthreads();
        } else {
            if (tid == 0) base_s = -1;
            __syncthreads();
        }
        const long long base = base_s;
        if (base >= 0) {
            const unsigned last_d2 = (unsigned)(ent[total - 1] >> 32);
            for (int t = tid; t < out_total; t += RL_THREADS) {
                const unsigned long long v = ent[t < total ? t : 0];
                p.out.pool[base + t] = t < total ? make_float2(__uint_as_float((unsigned)(v >> 32)), __uint_as_float((unsigned)v))
                                                 : make_float2(__uint_as_float(last_d2), __int_as_float(ROW_PAD_KEY));
            }
            if (tid < n) p.out.dmin[e0 + tid] = __int_as_float(dmin_s[tid]);
        }
        if (tid == 0) {
            p.out.rowdir[2 * slot] = make_int4((int)i, (int)a0, n, (int)c);
            p.out.rowdir[2 * slot + 1] = make_int4(base >= 0 ? (int)base : -1, chunks, (int)e0, 0);
            // rows with long lists are shared by the warps of a block, the others take one warp each: two task lists
            // (filled in the order in which the blocks get here, which is about the order of the row directory)
            const bool heavy = base >= 0 && chunks > p.coop_chunks;
            p.out.tasks[(heavy ? 0 : p.N) + atomicAdd(p.out.task_count + (heavy ? 0 : 1), 1u)] = (int)slot;
        }
    }
}

inline size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

}  // namespace

size_t row_list_workspace_bytes(long long N, long long E)
{
    return up256(sizeof(int4) * 2 * (size_t)N) + up256(sizeof(float) * (size_t)E) + up256(sizeof(unsigned) * 4 * ROW_SCHED_SLOTS) +
           up256(sizeof(int) * (size_t)N) + up256(sizeof(int) * 2 * (size_t)N) + 256 + sizeof(float2) * term_pool_entries(N, E);
}

RowListView row_list_carve(void *workspace, long long N, long long E)
{
    char *at = static_cast<char *>(workspace);
    RowListView v{};
    v.rowdir = reinterpret_cast<int4 *>(at); at += up256(sizeof(int4) * 2 * (size_t)N);
    v.dmin = reinterpret_cast<float *>(at); at += up256(sizeof(float) * (size_t)E);
    v.sched = reinterpret_cast<unsigned *>(at); at += up256(sizeof(unsigned) * 4 * ROW_SCHED_SLOTS);
    v.leftover = reinterpret_cast<int *>(at); at += up256(sizeof(int) * (size_t)N);
    v.tasks = reinterpret_cast<int *>(at); at += up256(sizeof(int) * 2 * (size_t)N);
    v.cursor = reinterpret_cast<unsigned long long *>(at);
    v.task_count = reinterpret_cast<unsigned *>(at + 8); at += 256;
    v.pool = reinterpret_cast<float2 *>(at);
    v.capacity = (long long)term_pool_entries(N, E);
    return v;
}

int launch_row_list_build(const RowListBuild &b, cudaStream_t s)
{
    if (b.N == 0) return CF_OK;
    // the scheduling blocks of the calls, and the pool cursor with the two task counters: two small memsets
    if (cudaMemsetAsync(b.out.sched, 0, sizeof(unsigned) * 4 * ROW_SCHED_SLOTS, s) != cudaSuccess ||
        cudaMemsetAsync(b.out.cursor, 0, 16, s) != cudaSuccess)
        return launch_status("row list scheduling words");
    static thread_local bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        if (cudaFuncSetAttribute(row_list_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)RL_SMEM) != cudaSuccess) {
            cudaGetLastError();
            return fail(CF_ERR_CUDA, "row list build: %zu bytes of shared memory not available", RL_SMEM);
        }
        configured[dev & 63] = true;
    }
    const long long cap = (long long)sm_count() * 3;
    row_list_build_kernel<<<(unsigned)(b.N < cap ? b.N : cap), RL_THREADS, RL_SMEM, s>>>(b);
    return launch_status("row_list_build_kernel");
}

}  // namespace cf

extern "C" int64_t cf_row_list_workspace_bytes(int64_t N, int64_t E) { return (int64_t)cf::row_list_workspace_bytes(N, E); }

extern "C" int cf_row_list_build(const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                                 const int64_t *edges, const int64_t *row_start, const int32_t *row_order, int64_t N,
                                 int64_t E, int64_t max_atoms, double cutoff_radius, int lattice_range, int minimum_range,
                                 double a_widest, void *workspace, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_row_list_build: negative size");
    CF_REQUIRE(a_widest < 0, CF_ERR_INVALID, "cf_row_list_build: a_widest must be negative");
    CF_REQUIRE(max_atoms >= 1 && max_atoms <= ROW_LIST_MAX_KEYS, CF_ERR_RANGE,
               "cf_row_list_build: max_atoms=%lld outside [1,%d]", (long long)max_atoms, ROW_LIST_MAX_KEYS);
    CF_REQUIRE(N < (1ll << 31) && E < (1ll << 31), CF_ERR_RANGE, "cf_row_list_build: N or E beyond 32-bit row records");
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_row_list_build: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (N == 0) return CF_OK;
    CF_REQUIRE(pos_ij && tvecs && batch && edges && row_start && workspace, CF_ERR_INVALID, "cf_row_list_build: null pointer");
    CF_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 15) == 0, CF_ERR_INVALID, "cf_row_list_build: workspace must be 16-byte aligned");
    RowListBuild b{};
    b.pos_ij = pos_ij; b.tvecs = tvecs; b.rvlen = cutoff_radius != 0.0 ? rvlen : nullptr;
    b.batch = batch; b.edges = edges; b.row_start = row_start; b.row_order = row_order;
    b.N = N; b.E = E;
    b.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    b.a_widest = (float)a_widest;
    b.window = term_window(weight_floor_log2(), (float)a_widest);
    b.coop_chunks = ROW_COOP_CHUNKS;
    b.out = row_list_carve(workspace, N, E);
    return launch_row_list_build(b, as_stream(stream));
}
