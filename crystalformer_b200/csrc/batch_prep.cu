// Batch preparation on the device: crystal offsets, the all-pairs edge list, its CSR, relative positions and the
// reciprocal-lattice quantities the cut-off rule needs.  Replaces the host loop over crystals and the tolist()
// synchronisations of the reference (models/indexed_latticeformer_encoder.py:15-32, 183-253).
#include "common.cuh"

namespace cf {
namespace {

constexpr int SCAN_THREADS = 1024;

// Exclusive prefix sums of sizes and sizes^2 with one block: each thread scans a contiguous chunk.
__global__ void __launch_bounds__(SCAN_THREADS) crystal_offsets_kernel(const int64_t *__restrict__ sizes, long long B,
                                                                       int64_t *__restrict__ atom_start,
                                                                       int64_t *__restrict__ edge_start)
{
    __shared__ long long part_n[SCAN_THREADS], part_e[SCAN_THREADS];
    const int t = threadIdx.x;
    const long long chunk = (B + SCAN_THREADS - 1) / SCAN_THREADS;
    const long long lo = min((long long)t * chunk, B), hi = min(lo + chunk, B);
    long long sn = 0, se = 0;
    for (long long b = lo; b < hi; ++b) {
        const long long n = sizes[b];
        sn += n;
        se += n * n;
    }
    part_n[t] = sn;
    part_e[t] = se;
    __syncthreads();
    // Hillis-Steele inclusive scan over the 1024 partials
    for (int off = 1; off < SCAN_THREADS; off <<= 1) {
        long long vn = 0, ve = 0;
        if (t >= off) {
            vn = part_n[t - off];
            ve = part_e[t - off];
        }
        __syncthreads();
        part_n[t] += vn;
        part_e[t] += ve;
        __syncthreads();
    }
    long long on = part_n[t] - sn, oe = part_e[t] - se;
    for (long long b = lo; b < hi; ++b) {
        atom_start[b] = on;
        edge_start[b] = oe;
        const long long n = sizes[b];
        on += n;
        oe += n * n;
    }
    if (t == SCAN_THREADS - 1) {
        atom_start[B] = part_n[t];
        edge_start[B] = part_e[t];
    }
}

// Largest b in [0, B) with start[b] <= x  (start is non-decreasing, start[0] = 0; empty crystals are skipped over).
__device__ __forceinline__ long long find_segment(const int64_t *__restrict__ start, long long B, long long x)
{
    long long lo = 0, hi = B;  // invariant: start[lo] <= x < start[hi]
    while (hi - lo > 1) {
        const long long mid = (lo + hi) >> 1;
        if (start[mid] <= x) lo = mid; else hi = mid;
    }
    return lo;
}

__device__ __forceinline__ void cell_body(long long b, const float *__restrict__ trans, long long B,
                                          float *__restrict__ rvecs, float *__restrict__ vcell, float *__restrict__ rvlen)
{
    if (b >= B) return;
    const float *m = trans + 9 * b;
    // determinant by the rule of Sarrus, term order as models/indexed_latticeformer_encoder.py:34-44
    const float v = __fadd_rn(__fadd_rn(__fmul_rn(__fmul_rn(m[0], m[4]), m[8]), __fmul_rn(__fmul_rn(m[1], m[5]), m[6])),
                              __fmul_rn(__fmul_rn(m[2], m[3]), m[7]))
                  - __fmul_rn(__fmul_rn(m[2], m[4]), m[6]) - __fmul_rn(__fmul_rn(m[0], m[5]), m[7])
                  - __fmul_rn(__fmul_rn(m[1], m[3]), m[8]);
    if (vcell) vcell[b] = v;
    const float scale = __fmul_rn(__frcp_rn(v), 6.283185307179586f);
#pragma unroll
    for (int r = 0; r < 3; ++r) {
        const float *u = m + 3 * ((r + 1) % 3), *w = m + 3 * ((r + 2) % 3);
        const float cx = __fsub_rn(__fmul_rn(u[1], w[2]), __fmul_rn(u[2], w[1]));
        const float cy = __fsub_rn(__fmul_rn(u[2], w[0]), __fmul_rn(u[0], w[2]));
        const float cz = __fsub_rn(__fmul_rn(u[0], w[1]), __fmul_rn(u[1], w[0]));
        const float x = __fmul_rn(cx, scale), y = __fmul_rn(cy, scale), z = __fmul_rn(cz, scale);
        if (rvecs) {
            rvecs[9 * b + 3 * r + 0] = x;
            rvecs[9 * b + 3 * r + 1] = y;
            rvecs[9 * b + 3 * r + 2] = z;
        }
        if (rvlen) rvlen[3 * b + r] = __fsqrt_rn(__fadd_rn(__fadd_rn(__fmul_rn(x, x), __fmul_rn(y, y)), __fmul_rn(z, z)));
    }
}

__global__ void cell_kernel(const float *__restrict__ trans, long long B, float *__restrict__ rvecs,
                            float *__restrict__ vcell, float *__restrict__ rvlen)
{
    cell_body((long long)blockIdx.x * blockDim.x + threadIdx.x, trans, B, rvecs, vcell, rvlen);
}

__device__ __forceinline__ void atom_body(long long i, const int64_t *__restrict__ atom_start,
                                          const int64_t *__restrict__ edge_start, long long B, long long N,
                                          int64_t *__restrict__ batch, int64_t *__restrict__ row_start, long long E)
{
    if (i > N) return;
    if (i == N) {
        if (row_start) row_start[N] = E;
        return;
    }
    const long long c = find_segment(atom_start, B, i);
    if (batch) batch[i] = c;
    if (row_start) row_start[i] = edge_start[c] + (i - atom_start[c]) * (atom_start[c + 1] - atom_start[c]);
}

__global__ void atom_kernel(const int64_t *__restrict__ atom_start, const int64_t *__restrict__ edge_start,
                            long long B, long long N, int64_t *__restrict__ batch, int64_t *__restrict__ row_start,
                            long long E)
{
    atom_body((long long)blockIdx.x * blockDim.x + threadIdx.x, atom_start, edge_start, B, N, batch, row_start, E);
}

__device__ __forceinline__ void edge_body(long long e, const float *__restrict__ pos, const int64_t *__restrict__ atom_start,
                                          const int64_t *__restrict__ edge_start, long long B, long long E,
                                          int64_t *__restrict__ edges, float *__restrict__ pos_ij)
{
    if (e >= E) return;
    const long long c = find_segment(edge_start, B, e);
    const long long n = atom_start[c + 1] - atom_start[c];
    const long long local = e - edge_start[c];
    const long long i = atom_start[c] + local / n, j = atom_start[c] + local % n;
    if (edges) {
        edges[e] = i;
        edges[E + e] = j;
    }
    if (pos_ij) {
        pos_ij[3 * e + 0] = __fsub_rn(pos[3 * j + 0], pos[3 * i + 0]);
        pos_ij[3 * e + 1] = __fsub_rn(pos[3 * j + 1], pos[3 * i + 1]);
        pos_ij[3 * e + 2] = __fsub_rn(pos[3 * j + 2], pos[3 * i + 2]);
    }
}

__global__ void edge_kernel(const float *__restrict__ pos, const int64_t *__restrict__ atom_start,
                            const int64_t *__restrict__ edge_start, long long B, long long E,
                            int64_t *__restrict__ edges, float *__restrict__ pos_ij)
{
    edge_body((long long)blockIdx.x * blockDim.x + threadIdx.x, pos, atom_start, edge_start, B, E, edges, pos_ij);
}

// Scheduling weight of an atom's row in the fused attention kernels: a fixed part plus the expected number of
// (key, translation) pairs within `reach` of the atom, n x (volume of the reach sphere) / (cell volume).
__global__ void row_cost_kernel(const int64_t *__restrict__ atom_start, const float *__restrict__ trans, long long B,
                                long long N, float sphere, float *__restrict__ cost)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const long long c = find_segment(atom_start, B, i);
    const float *m = trans + 9 * c;
    const float v = m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
    const float n = (float)(atom_start[c + 1] - atom_start[c]);
    cost[i] = 1500.0f + n * (1.0f + sphere / fmaxf(fabsf(v), 1e-3f));
}

// Atoms in descending order of their row cost, ties by atom index (what a stable descending sort of cf_row_cost gives).
// All rows of a crystal have the same cost, so it is the crystals that are sorted: one thread block, bitonic sort of
// (cost, crystal) keys in shared memory, exclusive scan of the sorted atom counts, then every crystal's atoms are
// written as one run.
constexpr int ORDER_THREADS = 1024;
constexpr int ORDER_MAX_CRYSTALS = 2048;

__device__ __forceinline__ void row_order_body(const int64_t *__restrict__ atom_start, const float *__restrict__ trans,
                                               int B, int padded, float sphere, int32_t *__restrict__ order)
{
    __shared__ unsigned long long key[ORDER_MAX_CRYSTALS];
    __shared__ int offset[ORDER_MAX_CRYSTALS];
    __shared__ int warp_tot[ORDER_THREADS / 32];
    const int tid = threadIdx.x;
    for (int c = tid; c < padded; c += ORDER_THREADS) {
        unsigned long long k = 0ull;  // padding sorts last
        if (c < B) {
            const float *m = trans + 9 * c;
            const float v = m[0] * (m[4] * m[8] - m[5] * m[7]) - m[1] * (m[3] * m[8] - m[5] * m[6]) + m[2] * (m[3] * m[7] - m[4] * m[6]);
            const float n = (float)(atom_start[c + 1] - atom_start[c]);
            const float cost = 1500.0f + n * (1.0f + sphere / fmaxf(fabsf(v), 1e-3f));
            // positive floats order like their bit patterns; the complemented index breaks ties towards low indices
            k = ((unsigned long long)__float_as_uint(cost) << 32) | (unsigned)(0x7fffffff - c);
        }
        key[c] = k;
    }
    __syncthreads();
    for (int size = 2; size <= padded; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = tid; t < (padded >> 1); t += ORDER_THREADS) {
                const int lo = 2 * t - (t & (stride - 1));  // index of the pair's first element
                const int hi = lo + stride;
                const bool descending = (lo & size) == 0;
                const unsigned long long a = key[lo], b = key[hi];
                if ((a < b) == descending) { key[lo] = b; key[hi] = a; }
            }
            __syncthreads();
        }
    }
    // exclusive scan of the sorted crystals' atom counts (chunks of ORDER_THREADS, carried over)
    int carry = 0;
    for (int base = 0; base < padded; base += ORDER_THREADS) {
        const int k = base + tid;
        int n = 0;
        if (k < padded && key[k] != 0ull) {
            const int c = 0x7fffffff - (int)(unsigned)(key[k] & 0xffffffffu);
            n = (int)(atom_start[c + 1] - atom_start[c]);
        }
        int incl = n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(FULL, incl, o);
            if ((tid & 31) >= o) incl += up;
        }
        if ((tid & 31) == 31) warp_tot[tid >> 5] = incl;
        __syncthreads();
        int before = 0;
        for (int w = 0; w < (tid >> 5); ++w) before += warp_tot[w];
        int total = 0;
        for (int w = 0; w < ORDER_THREADS / 32; ++w) total += warp_tot[w];
        if (k < padded) offset[k] = carry + before + incl - n;
        carry += total;
        __syncthreads();
    }
    // every sorted crystal's atoms as one run; a warp per crystal, lanes over its atoms
    for (int k = tid >> 5; k < padded; k += ORDER_THREADS / 32) {
        if (key[k] == 0ull) continue;
        const int c = 0x7fffffff - (int)(unsigned)(key[k] & 0xffffffffu);
        const int first = (int)atom_start[c], n = (int)(atom_start[c + 1] - atom_start[c]);
        for (int r = tid & 31; r < n; r += 32) order[offset[k] + r] = first + r;
    }
}

__global__ void __launch_bounds__(ORDER_THREADS) row_order_kernel(const int64_t *__restrict__ atom_start,
                                                                  const float *__restrict__ trans, int B, int padded,
                                                                  float sphere, int32_t *__restrict__ order)
{
    row_order_body(atom_start, trans, B, padded, sphere, order);
}

// The batch geometry in ONE launch of 1024-thread blocks: block 0 sorts the rows (when asked to), the other blocks
// cover the cells, then the atoms, then the edges.  For batches of up to 1024 crystals the offsets are part of it:
// every block scans the crystals' sizes itself (sizes != NULL; one crystal per thread), works from its copy in shared
// memory, and block 1 stores them; larger batches bring offsets computed by crystal_offsets_kernel.
constexpr int INLINE_OFFSETS_MAX = 1024;
struct PrepareAll {
    const float *pos, *trans;
    const int64_t *sizes;            // NULL: atom_start / edge_start are inputs
    int64_t *atom_start, *edge_start;
    long long B, N, E;
    int64_t *batch, *edges, *row_start;
    float *pos_ij, *rvecs, *vcell, *rvlen;
    int32_t *order;   // NULL: no ordering
    int padded;
    float sphere;
};

__global__ void __launch_bounds__(ORDER_THREADS) prepare_all_kernel(const PrepareAll p)
{
    __shared__ int64_t atom_sh[INLINE_OFFSETS_MAX + 1], edge_sh[INLINE_OFFSETS_MAX + 1];
    __shared__ long long warp_n[ORDER_THREADS / 32], warp_e[ORDER_THREADS / 32];
    const int64_t *atom_start = p.atom_start, *edge_start = p.edge_start;
    if (p.sizes != nullptr) {
        // exclusive prefix sums of sizes and sizes^2 (B <= 1024 = ORDER_THREADS): warp scans, then the warps' totals
        const int t = threadIdx.x, lane = t & 31, w = t >> 5;
        const long long n = t < p.B ? p.sizes[t] : 0;
        long long in = n, ie = n * n;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const long long un = __shfl_up_sync(FULL, in, o), ue = __shfl_up_sync(FULL, ie, o);
            if (lane >= o) { in += un; ie += ue; }
        }
        if (lane == 31) { warp_n[w] = in; warp_e[w] = ie; }
        __syncthreads();
        long long bn = 0, be = 0;
        for (int k = 0; k < w; ++k) { bn += warp_n[k]; be += warp_e[k]; }
        if (t < p.B) { atom_sh[t + 1] = bn + in; edge_sh[t + 1] = be + ie; }
        if (t == 0) { atom_sh[0] = 0; edge_sh[0] = 0; }
        __syncthreads();
        if (blockIdx.x == 1)
            for (long long b = t; b <= p.B; b += ORDER_THREADS) { p.atom_start[b] = atom_sh[b]; p.edge_start[b] = edge_sh[b]; }
        atom_start = atom_sh;
        edge_start = edge_sh;
    }
    if (blockIdx.x == 0) {
        if (p.order != nullptr) row_order_body(atom_start, p.trans, (int)p.B, p.padded, p.sphere, p.order);
        return;
    }
    const long long idx = (long long)(blockIdx.x - 1) * ORDER_THREADS + threadIdx.x;
    if (idx < p.B) {
        cell_body(idx, p.trans, p.B, p.rvecs, p.vcell, p.rvlen);
    } else if (idx < p.B + p.N + 1) {
        atom_body(idx - p.B, atom_start, edge_start, p.B, p.N, p.batch, p.row_start, p.E);
    } else {
        edge_body(idx - p.B - p.N - 1, p.pos, atom_start, edge_start, p.B, p.E, p.edges, p.pos_ij);
    }
}

}  // namespace

// cf_crystal_offsets, cf_batch_prepare and cf_row_order in one launch (the one-call model forward; two launches for
// batches of more than 1024 crystals); *ordered says whether row_order was written (batches of more than
// ORDER_MAX_CRYSTALS crystals are not ordered).
int launch_prepare_all(const float *pos, const float *trans, const int64_t *sizes, int64_t *atom_start,
                       int64_t *edge_start, long long B, long long N, long long E, int64_t *batch, int64_t *edges,
                       int64_t *row_start, float *pos_ij, float *rvlen, double reach, int32_t *row_order, bool *ordered,
                       cudaStream_t s)
{
    PrepareAll p{};
    p.pos = pos; p.trans = trans; p.atom_start = atom_start; p.edge_start = edge_start; p.B = B; p.N = N; p.E = E;
    if (B <= INLINE_OFFSETS_MAX) {
        p.sizes = sizes;
    } else {
        crystal_offsets_kernel<<<1, SCAN_THREADS, 0, s>>>(sizes, B, atom_start, edge_start);
    }
    p.batch = batch; p.edges = edges; p.row_start = row_start; p.pos_ij = pos_ij; p.rvlen = rvlen;
    *ordered = row_order != nullptr && B <= ORDER_MAX_CRYSTALS && N < (1ll << 31);
    p.order = *ordered ? row_order : nullptr;
    p.padded = 2;
    while (p.padded < B) p.padded <<= 1;
    p.sphere = (float)(4.18879020478639 * reach * reach * reach);
    const long long items = B + N + 1 + E;
    prepare_all_kernel<<<(unsigned)(1 + (items + ORDER_THREADS - 1) / ORDER_THREADS), ORDER_THREADS, 0, s>>>(p);
    return launch_status("prepare_all_kernel");
}

}  // namespace cf

extern "C" int cf_row_order(const int64_t *atom_start, const float *trans, int64_t B, int64_t N, double reach,
                            int32_t *row_order, void *stream)
{
    using namespace cf;
    CF_REQUIRE(B >= 0 && N >= 0 && reach >= 0, CF_ERR_INVALID, "cf_row_order: negative size");
    CF_REQUIRE(B <= ORDER_MAX_CRYSTALS, CF_ERR_RANGE, "cf_row_order: B=%lld above %d crystals (sort cf_row_cost instead)",
               (long long)B, ORDER_MAX_CRYSTALS);
    CF_REQUIRE(N < (1ll << 31), CF_ERR_RANGE, "cf_row_order: N=%lld does not fit 32-bit atom indices", (long long)N);
    if (N == 0 || B == 0) return CF_OK;
    CF_REQUIRE(atom_start && trans && row_order, CF_ERR_INVALID, "cf_row_order: null pointer");
    int padded = 2;
    while (padded < B) padded <<= 1;
    const float sphere = (float)(4.18879020478639 * reach * reach * reach);
    row_order_kernel<<<1, ORDER_THREADS, 0, as_stream(stream)>>>(atom_start, trans, (int)B, padded, sphere, row_order);
    return launch_status("cf_row_order");
}

extern "C" int cf_row_cost(const int64_t *atom_start, const float *trans, int64_t B, int64_t N, double reach,
                           float *cost, void *stream)
{
    using namespace cf;
    CF_REQUIRE(B >= 0 && N >= 0 && reach >= 0, CF_ERR_INVALID, "cf_row_cost: negative size");
    if (N == 0) return CF_OK;
    CF_REQUIRE(atom_start && trans && cost, CF_ERR_INVALID, "cf_row_cost: null pointer");
    const float sphere = (float)(4.18879020478639 * reach * reach * reach);
    row_cost_kernel<<<(unsigned)((N + 255) / 256), 256, 0, as_stream(stream)>>>(atom_start, trans, B, N, sphere, cost);
    return launch_status("cf_row_cost");
}

extern "C" int cf_crystal_offsets(const int64_t *sizes, int64_t B, int64_t *atom_start, int64_t *edge_start,
                                  void *stream)
{
    using namespace cf;
    CF_REQUIRE(B >= 0 && B <= (1 << 20), CF_ERR_RANGE, "cf_crystal_offsets: B=%lld outside [0, 2^20]", (long long)B);
    CF_REQUIRE(atom_start && edge_start && (sizes || B == 0), CF_ERR_INVALID, "cf_crystal_offsets: null pointer");
    crystal_offsets_kernel<<<1, SCAN_THREADS, 0, as_stream(stream)>>>(sizes, B, atom_start, edge_start);
    return launch_status("cf_crystal_offsets");
}

extern "C" int cf_batch_prepare(const float *pos, const float *trans, const int64_t *sizes, const int64_t *atom_start,
                                const int64_t *edge_start, int64_t B, int64_t N, int64_t E, int64_t *batch,
                                int64_t *edges, int64_t *row_start, float *pos_ij, float *rvecs, float *vcell,
                                float *rvlen, void *stream)
{
    using namespace cf;
    (void)sizes;
    CF_REQUIRE(B >= 0 && N >= 0 && E >= 0, CF_ERR_INVALID, "cf_batch_prepare: negative size");
    CF_REQUIRE(atom_start && edge_start, CF_ERR_INVALID, "cf_batch_prepare: offsets are null");
    CF_REQUIRE(!pos_ij || pos, CF_ERR_INVALID, "cf_batch_prepare: pos_ij requested without pos");
    CF_REQUIRE(!(rvecs || vcell || rvlen) || trans, CF_ERR_INVALID, "cf_batch_prepare: cell outputs requested without trans");
    cudaStream_t s = as_stream(stream);
    if (B > 0 && (rvecs || vcell || rvlen)) cell_kernel<<<(unsigned)((B + 127) / 128), 128, 0, s>>>(trans, B, rvecs, vcell, rvlen);
    if (B > 0 && (batch || row_start)) atom_kernel<<<(unsigned)((N + 1 + 255) / 256), 256, 0, s>>>(atom_start, edge_start, B, N, batch, row_start, E);
    if (B > 0 && E > 0 && (edges || pos_ij)) edge_kernel<<<(unsigned)((E + 255) / 256), 256, 0, s>>>(pos, atom_start, edge_start, B, E, edges, pos_ij);
    return launch_status("cf_batch_prepare");
}
