// Real-space lattice sum, forward: phi (E,H) and psi (E,H,K) or W psi (E,H,16) per edge.
//
// One warp owns one edge (i,j) and all eight heads.  The reference gives every (edge, head) its own thread, which
// repeats the geometry and the 64 radial-basis exponentials eight times; here they are computed once per
// (edge, translation) and shared by the heads.
//
//   pass 0  lanes <-> translations : d^2 of every translation in the box, running minimum per head
//   pass 1  lanes <-> translations : the eight Gaussian weights w_h = 2^(a_h log2e (d^2 - d^2_min,h)), partial sums
//           for the log-sum-exp; translations whose weights all fall below the floor, or whose distance is so far
//           beyond the last bin that every basis value underflows, are dropped, the rest are compacted with a ballot
//           into a small per-warp staging area in shared memory (x = scaled distance, w_0..7)
//   pass 2  lanes <-> bins : each lane owns bins (lane, lane+32) of all eight heads = 16 accumulators in
//           registers; per staged translation it evaluates its two basis values (2 MUFU) and does 16 FMAs
//
// The box of a head follows the reference rule exactly (common.cuh); heads of one edge may have different boxes,
// in which case the union box is enumerated and each head masks the translations outside its own.
#include "common.cuh"

namespace cf {

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int PSI_STRIDE = 68;                            // floats per head row of the per-warp psi tile (bank skew)
constexpr int WT_HEAD_STRIDE = 64 * HEAD_DIM + 16;        // floats per head of the transposed projection (bank skew)
constexpr int WARP_SMEM_FLOATS = 32 * 8 + 32 + 8 * PSI_STRIDE;

struct FwdArgs {
    const float *a;
    const float *pos_ij;
    const float *tvecs;
    const int64_t *batch;
    const int64_t *edges;
    const float *W;
    const float *rvlen;
    float *z;
    float *v;
    long long N, E, W_num;
    BoxRule rule;
    float bin_step;   // spacing of bin centres in basis units: sqrt(log2 e) / (sqrt2 wscale)
    float bin_scale;  // bin_step / mu0: distance -> basis units
    float x_cut;      // beyond this scaled distance every basis value underflows
    float w_floor;
    int a_per_edge;
    int stage_w;      // 1: W (1,H,16,K) is staged transposed in shared memory
};

template <bool MASKED>
__device__ __forceinline__ bool in_box(int packed, int n1, int n2, int n3)
{
    if (!MASKED) return true;
    return abs(n1) <= (packed & 0xff) && abs(n2) <= ((packed >> 8) & 0xff) && abs(n3) <= ((packed >> 16) & 0xff);
}

// out[h][4 mq .. 4 mq + 3] = sum_k W[h][m][k] psi[h][k] for the lane's (h, mq); psi in shared memory.
template <int K, bool STAGED>
__device__ __forceinline__ float4 project(const float *__restrict__ Wsrc, const float *__restrict__ psi, int lane)
{
    const int h = lane >> 2, mq = lane & 3;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    const float *ps = psi + h * PSI_STRIDE;
    if (STAGED) {
        const float *wt = Wsrc + h * WT_HEAD_STRIDE + 4 * mq;  // [k][m]
#pragma unroll 4
        for (int k = 0; k < K; k += 4) {
            const float4 pv = *reinterpret_cast<const float4 *>(ps + k);
            const float4 w0 = *reinterpret_cast<const float4 *>(wt + (k + 0) * HEAD_DIM);
            const float4 w1 = *reinterpret_cast<const float4 *>(wt + (k + 1) * HEAD_DIM);
            const float4 w2 = *reinterpret_cast<const float4 *>(wt + (k + 2) * HEAD_DIM);
            const float4 w3 = *reinterpret_cast<const float4 *>(wt + (k + 3) * HEAD_DIM);
            o0 = fmaf(w0.x, pv.x, o0); o1 = fmaf(w0.y, pv.x, o1); o2 = fmaf(w0.z, pv.x, o2); o3 = fmaf(w0.w, pv.x, o3);
            o0 = fmaf(w1.x, pv.y, o0); o1 = fmaf(w1.y, pv.y, o1); o2 = fmaf(w1.z, pv.y, o2); o3 = fmaf(w1.w, pv.y, o3);
            o0 = fmaf(w2.x, pv.z, o0); o1 = fmaf(w2.y, pv.z, o1); o2 = fmaf(w2.z, pv.z, o2); o3 = fmaf(w2.w, pv.z, o3);
            o0 = fmaf(w3.x, pv.w, o0); o1 = fmaf(w3.y, pv.w, o1); o2 = fmaf(w3.z, pv.w, o2); o3 = fmaf(w3.w, pv.w, o3);
        }
    } else {
        const float *w = Wsrc + (size_t)(h * HEAD_DIM + 4 * mq) * K;  // [m][k], global memory
#pragma unroll 2
        for (int k = 0; k < K; k += 4) {
            const float4 pv = *reinterpret_cast<const float4 *>(ps + k);
            const float4 w0 = __ldg(reinterpret_cast<const float4 *>(w + 0 * K + k));
            const float4 w1 = __ldg(reinterpret_cast<const float4 *>(w + 1 * K + k));
            const float4 w2 = __ldg(reinterpret_cast<const float4 *>(w + 2 * K + k));
            const float4 w3 = __ldg(reinterpret_cast<const float4 *>(w + 3 * K + k));
            o0 += w0.x * pv.x + w0.y * pv.y + w0.z * pv.z + w0.w * pv.w;
            o1 += w1.x * pv.x + w1.y * pv.y + w1.z * pv.z + w1.w * pv.w;
            o2 += w2.x * pv.x + w2.y * pv.y + w2.z * pv.z + w2.w * pv.w;
            o3 += w3.x * pv.x + w3.y * pv.y + w3.z * pv.z + w3.w * pv.w;
        }
    }
    return make_float4(o0, o1, o2, o3);
}

template <int K, bool MASKED>
__device__ __forceinline__ void edge_sums(const FwdArgs &p, const TermGrid &grid, const Cell &cell, float rx, float ry,
                                          float rz, const float (&a2)[8], const int (&pk)[8], float (&dmin)[8],
                                          float (&sum)[8], float (&acc)[8][2], float *sw, float *sx, int lane)
{
    // pass 0: minimum squared distance, per head when the boxes differ
#pragma unroll
    for (int h = 0; h < 8; ++h) dmin[h] = 1e10f;
    for (int base = 0; base < grid.count; base += 32) {
        const int t = base + lane;
        int n1, n2, n3;
        grid.decode(min(t, grid.count - 1), n1, n2, n3);
        const float d2 = cell.dist2(rx, ry, rz, n1, n2, n3);
        if (MASKED) {
#pragma unroll
            for (int h = 0; h < 8; ++h)
                if (in_box<true>(pk[h], n1, n2, n3)) dmin[h] = fminf(dmin[h], d2);
        } else {
            dmin[0] = fminf(dmin[0], d2);
        }
    }
    if (MASKED) {
#pragma unroll
        for (int h = 0; h < 8; ++h) dmin[h] = warp_min(dmin[h]);
    } else {
        const float m = warp_min(dmin[0]);
#pragma unroll
        for (int h = 0; h < 8; ++h) dmin[h] = m;
    }

    const float c0 = (float)(lane + 1) * p.bin_step, c1 = (float)(lane + 33) * p.bin_step;
#pragma unroll
    for (int h = 0; h < 8; ++h) {
        sum[h] = 0.f;
        acc[h][0] = acc[h][1] = 0.f;
    }

    for (int base = 0; base < grid.count; base += 32) {
        // pass 1: one translation per lane
        const int t = base + lane;
        const bool valid = t < grid.count;
        int n1, n2, n3;
        grid.decode(valid ? t : 0, n1, n2, n3);
        const float d2 = cell.dist2(rx, ry, rz, n1, n2, n3);
        float w[8];
        float wmax = 0.f;
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            float wh = ex2(a2[h] * (d2 - dmin[h]));
            if (!valid || !in_box<MASKED>(pk[h], n1, n2, n3)) wh = 0.f;
            w[h] = wh;
            sum[h] += wh;
            wmax = fmaxf(wmax, wh);
        }
        if (K > 0) {
            const float x = sqrtf(d2) * p.bin_scale;
            const bool keep = wmax > p.w_floor && x < p.x_cut;
            const unsigned mask = __ballot_sync(FULL, keep);
            if (keep) {
                const int slot = __popc(mask & ((1u << lane) - 1u));
                sx[slot] = x;
                reinterpret_cast<float4 *>(sw)[2 * slot] = make_float4(w[0], w[1], w[2], w[3]);
                reinterpret_cast<float4 *>(sw)[2 * slot + 1] = make_float4(w[4], w[5], w[6], w[7]);
            }
            __syncwarp();
            // pass 2: two bins per lane, all heads
            const int cnt = __popc(mask);
#pragma unroll 2
            for (int m = 0; m < cnt; ++m) {
                const float x_m = sx[m];
                const float4 wa = reinterpret_cast<const float4 *>(sw)[2 * m];
                const float4 wb = reinterpret_cast<const float4 *>(sw)[2 * m + 1];
                const float t0 = c0 - x_m, t1 = c1 - x_m;
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
    }
#pragma unroll
    for (int h = 0; h < 8; ++h) sum[h] = warp_sum(sum[h]);
}

template <int K>
__global__ void __launch_bounds__(THREADS) lattice_sum_fwd_kernel(const FwdArgs p)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *wt = smem;
    float *mine = smem + (p.stage_w ? HEADS * WT_HEAD_STRIDE : 0) + warp * WARP_SMEM_FLOATS;
    float *sw = mine, *sx = mine + 32 * 8, *psi = mine + 32 * 8 + 32;

    if (K > 0 && p.stage_w) {
        // W[h][m][k] -> wt[h][k][m] so that a lane reads its four outputs' weights as one float4
        constexpr int KK = K > 0 ? K : 1;
        for (int idx = threadIdx.x; idx < HEADS * HEAD_DIM * K; idx += THREADS) {
            const int h = idx / (HEAD_DIM * KK), m = (idx / KK) % HEAD_DIM, k = idx % KK;
            wt[h * WT_HEAD_STRIDE + k * HEAD_DIM + m] = p.W[idx];
        }
        __syncthreads();
    }

    for (long long e = (long long)blockIdx.x * WARPS + warp; e < p.E; e += (long long)gridDim.x * WARPS) {
        const long long i = p.edges[e];
        const long long c = p.batch[i];
        const float rx = p.pos_ij[3 * e], ry = p.pos_ij[3 * e + 1], rz = p.pos_ij[3 * e + 2];
        Cell cell;
        cell.load(p.tvecs + 9 * c);

        const float a_own = p.a[(p.a_per_edge ? e : i) * HEADS + (lane & 7)];
        int R1, R2, R3;
        box_half_widths(p.rule, a_own, p.rvlen ? p.rvlen + 3 * c : nullptr, R1, R2, R3);
        const int M1 = warp_max_int(R1), M2 = warp_max_int(R2), M3 = warp_max_int(R3);
        const bool uniform = __all_sync(FULL, R1 == M1 && R2 == M2 && R3 == M3);
        const int packed = R1 | (R2 << 8) | (R3 << 16);
        float a2[8];
        int pk[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            a2[h] = __shfl_sync(FULL, a_own, h) * LOG2E;
            pk[h] = __shfl_sync(FULL, packed, h);
        }
        TermGrid grid;
        grid.set(M1, M2, M3);

        float dmin[8], sum[8], acc[8][2];
        if (uniform) edge_sums<K, false>(p, grid, cell, rx, ry, rz, a2, pk, dmin, sum, acc, sw, sx, lane);
        else edge_sums<K, true>(p, grid, cell, rx, ry, rz, a2, pk, dmin, sum, acc, sw, sx, lane);

        if (lane < 8) {
            const float s = pick8(sum, lane), dm = pick8(dmin, lane);
            p.z[e * HEADS + lane] = fmaf(dm, a_own, logf(s));
        }
        if (K > 0) {
            if (p.W == nullptr) {
                float *dst = p.v + (size_t)e * HEADS * K + lane;
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float inv = __frcp_rn(sum[h]);
                    dst[h * K] = acc[h][0] * inv;
                    dst[h * K + 32] = acc[h][1] * inv;
                }
            } else {
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    const float inv = __frcp_rn(sum[h]);
                    psi[h * PSI_STRIDE + lane] = acc[h][0] * inv;
                    psi[h * PSI_STRIDE + lane + 32] = acc[h][1] * inv;
                }
                __syncwarp();
                float4 o;
                if (p.stage_w) {
                    o = project<(K > 0 ? K : 4), true>(wt, psi, lane);
                } else {
                    const long long wi = (p.W_num == 1) ? 0 : (p.W_num == p.E ? e : i);
                    o = project<(K > 0 ? K : 4), false>(p.W + (size_t)wi * HEADS * HEAD_DIM * K, psi, lane);
                }
                reinterpret_cast<float4 *>(p.v + (size_t)e * HEADS * HEAD_DIM)[lane] = o;
                __syncwarp();
            }
        }
    }
}

__global__ void lattice_box_kernel(const float *a, int a_per_edge, const int64_t *batch, const int64_t *edges,
                                   long long E, const float *rvlen, BoxRule rule, int32_t *box)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= E * HEADS) return;
    const long long e = tid / HEADS;
    const int h = (int)(tid % HEADS);
    const long long i = edges[e];
    const long long c = batch[i];
    int R1, R2, R3;
    box_half_widths(rule, a[(a_per_edge ? e : i) * HEADS + h], rvlen ? rvlen + 3 * c : nullptr, R1, R2, R3);
    box[3 * tid + 0] = R1;
    box[3 * tid + 1] = R2;
    box[3 * tid + 2] = R3;
}

template <int K>
int launch_fwd(const FwdArgs &p, cudaStream_t stream)
{
    const size_t smem = sizeof(float) * ((p.stage_w ? HEADS * WT_HEAD_STRIDE : 0) + WARPS * WARP_SMEM_FLOATS);
    static thread_local int per_sm[2] = {0, 0};
    int &occ = per_sm[p.stage_w ? 1 : 0];
    if (occ == 0) {
        cudaFuncSetAttribute(lattice_sum_fwd_kernel<K>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(sizeof(float) * (HEADS * WT_HEAD_STRIDE + WARPS * WARP_SMEM_FLOATS)));
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, lattice_sum_fwd_kernel<K>, THREADS, smem) != cudaSuccess || occ <= 0)
            occ = 4;
    }
    const long long want = (p.E + WARPS - 1) / WARPS;
    const long long cap = (long long)sm_count() * occ;
    const int blocks = (int)(want < cap ? want : cap);
    lattice_sum_fwd_kernel<K><<<blocks, THREADS, smem, stream>>>(p);
    return launch_status("cf_lattice_sum_fwd");
}

}  // namespace

}  // namespace cf

extern "C" int cf_lattice_box(const float *a, int a_per_edge, const int64_t *batch, const int64_t *edges, int64_t N,
                              int64_t H, int64_t E, const float *rvlen, double cutoff_radius, int lattice_range,
                              int minimum_range, int32_t *box, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_lattice_box: negative size");
    CF_REQUIRE(H == HEADS, CF_ERR_UNSUPPORTED, "cf_lattice_box: H=%lld, only H=8 is compiled", (long long)H);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_lattice_box: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (E == 0) return CF_OK;
    CF_REQUIRE(a && batch && edges && box, CF_ERR_INVALID, "cf_lattice_box: null pointer");
    BoxRule rule{(float)cutoff_radius, lattice_range, minimum_range};
    const long long total = (long long)E * HEADS;
    lattice_box_kernel<<<(unsigned)((total + 255) / 256), 256, 0, as_stream(stream)>>>(a, a_per_edge, batch, edges, E, rvlen, rule, box);
    return launch_status("cf_lattice_box");
}

extern "C" int cf_lattice_sum_fwd(const float *a, int a_per_edge, const float *pos_ij, const float *tvecs,
                                  const int64_t *batch, const int64_t *edges, int64_t N, int64_t H, int64_t E,
                                  int64_t K, double dist_max, double wscale, const float *W, int64_t W_num, int64_t Dv,
                                  const float *rvlen, double cutoff_radius, int lattice_range, int minimum_range,
                                  float *z, float *v, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_lattice_sum_fwd: negative size");
    CF_REQUIRE(H == HEADS, CF_ERR_UNSUPPORTED, "cf_lattice_sum_fwd: H=%lld, only H=8 is compiled", (long long)H);
    CF_REQUIRE(K == 0 || K == 64, CF_ERR_UNSUPPORTED, "cf_lattice_sum_fwd: K=%lld, only K in {0,64} is compiled", (long long)K);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_lattice_sum_fwd: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (E == 0) return CF_OK;
    CF_REQUIRE(a && pos_ij && tvecs && batch && edges && z, CF_ERR_INVALID, "cf_lattice_sum_fwd: null pointer");
    if (K > 0) {
        CF_REQUIRE(v != nullptr, CF_ERR_INVALID, "cf_lattice_sum_fwd: v is null but K > 0");
        CF_REQUIRE(dist_max > 0 && wscale > 0, CF_ERR_INVALID, "cf_lattice_sum_fwd: dist_max and wscale must be positive");
        if (W) {
            CF_REQUIRE(Dv == HEAD_DIM, CF_ERR_UNSUPPORTED, "cf_lattice_sum_fwd: Dv=%lld, only 16 is compiled", (long long)Dv);
            CF_REQUIRE(W_num == 1 || W_num == E || W_num == N, CF_ERR_INVALID,
                       "cf_lattice_sum_fwd: W_num=%lld must be 1, E or N", (long long)W_num);
        }
    }
    FwdArgs p{};
    p.a = a; p.pos_ij = pos_ij; p.tvecs = tvecs; p.batch = batch; p.edges = edges;
    p.W = (K > 0) ? W : nullptr; p.rvlen = rvlen; p.z = z; p.v = v;
    p.N = N; p.E = E; p.W_num = W_num;
    p.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    p.a_per_edge = a_per_edge;
    p.w_floor = weight_floor();
    p.stage_w = (p.W != nullptr && W_num == 1) ? 1 : 0;
    if (K > 0) {
        const double step = sqrt(1.4426950408889634) / (sqrt(2.0) * (double)(float)wscale);
        const double mu0 = (double)(float)dist_max / (double)K;
        p.bin_step = (float)step;
        p.bin_scale = (float)(step / mu0);
        p.x_cut = (float)((double)K * step + 11.3);  // (x - K step)^2 > 126 => every 2^-(..)^2 < 2^-126
    }
    return K == 0 ? launch_fwd<0>(p, as_stream(stream)) : launch_fwd<64>(p, as_stream(stream));
}
