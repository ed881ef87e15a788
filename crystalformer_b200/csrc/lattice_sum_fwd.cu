// Real-space lattice sum, forward: phi (E,H) and psi (E,H,K) or W psi (E,H,16) per edge.
//
// Two kernels (building blocks in lattice_core.cuh):
//   lattice_phi_kernel   one thread per edge, all eight heads: z = log sum_n exp(a |r + n.T|^2).  MUFU-bound.
//   lattice_psi_kernel   one warp per edge: the radial-basis expansion psi, with the Gaussian weights already
//                        normalised by z, so no second reduction is needed.  The reference gives every (edge, head)
//                        its own thread and so repeats the geometry and the 64 basis exponentials eight times; here
//                        they are evaluated once per (edge, translation) and shared by the heads.
// The box of a head follows the reference rule exactly; heads of one edge may have different boxes, in which case
// the union box is enumerated and each head masks the translations outside its own.
#include "lattice_core.cuh"

namespace cf {

namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int PSI_STRIDE = 68;                            // floats per head row of the per-warp psi tile (bank skew)
constexpr int WT_HEAD_STRIDE = 64 * HEAD_DIM + 16;        // floats per head of the transposed projection (bank skew)
constexpr int WARP_SMEM_FLOATS = STAGE_FLOATS + 8 * PSI_STRIDE;

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
    BasisParams basis;
    int a_per_edge;
    int stage_w;      // 1: W (1,H,16,K) is staged transposed in shared memory
};

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


template <int TPE>
__global__ void __launch_bounds__(128) lattice_phi_kernel(const PhiArgs p)
{
    const long long gtid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (gtid == 0 && p.zero_word) *p.zero_word = 0u;
    const long long e_raw = gtid / TPE;
    const int sub = (int)(gtid % TPE);
    const bool live = e_raw < p.E;
    const long long e = live ? e_raw : p.E - 1;  // idle tail threads shadow the last edge so that shuffles stay full
    const long long i = p.edges[e];
    const long long c = p.batch[i];
    Cell cell;
    cell.load(p.tvecs + 9 * c);
    const float4 *ap = reinterpret_cast<const float4 *>(p.a + (p.a_per_edge ? e : i) * HEADS);
    const float4 a_lo = __ldg(ap), a_hi = __ldg(ap + 1);
    const float a[8] = {a_lo.x, a_lo.y, a_lo.z, a_lo.w, a_hi.x, a_hi.y, a_hi.z, a_hi.w};
    float rx, ry, rz;
    if (p.pos_ij) {
        rx = p.pos_ij[3 * e]; ry = p.pos_ij[3 * e + 1]; rz = p.pos_ij[3 * e + 2];
    } else {
        const long long j = p.edges[p.E + e];
        rx = __fsub_rn(p.pos[3 * j], p.pos[3 * i]);
        ry = __fsub_rn(p.pos[3 * j + 1], p.pos[3 * i + 1]);
        rz = __fsub_rn(p.pos[3 * j + 2], p.pos[3 * i + 2]);
    }
    float z[8];
    edge_phi<TPE>(p.rule, a, p.rvlen ? p.rvlen + 3 * c : nullptr, cell, rx, ry, rz, p.floor_log2, sub, z);
    if (live && sub == 0) {
        float4 *zp = reinterpret_cast<float4 *>(p.z + e * HEADS);
        zp[0] = make_float4(z[0], z[1], z[2], z[3]);
        zp[1] = make_float4(z[4], z[5], z[6], z[7]);
    }
}

template <int K>
__global__ void __launch_bounds__(THREADS, 5) lattice_psi_kernel(const FwdArgs p)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *wt = smem;
    float *mine = smem + (p.stage_w ? HEADS * WT_HEAD_STRIDE : 0) + warp * WARP_SMEM_FLOATS;
    float *psi = mine + STAGE_FLOATS;

    if (p.stage_w) {
        // W[h][m][k] -> wt[h][k][m] so that a lane reads its four outputs' weights as one float4
        for (int idx = threadIdx.x; idx < HEADS * HEAD_DIM * K; idx += THREADS) {
            const int h = idx / (HEAD_DIM * K), m = (idx / K) % HEAD_DIM, k = idx % K;
            wt[h * WT_HEAD_STRIDE + k * HEAD_DIM + m] = p.W[idx];
        }
        __syncthreads();
    }
    BinAccumulator<K> bins;
    bins.init(mine, lane, p.basis);

    for (long long e = (long long)blockIdx.x * WARPS + warp; e < p.E; e += (long long)gridDim.x * WARPS) {
        const long long i = p.edges[e];
        const long long c = p.batch[i];
        const float rx = p.pos_ij[3 * e], ry = p.pos_ij[3 * e + 1], rz = p.pos_ij[3 * e + 2];
        Cell cell;
        cell.load(p.tvecs + 9 * c);

        // lanes 0..7 (and their copies) hold head (lane & 7): its width, its box and the log-normaliser from phi
        const float a_own = p.a[(p.a_per_edge ? e : i) * HEADS + (lane & 7)];
        const float z_own = p.z[e * HEADS + (lane & 7)];
        const int pk_own = packed_box(p.rule, a_own, p.rvlen ? p.rvlen + 3 * c : nullptr);
        int uni = pk_own;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) uni = box_union(uni, __shfl_xor_sync(FULL, uni, o));
        const bool masked = !__all_sync(FULL, pk_own == uni);
        float a2[8], off[8];
        int pk[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            a2[h] = __shfl_sync(FULL, a_own, h) * LOG2E;
            off[h] = -__shfl_sync(FULL, z_own, h) * LOG2E;
            pk[h] = __shfl_sync(FULL, pk_own, h);
        }
        const int R1 = box_r1(uni), R2 = box_r2(uni), R3 = box_r3(uni);
        const int count = (2 * R1 + 1) * (2 * R2 + 1) * (2 * R3 + 1);
        TermWalker walk;
        walk.init(R1, R2, R3, (unsigned)lane);
        const float F1 = (float)R1, F2 = (float)R2, F3 = (float)R3;
        bins.clear();
        for (int base = 0; base < count; base += 32) {
            const bool valid = base + lane < count;
            const float f1 = walk.u1 - F1, f2 = walk.u2 - F2, f3 = walk.u3 - F3;
            const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, rx)));
            const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, ry)));
            const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, rz)));
            const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
            int i1 = 0, i2 = 0, i3 = 0;
            if (masked) {
                i1 = abs(__float2int_rn(f1)); i2 = abs(__float2int_rn(f2)); i3 = abs(__float2int_rn(f3));
            }
            float w[8];
            float emax = -INFINITY;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                float eh = fmaf(a2[h], d2, off[h]);
                if (masked && !(i1 <= box_r1(pk[h]) && i2 <= box_r2(pk[h]) && i3 <= box_r3(pk[h]))) eh = -INFINITY;
                w[h] = ex2(eh);
                emax = fmaxf(emax, eh);
            }
            const float x = fast_sqrt(d2) * p.basis.bin_scale;
            bins.push(valid && emax > p.basis.floor_log2 && d2 < p.basis.d2_cut, x, w);
            walk.step();
        }

        bins.flush(psi, PSI_STRIDE);
        if (p.W == nullptr) {
            float *dst = p.v + (size_t)e * HEADS * K + lane;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                dst[h * K] = psi[h * PSI_STRIDE + lane];
                dst[h * K + 32] = psi[h * PSI_STRIDE + lane + 32];
            }
            __syncwarp();
        } else {
            float4 o;
            if (p.stage_w) {
                o = project<K, true>(wt, psi, lane);
            } else {
                const long long wi = (p.W_num == 1) ? 0 : (p.W_num == p.E ? e : i);
                o = project<K, false>(p.W + (size_t)wi * HEADS * HEAD_DIM * K, psi, lane);
            }
            reinterpret_cast<float4 *>(p.v + (size_t)e * HEADS * HEAD_DIM)[lane] = o;
            __syncwarp();
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
    // the very function the lattice-sum kernels call, so that the bit-exactness test covers what they enumerate
    const int pk = packed_box(rule, a[(a_per_edge ? e : i) * HEADS + h], rvlen ? rvlen + 3 * c : nullptr);
    box[3 * tid + 0] = box_r1(pk);
    box[3 * tid + 1] = box_r2(pk);
    box[3 * tid + 2] = box_r3(pk);
}


int launch_fwd(const FwdArgs &p, long long K, cudaStream_t stream)
{
    PhiArgs phi{};
    phi.a = p.a; phi.pos_ij = p.pos_ij; phi.tvecs = p.tvecs; phi.batch = p.batch; phi.edges = p.edges;
    phi.rvlen = p.rvlen; phi.z = p.z; phi.E = p.E; phi.rule = p.rule; phi.a_per_edge = p.a_per_edge;
    phi.floor_log2 = p.basis.floor_log2;
    launch_lattice_phi(phi, stream);
    if (K > 0) {
        const size_t smem = sizeof(float) * ((p.stage_w ? HEADS * WT_HEAD_STRIDE : 0) + WARPS * WARP_SMEM_FLOATS);
        static thread_local int per_sm[2] = {0, 0};
        int &occ = per_sm[p.stage_w ? 1 : 0];
        if (occ == 0) {
            cudaFuncSetAttribute(lattice_psi_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(sizeof(float) * (HEADS * WT_HEAD_STRIDE + WARPS * WARP_SMEM_FLOATS)));
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, lattice_psi_kernel<64>, THREADS, smem) != cudaSuccess || occ <= 0)
                occ = 4;
        }
        const long long want = (p.E + WARPS - 1) / WARPS;
        const long long cap = (long long)sm_count() * occ;
        lattice_psi_kernel<64><<<(int)(want < cap ? want : cap), THREADS, smem, stream>>>(p);
    }
    return launch_status("cf_lattice_sum_fwd");
}

}  // namespace

int launch_lattice_phi(const PhiArgs &p, cudaStream_t stream)
{
    if (p.E > 0) {
        // enough threads to give every SM about 24 warps: small batches split each edge over up to 8 threads
        const long long target = (long long)sm_count() * 24 * 32;
        int tpe = 1;
        while (tpe < 8 && p.E * tpe < target) tpe *= 2;
        const unsigned blocks = (unsigned)((p.E * tpe + 127) / 128);
        switch (tpe) {
            case 1: lattice_phi_kernel<1><<<blocks, 128, 0, stream>>>(p); break;
            case 2: lattice_phi_kernel<2><<<blocks, 128, 0, stream>>>(p); break;
            case 4: lattice_phi_kernel<4><<<blocks, 128, 0, stream>>>(p); break;
            default: lattice_phi_kernel<8><<<blocks, 128, 0, stream>>>(p); break;
        }
    }
    return launch_status("lattice_phi_kernel");
}

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
    p.basis = make_basis_params(K, dist_max, wscale, weight_floor_log2());
    p.stage_w = (p.W != nullptr && W_num == 1) ? 1 : 0;
    return launch_fwd(p, K, as_stream(stream));
}
