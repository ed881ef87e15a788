// Real-space lattice sum, backward with respect to the Gaussian parameter a (N,H).
//
// Per edge e = (i,j) and head h, with p_n = exp(a d2_n - z_e) (z from the forward) and c_n = sum_k u_e[k] g_k(d_n)
// (u = gradient arriving at psi_e):
//     C0 = sum_n p_n c_n,  C1 = sum_n p_n d2_n,  C2 = sum_n p_n d2_n c_n
//     d loss / d a_i  +=  gz_e C1 + C2 - C1 C0
// (the formula of models/kernels/real_enc_bwd.cu:80-156).  One warp owns one edge; lanes run over its translations.
// The per-edge contributions are written out and summed per source atom by a second kernel in edge order, so the
// result does not depend on scheduling.  Optionally psi_e itself is recomputed and written (the gradient of a
// projection W needs it); phi and psi are never stored by the forward.
#include "lattice_bwd_core.cuh"

namespace cf {
namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int KBINS = 64;
constexpr int WARP_SMEM_FLOATS = HEADS * U_STRIDE + HEADS * KBINS + (STAGE_FLOATS > BWD_STAGE_FLOATS ? STAGE_FLOATS : BWD_STAGE_FLOATS);

struct BwdArgs {
    const float *a, *pos_ij, *tvecs, *rvlen, *z, *gz, *gpsi;
    const int64_t *batch, *edges;
    float *edge_out, *psi_out;
    long long E;
    BoxRule rule;
    BasisParams basis;
};

template <int K>
__global__ void __launch_bounds__(THREADS) lattice_bwd_edges_kernel(const BwdArgs p)
{
    extern __shared__ __align__(16) float smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float *u = smem + warp * WARP_SMEM_FLOATS;
    float *tile = u + HEADS * U_STRIDE;      // per-bin totals of the recomputed psi
    float *stage = tile + HEADS * KBINS;
    BinAccumulator<KBINS> bins;
    if (K > 0) bins.init(stage, lane, p.basis);

    for (long long e = (long long)blockIdx.x * WARPS + warp; e < p.E; e += (long long)gridDim.x * WARPS) {
        const long long i = p.edges[e];
        const long long c = p.batch[i];
        const float rx = p.pos_ij[3 * e], ry = p.pos_ij[3 * e + 1], rz = p.pos_ij[3 * e + 2];
        Cell cell;
        cell.load(p.tvecs + 9 * c);
        const float a_own = p.a[i * HEADS + (lane & 7)];
        const float z_own = p.z[e * HEADS + (lane & 7)];
        const float gz_own = p.gz[e * HEADS + (lane & 7)];
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
        const float F1 = (float)R1, F2 = (float)R2, F3 = (float)R3;
        const bool with_u = K > 0 && p.gpsi != nullptr;
        if (with_u) {
            const float4 *src = reinterpret_cast<const float4 *>(p.gpsi + (size_t)e * HEADS * K);
#pragma unroll
            for (int t = 0; t < HEADS * K / 128; ++t) reinterpret_cast<float4 *>(u)[lane + 32 * t] = __ldg(src + lane + 32 * t);
        }
        __syncwarp();

        float C0[8], C1[8], C2[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) C0[h] = C1[h] = C2[h] = 0.f;

        for (int pass = (K > 0 && p.psi_out) ? 0 : 1; pass < 2; ++pass) {
            TermWalker walk;
            walk.init(R1, R2, R3, (unsigned)lane);
            if (pass == 0) bins.clear();
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
                    if (!valid || (masked && !(i1 <= box_r1(pk[h]) && i2 <= box_r2(pk[h]) && i3 <= box_r3(pk[h])))) eh = -INFINITY;
                    w[h] = ex2(eh);
                    emax = fmaxf(emax, eh);
                }
                const float x = fast_sqrt(d2) * p.basis.bin_scale;
                const bool keep = K > 0 && emax > p.basis.floor_log2 && d2 < p.basis.d2_cut;
                if (pass == 0) {
                    bins.push(keep, x, w);
                } else {
#pragma unroll
                    for (int h = 0; h < 8; ++h) C1[h] = fmaf(w[h], d2, C1[h]);
                    if (with_u) {
                        const int cnt = stage_terms(stage, lane, keep, x, d2, 0, w);
                        if (lane < cnt) {
                            const float4 *row = reinterpret_cast<const float4 *>(stage + BWD_ENTRY_FLOATS * lane);
                            const float4 hd = row[0], pa = row[1], pb = row[2];
                            const float pw[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
                            float cd[8];
                            if (K == 64 && p.basis.windowed) basis_dot_window(u, hd.x, p.basis.bin_step, cd);
                            else basis_dot<(K > 0 ? K : 4)>(u, hd.x, p.basis.bin_step, cd);
#pragma unroll
                            for (int h = 0; h < 8; ++h) {
                                const float pc = pw[h] * cd[h];
                                C0[h] += pc;
                                C2[h] = fmaf(pc, hd.y, C2[h]);
                            }
                        }
                        __syncwarp();
                    }
                }
                walk.step();
            }
            if (pass == 0) {
                // per-bin totals go through the warp's own tile (u must stay intact for the second pass)
                float *dst = p.psi_out + (size_t)e * HEADS * KBINS + lane;
                bins.flush(tile, KBINS);
#pragma unroll
                for (int h = 0; h < 8; ++h) {
                    dst[h * KBINS] = tile[h * KBINS + lane];
                    dst[h * KBINS + 32] = tile[h * KBINS + lane + 32];
                }
                __syncwarp();
            }
        }
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            C0[h] = warp_sum(C0[h]);
            C1[h] = warp_sum(C1[h]);
            C2[h] = warp_sum(C2[h]);
        }
        if (lane < 8) {
            const float c0 = pick8(C0, lane), c1 = pick8(C1, lane), c2 = pick8(C2, lane);
            p.edge_out[e * HEADS + lane] = fmaf(gz_own, c1, c2 - c1 * c0);
        }
        __syncwarp();
    }
}

// ga[i][h] = sum of the contributions of atom i's edges, in edge order.
__global__ void row_sum_kernel(const float *__restrict__ edge_out, const int64_t *__restrict__ row_start, long long N,
                               float *__restrict__ ga)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= N * HEADS) return;
    const long long i = tid / HEADS;
    const int h = (int)(tid % HEADS);
    float s = 0.f;
    for (long long e = row_start[i]; e < row_start[i + 1]; ++e) s += edge_out[e * HEADS + h];
    ga[tid] = s;
}

}  // namespace
}  // namespace cf

extern "C" int cf_lattice_sum_bwd(const float *a, const float *pos_ij, const float *tvecs, const int64_t *batch,
                                  const int64_t *edges, const int64_t *row_start, const float *z, const float *gz,
                                  const float *gpsi, int64_t N, int64_t H, int64_t E, int64_t K, double dist_max,
                                  double wscale, const float *rvlen, double cutoff_radius, int lattice_range,
                                  int minimum_range, float *ga, float *psi_out, float *edge_scratch, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_lattice_sum_bwd: negative size");
    CF_REQUIRE(H == HEADS, CF_ERR_UNSUPPORTED, "cf_lattice_sum_bwd: H=%lld, only H=8 is compiled", (long long)H);
    CF_REQUIRE(K == 0 || K == 64, CF_ERR_UNSUPPORTED, "cf_lattice_sum_bwd: K=%lld, only K in {0,64} is compiled", (long long)K);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_lattice_sum_bwd: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    if (N == 0) return CF_OK;
    CF_REQUIRE(ga && row_start, CF_ERR_INVALID, "cf_lattice_sum_bwd: null pointer");
    cudaStream_t s = as_stream(stream);
    if (E > 0) {
        CF_REQUIRE(a && pos_ij && tvecs && batch && edges && z && gz && edge_scratch, CF_ERR_INVALID,
                   "cf_lattice_sum_bwd: null pointer");
        CF_REQUIRE(K == 0 || (dist_max > 0 && wscale > 0), CF_ERR_INVALID, "cf_lattice_sum_bwd: dist_max and wscale must be positive");
        BwdArgs p{};
        p.a = a; p.pos_ij = pos_ij; p.tvecs = tvecs; p.rvlen = rvlen; p.z = z; p.gz = gz; p.gpsi = K > 0 ? gpsi : nullptr;
        p.batch = batch; p.edges = edges; p.edge_out = edge_scratch; p.psi_out = K > 0 ? psi_out : nullptr; p.E = E;
        p.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
        p.basis = make_basis_params(K, dist_max, wscale, weight_floor_log2());
        const size_t smem = sizeof(float) * WARPS * WARP_SMEM_FLOATS;
        const long long want = (E + WARPS - 1) / WARPS, cap = (long long)sm_count() * 8;
        const int blocks = (int)(want < cap ? want : cap);
        if (K > 0) lattice_bwd_edges_kernel<64><<<blocks, THREADS, smem, s>>>(p);
        else lattice_bwd_edges_kernel<0><<<blocks, THREADS, smem, s>>>(p);
    }
    const long long total = (long long)N * HEADS;
    row_sum_kernel<<<(unsigned)((total + 127) / 128), 128, 0, s>>>(edge_scratch, row_start, N, ga);
    return launch_status("cf_lattice_sum_bwd");
}

// ------------------------------------------------------------------------------------------------------------------
// cf_lattice_sum_bwd_static: the same computation for callers that cannot hand over a scratch buffer.
//
// Some embedders are not in a position to allocate device memory at the moment they call: a serving process that
// sized all of its device memory at start-up and gives libraries none afterwards, a binding from a language runtime
// that has no device allocator at hand, or a latency-critical loop in which an allocation (which may synchronise the
// whole device) is not acceptable.  For them the per-edge contributions live in a fixed array that is part of the
// library image itself: it costs CF_STATIC_SCRATCH_MAX_EDGES * 8 floats (8 MiB) on every GPU that loads the library,
// for as long as the process lives, and bounds the number of edges one call may have.
//
// The array's name is only meaningful to device code; host code must ask the runtime for its device address.  That
// is done once per device, on the first call made with that device current (so make the first call on each device
// outside any stream capture), and the address is remembered.  Every call on a device uses the same array: two calls
// whose kernels may overlap on the GPU (different streams) would overwrite each other's contributions, so callers
// must serialise them.  Nothing in the array needs clearing between calls: every element a call reads (edges
// 0..E-1) is written by that same call first.
// ------------------------------------------------------------------------------------------------------------------
#include <mutex>

static __device__ __align__(256) float g_static_edge_scratch[(size_t)CF_STATIC_SCRATCH_MAX_EDGES * 8];

extern "C" int cf_lattice_sum_bwd_static(const float *a, const float *pos_ij, const float *tvecs, const int64_t *batch,
                                         const int64_t *edges, const int64_t *row_start, const float *z,
                                         const float *gz, const float *gpsi, int64_t N, int64_t H, int64_t E, int64_t K,
                                         double dist_max, double wscale, const float *rvlen, double cutoff_radius,
                                         int lattice_range, int minimum_range, float *ga, float *psi_out, void *stream)
{
    using namespace cf;
    CF_REQUIRE(E <= (int64_t)CF_STATIC_SCRATCH_MAX_EDGES, CF_ERR_RANGE,
               "cf_lattice_sum_bwd_static: E=%lld exceeds the built-in scratch of %lld edges; use cf_lattice_sum_bwd "
               "with a caller-provided scratch buffer", (long long)E, (long long)CF_STATIC_SCRATCH_MAX_EDGES);
    constexpr int MAX_DEVICES = 64;
    static std::mutex lock;
    static float *address_on_device[MAX_DEVICES] = {};
    int dev = -1;
    cudaError_t err = cudaGetDevice(&dev);
    if (err != cudaSuccess || dev < 0 || dev >= MAX_DEVICES)
        return fail(CF_ERR_CUDA, "cf_lattice_sum_bwd_static: cudaGetDevice: %s", cudaGetErrorString(err));
    float *scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(lock);
        if (address_on_device[dev] == nullptr) {
            float *ptr = nullptr;
            err = cudaGetSymbolAddress((void **)&ptr, g_static_edge_scratch);
            if (err != cudaSuccess || ptr == nullptr) {
                cudaGetLastError();
                return fail(CF_ERR_CUDA, "cf_lattice_sum_bwd_static: cudaGetSymbolAddress: %s", cudaGetErrorString(err));
            }
            address_on_device[dev] = ptr;
        }
        scratch = address_on_device[dev];
    }
    return cf_lattice_sum_bwd(a, pos_ij, tvecs, batch, edges, row_start, z, gz, gpsi, N, H, E, K, dist_max, wscale, rvlen,
                              cutoff_radius, lattice_range, minimum_range, ga, psi_out, scratch, stream);
}
