// Reciprocal-space lattice sum (the `reci` half of the reference's position encoding), forward and backward:
//     S[e,h]   = sum over n1 in [0,R], n2, n3 in [-R,R] of w(n1) exp(a_ih |k_n|^2) cos(kr_e . n),   w(0) = 1, else 2
//     phi[e,h] = log max(S, 1e-6) + 1.5 log(-4 pi a_ih) - log V
//     ga[i,h]  = sum_{e in row i} gz[e,h] (S < 1e-6 ? 0 : 1/S) sum_n w |k_n|^2 exp(a |k_n|^2) cos(kr_e . n)
// with k_n = n1 r1 + n2 r2 + n3 r3 (reciprocal rows of the edge's crystal) and kr_e = rvecs . pos_ij.
// (models/kernels/reci_enc_fwd.cu:16-67, reci_enc_bwd.cu:19-70; the backward leaves the 1.5 log(-4 pi a) term
// undifferentiated exactly as the reference does.)
//
// The reference spends (R+1)(2R+1)^2 exp + cos per (edge, head).  Here the sum is factorised: exp(a |k|^2) depends
// on the row's atom and the head only, cos(kr . n) on the edge only.
//   thread block per atom row:  1. all threads fill E[n][h] = w exp(a_h |k_n|^2) (or w |k_n|^2 exp(...)) in shared
//                                  memory, one (translation, head) pair each;
//                               2. one key per thread: three sincos, then cos(kr . n) for every n by complex
//                                  rotations (6 FMAs per term, no further transcendental), contracted with the
//                                  eight E[n][.] read as shared-memory broadcasts.
// Every sum has a fixed order: results are bitwise reproducible.
#include "common.cuh"

namespace cf {
namespace {

constexpr int RECI_THREADS = 128;
constexpr int RECI_MAX_RANGE = 6;  // (R+1)(2R+1)^2 x 8 floats of shared memory: 37 KB at R = 6

struct ReciArgs {
    const float *a, *kr_base, *rvecs, *vcell, *gz, *sum_in;
    const int64_t *batch, *row_start;
    float *z, *sum_out, *ga;
    long long N;
    int R;
};

// E[n][h] for the row's atom; n enumerates (n1, n2, n3) with n3 fastest, n1 from 0.
template <bool WEIGHTED>
__device__ __forceinline__ void fill_table(float *table, const float *__restrict__ r, const float *__restrict__ a_row,
                                           int R, int terms)
{
    const int S = 2 * R + 1;
    for (int idx = threadIdx.x; idx < terms * HEADS; idx += RECI_THREADS) {
        const int h = idx & 7, n = idx >> 3;
        const int n3 = n % S - R, n2 = (n / S) % S - R, n1 = n / (S * S);
        const float f1 = (float)n1, f2 = (float)n2, f3 = (float)n3;
        const float k1 = fmaf(r[6], f3, fmaf(r[3], f2, r[0] * f1));
        const float k2 = fmaf(r[7], f3, fmaf(r[4], f2, r[1] * f1));
        const float k3 = fmaf(r[8], f3, fmaf(r[5], f2, r[2] * f1));
        const float kk = fmaf(k3, k3, fmaf(k2, k2, k1 * k1));
        const float e = ex2(a_row[h] * LOG2E * kk) * (n1 == 0 ? 1.0f : 2.0f);
        table[idx] = WEIGHTED ? kk * e : e;
    }
}

// sum_n table[n][h] cos(kr . n) for all heads; cos by rotations from three sincos.
__device__ __forceinline__ void contract(const float *table, float kr1, float kr2, float kr3, int R, float (&out)[8])
{
    float c1, s1, c2, s2, c3, s3;  // unit rotations
    sincosf(kr1, &s1, &c1);
    sincosf(kr2, &s2, &c2);
    sincosf(kr3, &s3, &c3);
    float c2s, s2s, c3s, s3s;      // exp(-i R kr2), exp(-i R kr3): where the inner loops start
    sincosf(-(float)R * kr2, &s2s, &c2s);
    sincosf(-(float)R * kr3, &s3s, &c3s);
#pragma unroll
    for (int h = 0; h < 8; ++h) out[h] = 0.f;
    const float4 *t4 = reinterpret_cast<const float4 *>(table);
    float ar = 1.f, ai = 0.f;  // exp(i n1 kr1)
    for (int n1 = 0; n1 <= R; ++n1) {
        float br = c2s, bi = s2s;  // exp(i n2 kr2)
        for (int n2 = -R; n2 <= R; ++n2) {
            const float pr = ar * br - ai * bi, pi = ar * bi + ai * br;  // exp(i (n1 kr1 + n2 kr2))
            float gr = c3s, gi = s3s;                                      // exp(i n3 kr3)
            for (int n3 = -R; n3 <= R; ++n3) {
                const float cosv = pr * gr - pi * gi;
                const float4 e0 = t4[0], e1 = t4[1];
                t4 += 2;
                out[0] = fmaf(e0.x, cosv, out[0]); out[1] = fmaf(e0.y, cosv, out[1]);
                out[2] = fmaf(e0.z, cosv, out[2]); out[3] = fmaf(e0.w, cosv, out[3]);
                out[4] = fmaf(e1.x, cosv, out[4]); out[5] = fmaf(e1.y, cosv, out[5]);
                out[6] = fmaf(e1.z, cosv, out[6]); out[7] = fmaf(e1.w, cosv, out[7]);
                const float nr = gr * c3 - gi * s3;
                gi = gr * s3 + gi * c3;
                gr = nr;
            }
            const float nr = br * c2 - bi * s2;
            bi = br * s2 + bi * c2;
            br = nr;
        }
        const float nr = ar * c1 - ai * s1;
        ai = ar * s1 + ai * c1;
        ar = nr;
    }
}

__global__ void __launch_bounds__(RECI_THREADS) reci_fwd_kernel(const ReciArgs p)
{
    extern __shared__ __align__(16) float table[];
    const int terms = (p.R + 1) * (2 * p.R + 1) * (2 * p.R + 1);
    for (long long i = blockIdx.x; i < p.N; i += gridDim.x) {
        const long long c = p.batch[i];
        const long long e0 = p.row_start[i], e1 = p.row_start[i + 1];
        __syncthreads();  // the previous row's readers are done with the table
        fill_table<false>(table, p.rvecs + 9 * c, p.a + i * HEADS, p.R, terms);
        __syncthreads();
        const float log_v = logf(p.vcell[c]);
        for (long long e = e0 + threadIdx.x; e < e1; e += RECI_THREADS) {
            float s[8];
            contract(table, p.kr_base[3 * e], p.kr_base[3 * e + 1], p.kr_base[3 * e + 2], p.R, s);
            float z[8];
#pragma unroll
            for (int h = 0; h < 8; ++h)
                z[h] = logf(fmaxf(s[h], 1e-6f)) + (1.5f * logf(-12.5663706144f * p.a[i * HEADS + h]) - log_v);
            float4 *zo = reinterpret_cast<float4 *>(p.z + e * HEADS);
            zo[0] = make_float4(z[0], z[1], z[2], z[3]);
            zo[1] = make_float4(z[4], z[5], z[6], z[7]);
            if (p.sum_out) {
                float4 *so = reinterpret_cast<float4 *>(p.sum_out + e * HEADS);
                so[0] = make_float4(s[0], s[1], s[2], s[3]);
                so[1] = make_float4(s[4], s[5], s[6], s[7]);
            }
        }
    }
}

__global__ void __launch_bounds__(RECI_THREADS) reci_bwd_kernel(const ReciArgs p)
{
    extern __shared__ __align__(16) float table[];
    __shared__ float partial[RECI_THREADS / 32][HEADS];
    const int terms = (p.R + 1) * (2 * p.R + 1) * (2 * p.R + 1);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long long i = blockIdx.x; i < p.N; i += gridDim.x) {
        const long long c = p.batch[i];
        const long long e0 = p.row_start[i], e1 = p.row_start[i + 1];
        __syncthreads();
        fill_table<true>(table, p.rvecs + 9 * c, p.a + i * HEADS, p.R, terms);
        __syncthreads();
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (long long e = e0 + threadIdx.x; e < e1; e += RECI_THREADS) {
            float s[8];
            contract(table, p.kr_base[3 * e], p.kr_base[3 * e + 1], p.kr_base[3 * e + 2], p.R, s);
            const float4 *gp = reinterpret_cast<const float4 *>(p.gz + e * HEADS);
            const float4 *sp = reinterpret_cast<const float4 *>(p.sum_in + e * HEADS);
            const float4 g0 = gp[0], g1 = gp[1], q0 = sp[0], q1 = sp[1];
            const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            const float q[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int h = 0; h < 8; ++h) acc[h] += s[h] * g[h] * (q[h] < 1e-6f ? 0.f : 1.0f / q[h]);
        }
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            const float t = warp_sum(acc[h]);
            if (lane == 0) partial[warp][h] = t;
        }
        __syncthreads();
        if (threadIdx.x < HEADS) {
            const int h = threadIdx.x;
            p.ga[i * HEADS + h] = (partial[0][h] + partial[1][h]) + (partial[2][h] + partial[3][h]);
        }
    }
}

__global__ void reci_phase_kernel(const float *__restrict__ pos_ij, const float *__restrict__ rvecs,
                                  const int64_t *__restrict__ batch, const int64_t *__restrict__ edges, long long E,
                                  float *__restrict__ kr_base)
{
    const long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    const float *r = rvecs + 9 * batch[edges[e]];
    const float x = pos_ij[3 * e], y = pos_ij[3 * e + 1], z = pos_ij[3 * e + 2];
#pragma unroll
    for (int d = 0; d < 3; ++d) kr_base[3 * e + d] = fmaf(r[3 * d + 2], z, fmaf(r[3 * d + 1], y, r[3 * d] * x));
}

int launch(const ReciArgs &p, bool backward, cudaStream_t s, const char *what)
{
    const size_t smem = sizeof(float) * HEADS * (p.R + 1) * (2 * p.R + 1) * (2 * p.R + 1);
    const long long cap = (long long)sm_count() * 8;
    const int blocks = (int)(p.N < cap ? p.N : cap);
    if (backward)
        reci_bwd_kernel<<<blocks, RECI_THREADS, smem, s>>>(p);
    else
        reci_fwd_kernel<<<blocks, RECI_THREADS, smem, s>>>(p);
    return launch_status(what);
}

}  // namespace
}  // namespace cf

extern "C" int cf_reci_phase(const float *pos_ij, const float *rvecs, const int64_t *batch, const int64_t *edges,
                             int64_t E, float *kr_base, void *stream)
{
    using namespace cf;
    CF_REQUIRE(E >= 0, CF_ERR_INVALID, "cf_reci_phase: negative size");
    if (E == 0) return CF_OK;
    CF_REQUIRE(pos_ij && rvecs && batch && edges && kr_base, CF_ERR_INVALID, "cf_reci_phase: null pointer");
    reci_phase_kernel<<<(unsigned)((E + 255) / 256), 256, 0, as_stream(stream)>>>(pos_ij, rvecs, batch, edges, E, kr_base);
    return launch_status("cf_reci_phase");
}

extern "C" int cf_reci_sum_fwd(const float *a, const float *kr_base, const float *rvecs, const float *vcell,
                               const int64_t *batch, const int64_t *row_start, int64_t N, int64_t H, int64_t E,
                               int lattice_range, float *z, float *sumexp, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_reci_sum_fwd: negative size");
    CF_REQUIRE(H == HEADS, CF_ERR_UNSUPPORTED, "cf_reci_sum_fwd: H=%lld, only H=8 is compiled", (long long)H);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= RECI_MAX_RANGE, CF_ERR_RANGE,
               "cf_reci_sum_fwd: lattice_range %d outside [0,%d]", lattice_range, RECI_MAX_RANGE);
    if (N == 0 || E == 0) return CF_OK;
    CF_REQUIRE(a && kr_base && rvecs && vcell && batch && row_start && z, CF_ERR_INVALID, "cf_reci_sum_fwd: null pointer");
    ReciArgs p{};
    p.a = a; p.kr_base = kr_base; p.rvecs = rvecs; p.vcell = vcell; p.batch = batch; p.row_start = row_start;
    p.z = z; p.sum_out = sumexp; p.N = N; p.R = lattice_range;
    return launch(p, false, as_stream(stream), "cf_reci_sum_fwd");
}

extern "C" int cf_reci_sum_bwd(const float *a, const float *kr_base, const float *rvecs, const int64_t *batch,
                               const int64_t *row_start, const float *gz, const float *sumexp, int64_t N, int64_t H,
                               int64_t E, int lattice_range, float *ga, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_reci_sum_bwd: negative size");
    CF_REQUIRE(H == HEADS, CF_ERR_UNSUPPORTED, "cf_reci_sum_bwd: H=%lld, only H=8 is compiled", (long long)H);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= RECI_MAX_RANGE, CF_ERR_RANGE,
               "cf_reci_sum_bwd: lattice_range %d outside [0,%d]", lattice_range, RECI_MAX_RANGE);
    if (N == 0) return CF_OK;
    CF_REQUIRE(a && rvecs && batch && row_start && ga && (E == 0 || (kr_base && gz && sumexp)), CF_ERR_INVALID,
               "cf_reci_sum_bwd: null pointer");
    ReciArgs p{};
    p.a = a; p.kr_base = kr_base; p.rvecs = rvecs; p.batch = batch; p.row_start = row_start; p.gz = gz; p.sum_in = sumexp;
    p.ga = ga; p.N = N; p.R = lattice_range;
    return launch(p, true, as_stream(stream), "cf_reci_sum_bwd");
}
