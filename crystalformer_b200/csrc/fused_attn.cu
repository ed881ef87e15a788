// Edge-indexed softmax attention with the position terms given as tensors (the reference's operator split):
//   prob = softmax_j(q_i.k_j + aij),  out_i = sum_j prob_ij (v_j + bij)
// and its backward.  One warp owns one (atom, head) pair; lanes first run over the keys (logits, soft-max
// statistics), then split as (key parity, channel) for the weighted sums over 16-wide vectors.  The backward reads
// the per-edge tensors of a crystal's n x n block in both orders by index arithmetic, e(i,j) = c + i_local n +
// j_local, so no transposed copies are made (the reference transposes prob, bij and the gradients with a separate
// kernel, models/cuda_funcs/fused_dpa.py:157-191).  No atomics: every output element has one owner.
#include "common.cuh"

namespace cf {
namespace {

constexpr int THREADS = 256;  // 8 warps = the 8 heads of one atom

struct AttnArgs {
    const float *q, *k, *v, *aij, *bij;
    const int64_t *edges, *row_start;
    const float *prob_in, *out_in, *gout;
    float *prob, *out, *gq, *gk, *gv, *gaij, *gbij;
    long long N, E;
};

__device__ __forceinline__ float dot16(const float4 (&x)[4], const float *__restrict__ y)
{
    const float4 *y4 = reinterpret_cast<const float4 *>(y);
    float s = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const float4 b = __ldg(y4 + c);
        s = fmaf(x[c].x, b.x, s); s = fmaf(x[c].y, b.y, s); s = fmaf(x[c].z, b.z, s); s = fmaf(x[c].w, b.w, s);
    }
    return s;
}

__device__ __forceinline__ void load16(float4 (&x)[4], const float *__restrict__ src)
{
#pragma unroll
    for (int c = 0; c < 4; ++c) x[c] = __ldg(reinterpret_cast<const float4 *>(src) + c);
}

__global__ void __launch_bounds__(THREADS) fused_attn_fwd_kernel(const AttnArgs p)
{
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    for (long long i = blockIdx.x; i < p.N; i += gridDim.x) {
        const long long e0 = p.row_start[i];
        const int n = (int)(p.row_start[i + 1] - e0);
        float4 qi[4];
        load16(qi, p.q + (i * HEADS + h) * HEAD_DIM);
        // pass 1: logits into prob (used as scratch), running maximum
        float mx = -1e20f;
        for (int t = lane; t < n; t += 32) {
            const long long e = e0 + t, j = p.edges[p.E + e];
            float s = dot16(qi, p.k + (j * HEADS + h) * HEAD_DIM);
            if (p.aij) s += p.aij[e * HEADS + h];
            p.prob[e * HEADS + h] = s;
            mx = fmaxf(mx, s);
        }
        mx = warp_max(mx);
        float den = 0.f;
        for (int t = lane; t < n; t += 32) {
            const long long e = e0 + t;
            const float w = ex2((p.prob[e * HEADS + h] - mx) * LOG2E);
            p.prob[e * HEADS + h] = w;
            den += w;
        }
        den = warp_sum(den);
        const float inv = __frcp_rn(den);
        for (int t = lane; t < n; t += 32) p.prob[(e0 + t) * HEADS + h] *= inv;
        __syncwarp();
        // pass 2: lanes = (key parity, channel)
        const int d = lane & 15, half = lane >> 4;
        float acc = 0.f;
        for (int t = half; t < n; t += 2) {
            const long long e = e0 + t, j = p.edges[p.E + e];
            float val = __ldg(p.v + (j * HEADS + h) * HEAD_DIM + d);
            if (p.bij) val += __ldg(p.bij + (e * HEADS + h) * HEAD_DIM + d);
            acc = fmaf(p.prob[e * HEADS + h], val, acc);
        }
        acc += __shfl_xor_sync(FULL, acc, 16);
        if (half == 0) p.out[(i * HEADS + h) * HEAD_DIM + d] = acc;
    }
}

// Row pass of the backward: per (query i, head): gA_ij, gB_ij for every key and gQ_i.
__global__ void __launch_bounds__(THREADS) fused_attn_bwd_rows_kernel(const AttnArgs p)
{
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    for (long long i = blockIdx.x; i < p.N; i += gridDim.x) {
        const long long e0 = p.row_start[i];
        const int n = (int)(p.row_start[i + 1] - e0);
        float4 go[4], oi[4];
        load16(go, p.gout + (i * HEADS + h) * HEAD_DIM);
        load16(oi, p.out_in + (i * HEADS + h) * HEAD_DIM);
        float go_o = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) go_o += go[c].x * oi[c].x + go[c].y * oi[c].y + go[c].z * oi[c].z + go[c].w * oi[c].w;
        for (int t = lane; t < n; t += 32) {
            const long long e = e0 + t, j = p.edges[p.E + e];
            const float pr = p.prob_in[e * HEADS + h];
            float s = dot16(go, p.v + (j * HEADS + h) * HEAD_DIM);
            if (p.bij) s += dot16(go, p.bij + (e * HEADS + h) * HEAD_DIM);
            p.gaij[e * HEADS + h] = pr * (s - go_o);
            if (p.gbij) {
                float4 *dst = reinterpret_cast<float4 *>(p.gbij + (e * HEADS + h) * HEAD_DIM);
#pragma unroll
                for (int c = 0; c < 4; ++c) dst[c] = make_float4(go[c].x * pr, go[c].y * pr, go[c].z * pr, go[c].w * pr);
            }
        }
        __syncwarp();
        const int d = lane & 15, half = lane >> 4;
        float acc = 0.f;
        for (int t = half; t < n; t += 2) {
            const long long e = e0 + t, j = p.edges[p.E + e];
            acc = fmaf(p.gaij[e * HEADS + h], __ldg(p.k + (j * HEADS + h) * HEAD_DIM + d), acc);
        }
        acc += __shfl_xor_sync(FULL, acc, 16);
        if (half == 0) p.gq[(i * HEADS + h) * HEAD_DIM + d] = acc;
    }
}

// Column pass: per (key j, head): gV_j = sum_i p_ij go_i, gK_j = sum_i gA_ij q_i.
__global__ void __launch_bounds__(THREADS) fused_attn_bwd_cols_kernel(const AttnArgs p)
{
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    const int d = lane & 15, half = lane >> 4;
    for (long long j = blockIdx.x; j < p.N; j += gridDim.x) {
        const long long r0 = p.row_start[j];
        const int n = (int)(p.row_start[j + 1] - r0);
        const long long first = p.edges[p.E + r0];  // first atom of j's crystal
        const long long c = p.row_start[first];     // first edge of the crystal
        const long long jl = j - first;
        float av = 0.f, ak = 0.f;
        for (int il = half; il < n; il += 2) {
            const long long i = first + il, e = c + (long long)il * n + jl;
            av = fmaf(p.prob_in[e * HEADS + h], __ldg(p.gout + (i * HEADS + h) * HEAD_DIM + d), av);
            ak = fmaf(p.gaij[e * HEADS + h], __ldg(p.q + (i * HEADS + h) * HEAD_DIM + d), ak);
        }
        av += __shfl_xor_sync(FULL, av, 16);
        ak += __shfl_xor_sync(FULL, ak, 16);
        if (half == 0) {
            p.gv[(j * HEADS + h) * HEAD_DIM + d] = av;
            p.gk[(j * HEADS + h) * HEAD_DIM + d] = ak;
        }
    }
}

int grid_for(long long N) { const long long cap = (long long)sm_count() * 8; return (int)(N < cap ? N : cap); }

}  // namespace
}  // namespace cf

extern "C" int cf_fused_attn_fwd(const float *q, const float *k, const float *v, const float *aij, const float *bij,
                                 const int64_t *edges, const int64_t *row_start, int64_t N, int64_t H, int64_t D,
                                 int64_t E, float *prob, float *out, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_fused_attn_fwd: negative size");
    CF_REQUIRE(H == HEADS && D == HEAD_DIM, CF_ERR_UNSUPPORTED, "cf_fused_attn_fwd: H=%lld D=%lld, only H=8 D=16 is compiled",
               (long long)H, (long long)D);
    if (N == 0) return CF_OK;
    CF_REQUIRE(q && k && v && edges && row_start && prob && out, CF_ERR_INVALID, "cf_fused_attn_fwd: null pointer");
    AttnArgs p{};
    p.q = q; p.k = k; p.v = v; p.aij = aij; p.bij = bij; p.edges = edges; p.row_start = row_start;
    p.prob = prob; p.out = out; p.N = N; p.E = E;
    fused_attn_fwd_kernel<<<grid_for(N), THREADS, 0, as_stream(stream)>>>(p);
    return launch_status("cf_fused_attn_fwd");
}

extern "C" int cf_fused_attn_bwd(const float *q, const float *k, const float *v, const float *bij, const int64_t *edges,
                                 const int64_t *row_start, int64_t N, int64_t H, int64_t D, int64_t E,
                                 const float *prob, const float *out, const float *gout, float *gq, float *gk,
                                 float *gv, float *gaij, float *gbij, void *stream)
{
    using namespace cf;
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_fused_attn_bwd: negative size");
    CF_REQUIRE(H == HEADS && D == HEAD_DIM, CF_ERR_UNSUPPORTED, "cf_fused_attn_bwd: H=%lld D=%lld, only H=8 D=16 is compiled",
               (long long)H, (long long)D);
    if (N == 0) return CF_OK;
    CF_REQUIRE(q && k && v && edges && row_start && prob && out && gout && gq && gk && gv && gaij, CF_ERR_INVALID,
               "cf_fused_attn_bwd: null pointer");
    CF_REQUIRE((bij != nullptr) == (gbij != nullptr), CF_ERR_INVALID, "cf_fused_attn_bwd: bij and gbij must both be given or both be null");
    AttnArgs p{};
    p.q = q; p.k = k; p.v = v; p.bij = bij; p.edges = edges; p.row_start = row_start; p.prob_in = prob; p.out_in = out;
    p.gout = gout; p.gq = gq; p.gk = gk; p.gv = gv; p.gaij = gaij; p.gbij = gbij; p.N = N; p.E = E;
    fused_attn_bwd_rows_kernel<<<grid_for(N), THREADS, 0, as_stream(stream)>>>(p);
    fused_attn_bwd_cols_kernel<<<grid_for(N), THREADS, 0, as_stream(stream)>>>(p);
    return launch_status("cf_fused_attn_bwd");
}
