// Fused infinitely connected attention, backward.  phi and psi are recomputed from the geometry.
//
// With the joint weight of a (key, translation) term  P_jn = p_ij p(n|ij) = exp(q_i.k_j - lse_i + a_i d2_jn),
// u_i = W^T gout_i (8 x 64), c(d) = sum_k u_i[k] g_k(d), delta_i = gout_i . out_i and gov_j = gout_i . v_j:
//     glogit_ij = p_ij (gov_j - delta_i) + sum_n P_jn c(d_jn)
//     ga_i      = sum_{j,n} P_jn d2_jn (gov_j - delta_i + c(d_jn))          (the products of per-edge sums cancel)
//     gq_i      = sum_j glogit_ij k_j          gk_j = sum_i glogit_ij q_i          gv_j = sum_i p_ij gout_i
// which is the chain of models/kernels/fused_dpa_bwd.cu:53-114 and real_enc_proj_bwd.cu:153-218 written for the
// hoisted projection.  The gradient of W is sum_i gout_i (x) psi_row_i, a GEMM done by the caller.
//
//   infinite_attn_bwd_rows_kernel  CTA per atom i: recompute q.k, p_ij, then each warp takes a contiguous range of the
//                                  row's keys; lanes run over (key, translation) terms, survivors are compacted and each
//                                  lane contracts the 64 basis values of its own term with u_i (shared memory, broadcast
//                                  reads).  Per-key sums are formed by walking the staged entries in order, so nothing
//                                  depends on scheduling.  Writes glogit (E,H), ga (N,H), gq (N,H,D).
//   infinite_attn_bwd_cols_kernel  warp per (key j, head): gk_j, gv_j from glogit and p_ij = exp(logit - lse_i), reading
//                                  the crystal's n x n block in column order by index arithmetic.
#include "lattice_bwd_core.cuh"
#include "term_list.cuh"

namespace cf {
namespace {

constexpr int THREADS = 128;
constexpr int WARPS = THREADS / 32;
constexpr int KBINS = 64;

struct BwdRowArgs {
    const float *q, *k, *v, *a, *pos, *pos_ij, *tvecs, *rvlen, *W, *logit, *lse, *out, *gout;
    const int64_t *batch, *edges, *row_start;
    const int32_t *row_order;
    float *gq, *gk, *gv, *ga, *glogit;
    long long N, E;
    int max_atoms;
    BoxRule rule;
    BasisParams basis;
    TermList list;  // optional (pool == NULL: none): the rows' terms, found once per batch (term_list.cuh)
};

__host__ __device__ inline size_t bwd_row_smem_floats(int max_atoms, bool with_basis)
{
    // per atom: rel (4) + c (8) + p (8) + gov (8) + s0 (8); then u (8 x 64), per-warp staging and results, ga partials
    return (size_t)max_atoms * 36 + (with_basis ? HEADS * U_STRIDE + WARPS * (BWD_STAGE_FLOATS + 32 * 8) : 0) + WARPS * 8 + 16;
}

template <int K>
__global__ void __launch_bounds__(THREADS) infinite_attn_bwd_rows_kernel(const BwdRowArgs p)
{
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float4 *rel = reinterpret_cast<float4 *>(smem);                    // [max_atoms]
    float *cj = smem + (size_t)p.max_atoms * 4;                        // [max_atoms][8] (q.k - lse) log2e
    float *pj = cj + (size_t)p.max_atoms * 8;                          // [max_atoms][8] p_ij
    float *gov = pj + (size_t)p.max_atoms * 8;                         // [max_atoms][8] gout_i . v_j - delta_i
    float *s0 = gov + (size_t)p.max_atoms * 8;                         // [max_atoms][8] sum_n P c, then glogit
    float *u = s0 + (size_t)p.max_atoms * 8;                           // [8][64]
    float *stage = u + (K > 0 ? HEADS * U_STRIDE : 0) + (K > 0 ? warp * (BWD_STAGE_FLOATS + 32 * 8) : 0);
    float *res = stage + BWD_STAGE_FLOATS;                             // [32][8] P c of the staged entries
    float *ga_part = u + (K > 0 ? HEADS * U_STRIDE + WARPS * (BWD_STAGE_FLOATS + 32 * 8) : 0);  // [WARPS][8]
    float *delta_s = ga_part + WARPS * 8;                              // [8]

    for (long long slot = blockIdx.x; slot < p.N; slot += gridDim.x) {
        const long long i = p.row_order ? p.row_order[slot] : slot;
        const long long c = p.batch[i];
        const long long e0 = p.row_start[i];
        const int n = (int)(p.row_start[i + 1] - e0);
        const long long a0 = n > 0 ? p.edges[p.E + e0] : 0;
        if (n > p.max_atoms) {
            p.gq[i * HEADS * HEAD_DIM + tid] = __int_as_float(0x7fc00000);
            if (tid < HEADS) p.ga[i * HEADS + tid] = __int_as_float(0x7fc00000);
            continue;
        }
        // ---- relative positions, delta_i = gout_i . out_i, u_i = W^T gout_i
        if (p.pos_ij) {
            for (int j = tid; j < n; j += THREADS) {
                const float *pp = p.pos_ij + 3 * (e0 + j);
                rel[j] = make_float4(pp[0], pp[1], pp[2], 0.f);
            }
        } else {
            const float pix = p.pos[3 * i], piy = p.pos[3 * i + 1], piz = p.pos[3 * i + 2];
            for (int j = tid; j < n; j += THREADS) {
                const float *pp = p.pos + 3 * (a0 + j);
                rel[j] = make_float4(__fsub_rn(pp[0], pix), __fsub_rn(pp[1], piy), __fsub_rn(pp[2], piz), 0.f);
            }
        }
        {
            // thread = (h, m): one element of gout_i and out_i; reduce the products over the 16 lanes of a head
            float prod = p.gout[i * HEADS * HEAD_DIM + tid] * p.out[i * HEADS * HEAD_DIM + tid];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) prod += __shfl_xor_sync(FULL, prod, o);
            if ((tid & 15) == 0) delta_s[tid >> 4] = prod;
        }
        if (K > 0) {
            for (int idx = tid; idx < HEADS * KBINS; idx += THREADS) {
                const int h = idx / KBINS, k = idx % KBINS;
                const float *go = p.gout + (i * HEADS + h) * HEAD_DIM;
                const float *w = p.W + (size_t)h * HEAD_DIM * KBINS + k;
                float acc = 0.f;
#pragma unroll
                for (int m = 0; m < HEAD_DIM; ++m) acc = fmaf(__ldg(w + m * KBINS), go[m], acc);
                u[h * U_STRIDE + k] = acc;
            }
        }
        __syncthreads();
        // ---- per key: q.k - lse, p_ij, gout_i.v_j - delta_i; warp w owns heads 2w and 2w+1
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const int h = 2 * warp + hh;
            float4 qv[4], gv4[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                qv[t] = __ldg(reinterpret_cast<const float4 *>(p.q + (i * HEADS + h) * HEAD_DIM) + t);
                gv4[t] = __ldg(reinterpret_cast<const float4 *>(p.gout + (i * HEADS + h) * HEAD_DIM) + t);
            }
            const float lse = p.lse[i * HEADS + h], dl = delta_s[h];
            for (int j = lane; j < n; j += 32) {
                const float4 *kp = reinterpret_cast<const float4 *>(p.k + ((a0 + j) * HEADS + h) * HEAD_DIM);
                const float4 *vp = reinterpret_cast<const float4 *>(p.v + ((a0 + j) * HEADS + h) * HEAD_DIM);
                float s = 0.f, g = 0.f;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    const float4 kv = __ldg(kp + t), vv = __ldg(vp + t);
                    s = fmaf(qv[t].x, kv.x, s); s = fmaf(qv[t].y, kv.y, s); s = fmaf(qv[t].z, kv.z, s); s = fmaf(qv[t].w, kv.w, s);
                    g = fmaf(gv4[t].x, vv.x, g); g = fmaf(gv4[t].y, vv.y, g); g = fmaf(gv4[t].z, vv.z, g); g = fmaf(gv4[t].w, vv.w, g);
                }
                cj[j * 8 + h] = (s - lse) * LOG2E;
                pj[j * 8 + h] = ex2((p.logit[(e0 + j) * HEADS + h] - lse) * LOG2E);
                gov[j * 8 + h] = g - dl;
                s0[j * 8 + h] = 0.f;
            }
        }
        __syncthreads();

        // ---- main pass: each warp takes a contiguous range of keys and all their translations
        const float a_own = p.a[i * HEADS + (lane & 7)];
        const int pk_own = packed_box(p.rule, a_own, p.rvlen ? p.rvlen + 3 * c : nullptr);
        int uni = pk_own;
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) uni = box_union(uni, __shfl_xor_sync(FULL, uni, o));
        const bool masked = !__all_sync(FULL, pk_own == uni);
        float a2[8];
        int pk[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) {
            a2[h] = __shfl_sync(FULL, a_own, h) * LOG2E;
            pk[h] = __shfl_sync(FULL, pk_own, h);
        }
        float G[8];
#pragma unroll
        for (int h = 0; h < 8; ++h) G[h] = 0.f;
        // lanes 0..7 carry the running per-key sum of head (lane) while walking the staged entries in order
        float run = 0.f;
        int run_key = -1;
        // one term per lane: the eight joint weights, their part of ga, and (K > 0) the contraction of the basis with u
        auto term = [&](bool valid, int j, float d2, int key) {
            const float4 ca = *reinterpret_cast<const float4 *>(cj + j * 8);
            const float4 cb = *reinterpret_cast<const float4 *>(cj + j * 8 + 4);
            const float4 ga4 = *reinterpret_cast<const float4 *>(gov + j * 8);
            const float4 gb4 = *reinterpret_cast<const float4 *>(gov + j * 8 + 4);
            const float off[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
            const float gj[8] = {ga4.x, ga4.y, ga4.z, ga4.w, gb4.x, gb4.y, gb4.z, gb4.w};
            float w[8];
            float emax = -INFINITY;
#pragma unroll
            for (int h = 0; h < 8; ++h) {
                float eh = fmaf(a2[h], d2, off[h]);
                if (!valid || (masked && !key_in_box(key, pk[h]))) eh = -INFINITY;
                w[h] = ex2(eh);
                emax = fmaxf(emax, eh);
                G[h] = fmaf(w[h] * d2, gj[h], G[h]);
            }
            if (K > 0) {
                const float x = fast_sqrt(d2) * p.basis.bin_scale;
                const bool keep = emax > p.basis.floor_log2 && d2 < p.basis.d2_cut;
                const int cnt = stage_terms(stage, lane, keep, x, d2, j, w);
                if (cnt > 0) {
                    if (lane < cnt) {
                        const float4 *row = reinterpret_cast<const float4 *>(stage + BWD_ENTRY_FLOATS * lane);
                        const float4 hd = row[0], pa = row[1], pb = row[2];
                        const float pw[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
                        float cd[8];
                        if (K == 64 && p.basis.windowed) basis_dot_window(u, hd.x, p.basis.bin_step, cd);
                        else basis_dot<(K > 0 ? K : 4)>(u, hd.x, p.basis.bin_step, cd);
                        float pc[8];
#pragma unroll
                        for (int h = 0; h < 8; ++h) {
                            pc[h] = pw[h] * cd[h];
                            G[h] = fmaf(pc[h], hd.y, G[h]);
                        }
                        reinterpret_cast<float4 *>(res + 8 * lane)[0] = make_float4(pc[0], pc[1], pc[2], pc[3]);
                        reinterpret_cast<float4 *>(res + 8 * lane)[1] = make_float4(pc[4], pc[5], pc[6], pc[7]);
                    }
                    __syncwarp();
                    if (lane < 8) {  // ordered walk: entries are sorted by key
                        for (int m = 0; m < cnt; ++m) {
                            const int key_m = __float_as_int(stage[BWD_ENTRY_FLOATS * m + 2]);
                            if (key_m != run_key) {
                                if (run_key >= 0) s0[run_key * 8 + lane] = run;
                                run = 0.f;
                                run_key = key_m;
                            }
                            run += res[8 * m + lane];
                        }
                    }
                }
                __syncwarp();
            }
        };
        const int list_first = (p.list.pool != nullptr && n > 0) ? p.list.start[e0] : -1;
        if (list_first >= 0) {
            // ---- terms from the row's list (entries contiguous, keys ascending).  A warp takes whole keys, so that
            //      every per-key sum has one owner: warp w gets the keys whose first entry lies in its equal share
            const int list_end = p.list.start[e0 + n - 1] + p.list.count[e0 + n - 1];
            const int span = list_end - list_first, share = (span + WARPS - 1) / WARPS;
            auto keys_before = [&](int target) {  // number of keys whose entries start before `target` (warp-uniform)
                int cnt = 0;
                for (int j0 = 0; j0 < n; j0 += 32) {
                    const int j = j0 + lane;
                    const bool before = j < n && p.list.start[e0 + j] - list_first < target;
                    cnt += __popc(__ballot_sync(FULL, before));
                }
                return cnt;
            };
            const int k_lo = warp == 0 ? 0 : keys_before(warp * share);
            const int k_hi = warp == WARPS - 1 ? n : keys_before((warp + 1) * share);
            const int w_lo = k_lo < n ? p.list.start[e0 + k_lo] : list_end;
            const int w_hi = k_hi < n ? p.list.start[e0 + k_hi] : list_end;
            float2 ahead = make_float2(0.f, 0.f);  // the entries of the next step, requested one step early
            if (w_lo + lane < w_hi) ahead = __ldg(p.list.pool + w_lo + lane);
            for (int at = w_lo; at < w_hi; at += 32) {
                const bool live = at + lane < w_hi;
                const float2 en = ahead;
                if (at + 32 + lane < w_hi) ahead = __ldg(p.list.pool + at + 32 + lane);
                const int key = __float_as_int(en.y);
                // (the lists are built for a box that contains every head's: terms outside this row's boxes drop out here)
                term(live && key_in_box(key, uni), live ? (key & 2047) : k_lo, en.x, key);
            }
        } else {
            const int R1 = box_r1(uni), R2 = box_r2(uni), R3 = box_r3(uni);
            const unsigned per_key = (unsigned)((2 * R1 + 1) * (2 * R2 + 1) * (2 * R3 + 1));
            const int keys_per_warp = (n + WARPS - 1) / WARPS;
            const int j_begin = min(warp * keys_per_warp, n), j_end = min(j_begin + keys_per_warp, n);
            const unsigned begin = (unsigned)j_begin * per_key, end = (unsigned)j_end * per_key;
            Cell cell;
            cell.load(p.tvecs + 9 * c);
            const float F1 = (float)R1, F2 = (float)R2, F3 = (float)R3;
            TermWalker walk;
            walk.init(R1, R2, R3, begin + lane);
            for (unsigned base = begin; base < end; base += 32) {
                const bool valid = base + lane < end;
                const int j = valid ? walk.row : j_begin;
                const float4 r = rel[j];
                const float f1 = walk.u1 - F1, f2 = walk.u2 - F2, f3 = walk.u3 - F3;
                const float dx = fmaf(cell.t3x, f3, fmaf(cell.t2x, f2, fmaf(cell.t1x, f1, r.x)));
                const float dy = fmaf(cell.t3y, f3, fmaf(cell.t2y, f2, fmaf(cell.t1y, f1, r.y)));
                const float dz = fmaf(cell.t3z, f3, fmaf(cell.t2z, f2, fmaf(cell.t1z, f1, r.z)));
                const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
                int key = 0;
                if (masked) key = pack_key(0, abs(__float2int_rn(f1)), abs(__float2int_rn(f2)), abs(__float2int_rn(f3)));
                term(valid, j, d2, key);
                walk.step();
            }
        }
        if (K > 0 && lane < 8 && run_key >= 0) s0[run_key * 8 + lane] = run;
#pragma unroll
        for (int h = 0; h < 8; ++h) G[h] = warp_sum(G[h]);
        if (lane < 8) ga_part[warp * 8 + lane] = pick8(G, lane);
        __syncthreads();
        if (tid < HEADS)
            p.ga[i * HEADS + tid] = (ga_part[tid] + ga_part[8 + tid]) + (ga_part[16 + tid] + ga_part[24 + tid]);
        // ---- glogit_ij = p_ij (gov_j - delta) + S0_ij ; keep it in shared memory for gq
        for (int idx = tid; idx < n * HEADS; idx += THREADS) {
            const float g = fmaf(pj[idx], gov[idx], s0[idx]);
            s0[idx] = g;
            p.glogit[e0 * HEADS + idx] = g;
        }
        __syncthreads();
        {
            const int h = tid >> 4;
            float acc = 0.f;
            const float *kp = p.k + a0 * HEADS * HEAD_DIM + tid;
            for (int j = 0; j < n; ++j) acc = fmaf(s0[j * 8 + h], __ldg(kp + (size_t)j * HEADS * HEAD_DIM), acc);
            p.gq[i * HEADS * HEAD_DIM + tid] = acc;
        }
        __syncthreads();
    }
}

// gk_j = sum_i glogit_ij q_i, gv_j = sum_i p_ij gout_i with p_ij = exp(logit_ij - lse_i); warp per (key, head).
__global__ void __launch_bounds__(256) infinite_attn_bwd_cols_kernel(const BwdRowArgs p)
{
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    const int d = lane & 15, half = lane >> 4;
    for (long long j = blockIdx.x; j < p.N; j += gridDim.x) {
        const long long r0 = p.row_start[j];
        const int n = (int)(p.row_start[j + 1] - r0);
        if (n == 0) continue;
        const long long first = p.edges[p.E + r0];
        const long long c0 = p.row_start[first];
        const long long jl = j - first;
        float av = 0.f, ak = 0.f;
        for (int il = half; il < n; il += 2) {
            const long long i = first + il, e = c0 + (long long)il * n + jl;
            const float pr = ex2((p.logit[e * HEADS + h] - p.lse[i * HEADS + h]) * LOG2E);
            av = fmaf(pr, __ldg(p.gout + (i * HEADS + h) * HEAD_DIM + d), av);
            ak = fmaf(p.glogit[e * HEADS + h], __ldg(p.q + (i * HEADS + h) * HEAD_DIM + d), ak);
        }
        av += __shfl_xor_sync(FULL, av, 16);
        ak += __shfl_xor_sync(FULL, ak, 16);
        if (half == 0) {
            p.gv[(j * HEADS + h) * HEAD_DIM + d] = av;
            p.gk[(j * HEADS + h) * HEAD_DIM + d] = ak;
        }
    }
}

}  // namespace

int infinite_attn_bwd_impl(const float *q, const float *k, const float *v, const float *a, const float *pos,
                           const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                           const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D,
                           int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                           double cutoff_radius, int lattice_range, int minimum_range, const float *logit,
                           const float *lse, const float *out, const float *gout, float *gq, float *gk, float *gv,
                           float *ga, float *glogit, const int32_t *row_order, const TermList *list, void *stream);

}  // namespace cf

extern "C" int cf_infinite_attn_bwd(const float *q, const float *k, const float *v, const float *a, const float *pos,
                                    const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                                    const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                                    int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                                    const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                                    const float *logit, const float *lse, const float *out, const float *gout, float *gq,
                                    float *gk, float *gv, float *ga, float *glogit, const int32_t *row_order,
                                    void *stream)
{
    return cf::infinite_attn_bwd_impl(q, k, v, a, pos, pos_ij, tvecs, rvlen, batch, edges, row_start, N, B, H, D, E, K,
                                      max_atoms, dist_max, wscale, W, cutoff_radius, lattice_range, minimum_range, logit,
                                      lse, out, gout, gq, gk, gv, ga, glogit, row_order, nullptr, stream);
}

extern "C" int cf_infinite_attn_bwd_listed(const float *q, const float *k, const float *v, const float *a,
                                           const float *pos_ij, const float *tvecs, const float *rvlen,
                                           const int64_t *batch, const int64_t *edges, const int64_t *row_start,
                                           int64_t N, int64_t B, int64_t H, int64_t D, int64_t E, int64_t K,
                                           int64_t max_atoms, double dist_max, double wscale, const float *W,
                                           double cutoff_radius, int lattice_range, int minimum_range,
                                           const float *logit, const float *lse, const float *out, const float *gout,
                                           float *gq, float *gk, float *gv, float *ga, float *glogit,
                                           const int32_t *row_order, void *term_lists, double a_widest, void *stream)
{
    using namespace cf;
    CF_REQUIRE(term_lists != nullptr && pos_ij != nullptr && a_widest < 0, CF_ERR_INVALID,
               "cf_infinite_attn_bwd_listed: needs term lists, pos_ij and a negative a_widest");
    CF_REQUIRE(N >= 0 && E >= 0, CF_ERR_INVALID, "cf_infinite_attn_bwd_listed: negative size");
    TermList list{};
    int *start, *count;
    float *dmin;
    unsigned long long *cursor;
    float2 *pool;
    term_list_carve(term_lists, N, E, &start, &count, &dmin, &cursor, &pool);
    list.pool = pool; list.start = start; list.count = count; list.dmin = dmin;
    list.window = term_window(weight_floor_log2(), (float)a_widest);
    return infinite_attn_bwd_impl(q, k, v, a, nullptr, pos_ij, tvecs, rvlen, batch, edges, row_start, N, B, H, D, E, K,
                                  max_atoms, dist_max, wscale, W, cutoff_radius, lattice_range, minimum_range, logit, lse,
                                  out, gout, gq, gk, gv, ga, glogit, row_order, &list, stream);
}

int cf::infinite_attn_bwd_impl(const float *q, const float *k, const float *v, const float *a, const float *pos,
                               const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                               const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                               int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                               const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                               const float *logit, const float *lse, const float *out, const float *gout, float *gq,
                               float *gk, float *gv, float *ga, float *glogit, const int32_t *row_order,
                               const TermList *list, void *stream)
{
    CF_REQUIRE(N >= 0 && E >= 0 && B >= 0, CF_ERR_INVALID, "cf_infinite_attn_bwd: negative size");
    CF_REQUIRE(H == HEADS && D == HEAD_DIM, CF_ERR_UNSUPPORTED, "cf_infinite_attn_bwd: H=%lld D=%lld, only H=8 D=16 is compiled",
               (long long)H, (long long)D);
    CF_REQUIRE(K == 0 || K == 64, CF_ERR_UNSUPPORTED, "cf_infinite_attn_bwd: K=%lld, only K in {0,64} is compiled", (long long)K);
    CF_REQUIRE(lattice_range >= 0 && lattice_range <= CF_MAX_RANGE && minimum_range >= 0, CF_ERR_RANGE,
               "cf_infinite_attn_bwd: lattice_range %d outside [0,%d]", lattice_range, CF_MAX_RANGE);
    CF_REQUIRE(max_atoms >= 1 && max_atoms <= 1024, CF_ERR_RANGE, "cf_infinite_attn_bwd: max_atoms=%lld outside [1,1024]",
               (long long)max_atoms);
    if (N == 0) return CF_OK;
    CF_REQUIRE(q && k && v && a && (pos || pos_ij) && tvecs && batch && edges && row_start && logit && lse && out && gout &&
                   gq && gk && gv && ga && glogit, CF_ERR_INVALID, "cf_infinite_attn_bwd: null pointer");
    CF_REQUIRE(K == 0 || (W != nullptr && dist_max > 0 && wscale > 0), CF_ERR_INVALID,
               "cf_infinite_attn_bwd: K > 0 needs W and positive dist_max, wscale");
    cudaStream_t s = as_stream(stream);
    BwdRowArgs p{};
    p.q = q; p.k = k; p.v = v; p.a = a; p.pos = pos; p.pos_ij = pos_ij; p.tvecs = tvecs; p.rvlen = rvlen; p.W = W;
    p.logit = logit; p.lse = lse; p.out = out; p.gout = gout; p.batch = batch; p.edges = edges; p.row_start = row_start;
    p.gq = gq; p.gk = gk; p.gv = gv; p.ga = ga; p.glogit = glogit; p.row_order = row_order; p.N = N; p.E = E; p.max_atoms = (int)max_atoms;
    p.rule = BoxRule{(float)cutoff_radius, lattice_range, minimum_range};
    p.basis = make_basis_params(K, dist_max, wscale, weight_floor_log2());
    if (list != nullptr) p.list = *list;
    const size_t smem = sizeof(float) * bwd_row_smem_floats((int)max_atoms, K > 0);
    auto kernel = K > 0 ? infinite_attn_bwd_rows_kernel<64> : infinite_attn_bwd_rows_kernel<0>;
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
            cudaGetLastError();
            return fail(CF_ERR_RANGE, "cf_infinite_attn_bwd: %zu bytes of shared memory for max_atoms=%lld not available",
                        smem, (long long)max_atoms);
        }
    }
    int occ = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, kernel, THREADS, smem) != cudaSuccess || occ <= 0) occ = 1;
    const long long cap = (long long)sm_count() * occ;
    kernel<<<(int)(N < cap ? N : cap), THREADS, smem, s>>>(p);
    const long long cap2 = (long long)sm_count() * 8;
    infinite_attn_bwd_cols_kernel<<<(int)(N < cap2 ? N : cap2), 256, 0, s>>>(p);
    return launch_status("cf_infinite_attn_bwd");
}
