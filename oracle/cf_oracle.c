/*
 * CPU oracle for the infinitely-connected-attention hot path.  TEST INFRASTRUCTURE ONLY:
 * nothing in the shipped package may link or call this file; it exists so that tests, the
 * smoke check and the benchmark's CPU-baseline leg have an independent statement of what
 * the CUDA kernels must compute.
 *
 * It restates, in plain C with the same loop order and (in the _f32 build) the same float
 * arithmetic, the algorithms of the reference project's device kernels and host helpers.
 * Every function names the reference file:line it follows (paths relative to the
 * reference project root).  The file is compiled twice, with REAL = float (symbols *_f32)
 * and REAL = double (symbols *_f64, the arbiter for tolerance questions).
 *
 * Pinning: tests/test_oracle_golden.py checks this file against vectors produced by the
 * reference's own PyTorch implementation (tests/golden/make_golden.py) and, where the
 * reference kernels themselves were compiled for the CPU (oracle/_ref), against those.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifndef REAL
#define REAL float
#define SUFFIX _f32
#endif
#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

typedef long long i64;

#define CFO_PI_F 3.141592654f /* the single-precision pi constant the reference kernels use */

static inline REAL r_exp(REAL x) { return sizeof(REAL) == 4 ? (REAL)expf((float)x) : (REAL)exp((double)x); }
static inline REAL r_log(REAL x) { return sizeof(REAL) == 4 ? (REAL)logf((float)x) : (REAL)log((double)x); }
static inline REAL r_sqrt(REAL x) { return sizeof(REAL) == 4 ? (REAL)sqrtf((float)x) : (REAL)sqrt((double)x); }

/* ------------------------------------------------------------------------------------------
 * Translation box of one (atom, head).
 * Follows models/kernels/real_enc_fwd.cu:63-85 (identical text in real_enc_proj_fwd.cu:66-88,
 * real_enc_bwd.cu:60-82, real_enc_proj_bwd.cu:63-86).  Always evaluated in the kernels' mixed
 * float/double arithmetic so that the integers are reproduced exactly:
 *   cutoff_radius == 0 : R = lattice_range in every direction
 *   cutoff_radius <  0 : radius = sqrtf(-0.5f / a) * (-cutoff_radius)      (float)
 *   cutoff_radius >  0 : radius = (float)cutoff_radius
 *   R_d = ceil( (double)((radius + 0.01f) * rvlen_d) / (2.0 * (double)pi_f) ), then max(R_d, minimum_range).
 * ---------------------------------------------------------------------------------------- */
static void box_of(float a, const float *rvlen3, double cutoff_radius, int lattice_range, int minimum_range, int R[3])
{
    float cutoff = (float)cutoff_radius;
    R[0] = R[1] = R[2] = lattice_range;
    if (cutoff != 0.0f) {
        if (cutoff < 0) cutoff = sqrtf(-0.5f / a) * (-cutoff);
        const double two_pi = 2.0 * CFO_PI_F;
        for (int d = 0; d < 3; d++) {
            float reach = (cutoff + 0.01f) * rvlen3[d];
            int r = (int)ceil((double)reach / two_pi);
            if (minimum_range > 0 && r < minimum_range) r = minimum_range;
            R[d] = r;
        }
    }
}

void FN(cfo_box)(const float *a, i64 count, const float *rvlen3, double cutoff_radius, int lattice_range,
                 int minimum_range, int *R_out)
{
    for (i64 t = 0; t < count; t++) box_of(a[t], rvlen3, cutoff_radius, lattice_range, minimum_range, R_out + 3 * t);
}

/* ------------------------------------------------------------------------------------------
 * All-pairs edge list.  Follows models/indexed_latticeformer_encoder.py:15-32.
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_edge_index)(const i64 *sizes, i64 B, i64 *edges /* (2,E) */, i64 E)
{
    i64 e = 0, c = 0;
    for (i64 b = 0; b < B; b++) {
        i64 n = sizes[b];
        for (i64 i = 0; i < n; i++)
            for (i64 j = 0; j < n; j++, e++) {
                edges[e] = c + i;
                edges[E + e] = c + j;
            }
        c += n;
    }
}

/* ------------------------------------------------------------------------------------------
 * Geometry handed to the kernels.  Follows models/indexed_latticeformer_encoder.py:183-253
 * (pos_ij :215, cell volume via det_3x3 :34-44,206, reciprocal rows 2*pi*(t_b x t_c)/V :208-213) and
 * the row norms taken in models/indexed_lattice_multi_head_attention_cuda.py:400.  float32 like torch.
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_geometry)(const float *pos, const float *trans, const i64 *edges, i64 B, i64 E,
                      float *pos_ij, float *rvecs, float *vcell, float *rvlen)
{
    for (i64 e = 0; e < E; e++)
        for (int d = 0; d < 3; d++) pos_ij[3 * e + d] = pos[3 * edges[E + e] + d] - pos[3 * edges[e] + d];
    for (i64 b = 0; b < B; b++) {
        const float *m = trans + 9 * b;
        float v = m[0] * m[4] * m[8] + m[1] * m[5] * m[6] + m[2] * m[3] * m[7]
                - m[2] * m[4] * m[6] - m[0] * m[5] * m[7] - m[1] * m[3] * m[8];
        vcell[b] = v;
        float scale = (float)(2.0 * M_PI) / v; /* torch: python double 2*pi divided into a float tensor */
        for (int r = 0; r < 3; r++) {
            const float *u = m + 3 * ((r + 1) % 3), *w = m + 3 * ((r + 2) % 3);
            float c[3] = { u[1] * w[2] - u[2] * w[1], u[2] * w[0] - u[0] * w[2], u[0] * w[1] - u[1] * w[0] };
            float s = 0;
            for (int d = 0; d < 3; d++) {
                float x = c[d] * scale;
                rvecs[9 * b + 3 * r + d] = x;
                s += x * x;
            }
            rvlen[3 * b + r] = sqrtf(s);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Real-space lattice sum, forward.
 * Follows models/kernels/real_enc_fwd.cu:22-144 (psi written as is) and real_enc_proj_fwd.cu:24-169
 * (W psi written); `nested` selects the per-loop partial sums of the *_v2 files (real_enc_fwd_v2.cu:109-122).
 *   phi[e,h] = log sum_n exp(a (d2_n - d2min)) + a d2min
 *   psi[e,h,k] = sum_n exp(a (d2_n - d2min)) exp(-b_k(n)^2) / sum_n exp(a (d2_n - d2min)),
 *   b_k = ((k+1) - d_n/mu0) / (sqrt2 wscale), mu0 = dist_max/K, advanced as b += 1/(wscale sqrt2).
 * `a` is indexed by the edge's source atom (reference) or, when a_per_edge != 0, by the edge itself
 * (needed by the kernel microbenchmark, which draws one width per (edge, head)).
 * W: (W_num, H, Dv, K) with W_num in {1, E, N} (real_enc_proj_fwd.cu:139-148); W == NULL writes psi (E,H,K).
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_lattice_sum_fwd)(const float *a_in, int a_per_edge, const float *pos_ij, const float *tvecs,
                             const i64 *batch, const i64 *edges, i64 N, i64 H, i64 E, i64 K, double dist_max,
                             double wscale, const float *W, i64 W_num, i64 Dv, const float *rvlen,
                             double cutoff_radius, int lattice_range, int minimum_range, int nested,
                             REAL *z_out, REAL *v_out, int *box_out /* (E,H,3) or NULL */)
{
#pragma omp parallel
    {
        REAL *sv = (REAL *)malloc(sizeof(REAL) * (size_t)(K > 0 ? K : 1));
#pragma omp for schedule(dynamic, 16)
        for (i64 e = 0; e < E; e++) {
            const i64 i = edges[e];
            const i64 c = batch[i];
            const REAL rx = pos_ij[3 * e], ry = pos_ij[3 * e + 1], rz = pos_ij[3 * e + 2];
            const float *t = tvecs + 9 * c;
            for (i64 h = 0; h < H; h++) {
                const float af = a_per_edge ? a_in[e * H + h] : a_in[i * H + h];
                const REAL a = af;
                int R[3];
                box_of(af, rvlen ? rvlen + 3 * c : NULL, rvlen ? cutoff_radius : 0.0, lattice_range, minimum_range, R);
                if (box_out) memcpy(box_out + 3 * (e * H + h), R, sizeof(R));

                REAL d2min = (REAL)1e10;
                for (int n1 = -R[0]; n1 <= R[0]; n1++)
                    for (int n2 = -R[1]; n2 <= R[1]; n2++)
                        for (int n3 = -R[2]; n3 <= R[2]; n3++) {
                            REAL dx = rx + (REAL)t[0] * n1 + (REAL)t[3] * n2 + (REAL)t[6] * n3;
                            REAL dy = ry + (REAL)t[1] * n1 + (REAL)t[4] * n2 + (REAL)t[7] * n3;
                            REAL dz = rz + (REAL)t[2] * n1 + (REAL)t[5] * n2 + (REAL)t[8] * n3;
                            REAL d2 = dx * dx + dy * dy + dz * dz;
                            if (d2 < d2min) d2min = d2;
                        }

                const REAL step = (REAL)1.0 / ((REAL)(float)wscale * r_sqrt((REAL)2.0));
                const REAL mu0 = K > 0 ? (REAL)(float)dist_max / (REAL)K : (REAL)1;
                for (i64 k = 0; k < K; k++) sv[k] = 0;
                REAL sum = 0;
                for (int n1 = -R[0]; n1 <= R[0]; n1++) {
                    REAL s1 = 0;
                    for (int n2 = -R[1]; n2 <= R[1]; n2++) {
                        REAL s2 = 0;
                        for (int n3 = -R[2]; n3 <= R[2]; n3++) {
                            REAL dx = rx + (REAL)t[0] * n1 + (REAL)t[3] * n2 + (REAL)t[6] * n3;
                            REAL dy = ry + (REAL)t[1] * n1 + (REAL)t[4] * n2 + (REAL)t[7] * n3;
                            REAL dz = rz + (REAL)t[2] * n1 + (REAL)t[5] * n2 + (REAL)t[8] * n3;
                            REAL d2 = dx * dx + dy * dy + dz * dz;
                            REAL w = r_exp(a * (d2 - d2min));
                            if (nested) s2 += w; else sum += w;
                            if (K > 0) {
                                REAL b = -r_sqrt(d2) / mu0 * step;
                                for (i64 k = 0; k < K; k++) {
                                    b += step;
                                    sv[k] += r_exp(-b * b) * w;
                                }
                            }
                        }
                        if (nested) s1 += s2;
                    }
                    if (nested) sum += s1;
                }
                z_out[e * H + h] = r_log(sum) + d2min * a;
                if (K > 0 && v_out) {
                    if (!W) {
                        for (i64 k = 0; k < K; k++) v_out[(e * H + h) * K + k] = sv[k] / sum;
                    } else {
                        i64 wi = (W_num == 1) ? 0 : (W_num == E ? e : i);
                        const float *Wh = W + (wi * H + h) * Dv * K;
                        if (nested) for (i64 k = 0; k < K; k++) sv[k] = sv[k] / sum;
                        for (i64 m = 0; m < Dv; m++) {
                            REAL acc = 0;
                            for (i64 k = 0; k < K; k++) acc += (REAL)Wh[m * K + k] * sv[k];
                            v_out[(e * H + h) * Dv + m] = nested ? acc : acc / sum;
                        }
                    }
                }
            }
        }
        free(sv);
    }
    (void)N;
}

/* ------------------------------------------------------------------------------------------
 * Real-space lattice sum, backward with respect to `a` (N,H) and the projection W.
 * Follows models/kernels/real_enc_bwd.cu:80-156 (gv is the gradient of psi itself, W == NULL) and
 * real_enc_proj_bwd.cu:88-221 (gv is the gradient of W psi; u = W^T gv :108-131; gW += gv (x) psi :205-218).
 * With p_n = exp(a d2_n - phi) and c_n = sum_k exp(-b_k(n)^2) u_k:
 *   ga[i,h] = sum_{e in row i} [ gz_e C1 + C2 - C1 C0 ],  C0 = sum_n p_n c_n, C1 = sum_n d2_n p_n, C2 = sum_n d2_n p_n c_n.
 * gW_out, when not NULL, receives one (H,Dv,K) block per W instance (W_num in {1,N,E}): for W_num == 1 the
 * per-atom blocks the reference writes (real_enc_proj_bwd.cu:51-55) are already summed over atoms here, which is
 * what autograd does with them afterwards.
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_lattice_sum_bwd)(const float *a_in, const float *pos_ij, const float *tvecs, const i64 *batch,
                             const i64 *edges, const i64 *e_start, const REAL *z, const REAL *gz, const REAL *gv,
                             i64 N, i64 H, i64 E, i64 K, double dist_max, double wscale, const float *W, i64 W_num,
                             i64 Dv, const float *rvlen, double cutoff_radius, int lattice_range, int minimum_range,
                             REAL *ga_out, REAL *gW_out)
{
    const size_t wblk = (size_t)(H * Dv * K);
    REAL *gW_atoms = NULL;
    if (gW_out && W && W_num == 1) gW_atoms = (REAL *)calloc((size_t)N * wblk, sizeof(REAL));
    if (gW_out && W) memset(gW_out, 0, sizeof(REAL) * wblk * (size_t)W_num);
#pragma omp parallel
    {
        REAL *u = (REAL *)malloc(sizeof(REAL) * (size_t)(K > 0 ? K : 1));
        REAL *sv = (REAL *)malloc(sizeof(REAL) * (size_t)(K > 0 ? K : 1));
#pragma omp for schedule(dynamic, 4)
        for (i64 i = 0; i < N; i++) {
            const i64 c = batch[i];
            const float *t = tvecs + 9 * c;
            for (i64 h = 0; h < H; h++) {
                const float af = a_in[i * H + h];
                const REAL a = af;
                int R[3];
                box_of(af, rvlen ? rvlen + 3 * c : NULL, rvlen ? cutoff_radius : 0.0, lattice_range, minimum_range, R);
                const REAL step = (REAL)1.0 / ((REAL)(float)wscale * r_sqrt((REAL)2.0));
                const REAL mu0 = K > 0 ? (REAL)(float)dist_max / (REAL)K : (REAL)1;
                REAL total = 0, total_v = 0;
                for (i64 e = e_start[i]; e < e_start[i + 1]; e++) {
                    const REAL rx = pos_ij[3 * e], ry = pos_ij[3 * e + 1], rz = pos_ij[3 * e + 2];
                    const i64 eh = e * H + h;
                    const REAL *g = NULL;
                    const float *Wh = NULL;
                    REAL *gWh = NULL;
                    if (K > 0 && gv) {
                        if (!W) {
                            for (i64 k = 0; k < K; k++) u[k] = gv[eh * K + k];
                        } else {
                            i64 wi = (W_num == 1) ? 0 : (W_num == E ? e : i);
                            Wh = W + (wi * H + h) * Dv * K;
                            g = gv + eh * Dv;
                            for (i64 k = 0; k < K; k++) u[k] = 0;
                            for (i64 m = 0; m < Dv; m++)
                                for (i64 k = 0; k < K; k++) u[k] += (REAL)Wh[m * K + k] * g[m];
                            if (gW_out) {
                                if (W_num == 1) gWh = gW_atoms + (size_t)i * wblk + (size_t)h * Dv * K;
                                else gWh = gW_out + (size_t)wi * wblk + (size_t)h * Dv * K;
                            }
                        }
                        for (i64 k = 0; k < K; k++) sv[k] = 0;
                    }
                    REAL c0 = 0, c1 = 0;
                    for (int n1 = -R[0]; n1 <= R[0]; n1++)
                        for (int n2 = -R[1]; n2 <= R[1]; n2++)
                            for (int n3 = -R[2]; n3 <= R[2]; n3++) {
                                REAL dx = rx + (REAL)t[0] * n1 + (REAL)t[3] * n2 + (REAL)t[6] * n3;
                                REAL dy = ry + (REAL)t[1] * n1 + (REAL)t[4] * n2 + (REAL)t[7] * n3;
                                REAL dz = rz + (REAL)t[2] * n1 + (REAL)t[5] * n2 + (REAL)t[8] * n3;
                                REAL d2 = dx * dx + dy * dy + dz * dz;
                                REAL p = r_exp(a * d2 - z[eh]);
                                REAL px = d2 * p;
                                c1 += px;
                                if (K > 0 && gv) {
                                    REAL cn = 0;
                                    REAL b = -r_sqrt(d2) / mu0 * step;
                                    for (i64 k = 0; k < K; k++) {
                                        b += step;
                                        REAL gk = r_exp(-b * b);
                                        cn += gk * u[k];
                                        sv[k] += gk * p;
                                    }
                                    total_v += px * cn;
                                    c0 += p * cn;
                                }
                            }
                    total += c1 * gz[eh];
                    total_v -= c1 * c0;
                    if (gWh)
                        for (i64 m = 0; m < Dv; m++)
                            for (i64 k = 0; k < K; k++) gWh[m * K + k] += sv[k] * g[m];
                }
                ga_out[i * H + h] = total + total_v;
            }
        }
        free(u);
        free(sv);
    }
    if (gW_atoms) {
        for (i64 i = 0; i < N; i++)
            for (size_t x = 0; x < wblk; x++) gW_out[x] += gW_atoms[(size_t)i * wblk + x];
        free(gW_atoms);
    }
}

/* ------------------------------------------------------------------------------------------
 * Fixed-shape pairwise summation tree.  Follows models/kernels/pairwise_sum.cuh:37-75
 * (halves recursively; lengths here are powers of two).
 * ---------------------------------------------------------------------------------------- */
static REAL tree_sum(const REAL *x, int n)
{
    if (n == 1) return x[0];
    if (n == 2) return x[0] + x[1];
    return tree_sum(x, n / 2) + tree_sum(x + n / 2, n / 2);
}

/* ------------------------------------------------------------------------------------------
 * Edge-indexed softmax attention, forward.
 * Follows models/kernels/fused_dpa_fwd.cu:19-125 and fused_dpa_fwd_v3.cu:19-136 (`run_len` > 0 selects the
 * v3 running partial sums of that length, :81-132).  q is already divided by sqrt(D) by the caller
 * (models/indexed_lattice_multi_head_attention_cuda.py:179).
 *   logit_ij = q_i . k_j + phi_ij ; p = softmax_j (max-subtracted, denominator summed pairwise in 64-blocks)
 *   out_i = sum_j p_ij (v_j + b_ij)
 * `max_sys_pow2` is the padded length of the second summation level (512 in the reference).
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_fused_attn_fwd)(const REAL *q, const REAL *k, const REAL *v, const REAL *aij, const REAL *bij,
                            const i64 *edges, const i64 *e_start, i64 N, i64 H, i64 E, i64 D, int run_len,
                            int max_sys_pow2, REAL *prob, REAL *out)
{
    enum { BS = 64 };
#pragma omp parallel
    {
        i64 cap = 0;
        REAL *w = NULL;
        REAL *blocks = (REAL *)malloc(sizeof(REAL) * (size_t)(max_sys_pow2 / BS));
        REAL *o = (REAL *)malloc(sizeof(REAL) * (size_t)D), *run = (REAL *)malloc(sizeof(REAL) * (size_t)D);
#pragma omp for schedule(dynamic, 8)
        for (i64 i = 0; i < N; i++) {
            const i64 e0 = e_start[i], cnt = e_start[i + 1] - e0;
            const i64 padded = (cnt + BS - 1) / BS * BS;
            if (padded > cap) { cap = padded; w = (REAL *)realloc(w, sizeof(REAL) * (size_t)cap); }
            for (i64 h = 0; h < H; h++) {
                const REAL *qi = q + (i * H + h) * D;
                REAL mx = (REAL)-1e20;
                for (i64 t = 0; t < cnt; t++) {
                    const i64 e = e0 + t, j = edges[E + e];
                    const REAL *kj = k + (j * H + h) * D;
                    REAL s = 0;
                    for (i64 d = 0; d < D; d++) s += qi[d] * kj[d];
                    if (aij) s += aij[e * H + h];
                    if (s > mx) mx = s;
                    w[t] = s;
                }
                for (i64 t = 0; t < cnt; t++) w[t] = r_exp(w[t] - mx);
                for (i64 t = cnt; t < padded; t++) w[t] = 0;
                const int nblk = max_sys_pow2 / BS;
                for (int b = 0; b < nblk; b++) blocks[b] = (b < padded / BS) ? tree_sum(w + b * BS, BS) : 0;
                const REAL denom = tree_sum(blocks, nblk);
                for (i64 t = 0; t < cnt; t++) {
                    w[t] /= denom;
                    if (prob) prob[(e0 + t) * H + h] = w[t];
                }
                for (i64 d = 0; d < D; d++) o[d] = run[d] = 0;
                for (i64 t = 0; t < cnt; t++) {
                    const i64 e = e0 + t, j = edges[E + e];
                    const REAL *vj = v + (j * H + h) * D;
                    const REAL *be = bij ? bij + (e * H + h) * D : NULL;
                    for (i64 d = 0; d < D; d++) run[d] += (be ? vj[d] + be[d] : vj[d]) * w[t];
                    if (run_len <= 0 || ((t + 1) % run_len) == 0 || t == cnt - 1)
                        for (i64 d = 0; d < D; d++) { o[d] += run[d]; run[d] = 0; }
                }
                for (i64 d = 0; d < D; d++) out[(i * H + h) * D + d] = o[d];
            }
        }
        free(w); free(blocks); free(o); free(run);
    }
}

/* ------------------------------------------------------------------------------------------
 * Edge-indexed softmax attention, backward.
 * Follows models/kernels/fused_dpa_bwd.cu:23-125 (per key j: gV, gK, the per-edge softmax gradient and gB),
 * fused_dpa_bwd_q.cu:12-53 (per query i: gQ) and the host code around them, which transposes prob / b into
 * key-major order before and the per-edge gradients back after (models/cuda_funcs/fused_dpa.py:136-191).
 * Here the transposition is plain index arithmetic: edges of a crystal with n atoms starting at edge offset c
 * satisfy e(i,j) = c + i_local n + j_local.
 *   t_ij = go_i p_ij ; gV_j = sum_i t_ij ; gB_ij = t_ij ; gA_ij = sum_d (v_j + b_ij - o_i)_d t_ij,d
 *   gK_j = sum_i gA_ij q_i ; gQ_i = sum_j gA_ij k_j      (gQ is with respect to the pre-scaled q)
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_fused_attn_bwd)(const REAL *q, const REAL *k, const REAL *v, const REAL *bij, const i64 *edges,
                            const i64 *e_start, i64 N, i64 H, i64 E, i64 D, const REAL *prob, const REAL *out,
                            const REAL *go, REAL *gq, REAL *gk, REAL *gv, REAL *gaij, REAL *gbij)
{
#pragma omp parallel for schedule(dynamic, 8)
    for (i64 j = 0; j < N; j++) {
        /* row j of the all-pairs block lists the atoms of j's crystal in order: that is the set of queries i. */
        const i64 r0 = e_start[j], n = e_start[j + 1] - r0;
        const i64 first = edges[E + r0];             /* first atom of the crystal */
        const i64 c = e_start[first];                /* first edge of the crystal */
        const i64 jl = j - first;
        for (i64 h = 0; h < H; h++) {
            REAL *gvj = gv + (j * H + h) * D, *gkj = gk + (j * H + h) * D;
            const REAL *vj = v + (j * H + h) * D;
            for (i64 d = 0; d < D; d++) gvj[d] = gkj[d] = 0;
            for (i64 il = 0; il < n; il++) {
                const i64 i = first + il, e = c + il * n + jl;
                const REAL p = prob[e * H + h];
                const REAL *goi = go + (i * H + h) * D, *oi = out + (i * H + h) * D, *qi = q + (i * H + h) * D;
                const REAL *be = bij ? bij + (e * H + h) * D : NULL;
                REAL gs = 0;
                for (i64 d = 0; d < D; d++) {
                    REAL t = goi[d] * p;
                    gvj[d] += t;
                    if (gbij) gbij[(e * H + h) * D + d] = t;
                    gs += ((be ? vj[d] + be[d] : vj[d]) - oi[d]) * t;
                }
                gaij[e * H + h] = gs;
                for (i64 d = 0; d < D; d++) gkj[d] += gs * qi[d];
            }
        }
    }
#pragma omp parallel for schedule(dynamic, 8)
    for (i64 i = 0; i < N; i++)
        for (i64 h = 0; h < H; h++) {
            REAL *gqi = gq + (i * H + h) * D;
            for (i64 d = 0; d < D; d++) gqi[d] = 0;
            for (i64 e = e_start[i]; e < e_start[i + 1]; e++) {
                const i64 j = edges[E + e];
                const REAL gs = gaij[e * H + h];
                const REAL *kj = k + (j * H + h) * D;
                for (i64 d = 0; d < D; d++) gqi[d] += gs * kj[d];
            }
        }
}

/* ------------------------------------------------------------------------------------------
 * Per-crystal mean of atom features.  Follows models/kernels/irregular_mean_fwd.cu:4-90 together with
 * pairwise_sum.cuh:78-111: the row count is rounded up to a power of two 2^L; rows are summed in groups of
 * four by a fixed tree ((x0+x1)+(x2+x3), missing rows read as zero), and the 2^L/4 group sums by the same tree.
 * Counts 1 and 2 are summed directly (:56-60).
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_segment_mean)(const REAL *x, const i64 *start, i64 B, i64 D, REAL *out)
{
    for (i64 b = 0; b < B; b++) {
        const i64 s = start[b], len = start[b + 1] - s;
        int L = 0;
        while (((i64)1 << L) < len) L++;
        for (i64 d = 0; d < D; d++) {
            const REAL *src = x + s * D + d;
            REAL sum;
            if (L == 0) sum = len > 0 ? src[0] : 0;
            else if (L == 1) sum = src[0] + src[D];
            else {
                const int groups = (1 << L) > 4 ? (1 << L) / 4 : 1;
                REAL buf[1024];
                for (int g = 0; g < groups; g++) {
                    REAL m[4];
                    for (int t = 0; t < 4; t++) {
                        i64 idx = (i64)g * 4 + t;
                        m[t] = idx < len ? src[idx * D] : 0;
                    }
                    buf[g] = (m[0] + m[1]) + (m[2] + m[3]);
                }
                sum = tree_sum(buf, groups);
            }
            out[b * D + d] = sum / (REAL)len;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Reciprocal-space lattice sum, forward and backward.
 * Follows models/kernels/reci_enc_fwd.cu:16-67 and reci_enc_bwd.cu:19-70 (`nested` = the per-loop partial sums
 * of reci_enc_fwd_v2.cu:49-58 / reci_enc_bwd_v2.cu:57-66), and the phase handed to them,
 * kr_base = rvecs[b] . pos_ij (models/indexed_latticeformer_encoder.py:249-251).
 *   S[e,h]   = sum over n1 in [0,R], n2,n3 in [-R,R] of w(n1) exp(a |k_n|^2) cos(kr . n),  w(0) = 1, else 2,
 *              k_n = n1 r1 + n2 r2 + n3 r3 (rows of rvecs), a = a[i,h] < 0
 *   phi[e,h] = log max(S, 1e-6) + 1.5 log(-4 pi a) - log V
 *   ga[i,h]  = sum_{e of row i} gz[e,h] (S < 1e-6 ? 0 : 1/S) sum_n w |k_n|^2 exp(a |k_n|^2) cos(kr . n)
 * (the reference's backward does not differentiate the 1.5 log(-4 pi a) term; neither does this).
 * ---------------------------------------------------------------------------------------- */
void FN(cfo_reci_phase)(const float *pos_ij, const float *rvecs, const i64 *batch, const i64 *edges, i64 E,
                        float *kr_base)
{
    for (i64 e = 0; e < E; e++) {
        const float *r = rvecs + 9 * batch[edges[e]], *p = pos_ij + 3 * e;
        for (int d = 0; d < 3; d++) kr_base[3 * e + d] = r[3 * d] * p[0] + r[3 * d + 1] * p[1] + r[3 * d + 2] * p[2];
    }
}

static REAL reci_terms(REAL a, const float *kr, const float *r, int R, int nested, int weighted)
{
    REAL sum = 0;
    for (int n1 = 0; n1 <= R; n1++) {
        const REAL scale = n1 == 0 ? 1 : 2;
        REAL s1 = 0;
        for (int n2 = -R; n2 <= R; n2++) {
            REAL s2 = 0;
            for (int n3 = -R; n3 <= R; n3++) {
                const REAL k1 = (REAL)r[0] * n1 + (REAL)r[3] * n2 + (REAL)r[6] * n3;
                const REAL k2 = (REAL)r[1] * n1 + (REAL)r[4] * n2 + (REAL)r[7] * n3;
                const REAL k3 = (REAL)r[2] * n1 + (REAL)r[5] * n2 + (REAL)r[8] * n3;
                const REAL kk = k1 * k1 + k2 * k2 + k3 * k3;
                const REAL arg = (REAL)kr[0] * n1 + (REAL)kr[1] * n2 + (REAL)kr[2] * n3;
                const REAL c = sizeof(REAL) == 4 ? (REAL)cosf((float)arg) : (REAL)cos((double)arg);
                const REAL t = (weighted ? kk * r_exp(a * kk) : r_exp(a * kk)) * c * scale;
                if (nested) s2 += t; else sum += t;
            }
            if (nested) s1 += s2;
        }
        if (nested) sum += s1;
    }
    return sum;
}

void FN(cfo_reci_sum_fwd)(const float *a, const float *kr_base, const float *rvecs, const float *vcell,
                          const i64 *batch, const i64 *edges, i64 N, i64 H, i64 E, int lattice_range, int nested,
                          REAL *z_out, REAL *sum_out)
{
    (void)N;
#pragma omp parallel for schedule(dynamic, 64)
    for (i64 e = 0; e < E; e++) {
        const i64 i = edges[e], b = batch[i];
        for (i64 h = 0; h < H; h++) {
            const REAL ah = a[i * H + h];
            const REAL s = reci_terms(ah, kr_base + 3 * e, rvecs + 9 * b, lattice_range, nested, 0);
            const REAL c4pi = sizeof(REAL) == 4 ? (REAL)12.5663706144f : (REAL)12.5663706144;
            const REAL log_ci = (REAL)1.5 * r_log(-c4pi * ah) - r_log((REAL)vcell[b]);
            const REAL floor_ = sizeof(REAL) == 4 ? (REAL)1e-6f : (REAL)1e-6;
            z_out[e * H + h] = r_log(s > floor_ ? s : floor_) + log_ci;
            if (sum_out) sum_out[e * H + h] = s;
        }
    }
}

void FN(cfo_reci_sum_bwd)(const float *a, const float *kr_base, const float *rvecs, const i64 *batch,
                          const i64 *row_start, const REAL *gz, const REAL *sum_in, i64 N, i64 H, i64 E,
                          int lattice_range, int nested, REAL *ga)
{
    (void)E;
#pragma omp parallel for schedule(dynamic, 8)
    for (i64 i = 0; i < N; i++) {
        const i64 b = batch[i];
        for (i64 h = 0; h < H; h++) {
            const REAL ah = a[i * H + h];
            REAL acc = 0;
            for (i64 e = row_start[i]; e < row_start[i + 1]; e++) {
                const REAL s = reci_terms(ah, kr_base + 3 * e, rvecs + 9 * b, lattice_range, nested, 1);
                const REAL se = sum_in[e * H + h];
                const REAL floor_ = sizeof(REAL) == 4 ? (REAL)1e-6f : (REAL)1e-6;
                acc += s * gz[e * H + h] * (se < floor_ ? (REAL)0 : (REAL)1 / se);
            }
            ga[i * H + h] = acc;
        }
    }
}
