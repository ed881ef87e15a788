/*
 * Host launchers for the reference kernels compiled for the CPU (see cuda_on_cpu.h).  TEST INFRASTRUCTURE ONLY.
 * Each `cfref_<kernel>` runs the reference kernel of that name over a 1-D grid with OpenMP across blocks and takes
 * exactly the kernel's own arguments, preceded by (grid, block) as the reference's Python wrappers compute them
 * (models/cuda_funcs/real_space_enc.py:79,99 ; real_space_enc_proj.py:53,72 ; fused_dpa.py:39-57,162-206 ;
 * irregular_mean.py:43-55 ; reci_space_enc.py:41-56,76-95).
 */
#include "cuda_on_cpu.h"

thread_local cfref_dim3 blockDim, blockIdx, threadIdx;
typedef long long int lli;

template <class F>
static void run_grid(lli grid, unsigned block, F &&body)
{
#pragma omp parallel for schedule(dynamic, 64)
    for (lli b = 0; b < grid; b++) {
        blockDim = {block, 1u, 1u};
        blockIdx = {(unsigned)b, 0u, 0u};
        for (unsigned t = 0; t < block; t++) {
            threadIdx = {t, 0u, 0u};
            body();
        }
    }
}

extern "C" {
void real_enc_fwd(const float *, const float *, const float *, const float *, const lli *, const lli *, const lli,
                  const lli, const lli, const lli, const double, const double, const float *, const double, float *,
                  float *);
void real_enc_bwd(const float *, const float *, const float *, const float *, const lli *, const lli *, const lli *,
                  const float *, const float *, const float *, const lli, const lli, const lli, const lli, const double,
                  const double, const float *, const double, float *);
void real_enc_proj_fwd(const float *, const float *, const float *, const float *, const lli *, const lli *,
                       const lli, const lli, const lli, const lli, const double, const double, const float *,
                       const lli, const float *, const double, float *, float *);
void real_enc_proj_bwd(const float *, const float *, const float *, const lli *, const lli *, const lli *,
                       const float *, const float *, const float *, const lli, const lli, const lli, const double,
                       const double, const float *, const lli, const float *, const double, float *, float *);
void fused_dpa_fwd(const float *, const float *, const float *, const float *, const float *, const lli *,
                   const lli *, const lli, const lli, const lli, float *, float *);
void fused_dpa_fwd_v3(const float *, const float *, const float *, const float *, const float *, const lli *,
                      const lli *, const lli, const lli, const lli, float *, float *);
void fused_dpa_bwd(const float *, const float *, const float *, const float *, const float *, const lli *,
                   const lli *, const lli *, const lli, const lli, const lli, const float *, const float *,
                   const float *, float *, float *, float *, float *, float *);
void fused_dpa_bwd_q(const float *, const float *, const lli *, const lli *, const lli, const lli, const lli, float *);
void irregular_transpose(const float *, const lli *, const lli *, const lli *, const lli, const lli, float *);
void irregular_mean_fwd(const float *, const lli *, const lli, const lli, float *);
void reci_enc_fwd(const float *, const float *, const float *, const float *, const lli *, const lli *, const lli,
                  const lli, const lli, float *, float *);
void reci_enc_bwd(const float *, const float *, const float *, const float *, const lli *, const lli *, const lli *,
                  const float *, const float *, const float *, const lli, const lli, const lli, float *);

void cfref_real_enc_fwd(lli grid, int block, const float *a, const float *rpos, const float *d2min, const float *tv,
                        const lli *batch, const lli *edges, lli N, lli H, lli E, lli K, double dist_max, double wscale,
                        const float *rvlen, double cutoff, float *z, float *v)
{
    run_grid(grid, block, [&] { real_enc_fwd(a, rpos, d2min, tv, batch, edges, N, H, E, K, dist_max, wscale, rvlen, cutoff, z, v); });
}
void cfref_real_enc_bwd(lli grid, int block, const float *a, const float *rpos, const float *tv, const lli *batch,
                        const lli *edges, const lli *e_start, const float *z, const float *gz, const float *gv, lli N,
                        lli H, lli E, lli K, double dist_max, double wscale, const float *rvlen, double cutoff,
                        float *ga)
{
    run_grid(grid, block, [&] { real_enc_bwd(a, rpos, nullptr, tv, batch, edges, e_start, z, gz, gv, N, H, E, K, dist_max, wscale, rvlen, cutoff, ga); });
}
void cfref_real_enc_proj_fwd(lli grid, int block, const float *a, const float *rpos, const float *d2min,
                             const float *tv, const lli *batch, const lli *edges, lli N, lli H, lli E, lli K,
                             double dist_max, double wscale, const float *W, lli W_num, const float *rvlen,
                             double cutoff, float *z, float *v)
{
    run_grid(grid, block, [&] { real_enc_proj_fwd(a, rpos, d2min, tv, batch, edges, N, H, E, K, dist_max, wscale, W, W_num, rvlen, cutoff, z, v); });
}
void cfref_real_enc_proj_bwd(lli grid, int block, const float *a, const float *rpos, const float *tv, const lli *batch,
                             const lli *edges, const lli *e_start, const float *z, const float *gz, const float *gv,
                             lli N, lli H, lli E, double dist_max, double wscale, const float *W, lli W_num,
                             const float *rvlen, double cutoff, float *ga, float *gW)
{
    run_grid(grid, block, [&] { real_enc_proj_bwd(a, rpos, tv, batch, edges, e_start, z, gz, gv, N, H, E, dist_max, wscale, W, W_num, rvlen, cutoff, ga, gW); });
}
void cfref_fused_dpa_fwd(lli grid, int block, int v3, const float *q, const float *k, const float *v, const float *aij,
                         const float *bij, const lli *edges, const lli *e_start, lli N, lli H, lli E, float *prob,
                         float *out)
{
    if (v3) run_grid(grid, block, [&] { fused_dpa_fwd_v3(q, k, v, aij, bij, edges, e_start, N, H, E, prob, out); });
    else run_grid(grid, block, [&] { fused_dpa_fwd(q, k, v, aij, bij, edges, e_start, N, H, E, prob, out); });
}
void cfref_fused_dpa_bwd(lli grid, int block, const float *q, const float *k, const float *v, const float *taij,
                         const float *tbij, const lli *batch, const lli *edges, const lli *e_start, lli N, lli H, lli E,
                         const float *tprob, const float *out, const float *gout, float *gq, float *gk, float *gv,
                         float *tgaij, float *tgbij)
{
    run_grid(grid, block, [&] { fused_dpa_bwd(q, k, v, taij, tbij, batch, edges, e_start, N, H, E, tprob, out, gout, gq, gk, gv, tgaij, tgbij); });
}
void cfref_fused_dpa_bwd_q(lli grid, int block, const float *k, const float *gaij, const lli *edges,
                           const lli *e_start, lli N, lli H, lli E, float *gq)
{
    run_grid(grid, block, [&] { fused_dpa_bwd_q(k, gaij, edges, e_start, N, H, E, gq); });
}
void cfref_irregular_transpose(lli grid, int block, const float *src, const lli *upper_e, const lli *mat_sec,
                               const lli *dims, lli hE, lli C, float *dst)
{
    /* swaps pairs in place; pairs are disjoint, so any execution order is valid */
    run_grid(grid, block, [&] { irregular_transpose(src, upper_e, mat_sec, dims, hE, C, dst); });
}
void cfref_irregular_mean_fwd(lli grid, int block, const float *src, const lli *start, lli B, lli D, float *dst)
{
    run_grid(grid, block, [&] { irregular_mean_fwd(src, start, B, D, dst); });
}
void cfref_reci_enc_fwd(lli grid, int block, const float *a, const float *kr, const float *rvecs, const float *vcell,
                        const lli *batch, const lli *edges, lli N, lli H, lli E, float *z, float *sumexp)
{
    run_grid(grid, block, [&] { reci_enc_fwd(a, kr, rvecs, vcell, batch, edges, N, H, E, z, sumexp); });
}
void cfref_reci_enc_bwd(lli grid, int block, const float *a, const float *kr, const float *rvecs, const float *vcell,
                        const lli *batch, const lli *edges, const lli *e_start, const float *z, const float *gz,
                        const float *sumexp, lli N, lli H, lli E, float *ga)
{
    run_grid(grid, block, [&] { reci_enc_bwd(a, kr, rvecs, vcell, batch, edges, e_start, z, gz, sumexp, N, H, E, ga); });
}
}
