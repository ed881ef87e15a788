/*
 * crystalformer_b200 - C ABI of the sm_100a kernels for Crystalformer's infinitely connected attention.
 *
 * This library replaces the reference project's run-time compiled CuPy kernels (models/kernels/ *.cu, loaded by
 * models/cuda_funcs/kernel_manager.py) and the launch code of its autograd wrappers (models/cuda_funcs/ *.py).
 * Every entry point
 *   - takes raw DEVICE pointers to contiguous arrays (float32 data, int64 indices, as the reference kernels do),
 *     plain sizes and scalars, and the CUDA stream to launch on (a cudaStream_t passed as void*; NULL = default),
 *   - launches asynchronously on that stream of the CURRENT device and does not synchronise; outputs and scratch
 *     are the caller's (as with the reference wrappers, which allocate with torch.empty and hand pointers to the
 *     kernels).  The exceptions are named where they are declared: cf_peer_alloc / cf_peer_free allocate and free
 *     device memory and synchronise the device (set-up calls, never on the data path),
 *   - returns CF_OK or a negative CF_ERR_* code and never throws; cf_last_error() gives the message of the last
 *     failure on the calling thread.
 * State kept by the library: the process-wide switches (cf_set_weight_floor_log2, cf_set_sorted_rows,
 * cf_set_chained_launches, cf_set_row_stats), a
 * side stream and two events per (host thread, device) created by the first cf_encoder_forward / cf_model_forward,
 * the 8 MiB scratch array of cf_lattice_sum_bwd_static, and a pool of row tickets per device: 64 single counters
 * handed round-robin to the cf_infinite_attn_fwd[_listed] calls with K > 0 and 8 blocks of 16 handed round-robin to the
 * one-call forwards that use term lists.  A ticket is reused after 64 calls (8 forwards): at most that many such calls
 * may be PENDING on one device at a time, whatever streams they were issued on; beyond that two row kernels can share
 * a counter and rows would be skipped.  (The row-list path, cf_row_list_build / cf_infinite_attn_fwd_sorted and the
 * one-call forwards of batches of small crystals, keeps its counters in the caller's workspace and has no such limit.)
 * Otherwise no per-call state, so the library may be called concurrently from one host thread per GPU (the
 * reference's multi-GPU path does that: models/latticeformer.py:274).
 *
 * Compile-time constants of the reference (HEAD_NUM, K_HEAD_DIM, V_HEAD_DIM, VPE_DIM, LATTICE_RANGE, MINIMUM_RANGE;
 * kernel_manager.py:110-126) are run-time arguments here.  Supported shapes: H = 8 heads, head dim D = 16,
 * K = value_pe_dist_real in {0, 64}; anything else returns CF_ERR_UNSUPPORTED.
 *
 * Shapes: N atoms, E edges (all ordered pairs inside each crystal, row-major per crystal:
 * models/indexed_latticeformer_encoder.py:15-32), B crystals, H heads, D head dim, K radial-basis bins.
 */
#ifndef CRYSTALFORMER_B200_H
#define CRYSTALFORMER_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CF_OK 0
#define CF_ERR_INVALID (-1)     /* null pointer, negative size, inconsistent arguments */
#define CF_ERR_UNSUPPORTED (-2) /* shape outside the compiled set (H, D, K) */
#define CF_ERR_CUDA (-3)        /* a CUDA runtime call failed; message in cf_last_error() */
#define CF_ERR_RANGE (-4)       /* a size exceeds a documented limit */

/* Largest half-width of the translation box in any direction.  The reference loops over whatever the cut-off rule
 * yields; here a box wider than this is clamped so that a degenerate width (a -> 0) cannot stall the GPU. */
#define CF_MAX_RANGE 32

/* Library version as major*10000 + minor*100 + patch. */
int cf_version(void);

/* Message of the last error raised on the calling thread ("" if none). The pointer stays valid until the next
 * failing call on the same thread. */
const char *cf_last_error(void);

/* An approximation, not a bit-neutral skip: terms of a lattice sum whose weight is below 2^log2_floor of the sum's
 * largest term for every head are left out (and the backward contracts the radial basis over the 20 bins around a
 * term only):
 * in phi relative to the nearest image, in the radial-basis accumulation relative to the normalised total (in the
 * fused attention: relative to the whole row's soft-max total).  Default -30: such a term is below 1/64 ulp of a
 * float32 sum (measured change of the attention output 6e-8 relative, against 4e-9 at -40); pass -1000 to
 * accumulate every term.  Process-wide tuning knob, read at launch time. */
void cf_set_weight_floor_log2(double log2_floor);
double cf_get_weight_floor_log2(void);

/* Whether cf_encoder_forward / cf_model_forward may take the row-list path (cf_row_list_build +
 * cf_infinite_attn_fwd_sorted, below) for batches whose crystals have at most 64 atoms; 1 by default, 0 keeps the
 * term-list kernels for every batch.  Process-wide, read at launch time. */
void cf_set_sorted_rows(int enabled);
int cf_get_sorted_rows(void);

/* Whether the kernels of cf_encoder_forward / cf_model_forward are launched as a chain of programmatic dependent
 * launches (a kernel's blocks are scheduled and run their prologue - staging of weights - while its predecessor
 * drains, then wait for it to complete); 1 by default, 0 launches them the ordinary way.  Results are identical. */
void cf_set_chained_launches(int enabled);

/* Work counters of the sorted row kernel (diagnostic, for roofline accounting): while `device_words` (DEVICE memory,
 * four uint64, zeroed by the caller) is set, every cf_infinite_attn_fwd_sorted launch - also inside the one-call
 * forwards - adds { chunks of eight entries swept, (chunk, 16-bin tile) pairs whose basis values were evaluated,
 * rows processed, 0 }.  NULL (the default) switches the counting off.  Process-wide; the memory must stay valid
 * while set. */
void cf_set_row_stats(void *device_words);

/* ------------------------------------------------------------------------------------------------------------
 * Batch preparation.  Replaces get_edge_index and compute_lattice_distances_for_cuda
 * (models/indexed_latticeformer_encoder.py:15-32, 183-253) and the CSR construction repeated in every wrapper
 * (models/cuda_funcs/fused_dpa.py:24-26), without the host loop over crystals and without device->host syncs.
 *
 * cf_crystal_offsets: atom_start (B+1), edge_start (B+1) int64 exclusive prefix sums of sizes and sizes^2.
 *                     One block; B <= 2^20.
 * cf_batch_prepare  : from pos (N,3), trans (B,3,3), sizes (B) and the two offset arrays writes any of (NULL = skip)
 *     batch     (N)   int64  crystal of each atom
 *     edges     (2,E) int64  all-pairs edge list, bit-identical to get_edge_index
 *     row_start (N+1) int64  first edge of each source atom (CSR of edges[0])
 *     pos_ij    (E,3) f32    pos[j] - pos[i]
 *     rvecs (B,3,3), vcell (B), rvlen (B,3) f32: reciprocal rows 2 pi (t_b x t_c)/V, cell volume, |rvecs rows|
 * ---------------------------------------------------------------------------------------------------------- */
int cf_crystal_offsets(const int64_t *sizes, int64_t B, int64_t *atom_start, int64_t *edge_start, void *stream);
int cf_batch_prepare(const float *pos, const float *trans, const int64_t *sizes, const int64_t *atom_start,
                     const int64_t *edge_start, int64_t B, int64_t N, int64_t E, int64_t *batch, int64_t *edges,
                     int64_t *row_start, float *pos_ij, float *rvecs, float *vcell, float *rvlen, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Translation box of every (edge, head): box (E,H,3) int32 = (R1,R2,R3) of the reference's cut-off rule
 * (models/kernels/real_enc_fwd.cu:63-85), reproduced bit for bit:
 *   cutoff_radius == 0 or rvlen == NULL : R = lattice_range            (the fixed box of the PyTorch path)
 *   cutoff_radius <  0 : radius = sqrt(-0.5/a) * |cutoff_radius|       (per atom and head)
 *   cutoff_radius >  0 : radius = cutoff_radius
 *   R_d = ceil((radius + 0.01) * rvlen_d / 2pi), raised to minimum_range, clamped to CF_MAX_RANGE.
 * a is (N,H), or (E,H) when a_per_edge != 0.  Diagnostic / test entry; the kernels below apply the same rule.
 * ---------------------------------------------------------------------------------------------------------- */
int cf_lattice_box(const float *a, int a_per_edge, const int64_t *batch, const int64_t *edges, int64_t N, int64_t H,
                   int64_t E, const float *rvlen, double cutoff_radius, int lattice_range, int minimum_range,
                   int32_t *box, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Real-space lattice sum, forward.  Replaces real_enc_fwd / real_enc_proj_fwd (and their _v2 variants)
 * (models/kernels/real_enc_fwd.cu:4-144, real_enc_proj_fwd.cu:4-169) as launched by
 * RealPeriodicEncodingFuncCUDA.forward / RealPeriodicEncodingWithProjFuncCUDA.forward
 * (models/cuda_funcs/real_space_enc.py:19-138, real_space_enc_proj.py:20-97).
 *   z (E,H)   = log sum_n exp(a |r_ij + n.T|^2)
 *   v         = psi (E,H,K) when W == NULL, else W psi (E,H,Dv) with W (W_num,H,Dv,K), W_num in {1, N, E}
 *   psi[k]    = softmax_n-weighted Gaussian radial basis, centres (k+1) dist_max/K, width wscale dist_max/K
 * K == 0 writes z only (v may be NULL).  a_per_edge != 0 reads a as (E,H) instead of (N,H) (kernel benchmark).
 * ---------------------------------------------------------------------------------------------------------- */
int cf_lattice_sum_fwd(const float *a, int a_per_edge, const float *pos_ij, const float *tvecs, const int64_t *batch,
                       const int64_t *edges, int64_t N, int64_t H, int64_t E, int64_t K, double dist_max,
                       double wscale, const float *W, int64_t W_num, int64_t Dv, const float *rvlen,
                       double cutoff_radius, int lattice_range, int minimum_range, float *z, float *v, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Real-space lattice sum, backward.  Replaces real_enc_bwd / real_enc_proj_bwd
 * (models/kernels/real_enc_bwd.cu:4-157, real_enc_proj_bwd.cu:4-221) as launched by the wrappers' backward
 * (models/cuda_funcs/real_space_enc.py:141-247, real_space_enc_proj.py:100-178).  phi and psi are recomputed.
 *   in : z (E,H) from the forward, gz (E,H), gpsi (E,H,K) = gradient arriving at psi (NULL when K == 0); with a
 *        projection W the caller forms gpsi = W^T gv first, as the reference's real_space_enc.py:196-199 does
 *   out: ga (N,H)
 *        psi_out (E,H,K), optional: psi recomputed, from which the caller gets the gradient of W as
 *        sum_e gv_e (x) psi_e (one GEMM; the reference accumulates the same sum per atom inside its kernel)
 * row_start (N+1) is the CSR of edges[0].  edge_scratch: (E,H) floats of device scratch holding the per-edge
 * contributions, which a second kernel adds up per atom in edge order (run-to-run identical results).
 * ---------------------------------------------------------------------------------------------------------- */
int cf_lattice_sum_bwd(const float *a, const float *pos_ij, const float *tvecs, const int64_t *batch,
                       const int64_t *edges, const int64_t *row_start, const float *z, const float *gz,
                       const float *gpsi, int64_t N, int64_t H, int64_t E, int64_t K, double dist_max, double wscale,
                       const float *rvlen, double cutoff_radius, int lattice_range, int minimum_range, float *ga,
                       float *psi_out, float *edge_scratch, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * cf_lattice_sum_bwd without a scratch argument.  No counterpart in the reference (its wrappers always allocate
 * their temporaries with torch).
 *
 * Meant for callers that cannot allocate device memory when they call: processes that fixed their device-memory
 * budget at start-up, bindings from runtimes without a device allocator, loops where an allocation's possible
 * device-wide synchronisation is not tolerable.  The (E,H) per-edge contributions are kept in an array built into
 * the library, which occupies CF_STATIC_SCRATCH_MAX_EDGES * 8 * 4 bytes (8 MiB) on every GPU that loads the library
 * until the process exits, and limits a call to E <= CF_STATIC_SCRATCH_MAX_EDGES edges (CF_ERR_RANGE beyond that).
 * The call itself allocates and frees nothing.
 *
 * The first call made with a given device current looks up the array's device address (once per device); make that
 * first call outside any stream capture.  All calls on a device share the one array and it keeps the previous
 * call's contents: calls that can overlap on the GPU (e.g. on different streams) race and must be serialised by the
 * caller.  Nothing needs zeroing: a call writes every element it later reads.  Arguments and results are those of
 * cf_lattice_sum_bwd.
 * ---------------------------------------------------------------------------------------------------------- */
#define CF_STATIC_SCRATCH_MAX_EDGES 262144
int cf_lattice_sum_bwd_static(const float *a, const float *pos_ij, const float *tvecs, const int64_t *batch,
                              const int64_t *edges, const int64_t *row_start, const float *z, const float *gz,
                              const float *gpsi, int64_t N, int64_t H, int64_t E, int64_t K, double dist_max,
                              double wscale, const float *rvlen, double cutoff_radius, int lattice_range,
                              int minimum_range, float *ga, float *psi_out, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Edge-indexed softmax attention with given position terms.  Replaces fused_dpa_fwd[_v3], fused_dpa_bwd[_v3],
 * fused_dpa_bwd_q[_v3] and irregular_transpose (models/kernels/fused_dpa_fwd.cu, fused_dpa_bwd.cu,
 * fused_dpa_bwd_q.cu, irregular_transpose.cu) as launched by FusedDotProductAttentionCUDA
 * (models/cuda_funcs/fused_dpa.py:17-208).  q is already divided by sqrt(D) by the caller.
 *   fwd: prob (E,H) = softmax_j(q_i.k_j + aij), out (N,H,D) = sum_j prob (v_j + bij); aij, bij may be NULL
 *   bwd: gq, gk, gv (N,H,D), gaij (E,H), gbij (E,H,D) (NULL when bij is NULL); no transposed copies are made.
 * No limit on atoms per crystal (the reference stops at 320, kernel_manager.py:55).
 * ---------------------------------------------------------------------------------------------------------- */
int cf_fused_attn_fwd(const float *q, const float *k, const float *v, const float *aij, const float *bij,
                      const int64_t *edges, const int64_t *row_start, int64_t N, int64_t H, int64_t D, int64_t E,
                      float *prob, float *out, void *stream);
int cf_fused_attn_bwd(const float *q, const float *k, const float *v, const float *bij, const int64_t *edges,
                      const int64_t *row_start, int64_t N, int64_t H, int64_t D, int64_t E, const float *prob,
                      const float *out, const float *gout, float *gq, float *gk, float *gv, float *gaij,
                      float *gbij, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Per-crystal mean of atom features.  Replaces irregular_mean_fwd (models/kernels/irregular_mean_fwd.cu) as
 * launched by IrregularMeanCUDA.forward (models/cuda_funcs/irregular_mean.py:21-58); same fixed summation tree.
 * x (N,D) -> out (B,D); start (B+1) int64 atom offsets.  Crystals of up to 1024 atoms.
 * ---------------------------------------------------------------------------------------------------------- */
int cf_segment_mean_fwd(const float *x, const int64_t *start, int64_t B, int64_t D, float *out, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Fully fused infinitely connected attention (what the reference computes with real_enc_proj_fwd followed by
 * fused_dpa_fwd, models/indexed_lattice_multi_head_attention_cuda.py:393-421,181-185), without materialising any
 * per-edge tensor except the logits:
 *   out_i = sum_j softmax_j(q_i.k_j + phi_ij) (v_j + W psi_ij)
 * computed as  sum_j p_ij v_j + W_h (sum_j p_ij psi_ij)  (W is shared by all edges, W (H,D,K)).
 *   in : q (pre-scaled), k, v (N,H,D); a (N,H); the geometry either as pos_ij (E,3) (what the reference hands its
 *        kernels) or, when pos_ij is NULL, as pos (N,3) from which pos[j]-pos[i] is taken; tvecs (B,3,3);
 *        rvlen (B,3) or NULL; batch (N); edges (2,E); row_start (N+1);
 *        max_atoms >= the largest number of atoms in one crystal
 *        (it sizes the shared memory of a thread block; crystals of up to 2048 atoms)
 *   out: out (N,H,D)
 *        logit (E,H)  q.k + phi, kept for the backward
 *        lse (N,H)    log sum_j exp(logit)
 *        psi_row (N,H,K) = sum_j p_ij psi_ij (NULL to skip; needed for the gradient of W)
 *   row_order (N) int32, optional (NULL = 0..N-1): a permutation of the atoms giving the order in which thread blocks
 *        pick them up.  Atoms of large crystals cost more; listing them first (descending atoms per crystal) balances
 *        the load.  The results do not depend on it.
 * ---------------------------------------------------------------------------------------------------------- */
int cf_infinite_attn_fwd(const float *q, const float *k, const float *v, const float *a, const float *pos,
                         const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                         const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                         int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                         const float *W, double cutoff_radius, int lattice_range, int minimum_range, float *out,
                         float *logit, float *lse, float *psi_row, const int32_t *row_order, void *stream);

/* Backward of cf_infinite_attn_fwd; phi and psi are recomputed from the geometry.
 *   in : everything the forward read, plus logit, lse, out and gout (N,H,D)
 *   out: gq (w.r.t. the pre-scaled q), gk, gv (N,H,D); ga (N,H); glogit (E,H) = gradient of the logits (also the
 *        hand-over between the two kernels of this call); crystals of up to 1024 atoms
 * The gradient of W is sum_i gout_i (x) psi_row_i, a plain GEMM the caller does from psi_row. */
int cf_infinite_attn_bwd(const float *q, const float *k, const float *v, const float *a, const float *pos,
                         const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                         const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H,
                         int64_t D, int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale,
                         const float *W, double cutoff_radius, int lattice_range, int minimum_range,
                         const float *logit, const float *lse, const float *out, const float *gout, float *gq,
                         float *gk, float *gv, float *ga, float *glogit, const int32_t *row_order, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Term lists: the (key, translation) pairs of a batch that can matter to ANY layer, found once per batch (the
 * reference enumerates every head's translation box again in every layer, real_enc_proj_fwd.cu:63-134).
 * cf_term_list_build stores, per edge, the translations whose squared distance is within
 * D = -floor_log2 / (|a_widest| log2 e) of the edge's nearest image, together with |n1|,|n2|,|n3| so that every
 * (atom, head) still applies its own box; a_widest < 0 is the value closest to zero that the Gaussian parameter a can
 * take in any layer (gauss_lb_real x -0.5/scale_real^2 for the reference's positive functions).
 * cf_infinite_attn_fwd_listed is cf_infinite_attn_fwd reading those lists (phi as a sum over an edge's entries, the
 * row kernel's candidates from a row's entries) instead of enumerating; rows that did not fit the workspace are
 * enumerated as before, so the result never depends on the capacity.  workspace: cf_term_list_workspace_bytes(N, E)
 * bytes, 16-byte aligned; built with the weight floor in force at the time (cf_set_weight_floor_log2).
 * cf_infinite_attn_bwd_listed is cf_infinite_attn_bwd with its sums over translations running over the same lists
 * (the terms the listed forward summed), for a training step that builds the lists once and uses them in the forward
 * and backward of every layer.
 * ---------------------------------------------------------------------------------------------------------- */
int64_t cf_term_list_workspace_bytes(int64_t N, int64_t E);
int cf_term_list_build(const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                       const int64_t *edges, const int64_t *row_start, const int32_t *row_order, int64_t N, int64_t E,
                       int64_t max_atoms, double cutoff_radius, int lattice_range, int minimum_range, double a_widest,
                       void *workspace, void *stream);
int cf_infinite_attn_fwd_listed(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                                const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                                const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D, int64_t E,
                                int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                                double cutoff_radius, int lattice_range, int minimum_range, float *out, float *logit,
                                float *lse, float *psi_row, const int32_t *row_order, void *term_lists,
                                double a_widest, void *stream);
int cf_infinite_attn_bwd_listed(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                                const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                                const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D, int64_t E,
                                int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                                double cutoff_radius, int lattice_range, int minimum_range, const float *logit,
                                const float *lse, const float *out, const float *gout, float *gq, float *gk, float *gv,
                                float *ga, float *glogit, const int32_t *row_order, void *term_lists, double a_widest,
                                void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Row lists and the tensor-core row kernel for batches of small crystals (max_atoms <= 64; K = 64, or K = 0: no
 * radial basis, W may be NULL; inference).  The one-call forwards use them for K = 64 (without a basis the
 * enumerating kernel with term lists is the faster one).
 * Same function as cf_infinite_attn_fwd (real_enc_proj_fwd + fused_dpa_fwd of the reference,
 * models/kernels/real_enc_proj_fwd.cu:63-169, models/kernels/fused_dpa_fwd_v3.cu), other organisation:
 * cf_row_list_build stores, per ATOM ROW, all (key, translation) terms within the term-list window of their edge's
 * nearest image (same rule and a_widest as cf_term_list_build), sorted by distance.  cf_infinite_attn_fwd_sorted then
 * computes a row with one warp in a single sweep over its entries: weights exp2(a d2 + q.k - M) against an upper
 * bound M, so that phi, the soft-max statistics and the radial-basis histogram are plain sums over the entries, done
 * as mma.m16n8k8 products (TF32 operands split into high and low parts: fp32-level accuracy).  The sweep stops at the
 * first eight entries that are below the weight floor for every head of this layer.  Rows that do not fit the
 * workspace (more than 4096 entries, or the pool is full) and rows where a head's box misses every listed term are
 * processed by the enumerating kernel of cf_infinite_attn_fwd inside the same call (rows without a basis or of more
 * than 32 keys enumerate phi edge by edge there: slow, and rare): results do not depend on the capacities.  No logits are written (inference); lse (N,H) is.
 *   workspace: cf_row_list_workspace_bytes(N, E) bytes, 16-byte aligned, built with the weight floor in force at the
 *   time; it also holds the row counters of the calls that use it, so calls sharing a workspace must be ordered
 *   (one stream), and every build allows any number of calls.
 * ---------------------------------------------------------------------------------------------------------- */
int64_t cf_row_list_workspace_bytes(int64_t N, int64_t E);
int cf_row_list_build(const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                      const int64_t *edges, const int64_t *row_start, const int32_t *row_order, int64_t N, int64_t E,
                      int64_t max_atoms, double cutoff_radius, int lattice_range, int minimum_range, double a_widest,
                      void *workspace, void *stream);
int cf_infinite_attn_fwd_sorted(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                                const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                                const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D, int64_t E,
                                int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                                double cutoff_radius, int lattice_range, int minimum_range, float *out, float *lse,
                                void *row_lists, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Inference forward of the encoder stack (every layer of CrystalformerEncoderCUDA,
 * models/indexed_latticeformer_encoder.py:699-742 and :848-890, post-norm with LayerNorm = Identity) in one call:
 * per layer  x <- x + out_proj(attention(x)) ;  x <- x + W2 relu(W1 x + b1) + b2, with the attention of
 * cf_infinite_attn_fwd and the Gaussian-width pipeline of
 * models/indexed_lattice_multi_head_attention_cuda.py:640-722 (gauss_state 'q', normalised alpha with a stored
 * gauss_scale, positive_func 'elu=beta').  model_dim 128, 8 heads; dense products by cuBLAS SGEMM in plain fp32 on the
 * caller's handle (cublasHandle_t passed as void*; the library resolves cuBLAS from the copy loaded in the process).
 *   weights : HOST array of num_layers x 11 device pointers:
 *             Wqkv (384,128) [q,k,v rows stacked], bqkv (384), lattice_pos_weights (128), pe_dist_proj (8,16,K) or
 *             NULL, out_proj.weight (128,128), out_proj.bias (128), linear1.weight (ff,128), linear1.bias (ff),
 *             linear2.weight (128,ff), linear2.bias (128), packed (optional)
 *             packed: NULL, or Wqkv, out_proj.weight, linear1.weight, linear2.weight concatenated in the fragment
 *             order of the fused dense kernel: a weight W (out,in) as float4 entries
 *             [(nt * in/8 + ks) * 32 + lane] = (hi W[n,k], hi W[n,k+4], c W[n,k], c W[n,k+4]), n = 8 nt + lane/4,
 *             k = 8 ks + lane%4, hi = rounding to TF32 (ties away), c(w) = the 32-bit word { lower half:
 *             bfloat16(hi(w)), upper half: bfloat16(w - hi(w)) }.  When every layer has it and ff_dim is a multiple
 *             of 128, the four products and the element-wise steps of a layer boundary run as ONE tensor-core kernel
 *             (TF32 main product + bfloat16 correction product: fp32-level accuracy) instead of cuBLAS SGEMMs.
 *   scalars : HOST array of num_layers x 6 doubles: gauss_scale, gauss_shift, -0.5/scale_real^2, elu beta,
 *             gauss_lb_real, dist_max
 *   x       : (N,128) atom features, updated in place
 *   workspace: cf_encoder_workspace_floats(N, E, ff_dim) floats of device scratch
 *   attn_events: NULL, or a HOST array of 2 x num_layers cudaEvent_t recorded on `stream` immediately before and
 *             after each layer's attention kernels (lets a caller time them without splitting the call)
 * Geometry arguments as in cf_infinite_attn_fwd.  No gradient support (training uses the autograd path).
 * ---------------------------------------------------------------------------------------------------------- */
int64_t cf_encoder_workspace_floats(int64_t N, int64_t E, int64_t ff_dim);
int cf_encoder_forward(void *cublas_handle, int num_layers, const float *const *weights, const double *scalars, float *x,
                       const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                       const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t E,
                       int64_t max_atoms, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                       int lattice_range, int minimum_range, float *workspace, const int32_t *row_order,
                       void *const *attn_events, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Peer gather of the per-crystal outputs of data-parallel ranks (one process per GPU of one machine), without a
 * collective library on the data path.  The reference gathers inside one process (models/latticeformer.py:278-289).
 * Every rank allocates a gather buffer (cf_peer_alloc), hands its 64-byte handle to the other processes (any channel,
 * e.g. an all-gather of bytes at set-up) and maps theirs (cf_peer_open).  A buffer holds `slots` (>= 2) slots of
 * world * rows_per_rank * targets 8-byte cells; cell ((r * rows_per_rank + c) * targets + t) carries output t of
 * crystal c of rank r as { float bits (low word), step (high word) }, written by ONE 8-byte store, so that a reader
 * who sees the step has the value.  Step s (1, 2, 3, ...; the same sequence on every rank) uses slot s % slots.
 * A cf_peer_gather describes one step: cells[r] = the slot inside rank r's buffer as mapped in THIS process
 * (r = rank: the own buffer).  The producer - cf_model_forward given the descriptor, or cf_peer_gather_store for
 * outputs that exist already - stores this rank's rows into every rank's buffer; cf_peer_gather_collect, on the same
 * stream afterwards, waits until the cells of the own slot carry `step` and writes out[g] = value of row index[g] for
 * the `rows` crystals of the unsharded batch (index: int64 row numbers within the slot).  The wait is bounded: after
 * timeout_s the kernel writes status[0] = 1 + (a rank whose rows are missing), NaN for the missing values, and returns.
 * ---------------------------------------------------------------------------------------------------------- */
#define CF_MAX_PEERS 16
#define CF_PEER_HANDLE_BYTES 64
typedef struct cf_peer_gather {
    int32_t world, rank;
    int64_t rows_per_rank;
    uint32_t step, reserved;
    uint64_t *cells[CF_MAX_PEERS];
} cf_peer_gather;
int cf_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle);  /* zero-filled; handle: 64 bytes out */
int cf_peer_open(const unsigned char *handle, void **ptr);            /* maps another process's buffer */
int cf_peer_close(void *ptr);                                         /* unmaps (cf_peer_open) */
int cf_peer_free(void *ptr);                                          /* frees (cf_peer_alloc) */
int cf_peer_gather_store(const float *y, int64_t rows, int64_t targets, const cf_peer_gather *gather, void *stream);
int cf_peer_gather_collect(const uint64_t *cells, uint32_t step, const int64_t *index, int64_t rows, int64_t targets,
                           int64_t rows_per_rank, float *out, int32_t *status, double timeout_s, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Inference forward of the whole model in one host call (what Latticeformer.forward does in eval mode,
 * models/latticeformer.py:211-302, with pooling "avr", pre_pooling_op "no", norm_type "no" and a head of the form
 * Linear - ReLU - Linear): y (B, targets) from the species features (N, feature_dim), positions, lattices and sizes.
 * Runs the work of cf_crystal_offsets, cf_batch_prepare and cf_row_order (one launch), the embedding (W_embed
 * (128, feature_dim), no bias; one SGEMM unless W_embed_packed is given), cf_encoder_forward (same weights /
 * scalars / box arguments) and a fused mean + head kernel (W1 (hidden,128), b1, W2 (targets,hidden), b2; hidden <= 1024).  N, E = sum n, sum n^2 and max_atoms are host
 * integers the caller knows from the sizes.  workspace: cf_model_workspace_bytes(N, B, E, ff_dim) bytes, 256-byte
 * aligned.  order_reach: the reach handed to cf_row_order (about dist_max).
 * W_embed_packed (optional, NULL to skip): W_embed with its input columns zero-padded to 128, packed like slot 10 of
 * the layer weights (feature_dim <= 128).  When it is given and every layer brings packed weights, the embedding runs
 * inside the first dense block, the whole forward runs in this library's kernels and cublas_handle may be NULL.
 * gather (optional, NULL to skip): the pooling + head kernel also stores y into every rank's gather buffer (see
 * cf_peer_gather above; B <= gather->rows_per_rank).
 *   inputs_ready, slot_free: NULL, or cudaEvent_t (passed as void*) for pipelined use.  With inputs_ready given (an event
 *             after which features, pos, trans and sizes are valid) the batch preparation - the geometry launch and the
 *             list build, which depend on the inputs only - is issued on a stream of the library's own, ordered after
 *             inputs_ready and slot_free but NOT after the work already queued on `stream`: it then runs beside the
 *             previous batch's forward.  The caller must hand every forward that can be in flight its own workspace;
 *             slot_free is an event recorded on `stream` after the previous forward that used THIS workspace (NULL if
 *             there was none).  Only with packed weights (the cuBLAS-free path); otherwise ignored.
 * ---------------------------------------------------------------------------------------------------------- */
int64_t cf_model_workspace_bytes(int64_t N, int64_t B, int64_t E, int64_t ff_dim);
int cf_model_forward(void *cublas_handle, const float *features, int64_t feature_dim, const float *pos,
                     const float *trans, const int64_t *sizes, int64_t N, int64_t B, int64_t E, int64_t max_atoms,
                     const float *W_embed, const float *W_embed_packed, int num_layers, const float *const *weights,
                     const double *scalars, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius, int lattice_range,
                     int minimum_range, const float *W1, const float *b1, int64_t hidden, const float *W2,
                     const float *b2, int64_t targets, double order_reach, void *workspace, float *y,
                     void *const *attn_events, const cf_peer_gather *gather, void *inputs_ready, void *slot_free,
                     void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * One host call per batch of a streaming inference loop (no counterpart in the reference, whose demo and training
 * scripts call the model batch by batch from a DataLoader): pinned host inputs -> device on a copy stream, the
 * cf_model_forward of the batch on a compute stream with its preparation started as soon as the copy is done,
 * outputs -> pinned host memory, and the events that order them.  Everything a batch in flight needs is a slot owned
 * by the caller; nothing is allocated, kept or synchronised here.  Only the cuBLAS-free path (packed weights).
 *   cf_model_desc : the batch-independent arguments of cf_model_forward (same meaning); the two HOST arrays must
 *                   stay valid while calls are being made.
 *   cf_serve_slot : streams and events as void* (cudaStream_t / cudaEvent_t); device buffers x (max_atoms_total x
 *                   feature_dim), pos (max_atoms_total x 3), trans (max_crystals x 9) float32, sizes (max_crystals)
 *                   int64, workspace (cf_model_workspace_bytes of the three maxima), y (max_crystals x targets);
 *                   y_host: pinned, max_crystals x targets.  `copied` is recorded after the input copies,
 *                   `inputs_free` after the forward, `done` after the output copy (the caller waits for it, e.g.
 *                   cudaEventSynchronize, before reading y_host and before reusing the slot).
 *   inputs_in_use : 0 for a slot's first batch; else the copy stream first waits for the slot's `inputs_free`.
 *   gather        : null, or the peer gather of the step (one process per GPU, each with its shard of the batch):
 *                   `store` is the step's descriptor for cf_model_forward; the compute stream first waits for
 *                   `store_after` (if not null: the event after the collect that last read the slot the step
 *                   stores to); `stored` is recorded after the forward; the collect (cf_peer_gather_collect with
 *                   `own_cells`, `index`, `total_rows`, `status`, `timeout_s`) runs on `collect_stream` after
 *                   `stored`, writes y_all (total_rows x targets) and is followed by `collected`; y_all and the
 *                   status word then go to y_all_host / status_host (pinned) and the slot's `done` is recorded on
 *                   the collect stream.  The slot's y / y_host are not copied in that case.
 *   species_host  : with x_host == NULL: HOST array of N indices below feature_dim (the atoms' species, i.e. the
 *                   position of the 1 in a one-hot feature row): 8 N bytes are copied instead of 4 N feature_dim, into
 *                   the slot's `species` buffer (max_atoms_total int64, may be NULL in slots that never take indices),
 *                   and the first dense block builds the one-hot rows in shared memory; same outputs, bit for bit.
 *   cf_model_desc.dense_tile_rows : 0 = the dense blocks choose their row tile themselves (16 rows while that fills
 *                   one wave of SMs: shortest latency of a single forward); 32 = 32-row tiles (fewer, longer blocks
 *                   that read the weights half as often: more forwards per second when several streams keep the GPU
 *                   full); 16 = always 16.
 * x_host .. sizes_host: HOST memory (pinned for the copies to be asynchronous) of the batch: one-hot species (N x
 * feature_dim), positions, lattice rows, atoms per crystal; E = sum of sizes^2, max_atoms = largest size.
 * ---------------------------------------------------------------------------------------------------------- */
typedef struct cf_model_desc {
    int64_t feature_dim;
    const float *W_embed, *W_embed_packed;
    int32_t num_layers, lattice_range, minimum_range, dense_tile_rows;
    const float *const *weights;
    const double *scalars;
    int64_t K, ff_dim;
    double wscale, cutoff_radius;
    const float *W1, *b1;
    int64_t hidden;
    const float *W2, *b2;
    int64_t targets;
    double order_reach;
} cf_model_desc;
typedef struct cf_serve_slot {
    void *copy_stream, *compute_stream;
    void *copied, *inputs_free, *done;
    float *x, *pos, *trans;
    int64_t *sizes;
    void *workspace;
    float *y, *y_host;
    int64_t max_atoms_total, max_crystals, max_edges;
    int64_t *species;
} cf_serve_slot;
typedef struct cf_serve_gather {
    const cf_peer_gather *store;
    void *collect_stream;
    void *store_after, *stored, *collected;
    const uint64_t *own_cells;
    const int64_t *index;
    int64_t total_rows;
    float *y_all, *y_all_host;
    int32_t *status, *status_host;
    double timeout_s;
} cf_serve_gather;
int cf_serve_submit(const cf_model_desc *model, const cf_serve_slot *slot, const float *x_host, const float *pos_host,
                    const float *trans_host, const int64_t *sizes_host, int64_t N, int64_t B, int64_t E,
                    int64_t max_atoms, int inputs_in_use, const cf_serve_gather *gather, const int64_t *species_host);

/* ------------------------------------------------------------------------------------------------------------
 * Scheduling weight of every atom's row for the fused attention kernels (no counterpart in the reference, which
 * launches one thread per (atom, head) in index order): cost[i] = 1500 + n (1 + (4 pi / 3) reach^3 / |det trans|),
 * n the atom count of the atom's crystal; about the number of (key, translation) pairs within `reach` Angstrom.
 * Sorting atoms by descending cost gives the `row_order` argument of cf_infinite_attn_fwd / cf_encoder_forward.
 * ---------------------------------------------------------------------------------------------------------- */
int cf_row_cost(const int64_t *atom_start, const float *trans, int64_t B, int64_t N, double reach, float *cost,
                void *stream);
/* The atoms in descending order of cf_row_cost, ties by index (a stable descending sort of the costs), computed in
 * one launch for batches of up to 2048 crystals (CF_ERR_RANGE beyond: sort the costs instead).  row_order (N) int32. */
int cf_row_order(const int64_t *atom_start, const float *trans, int64_t B, int64_t N, double reach,
                 int32_t *row_order, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Reciprocal-space lattice sum (domains `reci`, `RECI`, `multihead` of the reference's attention module).
 * Replace reci_enc_fwd / reci_enc_bwd (models/kernels/reci_enc_fwd.cu, reci_enc_bwd.cu) as launched by
 * ReciPeriodicEncodingFuncCUDA (models/cuda_funcs/reci_space_enc.py:19-56, 59-99):
 *   S[e,h]   = sum_{n1 in [0,R], n2,n3 in [-R,R]} w(n1) exp(a[i,h] |n.rvecs|^2) cos(kr_base[e].n),  w(0)=1, else 2
 *   z[e,h]   = log max(S, 1e-6) + 1.5 log(-4 pi a[i,h]) - log vcell
 *   ga[i,h]  = sum_{e in row i} gz[e,h] (S < 1e-6 ? 0 : 1/S) sum_n w |k_n|^2 exp(a |k_n|^2) cos(kr_base[e].n)
 * a (N,8) < 0; kr_base (E,3); rvecs (B,3,3); vcell (B); batch (N); row_start (N+1) CSR offsets of the edge list by
 * source atom (the reference builds it in its backward, reci_space_enc.py:64-66); R = lattice_range <= 6 (the
 * reference compiles LATTICE_RANGE into the kernel).  sumexp (E,8) may be NULL in the forward.
 * cf_reci_phase computes kr_base = rvecs[crystal of e] . pos_ij[e] (models/indexed_latticeformer_encoder.py:249-251).
 * ---------------------------------------------------------------------------------------------------------- */
int cf_reci_phase(const float *pos_ij, const float *rvecs, const int64_t *batch, const int64_t *edges, int64_t E,
                  float *kr_base, void *stream);
int cf_reci_sum_fwd(const float *a, const float *kr_base, const float *rvecs, const float *vcell,
                    const int64_t *batch, const int64_t *row_start, int64_t N, int64_t H, int64_t E,
                    int lattice_range, float *z, float *sumexp, void *stream);
int cf_reci_sum_bwd(const float *a, const float *kr_base, const float *rvecs, const int64_t *batch,
                    const int64_t *row_start, const float *gz, const float *sumexp, int64_t N, int64_t H, int64_t E,
                    int lattice_range, float *ga, void *stream);

/* ------------------------------------------------------------------------------------------------------------
 * Pipe-throughput probes for the roofline denominators: `iters` dependent-free FFMA (kind 0) or MUFU.EX2 (kind 1)
 * instructions per thread over a full grid; sink (>= 1 float) receives a value so the loop is not elided.
 * Work per launch = blocks * threads * iters * 8 instructions.
 * ---------------------------------------------------------------------------------------------------------- */
int cf_pipe_probe(int kind, int blocks, int threads, int64_t iters, float *sink, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* CRYSTALFORMER_B200_H */
