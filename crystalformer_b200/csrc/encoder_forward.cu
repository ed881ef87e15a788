// Inference forward of the whole encoder stack in ONE host call.
//
// The reference runs an encoder layer as ~30 framework operators (in-projection, the Gaussian-width pipeline of
// models/indexed_lattice_multi_head_attention_cuda.py:640-722, q scaling, attention, out-projection, residual,
// feed-forward, residual; models/indexed_latticeformer_encoder.py:848-890 with LayerNorm = Identity under T-Fixup).
// At the sizes of a crystal batch each of them is launch-bound, and the host cannot issue them as fast as the GPU
// retires them.  Here a layer is eight launches issued back to back from C++:
//
//   SGEMM   qkv = x Wqkv^T                                   (cuBLAS, fp32)
//   qkv_post    + bias, alpha = q.w -> normalise -> elu -> a, q / sqrt(D); also x += out_proj.bias (used later)
//   lattice_phi_kernel, infinite_attn_rows_kernel           (cf_infinite_attn_fwd)
//   SGEMM   x += attn Wo^T                                   (beta = 1: the residual is the accumulator)
//   SGEMM   h = x W1^T
//   ffn_post    h = relu(h + b1); x += b2
//   SGEMM   x += h W2^T
//
// cuBLAS is resolved at run time from the copy already loaded in the process (the caller passes its handle), so that
// the handle and the functions come from the same library.  No training support: the autograd path stays in Python.
#include "blas_dyn.cuh"
#include "common.cuh"
#include "dense_block.cuh"
#include "row_list.cuh"
#include "term_list.cuh"

namespace cf {
int encoder_forward_impl(void *cublas_handle, int num_layers, const float *const *weights, const double *scalars,
                         float *x, const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                         const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t E,
                         int64_t max_atoms, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                         int lattice_range, int minimum_range, float *workspace, const int32_t *row_order,
                         void *const *attn_events, void *stream, const EmbedStage *embed, bool early_prep);
int infinite_attn_fwd_impl(const float *q, const float *k, const float *v, const float *a, const float *pos,
                           const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                           const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t H, int64_t D,
                           int64_t E, int64_t K, int64_t max_atoms, double dist_max, double wscale, const float *W,
                           double cutoff_radius, int lattice_range, int minimum_range, float *out, float *logit,
                           float *lse, float *psi_row, const int32_t *row_order, const TermList *list,
                           unsigned *ticket_ready, void *stream, bool chained);
unsigned *row_ticket_block(int count);
int sorted_attn_impl(const float *q, const float *k, const float *v, const float *a, const float *pos_ij,
                     const float *tvecs, const float *rvlen, const int64_t *batch, const int64_t *edges,
                     const int64_t *row_start, int64_t N, int64_t E, int64_t max_atoms, double dist_max, double wscale,
                     const float *W, double cutoff_radius, int lattice_range, int minimum_range, float *out, float *lse,
                     const RowListView &view, int sched_slot, bool zeroed, int64_t K, cudaStream_t s);
namespace {

// A second stream and two events per (host thread, device), created on first use and kept for the life of the
// process: the term-list build of a forward depends on the geometry only and runs beside the first dense block.
struct SideStream {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
    bool ok = false;
};
SideStream &side_stream()
{
    static thread_local SideStream per_device[64];
    int dev = 0;
    cudaGetDevice(&dev);
    SideStream &s = per_device[dev & 63];
    if (!s.ok && s.stream == nullptr) {
        s.ok = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess &&
               cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess &&
               cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) == cudaSuccess;
        if (!s.ok) {
            cudaGetLastError();
            s.stream = reinterpret_cast<cudaStream_t>(1);  // do not try again
        }
    }
    return s;
}

}  // namespace

// The side stream made to wait for the caller's events (either may be NULL), for cf_model_forward's early preparation;
// NULL if the side stream could not be created.
cudaStream_t early_prep_stream(void *inputs_ready, void *slot_free)
{
    SideStream &side = side_stream();
    if (!side.ok) return nullptr;
    if (inputs_ready != nullptr && cudaStreamWaitEvent(side.stream, reinterpret_cast<cudaEvent_t>(inputs_ready), 0) != cudaSuccess) return nullptr;
    if (slot_free != nullptr && cudaStreamWaitEvent(side.stream, reinterpret_cast<cudaEvent_t>(slot_free), 0) != cudaSuccess) return nullptr;
    return side.stream;
}

namespace {

struct LayerScalars {
    float gauss_scale, gauss_shift;  // alpha <- (alpha + shift) * scale
    float a_factor;                  // -0.5 / scale_real^2
    float elu_beta, lower_bound;     // positive_func 'elu=beta', gauss_lb_real
};

// One thread per (atom, head): bias, width parameter, scaled query, and the deferred out-projection bias.
__global__ void qkv_post_kernel(const float *__restrict__ qkv, const float *__restrict__ bias,
                                const float *__restrict__ w_pos, const float *__restrict__ out_bias, LayerScalars sc,
                                long long N, float *__restrict__ q, float *__restrict__ k, float *__restrict__ v,
                                float *__restrict__ a, float *__restrict__ x)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= N * HEADS) return;
    const long long i = tid / HEADS;
    const int h = (int)(tid % HEADS);
    const int col = h * HEAD_DIM;
    const float4 *src = reinterpret_cast<const float4 *>(qkv + i * 384 + col);
    const float4 *bq = reinterpret_cast<const float4 *>(bias + col);
    const float4 *wp = reinterpret_cast<const float4 *>(w_pos + col);
    float4 *qd = reinterpret_cast<float4 *>(q + i * 128 + col);
    float4 *kd = reinterpret_cast<float4 *>(k + i * 128 + col);
    float4 *vd = reinterpret_cast<float4 *>(v + i * 128 + col);
    float4 *xd = reinterpret_cast<float4 *>(x + i * 128 + col);
    const float4 *ob = reinterpret_cast<const float4 *>(out_bias + col);
    float alpha = 0.f;
#pragma unroll
    for (int t = 0; t < 4; ++t) {
        float4 qv = src[t];
        const float4 b0 = __ldg(bq + t), w = __ldg(wp + t);
        qv.x += b0.x; qv.y += b0.y; qv.z += b0.z; qv.w += b0.w;
        alpha = fmaf(qv.x, w.x, alpha); alpha = fmaf(qv.y, w.y, alpha); alpha = fmaf(qv.z, w.z, alpha); alpha = fmaf(qv.w, w.w, alpha);
        qd[t] = make_float4(qv.x * 0.25f, qv.y * 0.25f, qv.z * 0.25f, qv.w * 0.25f);  // 1/sqrt(16)
        float4 kv = src[32 + t];
        const float4 b1 = __ldg(bq + 32 + t);
        kd[t] = make_float4(kv.x + b1.x, kv.y + b1.y, kv.z + b1.z, kv.w + b1.w);
        float4 vv = src[64 + t];
        const float4 b2 = __ldg(bq + 64 + t);
        vd[t] = make_float4(vv.x + b2.x, vv.y + b2.y, vv.z + b2.z, vv.w + b2.w);
        float4 xv = xd[t];
        const float4 o = __ldg(ob + t);
        xd[t] = make_float4(xv.x + o.x, xv.y + o.y, xv.z + o.z, xv.w + o.w);
    }
    // (1 - lb) elu(x beta / (1 - lb)) + 1, x the normalised alpha
    const float xn = (alpha + sc.gauss_shift) * sc.gauss_scale;
    const float t = xn * (sc.elu_beta / (1.0f - sc.lower_bound));
    const float elu = t > 0.f ? t : expm1f(t);
    a[tid] = ((1.0f - sc.lower_bound) * elu + 1.0f) * sc.a_factor;
}

__global__ void ffn_post_kernel(float *__restrict__ h, const float *__restrict__ b1, long long N, int ff,
                                float *__restrict__ x, const float *__restrict__ b2)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total_h = N * (long long)(ff / 4);
    if (tid < total_h) {
        const int c = (int)(tid % (ff / 4));
        float4 hv = reinterpret_cast<float4 *>(h)[tid];
        const float4 b = __ldg(reinterpret_cast<const float4 *>(b1) + c);
        hv.x = fmaxf(hv.x + b.x, 0.f); hv.y = fmaxf(hv.y + b.y, 0.f); hv.z = fmaxf(hv.z + b.z, 0.f); hv.w = fmaxf(hv.w + b.w, 0.f);
        reinterpret_cast<float4 *>(h)[tid] = hv;
    }
    if (tid < N * 32) {
        const int c = (int)(tid % 32);
        float4 xv = reinterpret_cast<float4 *>(x)[tid];
        const float4 b = __ldg(reinterpret_cast<const float4 *>(b2) + c);
        xv.x += b.x; xv.y += b.y; xv.z += b.z; xv.w += b.w;
        reinterpret_cast<float4 *>(x)[tid] = xv;
    }
}

}  // namespace
}  // namespace cf

extern "C" int64_t cf_encoder_workspace_floats(int64_t N, int64_t E, int64_t ff_dim)
{
    // qkv (384) + q,k,v (3 x 128) + attention output (128) + a (8) + lse (8) + hidden (ff) per atom, logits per edge,
    // then the term lists: directory (2 ints per edge), allocation cursor, pool (2 floats per entry)
    // (or, for batches of small crystals, the row lists: whichever is larger)
    const size_t lists = cf::term_list_workspace_bytes(N, E), rows = cf::row_list_workspace_bytes(N, E);
    return N * (384 + 384 + 128 + 8 + 8 + ff_dim) + E * 8 + 64 + (int64_t)((lists > rows ? lists : rows) + 3) / 4;
}

extern "C" int cf_encoder_forward(void *cublas_handle, int num_layers, const float *const *weights, const double *scalars,
                                  float *x, const float *pos_ij, const float *tvecs, const float *rvlen,
                                  const int64_t *batch, const int64_t *edges, const int64_t *row_start, int64_t N,
                                  int64_t B, int64_t E, int64_t max_atoms, int64_t K, int64_t ff_dim, double wscale,
                                  double cutoff_radius, int lattice_range, int minimum_range, float *workspace,
                                  const int32_t *row_order, void *const *attn_events, void *stream)
{
    return cf::encoder_forward_impl(cublas_handle, num_layers, weights, scalars, x, pos_ij, tvecs, rvlen, batch, edges,
                                    row_start, N, B, E, max_atoms, K, ff_dim, wscale, cutoff_radius, lattice_range,
                                    minimum_range, workspace, row_order, attn_events, stream, nullptr, false);
}

// cf_encoder_forward with an optional embedding stage (dense path only): x is then written by the first dense block.
int cf::encoder_forward_impl(void *cublas_handle, int num_layers, const float *const *weights, const double *scalars,
                             float *x, const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                             const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t E,
                             int64_t max_atoms, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                             int lattice_range, int minimum_range, float *workspace, const int32_t *row_order,
                             void *const *attn_events, void *stream, const EmbedStage *embed, bool early_prep)
{
    CF_REQUIRE(N >= 0 && E >= 0 && num_layers >= 0, CF_ERR_INVALID, "cf_encoder_forward: negative size");
    CF_REQUIRE(ff_dim > 0 && ff_dim % 4 == 0, CF_ERR_UNSUPPORTED, "cf_encoder_forward: ff_dim must be a positive multiple of 4");
    CF_REQUIRE(N < (1ll << 31) / 512, CF_ERR_RANGE, "cf_encoder_forward: N=%lld too large for 32-bit GEMM sizes", (long long)N);
    if (N == 0 || num_layers == 0) return CF_OK;
    CF_REQUIRE(weights && scalars && x && workspace, CF_ERR_INVALID, "cf_encoder_forward: null pointer");
    const int ff = (int)ff_dim;
    const bool fused = dense_path_available(num_layers, weights, ff_dim);  // one launch per layer boundary, no cuBLAS
    CF_REQUIRE(fused || embed == nullptr, CF_ERR_INVALID, "cf_encoder_forward: embedding stage without the dense path");
    CF_REQUIRE(fused || cublas_handle, CF_ERR_INVALID, "cf_encoder_forward: null cuBLAS handle");
    cudaStream_t s = as_stream(stream);

    float *qkv = workspace;
    float *q = qkv + N * 384, *k = q + N * 128, *v = k + N * 128, *attn = v + N * 128;
    float *a = attn + N * 128, *lse = a + N * 8, *hidden = lse + N * 8, *logit = hidden + N * ff_dim;
    int rc = CF_OK;

    // Term lists (term_list.cuh): the geometry is the same for every layer, so the (key, translation) pairs that can
    // matter to any layer are found once.  The widest Gaussian any layer can produce has a = lower_bound x a_factor.
    TermList lists{};
    const TermList *list = nullptr;
    RowListView row_lists{};
    bool sorted_rows = false;  // batches of crystals of at most 32 atoms with a value encoding: row lists + sorted row kernel
    // The build runs on the side stream and the first attention waits for it.  early_prep: the caller has already put the
    // geometry launch on the side stream (cf_model_forward with an inputs-ready event), so the side stream is not made
    // to wait for this stream here.
    bool forked = early_prep;
    unsigned *tickets = nullptr;
    if (pos_ij != nullptr && weight_floor_log2() > -200.0f) {
        float a_widest = -INFINITY;
        for (int l = 0; l < num_layers; ++l) a_widest = fmaxf(a_widest, (float)(scalars[6 * l + 4] * scalars[6 * l + 2]));
        if (a_widest < 0.0f) {
            const BoxRule rule{(float)cutoff_radius, lattice_range, minimum_range};
            const float window = term_window(weight_floor_log2(), a_widest);
            SideStream &side = side_stream();
            if (!early_prep)
                forked = side.ok && cudaEventRecord(side.fork, s) == cudaSuccess &&
                         cudaStreamWaitEvent(side.stream, side.fork, 0) == cudaSuccess;
            // (without a basis the enumerating kernel with term lists is faster - 0.62 against 0.79 ms for a 7-layer
            // forward of 256 crystals of up to 60 atoms - so K = 0 keeps it)
            sorted_rows = sorted_rows_enabled() && K == 64 && max_atoms <= ROW_LIST_MAX_KEYS && N < (1ll << 31) && E < (1ll << 31);
            if (sorted_rows) {
                RowListBuild rb{};
                rb.pos_ij = pos_ij; rb.tvecs = tvecs; rb.rvlen = cutoff_radius != 0.0 ? rvlen : nullptr;
                rb.batch = batch; rb.edges = edges; rb.row_start = row_start; rb.row_order = row_order;
                rb.N = N; rb.E = E; rb.rule = rule; rb.a_widest = a_widest; rb.window = window; rb.coop_chunks = ROW_COOP_CHUNKS;
                rb.out = row_lists = row_list_carve(logit + E * 8 + 64, N, E);
                rc = launch_row_list_build(rb, forked ? side.stream : s);
            } else {
                TermListBuild tb{};
                tb.pos_ij = pos_ij; tb.tvecs = tvecs; tb.rvlen = cutoff_radius != 0.0 ? rvlen : nullptr;
                tb.batch = batch; tb.edges = edges; tb.row_start = row_start; tb.row_order = row_order;
                tb.N = N; tb.E = E; tb.max_atoms = (int)max_atoms;
                tb.rule = rule;
                tb.a_widest = a_widest;
                tb.window = window;
                term_list_carve(logit + E * 8 + 64, N, E, &tb.start, &tb.count, &tb.dmin, &tb.cursor, &tb.pool);
                tb.capacity = (long long)term_pool_entries(N, E);
                rc = launch_term_list_build(tb, forked ? side.stream : s);
                // the row tickets of all layers, zeroed once here instead of by a phi launch per layer (on the main
                // stream, ahead of the first dense block: the list build is the longer of the two branches)
                if (K > 0 && num_layers <= 16 && (tickets = row_ticket_block(num_layers)) != nullptr &&
                    cudaMemsetAsync(tickets, 0, sizeof(unsigned) * num_layers, s) != cudaSuccess)
                    tickets = nullptr;
                lists.pool = tb.pool; lists.start = tb.start; lists.count = tb.count; lists.dmin = tb.dmin; lists.window = tb.window;
                list = &lists;
            }
            if (rc != CF_OK) return rc;
        }
    }
    if (forked && cudaEventRecord(side_stream().join, side_stream().stream) != cudaSuccess) return launch_status("side stream join");
    // one attention call of layer l (dist_max, W of that layer)
    auto attention = [&](int l, double dist_max, const float *W, float *attn_out, float *lse_out) {
        if (sorted_rows)
            return sorted_attn_impl(q, k, v, a, pos_ij, tvecs, rvlen, batch, edges, row_start, N, E, max_atoms, dist_max, wscale,
                                    W, cutoff_radius, lattice_range, minimum_range, attn_out, lse_out, row_lists,
                                    l < ROW_SCHED_SLOTS - 1 ? l : ROW_SCHED_SLOTS - 1, l < ROW_SCHED_SLOTS - 1, K, s);
        return infinite_attn_fwd_impl(q, k, v, a, nullptr, pos_ij, tvecs, rvlen, batch, edges, row_start, N, B, HEADS, HEAD_DIM,
                                      E, K, max_atoms, dist_max, wscale, W, cutoff_radius, lattice_range, minimum_range,
                                      attn_out, logit, lse_out, nullptr, row_order, list, tickets ? tickets + l : nullptr, s, true);
    };

    // Fused dense path: every layer brings its weights packed for the tensor-core kernel (slot 10) and the
    // feed-forward width is a multiple of 128.  One launch per layer boundary instead of four GEMMs and two
    // element-wise passes; see dense_block.cu.
    if (fused) {
        auto head_of = [&](DenseArgs &d, int l) {
            const float *const *w = weights + 11 * l;
            const double *sc = scalars + 6 * l;
            d.head = 1;
            d.Wqkv = reinterpret_cast<const float4 *>(w[10]);
            d.bqkv = w[1];
            d.w_pos = w[2];
            d.gauss_scale = (float)sc[0]; d.gauss_shift = (float)sc[1]; d.a_factor = (float)sc[2];
            d.elu_beta = (float)sc[3]; d.lower_bound = (float)sc[4];
        };
        DenseArgs d{};
        d.N = N; d.ff = ff; d.x = x; d.q = q; d.k = k; d.v = v; d.a = a; d.attn = attn;
        head_of(d, 0);
        d.chained = 0;  // (first kernel of the forward on this stream: nothing to chain to)
        if (embed != nullptr) { d.features = embed->features; d.species = embed->species; d.feature_dim = embed->feature_dim; d.Wembed = embed->packed; }
        rc = launch_dense_block(d, s);
        if (forked) cudaStreamWaitEvent(s, side_stream().join, 0);
        for (int l = 0; l < num_layers && rc == CF_OK; ++l) {
            const float *const *w = weights + 11 * l;
            const double *sc = scalars + 6 * l;
            if (attn_events) cudaEventRecord(reinterpret_cast<cudaEvent_t>(attn_events[2 * l]), s);
            rc = attention(l, sc[5], w[3], attn, lse);
            if (attn_events) cudaEventRecord(reinterpret_cast<cudaEvent_t>(attn_events[2 * l + 1]), s);
            if (rc != CF_OK) break;
            DenseArgs t{};
            t.N = N; t.ff = ff; t.x = x; t.q = q; t.k = k; t.v = v; t.a = a; t.attn = attn;
            t.tail = 1;
            t.chained = 1;
            const float4 *packed = reinterpret_cast<const float4 *>(w[10]);
            t.Wo = packed + 48 * 16 * 32;                     // after Wqkv (48 column tiles x 16 k steps x 32 lanes)
            t.W1 = t.Wo + 16 * 16 * 32;
            t.W2 = t.W1 + (size_t)(ff / 8) * 16 * 32;
            t.bo = w[5]; t.b1 = w[7]; t.b2 = w[9];
            if (l + 1 < num_layers) head_of(t, l + 1);
            rc = launch_dense_block(t, s);
        }
        if (rc != CF_OK) return rc;
        return launch_status("cf_encoder_forward");
    }

    const Blas &bl = blas();
    CF_REQUIRE(bl.ok, CF_ERR_CUDA, "cf_encoder_forward: libcublas.so.12 could not be resolved in this process");
    cublasHandle_t handle = reinterpret_cast<cublasHandle_t>(cublas_handle);
    BlasScope scope(bl, handle, s);
    const int rows = (int)N;
    cublasStatus_t st = CUBLAS_STATUS_SUCCESS;
    if (forked) cudaStreamWaitEvent(s, side_stream().join, 0);
    for (int l = 0; l < num_layers && rc == CF_OK && st == CUBLAS_STATUS_SUCCESS; ++l) {
        const float *const *w = weights + 11 * l;  // Wqkv, bqkv, w_pos, Wpe, Wo, bo, W1, b1, W2, b2, packed (optional)
        const double *sc = scalars + 6 * l;        // gauss_scale, gauss_shift, a_factor, elu_beta, lower_bound, dist_max
        LayerScalars ls{(float)sc[0], (float)sc[1], (float)sc[2], (float)sc[3], (float)sc[4]};
        st = linear(bl, handle, x, w[0], qkv, rows, 128, 384, 0.0f);
        if (st != CUBLAS_STATUS_SUCCESS) break;
        const long long nh = N * HEADS;
        qkv_post_kernel<<<(unsigned)((nh + 127) / 128), 128, 0, s>>>(qkv, w[1], w[2], w[5], ls, N, q, k, v, a, x);
        if (attn_events) cudaEventRecord(reinterpret_cast<cudaEvent_t>(attn_events[2 * l]), s);
        rc = attention(l, sc[5], w[3], attn, lse);
        if (attn_events) cudaEventRecord(reinterpret_cast<cudaEvent_t>(attn_events[2 * l + 1]), s);
        if (rc != CF_OK) break;
        st = linear(bl, handle, attn, w[4], x, rows, 128, 128, 1.0f);
        if (st != CUBLAS_STATUS_SUCCESS) break;
        st = linear(bl, handle, x, w[6], hidden, rows, 128, ff, 0.0f);
        if (st != CUBLAS_STATUS_SUCCESS) break;
        const long long work = N * (long long)(ff / 4 > 32 ? ff / 4 : 32);
        ffn_post_kernel<<<(unsigned)((work + 255) / 256), 256, 0, s>>>(hidden, w[7], N, ff, x, w[9]);
        st = linear(bl, handle, hidden, w[8], x, rows, ff, 128, 1.0f);
    }
    if (st != CUBLAS_STATUS_SUCCESS) return fail(CF_ERR_CUDA, "cf_encoder_forward: cuBLAS SGEMM failed with status %d", (int)st);
    if (rc != CF_OK) return rc;
    return launch_status("cf_encoder_forward");
}
