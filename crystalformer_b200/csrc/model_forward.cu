// Inference forward of the whole model in ONE host call:
//   species features -> embedding -> batch geometry -> encoder stack -> per-crystal mean -> two-layer head.
//
// The reference's Latticeformer.forward (models/latticeformer.py:211-302) is a chain of framework calls; at the sizes
// of a crystal batch the host cannot issue them as fast as the GPU retires them.  Here the chain is issued back to
// back from C++ on one stream: one geometry launch, the embedding (inside the first dense block of the encoder when
// its packed weight is given, else one SGEMM), the encoder stack, and one fused kernel for the pooling (models/pooling.py:19-25 with the fixed summation tree of irregular_mean_fwd.cu) and the
// multi-layer-perceptron head (Linear - ReLU - Linear, models/latticeformer.py:176-209 with norm_type "no").
// No allocation, no synchronisation: scratch comes from the caller's workspace.
#include "blas_dyn.cuh"
#include "common.cuh"
#include "dense_block.cuh"
#include "peer_gather.cuh"
#include "segment_mean.cuh"

namespace cf {
int validate_peer_gather(const cf_peer_gather *g, long long rows, const char *who);
int launch_prepare_all(const float *pos, const float *trans, const int64_t *sizes, int64_t *atom_start,
                       int64_t *edge_start, long long B, long long N, long long E, int64_t *batch, int64_t *edges,
                       int64_t *row_start, float *pos_ij, float *rvlen, double reach, int32_t *row_order, bool *ordered,
                       cudaStream_t s);
int encoder_forward_impl(void *cublas_handle, int num_layers, const float *const *weights, const double *scalars,
                         float *x, const float *pos_ij, const float *tvecs, const float *rvlen, const int64_t *batch,
                         const int64_t *edges, const int64_t *row_start, int64_t N, int64_t B, int64_t E,
                         int64_t max_atoms, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                         int lattice_range, int minimum_range, float *workspace, const int32_t *row_order,
                         void *const *attn_events, void *stream, const EmbedStage *embed, bool early_prep);
cudaStream_t early_prep_stream(void *inputs_ready, void *slot_free);
namespace {

constexpr int MODEL_DIM = 128;
constexpr int HEAD_THREADS = 128;
constexpr int HEAD_MAX_HIDDEN = 1024;

// One thread block per crystal: mean of the atoms' features, hidden = relu(W1 mean + b1), y = W2 hidden + b2.
// GATHER: y also goes into every rank's gather buffer (peer_gather.cuh).
template <bool GATHER>
__global__ void __launch_bounds__(HEAD_THREADS) pool_head_kernel(const float *__restrict__ x,
                                                                 const int64_t *__restrict__ atom_start,
                                                                 const float *__restrict__ W1, const float *__restrict__ b1,
                                                                 const float *__restrict__ W2, const float *__restrict__ b2,
                                                                 int hidden, int targets, float *__restrict__ y,
                                                                 const cf_peer_gather gather)
{
    __shared__ __align__(16) float pooled[MODEL_DIM];
    __shared__ float hid[HEAD_MAX_HIDDEN];
    const long long c = blockIdx.x;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    grid_dependency_wait();  // (chained launch behind the last dense block)
    const long long s = atom_start[c], len = atom_start[c + 1] - s;
    pooled[tid] = len > 0 ? segment_mean_channel(x + s * MODEL_DIM + tid, MODEL_DIM, len) : 0.f;
    __syncthreads();
    const float4 *p4 = reinterpret_cast<const float4 *>(pooled);
    for (int u = tid; u < hidden; u += HEAD_THREADS) {
        const float4 *w4 = reinterpret_cast<const float4 *>(W1 + (size_t)u * MODEL_DIM);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 8
        for (int d = 0; d < MODEL_DIM / 4; ++d) {
            const float4 w = __ldg(w4 + d), v = p4[d];
            a0 = fmaf(w.x, v.x, a0); a1 = fmaf(w.y, v.y, a1); a2 = fmaf(w.z, v.z, a2); a3 = fmaf(w.w, v.w, a3);
        }
        hid[u] = fmaxf((a0 + a1) + (a2 + a3) + b1[u], 0.f);
    }
    __syncthreads();
    for (int t = warp; t < targets; t += HEAD_THREADS / 32) {
        float acc = 0.f;
        for (int u = lane; u < hidden; u += 32) acc = fmaf(W2[(size_t)t * hidden + u], hid[u], acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            y[c * targets + t] = acc + b2[t];
            if (GATHER) peer_store(gather, c, targets, t, acc + b2[t]);
        }
    }
}

inline size_t align_up(size_t v) { return (v + 255) & ~(size_t)255; }

struct Carve {
    char *base;
    size_t used = 0;
    template <class T>
    T *take(size_t count)
    {
        T *p = base ? reinterpret_cast<T *>(base + used) : nullptr;
        used += align_up(count * sizeof(T));
        return p;
    }
};

struct Scratch {
    int64_t *atom_start, *edge_start, *batch, *row_start, *edges;
    float *pos_ij, *rvlen, *x, *encoder;
    int32_t *row_order;
    size_t bytes;
};

Scratch carve(void *workspace, int64_t N, int64_t B, int64_t E, int64_t ff_dim)
{
    Carve c{static_cast<char *>(workspace)};
    Scratch s{};
    s.atom_start = c.take<int64_t>(B + 1);
    s.edge_start = c.take<int64_t>(B + 1);
    s.batch = c.take<int64_t>(N);
    s.row_start = c.take<int64_t>(N + 1);
    s.edges = c.take<int64_t>(2 * E);
    s.pos_ij = c.take<float>(3 * E);
    s.rvlen = c.take<float>(3 * B);
    s.row_order = c.take<int32_t>(N);
    s.x = c.take<float>(N * MODEL_DIM);
    s.encoder = c.take<float>((size_t)cf_encoder_workspace_floats(N, E, ff_dim));
    s.bytes = c.used;
    return s;
}

}  // namespace
}  // namespace cf

extern "C" int64_t cf_model_workspace_bytes(int64_t N, int64_t B, int64_t E, int64_t ff_dim)
{
    return (int64_t)cf::carve(nullptr, N, B, E, ff_dim).bytes;
}

namespace cf {

// cf_model_forward with the species of the atoms given either as feature rows (`features`, the reference's interface)
// or as indices (`species`: the embedding of atom i is column species[i] of W_embed, i.e. what a one-hot feature row
// gives; only with packed weights, where the first dense block builds the one-hot rows in shared memory).
int model_forward_impl(void *cublas_handle, const float *features, const int64_t *species, int64_t feature_dim, const float *pos,
                       const float *trans, const int64_t *sizes, int64_t N, int64_t B, int64_t E,
                       int64_t max_atoms, const float *W_embed, const float *W_embed_packed, int num_layers,
                       const float *const *weights, const double *scalars, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                       int lattice_range, int minimum_range, const float *W1, const float *b1, int64_t hidden,
                       const float *W2, const float *b2, int64_t targets, double order_reach, void *workspace,
                       float *y, void *const *attn_events, const cf_peer_gather *gather, void *inputs_ready,
                       void *slot_free, void *stream)
{
    CF_REQUIRE(N >= 0 && B >= 0 && E >= 0 && feature_dim > 0, CF_ERR_INVALID, "cf_model_forward: bad size");
    if (gather != nullptr) {
        const int grc = validate_peer_gather(gather, B, "cf_model_forward");
        if (grc != CF_OK) return grc;
    }
    CF_REQUIRE(hidden > 0 && hidden <= HEAD_MAX_HIDDEN && targets > 0, CF_ERR_UNSUPPORTED,
               "cf_model_forward: head of %lld hidden units, %lld targets (hidden <= %d)", (long long)hidden,
               (long long)targets, HEAD_MAX_HIDDEN);
    CF_REQUIRE(N < (1ll << 31) / 512, CF_ERR_RANGE, "cf_model_forward: N=%lld too large for 32-bit GEMM sizes", (long long)N);
    if (B == 0) return CF_OK;
    CF_REQUIRE((features || species) && pos && trans && sizes && W_embed && W1 && b1 && W2 && b2 && workspace && y, CF_ERR_INVALID,
               "cf_model_forward: null pointer");
    // With packed weights everywhere the whole forward runs in this library's kernels and cuBLAS is not touched.
    const bool embed_fused = W_embed_packed != nullptr && feature_dim <= MODEL_DIM && num_layers > 0 && N > 0 &&
                             dense_path_available(num_layers, weights, ff_dim);
    CF_REQUIRE(embed_fused || cublas_handle, CF_ERR_INVALID, "cf_model_forward: null cuBLAS handle");
    CF_REQUIRE(embed_fused || features, CF_ERR_UNSUPPORTED, "cf_model_forward: species indices need the packed weights");
    cudaStream_t s = as_stream(stream);
    Scratch w = carve(workspace, N, B, E, ff_dim);

    CF_REQUIRE(B <= (1 << 20), CF_ERR_RANGE, "cf_model_forward: B=%lld above 2^20 crystals", (long long)B);
    // Early preparation: given an event after which the inputs are valid, the geometry launch and the list build go to
    // the library's side stream, ordered after that event (and after slot_free: the previous use of this workspace) but
    // NOT after the work already queued on `stream`, so they run beside the previous batch's forward.
    cudaStream_t prep = nullptr;
    if (inputs_ready != nullptr && embed_fused && N > 0) prep = early_prep_stream(inputs_ready, slot_free);
    const bool early = prep != nullptr;
    bool ordered = false;  // batches beyond the one-launch sort are processed in index order
    int rc = launch_prepare_all(pos, trans, sizes, w.atom_start, w.edge_start, B, N, E, w.batch, w.edges, w.row_start, w.pos_ij, w.rvlen,
                            order_reach, w.row_order, &ordered, early ? prep : s);
    if (rc != CF_OK) return rc;
    const int32_t *order = ordered ? w.row_order : nullptr;
    if (N > 0 && !embed_fused) {
        const Blas &bl = blas();
        CF_REQUIRE(bl.ok, CF_ERR_CUDA, "cf_model_forward: libcublas.so.12 could not be resolved in this process");
        cublasHandle_t handle = reinterpret_cast<cublasHandle_t>(cublas_handle);
        BlasScope scope(bl, handle, s);
        const cublasStatus_t st = linear(bl, handle, features, W_embed, w.x, (int)N, (int)feature_dim, MODEL_DIM, 0.0f);
        if (st != CUBLAS_STATUS_SUCCESS) return fail(CF_ERR_CUDA, "cf_model_forward: cuBLAS SGEMM failed with status %d", (int)st);
    }
    const EmbedStage embed{features, species, (int)feature_dim, reinterpret_cast<const float4 *>(W_embed_packed)};
    rc = encoder_forward_impl(cublas_handle, num_layers, weights, scalars, w.x, w.pos_ij, trans,
                              cutoff_radius != 0.0 ? w.rvlen : nullptr, w.batch, w.edges, w.row_start, N, B, E, max_atoms, K,
                              ff_dim, wscale, cutoff_radius, lattice_range, minimum_range, w.encoder, order, attn_events,
                              stream, embed_fused ? &embed : nullptr, early);
    if (rc != CF_OK) return rc;
    const bool chained = num_layers > 0 && N > 0;  // behind the encoder's last dense block
    if (gather != nullptr)
        launch_chained(pool_head_kernel<true>, dim3((unsigned)B), dim3(HEAD_THREADS), 0, s, chained, (const float *)w.x,
                       (const int64_t *)w.atom_start, W1, b1, W2, b2, (int)hidden, (int)targets, y, *gather);
    else
        launch_chained(pool_head_kernel<false>, dim3((unsigned)B), dim3(HEAD_THREADS), 0, s, chained, (const float *)w.x,
                       (const int64_t *)w.atom_start, W1, b1, W2, b2, (int)hidden, (int)targets, y, cf_peer_gather{});
    return launch_status("cf_model_forward");
}

}  // namespace cf

extern "C" int cf_model_forward(void *cublas_handle, const float *features, int64_t feature_dim, const float *pos,
                                const float *trans, const int64_t *sizes, int64_t N, int64_t B, int64_t E,
                                int64_t max_atoms, const float *W_embed, const float *W_embed_packed, int num_layers,
                                const float *const *weights, const double *scalars, int64_t K, int64_t ff_dim, double wscale, double cutoff_radius,
                                int lattice_range, int minimum_range, const float *W1, const float *b1, int64_t hidden,
                                const float *W2, const float *b2, int64_t targets, double order_reach, void *workspace,
                                float *y, void *const *attn_events, const cf_peer_gather *gather, void *inputs_ready,
                                void *slot_free, void *stream)
{
    CF_REQUIRE(features != nullptr || B == 0, CF_ERR_INVALID, "cf_model_forward: null pointer");
    return cf::model_forward_impl(cublas_handle, features, nullptr, feature_dim, pos, trans, sizes, N, B, E, max_atoms, W_embed,
                                  W_embed_packed, num_layers, weights, scalars, K, ff_dim, wscale, cutoff_radius, lattice_range,
                                  minimum_range, W1, b1, hidden, W2, b2, targets, order_reach, workspace, y, attn_events, gather,
                                  inputs_ready, slot_free, stream);
}
