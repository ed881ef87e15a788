// Host entry points and the two small kernels of the peer gather (peer_gather.cuh): buffers that other processes
// can map, the store of a rank's outputs into every rank's buffer, and the collect that waits for all ranks.
#include <string.h>

#include "peer_gather.cuh"

namespace cf {
namespace {

// y (rows, targets) of this rank -> every rank's buffer (for outputs that were not produced by the fused pooling +
// head kernel).
__global__ void __launch_bounds__(256) peer_store_kernel(const float *__restrict__ y, long long rows, int targets,
                                                         const cf_peer_gather g)
{
    const long long total = rows * targets;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x)
        peer_store(g, idx / targets, targets, (int)(idx % targets), y[idx]);
}

// out[g] = value of cell index[g] for the `rows` crystals of the unsharded batch, each taken once its cell carries
// `step`.  One block; every thread polls its own cells.  The wait is bounded: on a timeout status[0] = 1 + the rank
// whose row is missing, the missing values become NaN and the kernel returns, so the context stays usable and the
// host reports the failure.
__global__ void __launch_bounds__(256) peer_collect_kernel(const unsigned long long *cells, uint32_t step,
                                                           const int64_t *__restrict__ index, long long rows,
                                                           int targets, long long rows_per_rank, float *__restrict__ out,
                                                           int *status, unsigned long long timeout_ns)
{
    const long long total = rows * targets;
    const unsigned long long t0 = global_timer_ns();
    for (long long idx = threadIdx.x; idx < total; idx += blockDim.x) {
        const long long r = idx / targets;
        const volatile unsigned long long *cell = cells + index[r] * targets + (idx % targets);
        unsigned long long v = *cell;
        while ((uint32_t)(v >> 32) != step) {
            if (global_timer_ns() - t0 > timeout_ns) break;
            __nanosleep(100);
            v = *cell;
        }
        if ((uint32_t)(v >> 32) == step) {
            out[idx] = __uint_as_float((uint32_t)v);
        } else {
            out[idx] = __int_as_float(0x7fc00000);
            atomicMax(status, 1 + (int)(index[r] / rows_per_rank));
        }
    }
}

}  // namespace

int validate_peer_gather(const cf_peer_gather *g, long long rows, const char *who)
{
    CF_REQUIRE(g != nullptr, CF_ERR_INVALID, "%s: null gather", who);
    CF_REQUIRE(g->world >= 1 && g->world <= CF_MAX_PEERS && g->rank >= 0 && g->rank < g->world, CF_ERR_INVALID,
               "%s: rank %d of %d (at most %d ranks)", who, g->rank, g->world, CF_MAX_PEERS);
    CF_REQUIRE(g->rows_per_rank >= 0 && g->step != 0, CF_ERR_INVALID, "%s: bad gather", who);
    for (int r = 0; r < g->world; ++r)
        CF_REQUIRE(g->cells[r] != nullptr, CF_ERR_INVALID, "%s: null buffer of rank %d", who, r);
    CF_REQUIRE(rows <= g->rows_per_rank, CF_ERR_RANGE, "%s: %lld rows for a gather of %lld rows per rank", who, rows,
               (long long)g->rows_per_rank);
    return CF_OK;
}

}  // namespace cf

extern "C" int cf_peer_alloc(int64_t bytes, void **ptr, unsigned char *handle)
{
    using namespace cf;
    CF_REQUIRE(bytes > 0 && ptr && handle, CF_ERR_INVALID, "cf_peer_alloc: bad argument");
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, (size_t)bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        if (p) cudaFree(p);
        return fail(CF_ERR_CUDA, "cf_peer_alloc: %s", cudaGetErrorString(e));
    }
    static_assert(sizeof(h) == CF_PEER_HANDLE_BYTES, "handle size");
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return CF_OK;
}

extern "C" int cf_peer_open(const unsigned char *handle, void **ptr)
{
    using namespace cf;
    CF_REQUIRE(handle && ptr, CF_ERR_INVALID, "cf_peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(CF_ERR_CUDA, "cf_peer_open: %s", cudaGetErrorString(e));
    *ptr = p;
    return CF_OK;
}

extern "C" int cf_peer_close(void *ptr)
{
    using namespace cf;
    if (ptr == nullptr) return CF_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) return fail(CF_ERR_CUDA, "cf_peer_close: %s", cudaGetErrorString(e));
    return CF_OK;
}

extern "C" int cf_peer_free(void *ptr)
{
    using namespace cf;
    if (ptr == nullptr) return CF_OK;
    const cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) return fail(CF_ERR_CUDA, "cf_peer_free: %s", cudaGetErrorString(e));
    return CF_OK;
}

extern "C" int cf_peer_gather_store(const float *y, int64_t rows, int64_t targets, const cf_peer_gather *gather,
                                    void *stream)
{
    using namespace cf;
    CF_REQUIRE(rows >= 0 && targets > 0, CF_ERR_INVALID, "cf_peer_gather_store: bad size");
    const int rc = validate_peer_gather(gather, rows, "cf_peer_gather_store");
    if (rc != CF_OK) return rc;
    if (rows == 0) return CF_OK;
    CF_REQUIRE(y != nullptr, CF_ERR_INVALID, "cf_peer_gather_store: null pointer");
    const long long total = rows * targets;
    const unsigned blocks = (unsigned)((total + 255) / 256 > 64 ? 64 : (total + 255) / 256);
    peer_store_kernel<<<blocks, 256, 0, as_stream(stream)>>>(y, rows, (int)targets, *gather);
    return launch_status("cf_peer_gather_store");
}

extern "C" int cf_peer_gather_collect(const uint64_t *cells, uint32_t step, const int64_t *index, int64_t rows,
                                      int64_t targets, int64_t rows_per_rank, float *out, int32_t *status,
                                      double timeout_s, void *stream)
{
    using namespace cf;
    CF_REQUIRE(rows >= 0 && targets > 0 && rows_per_rank > 0 && step != 0, CF_ERR_INVALID,
               "cf_peer_gather_collect: bad argument");
    if (rows == 0) return CF_OK;
    CF_REQUIRE(cells && status && index && out, CF_ERR_INVALID, "cf_peer_gather_collect: null pointer");
    CF_REQUIRE(timeout_s > 0.0 && timeout_s <= 60.0, CF_ERR_RANGE, "cf_peer_gather_collect: timeout of %g s (0..60]",
               timeout_s);
    peer_collect_kernel<<<1, 256, 0, as_stream(stream)>>>(reinterpret_cast<const unsigned long long *>(cells), step, index,
                                                         (long long)rows, (int)targets, (long long)rows_per_rank, out,
                                                         status, (unsigned long long)(timeout_s * 1e9));
    return launch_status("cf_peer_gather_collect");
}
