// Shared device helpers of the crystalformer_b200 kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "crystalformer_b200.h"

namespace cf {

constexpr int HEADS = 8;          // heads handled by the compiled kernels
constexpr int HEAD_DIM = 16;      // key / value head width
constexpr unsigned FULL = 0xffffffffu;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

// ---- host-side error plumbing (api.cu) --------------------------------------------------------------------
int fail(int code, const char *fmt, ...);
int launch_status(const char *what);
float weight_floor_log2();  // log2 of the weight below which a term is left out of the basis accumulation
unsigned long long *row_stats_words();  // device words that the sorted row kernel adds its work counts to, or NULL
int &dense_tile_rows_choice();  // this thread's row tile of the dense blocks: 0 = chosen per launch, 16, 32
struct DenseTileRows {           // sets it for a scope
    int saved;
    explicit DenseTileRows(int rows) : saved(dense_tile_rows_choice()) { dense_tile_rows_choice() = rows; }
    ~DenseTileRows() { dense_tile_rows_choice() = saved; }
};
bool sorted_rows_enabled();  // the one-call forwards may use row lists and the sorted row kernel (cf_set_sorted_rows)

#define CF_REQUIRE(cond, code, ...) \
    do {                            \
        if (!(cond)) return ::cf::fail(code, __VA_ARGS__); \
    } while (0)

// ---- fast transcendental wrappers ---------------------------------------------------------------------------
// One MUFU.EX2 each; arguments here are <= 0 and results below 2^-126 flush to zero, which is what the callers want
// (such weights contribute nothing at float precision).
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rsqrt_fast(float x)
{
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---- translation box ---------------------------------------------------------------------------------------
// Parameters of the reference's cut-off rule (models/kernels/real_enc_fwd.cu:63-85); evaluated by packed_box in
// lattice_core.cuh:  R = ceil( (double)((radius + 0.01f) * rvlen) / (2.0 * (double)pi_f) ).
struct BoxRule {
    float cutoff;       // 0: fixed box; <0: |cutoff| sigmas of each head's Gaussian; >0: radius in Angstrom
    int lattice_range;  // half-width of the fixed box
    int minimum_range;  // floor applied to adaptive half-widths (0 = none)
};

// Lattice rows and the squared length of r + n.T, contracted the way nvcc contracts the reference's expression
// r + t1*n1 + t2*n2 + t3*n3 (three dependent FMAs per component).
struct Cell {
    float t1x, t1y, t1z, t2x, t2y, t2z, t3x, t3y, t3z;
    __device__ __forceinline__ void load(const float *__restrict__ t)
    {
        t1x = t[0]; t1y = t[1]; t1z = t[2];
        t2x = t[3]; t2y = t[4]; t2z = t[5];
        t3x = t[6]; t3y = t[7]; t3z = t[8];
    }
};

__device__ __forceinline__ float warp_min(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
__device__ __forceinline__ int warp_max_int(int v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(FULL, v, o));
    return v;
}
// Sum over the warp in a fixed butterfly order: every lane ends with the same bits, run to run.
__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(FULL, v, o);
    return v;
}

// Picks x[idx] from eight registers without dynamic indexing.
__device__ __forceinline__ float pick8(const float (&x)[8], int idx)
{
    float r = x[0];
#pragma unroll
    for (int h = 1; h < 8; ++h) r = (idx == h) ? x[h] : r;
    return r;
}

// ---- chained launches (programmatic dependent launch) ------------------------------------------------------
// The one-call forwards issue a dozen short kernels back to back on one stream.  A kernel launched with
// launch_chained(..., chained = true) may be scheduled while its predecessor in the stream is still draining: its
// blocks run their prologue (staging of weights into shared memory, index setup), then grid_dependency_wait() blocks
// until the predecessor grid has completed and its writes are visible.  Every kernel launched this way calls
// grid_launch_dependents() first (which lets ITS successor be scheduled once all of this grid's blocks have started)
// and grid_dependency_wait() before it reads or overwrites anything an earlier kernel of the stream touches - and it
// calls the wait unconditionally, so that completion of a kernel always implies completion of all before it.  In a
// kernel launched the ordinary way both calls do nothing.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
bool chained_launches_enabled();  // cf_set_chained_launches

template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                  bool chained, Args &&...args)
{
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (chained && chained_launches_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }
int sm_count();

}  // namespace cf
