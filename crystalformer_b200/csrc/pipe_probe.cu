// Throughput probes for the two pipes that bound the lattice-sum kernels: FP32 FMA and MUFU (ex2).
// They give the roofline denominators measured on the device at hand instead of datasheet numbers.
#include "common.cuh"

namespace cf {
namespace {

template <int KIND>
__global__ void pipe_probe_kernel(long long iters, float *sink)
{
    float x0 = 1.0f + threadIdx.x * 1e-7f, x1 = x0 + 0.1f, x2 = x0 + 0.2f, x3 = x0 + 0.3f;
    float x4 = x0 + 0.4f, x5 = x0 + 0.5f, x6 = x0 + 0.6f, x7 = x0 + 0.7f;
    const float m = 0.999999f, c = 1e-7f;
    for (long long it = 0; it < iters; ++it) {
        if (KIND == 0) {
            x0 = fmaf(x0, m, c); x1 = fmaf(x1, m, c); x2 = fmaf(x2, m, c); x3 = fmaf(x3, m, c);
            x4 = fmaf(x4, m, c); x5 = fmaf(x5, m, c); x6 = fmaf(x6, m, c); x7 = fmaf(x7, m, c);
        } else {
            // x <- 2^-x stays in (0.5, 1); the negation is an operand modifier, not an instruction
            x0 = ex2(-x0); x1 = ex2(-x1); x2 = ex2(-x2); x3 = ex2(-x3);
            x4 = ex2(-x4); x5 = ex2(-x5); x6 = ex2(-x6); x7 = ex2(-x7);
        }
    }
    const float r = ((x0 + x1) + (x2 + x3)) + ((x4 + x5) + (x6 + x7));
    if (r == 123.456f) *sink = r;  // practically never true; keeps the loop alive
}

}  // namespace
}  // namespace cf

extern "C" int cf_pipe_probe(int kind, int blocks, int threads, int64_t iters, float *sink, void *stream)
{
    using namespace cf;
    CF_REQUIRE(kind == 0 || kind == 1, CF_ERR_INVALID, "cf_pipe_probe: kind must be 0 (FMA) or 1 (MUFU)");
    CF_REQUIRE(blocks > 0 && threads > 0 && threads <= 1024 && iters >= 0 && iters <= (1ll << 24), CF_ERR_RANGE,
               "cf_pipe_probe: launch shape out of range");
    CF_REQUIRE(sink != nullptr, CF_ERR_INVALID, "cf_pipe_probe: sink is null");
    if (kind == 0) pipe_probe_kernel<0><<<blocks, threads, 0, as_stream(stream)>>>(iters, sink);
    else pipe_probe_kernel<1><<<blocks, threads, 0, as_stream(stream)>>>(iters, sink);
    return launch_status("cf_pipe_probe");
}
