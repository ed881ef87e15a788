// Per-crystal mean of atom features with the reference's fixed summation tree (see segment_mean.cuh).
#include "common.cuh"
#include "segment_mean.cuh"

namespace cf {
namespace {

__global__ void segment_mean_kernel(const float *__restrict__ x, const int64_t *__restrict__ start, long long B,
                                    long long D, float *__restrict__ out)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= B * D) return;
    const long long b = tid / D, d = tid % D;
    const long long s = start[b], len = start[b + 1] - s;
    out[tid] = segment_mean_channel(x + s * D + d, D, len);
}

}  // namespace
}  // namespace cf

extern "C" int cf_segment_mean_fwd(const float *x, const int64_t *start, int64_t B, int64_t D, float *out,
                                   void *stream)
{
    using namespace cf;
    CF_REQUIRE(B >= 0 && D >= 0, CF_ERR_INVALID, "cf_segment_mean_fwd: negative size");
    if (B == 0 || D == 0) return CF_OK;
    CF_REQUIRE(x && start && out, CF_ERR_INVALID, "cf_segment_mean_fwd: null pointer");
    const long long total = (long long)B * D;
    segment_mean_kernel<<<(unsigned)((total + 127) / 128), 128, 0, as_stream(stream)>>>(x, start, B, D, out);
    return launch_status("cf_segment_mean_fwd");
}
