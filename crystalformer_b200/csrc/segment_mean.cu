// Per-crystal mean of atom features with the reference's fixed summation tree
// (models/kernels/irregular_mean_fwd.cu, pairwise_sum.cuh:78-111): rows are summed four at a time as
// (x0+x1)+(x2+x3), and the group sums are combined by a balanced binary tree over the next power of two of groups.
// The tree is evaluated without a buffer by keeping one partial sum per tree level (a binary counter); padding
// leaves are zero, so skipping them leaves every bit unchanged.
#include "common.cuh"

namespace cf {
namespace {

__global__ void segment_mean_kernel(const float *__restrict__ x, const int64_t *__restrict__ start, long long B,
                                    long long D, float *__restrict__ out)
{
    const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= B * D) return;
    const long long b = tid / D, d = tid % D;
    const long long s = start[b], len = start[b + 1] - s;
    const float *src = x + s * D + d;
    float total = 0.f;
    if (len == 1) total = src[0];
    else if (len == 2) total = src[0] + src[D];
    else if (len > 2) {
        float part[12];
        unsigned occupied = 0;
        const long long groups = (len + 3) / 4;
        for (long long g = 0; g < groups; ++g) {
            const long long r = 4 * g;
            const float m0 = src[r * D];
            const float m1 = (r + 1 < len) ? src[(r + 1) * D] : 0.f;
            const float m2 = (r + 2 < len) ? src[(r + 2) * D] : 0.f;
            const float m3 = (r + 3 < len) ? src[(r + 3) * D] : 0.f;
            float val = (m0 + m1) + (m2 + m3);
            int level = 0;
            while (occupied & (1u << level)) {
                val = part[level] + val;
                occupied &= ~(1u << level);
                ++level;
            }
            part[level] = val;
            occupied |= 1u << level;
        }
        bool first = true;
        for (int level = 0; level < 12; ++level)
            if (occupied & (1u << level)) {
                total = first ? part[level] : part[level] + total;
                first = false;
            }
    }
    out[tid] = total / (float)len;
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
