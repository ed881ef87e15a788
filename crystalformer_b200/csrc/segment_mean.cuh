// Mean over the rows of one crystal for one channel with the reference's fixed summation tree
// (models/kernels/irregular_mean_fwd.cu, pairwise_sum.cuh:78-111): rows are summed four at a time as
// (x0+x1)+(x2+x3), and the group sums are combined by a balanced binary tree over the next power of two of groups.
// The tree is evaluated without a buffer by keeping one partial sum per tree level (a binary counter); padding
// leaves are zero, so skipping them leaves every bit unchanged.
#pragma once
#include <cuda_runtime.h>

namespace cf {

// src: first row of the crystal at the wanted channel; D: row stride in floats; len: rows (up to 4096).
__device__ __forceinline__ float segment_mean_channel(const float *__restrict__ src, long long D, long long len)
{
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
    return total / (float)len;
}

}  // namespace cf
