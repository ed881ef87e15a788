/*
 * Lets the reference project's device kernels (plain SIMT CUDA C, one `extern "C" __global__` function per file)
 * be compiled by g++ as ordinary functions, so that the reference's own kernel sources can serve as a CPU oracle.
 * TEST INFRASTRUCTURE ONLY.  Nothing here is copied from the reference: its sources are compiled where they lie.
 *
 * A "thread" is one call of the kernel function with blockIdx/threadIdx set; threads of a block run one after the
 * other on the same host thread.  That is valid for the kernels used here because none of them synchronises or
 * communicates between threads: every `__shared__` array is indexed by threadIdx.x first, i.e. it is per-thread
 * scratch, which a static thread_local array reproduces.
 */
#pragma once
#include <algorithm>
#include <cmath>
#include <cstddef>

struct cfref_dim3 { unsigned int x, y, z; };
extern thread_local cfref_dim3 blockDim, blockIdx, threadIdx;

#define __global__
#define __device__
#define __forceinline__ inline
#define __shared__ static thread_local
using std::max;
using std::min;
/* In device code exp/log/sqrt of a float argument resolve to the single-precision overloads; make g++ do the same
 * instead of silently promoting to the C library's double versions. */
using std::exp;
using std::log;
using std::sqrt;
