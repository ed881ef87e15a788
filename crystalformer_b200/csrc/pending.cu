// Entry points declared in the public header whose kernels are still to be written.
#include "common.cuh"

extern "C" int64_t cf_lattice_sum_bwd_scratch_bytes(int64_t, int64_t, int64_t, int64_t) { return 0; }

extern "C" int cf_lattice_sum_bwd(const float *, const float *, const float *, const int64_t *, const int64_t *,
                                  const int64_t *, const float *, const float *, const float *, int64_t, int64_t,
                                  int64_t, int64_t, double, double, const float *, int64_t, int64_t, const float *,
                                  double, int, int, float *, float *, void *, void *)
{
    return cf::fail(CF_ERR_UNSUPPORTED, "cf_lattice_sum_bwd: not built yet");
}

extern "C" int cf_infinite_attn_bwd(const float *, const float *, const float *, const float *, const float *,
                                    const float *, const float *, const float *, const int64_t *, const int64_t *,
                                    const int64_t *,
                                    int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                    double, double, const float *,
                                    double, int, int, const float *, const float *, const float *, const float *,
                                    float *, float *, float *, float *, float *, void *)
{
    return cf::fail(CF_ERR_UNSUPPORTED, "cf_infinite_attn_bwd: not built yet");
}
