// Host-side plumbing shared by every entry point: error reporting, tuning knobs, device queries.
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>

#include "common.cuh"

namespace cf {

static thread_local char g_error[512] = "";
static std::atomic<double> g_floor_log2{-30.0};
static std::atomic<int> g_sorted_rows{1};
static std::atomic<int> g_chained{1};
static std::atomic<unsigned long long *> g_row_stats{nullptr};

int fail(int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return code;
}

int launch_status(const char *what)
{
    cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(CF_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
    }
    return CF_OK;
}

float weight_floor_log2()
{
    const double f = g_floor_log2.load();
    return f < -1e30 ? -1e30f : (float)f;
}

int &dense_tile_rows_choice()
{
    static thread_local int rows = 0;
    return rows;
}

bool sorted_rows_enabled() { return g_sorted_rows.load() != 0; }

bool chained_launches_enabled() { return g_chained.load() != 0; }

unsigned long long *row_stats_words() { return g_row_stats.load(); }

int sm_count()
{
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

}  // namespace cf

extern "C" {

int cf_version(void) { return 100; }

const char *cf_last_error(void) { return cf::g_error; }

void cf_set_weight_floor_log2(double log2_floor) { cf::g_floor_log2.store(log2_floor); }

double cf_get_weight_floor_log2(void) { return cf::g_floor_log2.load(); }

void cf_set_sorted_rows(int enabled) { cf::g_sorted_rows.store(enabled != 0); }

int cf_get_sorted_rows(void) { return cf::g_sorted_rows.load(); }

void cf_set_chained_launches(int enabled) { cf::g_chained.store(enabled != 0); }

void cf_set_row_stats(void *device_words) { cf::g_row_stats.store(static_cast<unsigned long long *>(device_words)); }

}  // extern "C"
