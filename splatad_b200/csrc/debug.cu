// Checks that stand in for a memory checker on hosts where none can be run: a kernel that
// validates the index lists the compositing kernels are about to follow (every index they derive
// from flatten ids, tile offsets and packed ids), reporting violations through a counter instead of
// faulting. The Python layer runs it, together with canary words behind every workspace, when
// SPLATAD_DEBUG=1. No counterpart in the reference.
#include "common.cuh"

namespace splatad {

// report[0] += violations; report[1..3] = {site, index, limit} of the first one seen.
__device__ __forceinline__ void dbg_report(unsigned long long *report, unsigned site, unsigned long long index,
                                           unsigned long long limit) {
    if (atomicAdd(report, 1ull) == 0ull) {
        report[1] = site;
        report[2] = index;
        report[3] = limit;
    }
}

enum { SITE_FLATTEN_ID = 1, SITE_OFFSET_ORDER = 2, SITE_OFFSET_RANGE = 3, SITE_GAUSSIAN_ID = 4, SITE_SENSOR_ID = 5 };

__global__ void __launch_bounds__(kThreads)
validate_lists_kernel(int64_t n_isects, const int32_t *__restrict__ flatten_ids, uint64_t n_rows,
                      const int32_t *__restrict__ tile_offsets, uint32_t n_tiles, int32_t total_follows,
                      const int64_t *__restrict__ sensor_ids, const int64_t *__restrict__ gaussian_ids,
                      uint64_t n_packed, uint32_t n_sensors, uint64_t n_gaussians,
                      unsigned long long *__restrict__ report) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    const int64_t t0 = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    // the list the tiles cover ends where the offsets say it ends
    int64_t n_listed = n_isects;
    if (tile_offsets != nullptr && total_follows && n_tiles > 0) n_listed = min(n_isects, (int64_t)tile_offsets[n_tiles]);
    for (int64_t i = t0; i < n_listed; i += stride) {
        const int64_t g = flatten_ids[i];
        if (g < 0 || (uint64_t)g >= n_rows) dbg_report(report, SITE_FLATTEN_ID, (unsigned long long)g, n_rows);
    }
    if (tile_offsets != nullptr) {
        for (int64_t t = t0; t < (int64_t)n_tiles; t += stride) {
            const int64_t a = tile_offsets[t];
            const int64_t b = (t + 1 < (int64_t)n_tiles || total_follows) ? (int64_t)tile_offsets[t + 1] : n_isects;
            if (a > b) dbg_report(report, SITE_OFFSET_ORDER, (unsigned long long)t, (unsigned long long)a);
            if (a < 0 || b > n_isects) dbg_report(report, SITE_OFFSET_RANGE, (unsigned long long)t, (unsigned long long)n_isects);
        }
    }
    for (int64_t r = t0; r < (int64_t)n_packed; r += stride) {
        if (gaussian_ids != nullptr && (gaussian_ids[r] < 0 || (uint64_t)gaussian_ids[r] >= n_gaussians))
            dbg_report(report, SITE_GAUSSIAN_ID, (unsigned long long)gaussian_ids[r], n_gaussians);
        if (sensor_ids != nullptr && (sensor_ids[r] < 0 || (uint64_t)sensor_ids[r] >= n_sensors))
            dbg_report(report, SITE_SENSOR_ID, (unsigned long long)sensor_ids[r], n_sensors);
    }
}

} // namespace splatad

using namespace splatad;

extern "C" int splatad_debug_validate_lists(int64_t n_isects, const int32_t *flatten_ids, uint64_t n_rows,
                                            const int32_t *tile_offsets, uint32_t n_tiles, int32_t total_follows,
                                            const int64_t *sensor_ids, const int64_t *gaussian_ids,
                                            uint64_t n_packed, uint32_t n_sensors, uint64_t n_gaussians,
                                            uint64_t *report, void *stream) {
    SPL_REQUIRE(report != nullptr, SPLATAD_ERR_BAD_ARG, "debug_validate_lists: the report array is required");
    SPL_REQUIRE(n_isects == 0 || flatten_ids != nullptr, SPLATAD_ERR_BAD_ARG, "debug_validate_lists: null list");
    const int64_t work = max(max(n_isects, (int64_t)n_tiles), (int64_t)n_packed);
    if (work <= 0) return SPLATAD_OK;
    const uint32_t grid = (uint32_t)min((int64_t)div_up((uint64_t)work, kThreads), (int64_t)kNumSMs * 16);
    validate_lists_kernel<<<grid, kThreads, 0, (cudaStream_t)stream>>>(
        n_isects, flatten_ids, n_rows, tile_offsets, n_tiles, total_follows, sensor_ids, gaussian_ids, n_packed,
        n_sensors, n_gaussians, (unsigned long long *)report);
    return check_launch("debug_validate_lists");
}
