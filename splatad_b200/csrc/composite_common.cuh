// Thresholds and small helpers shared by the compositing kernels and the index kernels.
#pragma once

#include "common.cuh"

namespace splatad {

constexpr float kAlphaMax = 0.999f;
constexpr float kAlphaMin = 1.f / 255.f;
constexpr float kTStop = 1e-4f;

// Exactly fmodf((a - b + 180), 360) - 180 with the reference's final fix-up, but without the
// fmodf call whenever |a - b + 180| stays within one turn of [0, 360).
__device__ __forceinline__ float angle_difference(float a, float b) {
    const float x = a - b + 180.f;
    float r;
    if (fabsf(x) < 360.f) r = x;
    else if (x >= 360.f && x < 720.f) r = x - 360.f;
    else r = fmodf(x, 360.f);
    const float d = r - 180.f;
    return d < -180.f ? d + 360.f : d;
}

struct TileRange { int32_t start, end; };

__device__ __forceinline__ TileRange tile_range(const int32_t *__restrict__ offsets, uint32_t tile,
                                                uint32_t n_tiles_total, int64_t n_isects) {
    TileRange r;
    r.start = offsets[tile];
    // n_isects < 0: the caller's offsets carry one more entry, the total, written on the device
    r.end = (tile + 1 == n_tiles_total && n_isects >= 0) ? (int32_t)n_isects : offsets[tile + 1];
    return r;
}

} // namespace splatad
