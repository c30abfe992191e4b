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

// Lower bound of sigma(dx, dy) = 0.5 (a dx^2 + c dy^2) + b dx dy over the box
// [dx_lo, dx_hi] x [dy_lo, dy_hi], for a positive definite conic (a, b, c): zero when the box holds
// the centre, otherwise the smallest of the four edge minima (each a clamped 1-D parabola).
__device__ __forceinline__ float sigma_min_over_box(float a, float b, float c, float dx_lo, float dx_hi,
                                                    float dy_lo, float dy_hi) {
    if (dx_lo <= 0.f && dx_hi >= 0.f && dy_lo <= 0.f && dy_hi >= 0.f) return 0.f;
    float best = 3.0e38f;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const float X = e ? dx_hi : dx_lo;            // edge dx = X: minimise over dy
        const float y = fminf(fmaxf(-b * X / c, dy_lo), dy_hi);
        best = fminf(best, 0.5f * (a * X * X + c * y * y) + b * X * y);
        const float Y = e ? dy_hi : dy_lo;            // edge dy = Y: minimise over dx
        const float x = fminf(fmaxf(-b * Y / a, dx_lo), dx_hi);
        best = fminf(best, 0.5f * (a * x * x + c * Y * Y) + b * x * Y);
    }
    return best;
}

// True when a Gaussian cannot reach alpha >= 1/255 at any sample whose offset from its (possibly
// shifted) mean lies in the given box, so that skipping it for all those samples changes nothing:
// alpha = min(0.999, opacity * exp(-sigma)) < 1/255 needs sigma > ln(255 * opacity). Decided with a
// margin far above the float32 rounding of either side; anything doubtful (a conic that is not
// positive definite, NaNs) is kept.
__device__ __forceinline__ bool never_visible_in_box(float a, float b, float c, float opacity, float dx_lo,
                                                     float dx_hi, float dy_lo, float dy_hi) {
    if (opacity * 1.0001f < kAlphaMin) return true;       // exp(-sigma) <= 1 wherever sigma >= 0
    if (!(a > 0.f && c > 0.f && a * c - b * b > 0.f)) return false;
    if (!(dx_lo <= dx_hi && dy_lo <= dy_hi)) return false;   // NaN offsets
    const float s_max = __logf(255.f * opacity) * 1.001f + 1e-3f;
    const float s_min = sigma_min_over_box(a, b, c, dx_lo, dx_hi, dy_lo, dy_hi);
    return s_min * 0.999f - 1e-3f > s_max;
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
