// Front-to-back alpha compositing of the depth-sorted per-tile Gaussian lists, to camera
// pixels (rasterize_to_pixels) and to lidar points (rasterize_to_points), forward and
// backward. FP32 on the CUDA cores; there is no dense contraction in this path.
//
// One CTA per tile, one thread per pixel / lidar point. A CTA walks its tile's list in
// batches of blockDim Gaussians staged into shared memory as two float4 (+ extras for lidar),
// stops as soon as every pixel of the tile is saturated, and a warp whose 32 pixels are all
// saturated skips the batch body. The backward pass starts at the last list position any
// pixel of the tile actually consumed instead of the end of the list. The camera forward kernel
// stages only Gaussians that can reach alpha >= 1/255 somewhere in the tile (an exact, conservative
// test of the quadratic form over the tile's box of pixel centres, once per tile and Gaussian): the
// bounding rectangles behind the tile lists are loose, a quarter to a third of their entries never
// touch a pixel of the tile. The same test did not pay for lidar tiles and is not used there.
//
// Semantics follow the reference kernels
//   pixels fwd  gsplat/cuda/csrc/rasterization.cu:1360-1518     bwd 2833-3089
//   points fwd  gsplat/cuda/csrc/rasterization.cu:2021-2219     bwd 3728-4054
//   angle wrap  gsplat/cuda/csrc/utils.cuh:552-555
// Thresholds kept: alpha cap 0.999, alpha < 1/255 skipped, sigma < 0 skipped, a pixel stops
// (exclusively) when T*(1-alpha) <= 1e-4, median depth where T crosses 0.5, points with
// range <= 0 are not rendered.
#include "common.cuh"
#include "composite_common.cuh"

namespace splatad {

// Copies row g of a [*, n] float table to dst (one thread per row), zero-padded to a multiple of
// four floats: 16-byte loads when the rows are 16-byte aligned.
__device__ __forceinline__ void stage_row(float *__restrict__ dst, const float *__restrict__ table,
                                          size_t g, uint32_t n, bool vec) {
    const float *src = table + g * n;
    if (vec) {
        for (uint32_t k = 0; k < n; k += 4)
            *reinterpret_cast<float4 *>(dst + k) = __ldg(reinterpret_cast<const float4 *>(src + k));
    } else {
        const uint32_t npad = (n + 3u) & ~3u;
        for (uint32_t k = 0; k < npad; ++k) dst[k] = k < n ? __ldg(src + k) : 0.f;
    }
}

// acc[0 .. 4 * ceil(n / 4)) += row * w for a staged (zero-padded, 16-byte aligned) row: one
// 16-byte shared-memory load and one uniform test per four channels.
template <int CDIM>
__device__ __forceinline__ void axpy_staged(float (&acc)[CDIM], const float *__restrict__ row, uint32_t n,
                                            float w) {
    const float4 *r4 = reinterpret_cast<const float4 *>(row);
#pragma unroll
    for (int k4 = 0; k4 < CDIM / 4; ++k4) {
        if ((uint32_t)(4 * k4) < n) {
            const float4 v = r4[k4];
            acc[4 * k4 + 0] += v.x * w;
            acc[4 * k4 + 1] += v.y * w;
            acc[4 * k4 + 2] += v.z * w;
            acc[4 * k4 + 3] += v.w * w;
        }
    }
}

// acc += row * w over a staged row of exactly CDIM floats (zero behind the channels in use).
template <int CDIM>
__device__ __forceinline__ void axpy_staged_full(float (&acc)[CDIM], const float *__restrict__ row, float w) {
    const float4 *r4 = reinterpret_cast<const float4 *>(row);
    const float2 w2 = make_float2(w, w);
#pragma unroll
    for (int k4 = 0; k4 < CDIM / 4; ++k4) {
        const float4 v = r4[k4];
        // two channels per instruction: the packed multiply-add rounds each half like fmaf does
        const float2 lo = __ffma2_rn(make_float2(v.x, v.y), w2, make_float2(acc[4 * k4 + 0], acc[4 * k4 + 1]));
        const float2 hi = __ffma2_rn(make_float2(v.z, v.w), w2, make_float2(acc[4 * k4 + 2], acc[4 * k4 + 3]));
        acc[4 * k4 + 0] = lo.x; acc[4 * k4 + 1] = lo.y;
        acc[4 * k4 + 2] = hi.x; acc[4 * k4 + 3] = hi.y;
    }
}

// ---------------------------------------------------------------------------------------
// Camera forward. __launch_bounds__(1024): a tile may have up to 1024 pixels, and 64 registers let
// four 256-thread CTAs share an SM (with 66 the lidar kernel got three: 2.05 rounds of its 912 CTAs
// instead of 1.54).
// ---------------------------------------------------------------------------------------
template <int CDIM>
__global__ void __launch_bounds__(1024) rasterize_to_pixels_fwd_kernel(
    uint32_t C, int64_t n_isects, const float2 *__restrict__ means2d,
    const float *__restrict__ conics, const float *__restrict__ colors, uint32_t channels,
    const float *__restrict__ opacities, const float2 *__restrict__ pix_vels,
    const float *__restrict__ rs_time, const float *__restrict__ backgrounds, uint32_t W,
    uint32_t H, uint32_t tile_size, uint32_t tile_w, uint32_t tile_h,
    const int32_t *__restrict__ offsets, const int32_t *__restrict__ flatten_ids,
    float *__restrict__ render_colors, float *__restrict__ render_alphas,
    int32_t *__restrict__ last_ids, uint32_t stage_colors) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t bs = blockDim.x;
    float4 *sA = reinterpret_cast<float4 *>(smem_raw);   // x, y, vx, vy
    float4 *sB = sA + bs;                                // conic a, b, c, opacity
    int32_t *sId = reinterpret_cast<int32_t *>(sB + bs);
    uint32_t *sPos = reinterpret_cast<uint32_t *>(sId + bs);   // list position of the staged entry
    // colour rows of the batch (when they fit): the inner loop then never waits on global memory
    float *sCol = reinterpret_cast<float *>(sPos + bs);
    __shared__ uint32_t s_warp_kept[32];
    const uint32_t cpad = (channels + 3u) & ~3u;
    const bool vec = (channels % 4u == 0u) && ((reinterpret_cast<uintptr_t>(colors) & 15u) == 0u);

    const uint32_t tiles_per_cam = tile_w * tile_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t ty = tile / tile_w, tx = tile - ty * tile_w;
    const uint32_t tr = threadIdx.x;
    const uint32_t i = ty * tile_size + tr / tile_size;
    const uint32_t j = tx * tile_size + tr % tile_size;
    const bool inside = (tr < tile_size * tile_size) && (i < H && j < W);
    const float px = (float)j + 0.5f, py = (float)i + 0.5f;
    const float rs = rs_time[cam];
    const float roll = rs * ((py - 0.5f) / (float)(H - 1) - 0.5f);

    // pixel centres of this tile and the rolling-shutter offsets of its first and last row: a
    // Gaussian that cannot be seen anywhere in that box is not staged at all
    const float box_x0 = (float)(tx * tile_size) + 0.5f;
    const float box_x1 = (float)min((tx + 1) * tile_size, W) - 0.5f;
    const float box_y0 = (float)(ty * tile_size) + 0.5f;
    const float box_y1 = (float)min((ty + 1) * tile_size, H) - 0.5f;
    const float roll_a = rs * ((box_y0 - 0.5f) / (float)(H - 1) - 0.5f);
    const float roll_b = rs * ((box_y1 - 0.5f) / (float)(H - 1) - 0.5f);
    const float roll_lo = fminf(roll_a, roll_b), roll_hi = fmaxf(roll_a, roll_b);
    const uint32_t lane = tr & 31u, warp = tr >> 5, n_warps = bs >> 5;

    const TileRange range = tile_range(offsets, blockIdx.x, C * tiles_per_cam, n_isects);
    const uint32_t num_batches = (uint32_t)(range.end - range.start + bs - 1) / bs;

    bool done = !inside;
    float T = 1.f;
    uint32_t cur_idx = 0;
    float pix_out[CDIM];
#pragma unroll
    for (int k = 0; k < CDIM; ++k) pix_out[k] = 0.f;

    for (uint32_t b = 0; b < num_batches; ++b) {
        if (__syncthreads_count(done) >= (int)bs) break;
        const uint32_t batch_start = (uint32_t)range.start + bs * b;
        const uint32_t idx = batch_start + tr;
        bool keep = false;
        int32_t g = 0;
        float4 A, B;
        if (idx < (uint32_t)range.end) {
            g = flatten_ids[idx];
            const float2 xy = means2d[g];
            const float2 v = pix_vels[g];
            A = make_float4(xy.x, xy.y, v.x, v.y);
            B = make_float4(conics[3 * (size_t)g], conics[3 * (size_t)g + 1],
                            conics[3 * (size_t)g + 2], opacities[g]);
            // offsets mean - pixel over the tile; the mean moves with the row's shutter time
            const float mx_a = A.x + roll_lo * A.z, mx_b = A.x + roll_hi * A.z;
            const float my_a = A.y + roll_lo * A.w, my_b = A.y + roll_hi * A.w;
            keep = !never_visible_in_box(B.x, B.y, B.z, B.w, fminf(mx_a, mx_b) - box_x1,
                                         fmaxf(mx_a, mx_b) - box_x0, fminf(my_a, my_b) - box_y1,
                                         fmaxf(my_a, my_b) - box_y0);
        }
        // compact the survivors to the front of the staging arrays, list order kept
        const uint32_t kept_mask = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) s_warp_kept[warp] = __popc(kept_mask);
        __syncthreads();
        uint32_t pos = __popc(kept_mask & ((1u << lane) - 1u)), batch_size = 0;
        for (uint32_t w = 0; w < n_warps; ++w) {
            const uint32_t cnt = s_warp_kept[w];
            if (w < warp) pos += cnt;
            batch_size += cnt;
        }
        if (keep) {
            sA[pos] = A;
            sB[pos] = B;
            sId[pos] = g;
            sPos[pos] = idx;
            if (stage_colors) stage_row(sCol + pos * cpad, colors, (size_t)g, channels, vec);
        }
        __syncthreads();
        if (__all_sync(0xffffffffu, done)) continue;
        for (uint32_t t = 0; t < batch_size && !done; ++t) {
            const float4 A = sA[t];
            const float4 B = sB[t];
            const float dx = A.x + roll * A.z - px;
            const float dy = A.y + roll * A.w - py;
            const float sigma = 0.5f * (B.x * dx * dx + B.z * dy * dy) + B.y * dx * dy;
            const float alpha = fminf(kAlphaMax, B.w * __expf(-sigma));
            if (sigma < 0.f || alpha < kAlphaMin) continue;
            const float next_T = T * (1.f - alpha);
            if (next_T <= kTStop) { done = true; break; }
            const float vis = alpha * T;
            if (stage_colors) {
                axpy_staged<CDIM>(pix_out, sCol + t * cpad, channels, vis);
            } else {
                const float *c_ptr = colors + (size_t)sId[t] * channels;
#pragma unroll
                for (int k = 0; k < CDIM; ++k)
                    if ((uint32_t)k < channels) pix_out[k] += __ldg(c_ptr + k) * vis;
            }
            cur_idx = sPos[t];
            T = next_T;
        }
    }
    if (inside) {
        const size_t pix = ((size_t)cam * H + i) * W + j;
        render_alphas[pix] = 1.f - T;
        const float *bg = backgrounds ? backgrounds + (size_t)cam * channels : nullptr;
#pragma unroll
        for (int k = 0; k < CDIM; ++k)
            if ((uint32_t)k < channels)
                render_colors[pix * channels + k] = bg ? (pix_out[k] + T * bg[k]) : pix_out[k];
        last_ids[pix] = (int32_t)cur_idx;
    }
}

// ---------------------------------------------------------------------------------------
// Lidar forward
// ---------------------------------------------------------------------------------------
template <int CDIM>
__global__ void __launch_bounds__(1024) rasterize_to_points_fwd_kernel(
    uint32_t C, int64_t n_isects, const float2 *__restrict__ means2d,
    const float *__restrict__ conics, const float *__restrict__ colors,
    const float *__restrict__ ranges /* optional: last channel comes from here */, uint32_t channels,
    const float *__restrict__ opacities, const float *__restrict__ pix_vels /* [.,3] */,
    const float2 *__restrict__ depth_comps, const float *__restrict__ backgrounds,
    const float4 *__restrict__ raster_pts, uint32_t W, uint32_t H, uint32_t tile_width,
    uint32_t tile_height, uint32_t grid_w, uint32_t grid_h, int compute_alpha_sum,
    float alpha_sum_threshold, const int32_t *__restrict__ offsets,
    const int32_t *__restrict__ flatten_ids, uint32_t depth_idx,
    float *__restrict__ render_colors, float *__restrict__ render_alphas,
    float *__restrict__ alpha_sum_out, int32_t *__restrict__ last_ids,
    float *__restrict__ median_depths, uint32_t stage_features) {
    chain_enter();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t bs = blockDim.x;
    float4 *sA = reinterpret_cast<float4 *>(smem_raw);   // az, el, v_az, v_el
    float4 *sB = sA + bs;                                // conic a, b, c, opacity
    float4 *sC = sB + bs;                                // v_range, dc.x, dc.y, range (depth channel)
    int32_t *sId = reinterpret_cast<int32_t *>(sC + bs);
    // feature rows of the batch (when they fit): the inner loop then never waits on global memory
    float *sFeat = reinterpret_cast<float *>(sId + bs);

    const uint32_t tiles_per_cam = grid_w * grid_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t ty = tile / grid_w, tx = tile - ty * grid_w;
    const uint32_t tr = threadIdx.x;
    const uint32_t i = ty * tile_height + tr / tile_width;
    const uint32_t j = tx * tile_width + tr % tile_width;
    const bool in_image = (tr < tile_width * tile_height) && (i < H && j < W);
    bool inside = in_image;
    const size_t pix = ((size_t)cam * H + i) * W + j;
    float px = 0.f, py = 0.f, pz = 0.f, roll = 0.f;
    if (inside) {
        const float4 rp = raster_pts[pix];
        px = rp.x; py = rp.y; pz = rp.z; roll = rp.w;
        if (pz <= 0.f) inside = false;
    }

    const TileRange range = tile_range(offsets, blockIdx.x, C * tiles_per_cam, n_isects);
    const uint32_t num_batches = (uint32_t)(range.end - range.start + bs - 1) / bs;

    // with a separate range array the feature rows hold channels - 1 columns
    const uint32_t fstride = ranges ? channels - 1 : channels;
    // a staged row holds all CDIM accumulated channels: the features, behind them the range when it
    // comes from its own array, then zeros, so that one unconditional multiply-add pass covers them
    constexpr uint32_t fpad = (uint32_t)CDIM;
    const bool vec = (fstride % 4u == 0u) && ((reinterpret_cast<uintptr_t>(colors) & 15u) == 0u);
    bool done = !inside;
    float T = 1.f;
    uint32_t cur_idx = 0;
    float depth_extra = 0.f, alpha_sum = 0.f, median = 0.f;
    float pix_out[CDIM];
#pragma unroll
    for (int k = 0; k < CDIM; ++k) pix_out[k] = 0.f;

    for (uint32_t b = 0; b < num_batches; ++b) {
        if (__syncthreads_count(done) >= (int)bs) break;
        const uint32_t batch_start = (uint32_t)range.start + bs * b;
        const uint32_t idx = batch_start + tr;
        if (idx < (uint32_t)range.end) {
            const int32_t g = flatten_ids[idx];
            const float2 xy = means2d[g];
            const float *v = pix_vels + 3 * (size_t)g;
            const float2 dc = depth_comps[g];
            sA[tr] = make_float4(xy.x, xy.y, v[0], v[1]);
            sB[tr] = make_float4(conics[3 * (size_t)g], conics[3 * (size_t)g + 1],
                                 conics[3 * (size_t)g + 2], opacities[g]);
            const float range = ranges ? ranges[g] : colors[(size_t)g * channels + depth_idx];
            sC[tr] = make_float4(v[2], dc.x, dc.y, range);
            sId[tr] = g;
            if (stage_features) {
                float *row = sFeat + tr * fpad;
                uint32_t filled = 0;
                if (fstride) {
                    stage_row(row, colors, (size_t)g, fstride, vec);
                    filled = (fstride + 3u) & ~3u;
                }
                if (ranges) {
                    row[fstride] = range;
                    filled = max(filled, fstride + 1u);
                }
                for (uint32_t k = filled; k < fpad; ++k) row[k] = 0.f;
            }
        }
        __syncthreads();
        if (__all_sync(0xffffffffu, done)) continue;
        const uint32_t batch_size = min(bs, (uint32_t)range.end - batch_start);
        for (uint32_t t = 0; t < batch_size && !done; ++t) {
            const float4 A = sA[t];
            const float4 B = sB[t];
            const float dx = angle_difference(A.x + roll * A.z, px);
            const float dy = angle_difference(A.y + roll * A.w, py);
            const float sigma = 0.5f * (B.x * dx * dx + B.z * dy * dy) + B.y * dx * dy;
            const float alpha = fminf(kAlphaMax, B.w * __expf(-sigma));
            if (sigma < 0.f || alpha < kAlphaMin) continue;
            const float next_T = T * (1.f - alpha);
            if (next_T <= kTStop) { done = true; break; }
            const float vis = alpha * T;
            const float4 Cc = sC[t];
            if (stage_features) {
                // the zero padding of a staged row adds nothing to the channels behind it
                axpy_staged_full<CDIM>(pix_out, sFeat + t * fpad, vis);
            } else {
                const float *c_ptr = colors + (size_t)sId[t] * fstride;
#pragma unroll
                for (int k = 0; k < CDIM; ++k) {
                    if ((uint32_t)k < fstride) pix_out[k] += __ldg(c_ptr + k) * vis;
                    else if ((uint32_t)k < channels) pix_out[k] += Cc.w * vis;
                }
            }
            const float dterm = Cc.y * dx + Cc.z * dy + Cc.x * roll;
            depth_extra += dterm * vis;
            if (T > 0.5f && next_T <= 0.5f) median = Cc.w + dterm;
            if (compute_alpha_sum && Cc.w < (pz - alpha_sum_threshold)) alpha_sum += alpha;
            cur_idx = batch_start + t;
            T = next_T;
        }
    }
    if (in_image) {
        // points that are not rendered (range <= 0) produce zeros everywhere
        render_alphas[pix] = inside ? 1.f - T : 0.f;
        const float *bg = backgrounds ? backgrounds + (size_t)cam * channels : nullptr;
#pragma unroll
        for (int k = 0; k < CDIM; ++k)
            if ((uint32_t)k < channels) {
                float v = pix_out[k];
                if ((uint32_t)k == depth_idx) v += depth_extra;
                if (bg) v += T * bg[k];
                render_colors[pix * channels + k] = inside ? v : 0.f;
            }
        last_ids[pix] = inside ? (int32_t)cur_idx : 0;
        median_depths[pix] = inside ? median : 0.f;
        if (alpha_sum_out != nullptr) alpha_sum_out[pix] = inside ? alpha_sum : 0.f;
    }
}

// ---------------------------------------------------------------------------------------
// Backward helpers
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// Sums kSlots (a power of two <= 32) per-lane values over the warp at once: every step halves the
// number of values a lane carries and swaps the other half with the partner lane, kSlots - 1
// shuffles in all (plus one per remaining lane bit) where one butterfly per value takes 5 * kSlots.
// Returns, on lane l, the warp total of value (l * kSlots) / 32; lanes that share an index return
// the same total. v is destroyed.
template <int kSlots>
__device__ __forceinline__ float warp_sum_slots(float (&v)[kSlots], uint32_t lane) {
    int off = 16;
#pragma unroll
    for (int half = kSlots / 2; half >= 1; half >>= 1) {
        const bool upper = (lane & (uint32_t)off) != 0u;
#pragma unroll
        for (int i = 0; i < half; ++i) {
            const float send = upper ? v[i] : v[i + half];
            const float keep = upper ? v[i + half] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
        off >>= 1;
    }
    float r = v[0];
#pragma unroll
    for (; off >= 1; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
    return r;
}

constexpr int pow2_at_least(int n) { return n <= 1 ? 1 : 2 * pow2_at_least((n + 1) / 2); }

__device__ __forceinline__ int block_max_int(int v, int *red /* [32] */) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, off));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    int m = red[0];
    for (uint32_t w = 1; w < (blockDim.x + 31) / 32; ++w) m = max(m, red[w]);
    __syncthreads();
    return m;
}

// ---------------------------------------------------------------------------------------
// Camera backward
// ---------------------------------------------------------------------------------------
template <int CDIM>
__global__ void rasterize_to_pixels_bwd_kernel(
    uint32_t C, int64_t n_isects, const float2 *__restrict__ means2d,
    const float *__restrict__ conics, const float *__restrict__ colors, uint32_t channels,
    const float *__restrict__ opacities, const float2 *__restrict__ pix_vels,
    const float *__restrict__ rs_time, const float *__restrict__ backgrounds, uint32_t W,
    uint32_t H, uint32_t tile_size, uint32_t tile_w, uint32_t tile_h,
    const int32_t *__restrict__ offsets, const int32_t *__restrict__ flatten_ids,
    const float *__restrict__ render_alphas, const int32_t *__restrict__ last_ids,
    const float *__restrict__ v_render_colors, const float *__restrict__ v_render_alphas,
    float *__restrict__ v_means2d_abs, float *__restrict__ v_means2d,
    float *__restrict__ v_conics, float *__restrict__ v_colors, float *__restrict__ v_opacities,
    float *__restrict__ v_pix_vels) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int red[32];
    const uint32_t bs = blockDim.x;
    float4 *sA = reinterpret_cast<float4 *>(smem_raw);
    float4 *sB = sA + bs;
    int32_t *sId = reinterpret_cast<int32_t *>(sB + bs);
    int32_t *sPos = sId + bs;                            // list position of the staged entry
    float *sRgb = reinterpret_cast<float *>(sPos + bs);  // [bs * CDIM]
    __shared__ uint32_t s_warp_kept[32];

    const uint32_t tiles_per_cam = tile_w * tile_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t ty = tile / tile_w, tx = tile - ty * tile_w;
    const uint32_t tr = threadIdx.x;
    const uint32_t i = ty * tile_size + tr / tile_size;
    const uint32_t j = tx * tile_size + tr % tile_size;
    const bool inside = (tr < tile_size * tile_size) && (i < H && j < W);
    const float px = (float)j + 0.5f, py = (float)i + 0.5f;
    const float rs = rs_time[cam];
    const float roll = rs * ((py - 0.5f) / (float)(H - 1) - 0.5f);
    const size_t pix = ((size_t)cam * H + min(i, H - 1)) * W + min(j, W - 1);
    // box of the tile's pixel centres and the shutter offsets of its first and last row, as in the
    // forward kernel: entries that cannot be seen anywhere in the tile are not staged
    const float box_x0 = (float)(tx * tile_size) + 0.5f;
    const float box_x1 = (float)min((tx + 1) * tile_size, W) - 0.5f;
    const float box_y0 = (float)(ty * tile_size) + 0.5f;
    const float box_y1 = (float)min((ty + 1) * tile_size, H) - 0.5f;
    const float roll_a = rs * ((box_y0 - 0.5f) / (float)(H - 1) - 0.5f);
    const float roll_b = rs * ((box_y1 - 0.5f) / (float)(H - 1) - 0.5f);
    const float roll_lo = fminf(roll_a, roll_b), roll_hi = fmaxf(roll_a, roll_b);

    const TileRange range = tile_range(offsets, blockIdx.x, C * tiles_per_cam, n_isects);
    const bool vec = (channels % 4u == 0u) && ((reinterpret_cast<uintptr_t>(colors) & 15u) == 0u);

    const float T_final = 1.f - render_alphas[pix];
    float T = T_final;
    const int32_t bin_final = inside ? last_ids[pix] : 0;
    float buffer[CDIM], v_render_c[CDIM];
    float bg_dot = 0.f;
#pragma unroll
    for (int k = 0; k < CDIM; ++k) {
        buffer[k] = 0.f;
        v_render_c[k] = ((uint32_t)k < channels && inside) ? v_render_colors[pix * channels + k] : 0.f;
        if (backgrounds != nullptr && (uint32_t)k < channels)
            bg_dot += backgrounds[(size_t)cam * channels + k] * v_render_c[k];
    }
    const float v_render_a = inside ? v_render_alphas[pix] : 0.f;

    // last list position consumed by any pixel of this tile
    const int32_t tile_last = block_max_int(bin_final, red);
    int32_t warp_bin_final = bin_final;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        warp_bin_final = max(warp_bin_final, __shfl_xor_sync(0xffffffffu, warp_bin_final, off));
    const int32_t eff_end = min(range.end, tile_last + 1);
    if (eff_end <= range.start) return;
    const uint32_t num_batches = (uint32_t)(eff_end - range.start + bs - 1) / bs;
    const uint32_t lane = tr & 31, warp = tr >> 5, n_warps = bs >> 5;

    for (uint32_t b = 0; b < num_batches; ++b) {
        __syncthreads();
        const int32_t batch_end = eff_end - 1 - (int32_t)(bs * b);
        const int32_t idx = batch_end - (int32_t)tr;
        bool keep = false;
        int32_t g = 0;
        float4 A, B0;
        if (idx >= range.start) {
            g = flatten_ids[idx];
            const float2 xy = means2d[g];
            const float2 v = pix_vels[g];
            A = make_float4(xy.x, xy.y, v.x, v.y);
            B0 = make_float4(conics[3 * (size_t)g], conics[3 * (size_t)g + 1],
                             conics[3 * (size_t)g + 2], opacities[g]);
            const float mx_a = A.x + roll_lo * A.z, mx_b = A.x + roll_hi * A.z;
            const float my_a = A.y + roll_lo * A.w, my_b = A.y + roll_hi * A.w;
            keep = !never_visible_in_box(B0.x, B0.y, B0.z, B0.w, fminf(mx_a, mx_b) - box_x1,
                                         fmaxf(mx_a, mx_b) - box_x0, fminf(my_a, my_b) - box_y1,
                                         fmaxf(my_a, my_b) - box_y0);
        }
        // survivors to the front, still back to front in list order
        const uint32_t kept_mask = __ballot_sync(0xffffffffu, keep);
        if (lane == 0) s_warp_kept[warp] = __popc(kept_mask);
        __syncthreads();
        uint32_t pos = __popc(kept_mask & ((1u << lane) - 1u)), n_kept = 0;
        for (uint32_t w = 0; w < n_warps; ++w) {
            const uint32_t cnt = s_warp_kept[w];
            if (w < warp) pos += cnt;
            n_kept += cnt;
        }
        if (keep) {
            sA[pos] = A;
            sB[pos] = B0;
            sId[pos] = g;
            sPos[pos] = idx;
            // rows of CDIM floats (channels, then zeros): the channel loops run in packed pairs
            float *row = sRgb + pos * CDIM;
            stage_row(row, colors, (size_t)g, channels, vec);
            for (uint32_t k = (channels + 3u) & ~3u; k < (uint32_t)CDIM; ++k) row[k] = 0.f;
        }
        __syncthreads();
        for (uint32_t t = 0; t < n_kept; ++t) {
            const int32_t entry = sPos[t];
            if (entry > warp_bin_final) continue;   // behind everything this warp consumed
            bool valid = inside && (entry <= bin_final);
            float alpha = 0.f, opac = 0.f, vis = 0.f, dx = 0.f, dy = 0.f;
            float4 B = make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid) {
                const float4 A = sA[t];
                B = sB[t];
                opac = B.w;
                dx = A.x + roll * A.z - px;
                dy = A.y + roll * A.w - py;
                const float sigma = 0.5f * (B.x * dx * dx + B.z * dy * dy) + B.y * dx * dy;
                vis = __expf(-sigma);
                alpha = fminf(kAlphaMax, opac * vis);
                if (sigma < 0.f || alpha < kAlphaMin) valid = false;
            }
            if (!__any_sync(0xffffffffu, valid)) continue;
            float v_rgb[CDIM];
#pragma unroll
            for (int k = 0; k < CDIM; ++k) v_rgb[k] = 0.f;
            float v_conic_x = 0.f, v_conic_y = 0.f, v_conic_z = 0.f;
            float v_x = 0.f, v_y = 0.f, v_ax = 0.f, v_ay = 0.f, v_vx = 0.f, v_vy = 0.f, v_o = 0.f;
            if (valid) {
                const float ra = 1.f / (1.f - alpha);
                T *= ra;
                const float fac = alpha * T;
                // two channels per instruction (packed FP32 multiply-adds); channels beyond the
                // rendered ones have zero rows, zero cotangents and zero buffers
                const float *rgb = sRgb + (uint32_t)t * CDIM;
                const float2 fac2 = make_float2(fac, fac), T2 = make_float2(T, T), nra2 = make_float2(-ra, -ra);
                float2 va2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int k = 0; k < CDIM; k += 4) {
                    const float4 c4 = *reinterpret_cast<const float4 *>(rgb + k);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int q = k + 2 * h;
                        const float2 c2 = h ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y);
                        const float2 vr2 = make_float2(v_render_c[q], v_render_c[q + 1]);
                        const float2 b2 = make_float2(buffer[q], buffer[q + 1]);
                        const float2 g2 = __fmul2_rn(fac2, vr2);
                        v_rgb[q] = g2.x; v_rgb[q + 1] = g2.y;
                        const float2 u2 = __ffma2_rn(c2, T2, __fmul2_rn(b2, nra2));   // rgb T - buffer ra
                        va2 = __ffma2_rn(u2, vr2, va2);
                        const float2 nb2 = __ffma2_rn(c2, fac2, b2);
                        buffer[q] = nb2.x; buffer[q + 1] = nb2.y;
                    }
                }
                float v_alpha = va2.x + va2.y;
                v_alpha += T_final * ra * v_render_a;
                if (backgrounds != nullptr) v_alpha += -T_final * ra * bg_dot;
                if (opac * vis <= kAlphaMax) {
                    const float v_sigma = -opac * vis * v_alpha;
                    v_conic_x = 0.5f * v_sigma * dx * dx;
                    v_conic_y = v_sigma * dx * dy;
                    v_conic_z = 0.5f * v_sigma * dy * dy;
                    v_x = v_sigma * (B.x * dx + B.y * dy);
                    v_y = v_sigma * (B.y * dx + B.z * dy);
                    v_vx = v_x * roll;
                    v_vy = v_y * roll;
                    v_ax = fabsf(v_x);
                    v_ay = fabsf(v_y);
                    v_o = vis * v_alpha;
                }
            }
            // warp totals by multi-value butterflies; each total then sits on its own lane, which adds it in
            const size_t g = (size_t)sId[t];
            float g_tot;
            uint32_t gi;   // index of the geometry gradient this lane ends up holding
            if (CDIM + 10 <= 16) {
                // up to 6 channels: colours and geometry share one 16-value butterfly
                float gs[16] = {v_conic_x, v_conic_y, v_conic_z, v_x, v_y, v_vx, v_vy, v_o, v_ax, v_ay,
                                0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int k = 0; k < CDIM && k < 6; ++k) gs[10 + k] = v_rgb[k];
                g_tot = warp_sum_slots<16>(gs, lane);
                gi = lane >> 1;
                if ((lane & 1u) == 0u && gi >= 10u && gi - 10u < channels)
                    atomicAdd(v_colors + g * channels + (gi - 10u), g_tot);
            } else {
                constexpr int kColorSlots = pow2_at_least(CDIM);
                float cs[kColorSlots];
#pragma unroll
                for (int k = 0; k < kColorSlots; ++k) cs[k] = k < CDIM ? v_rgb[k] : 0.f;
                float gs[16] = {v_conic_x, v_conic_y, v_conic_z, v_x, v_y, v_vx, v_vy, v_o, v_ax, v_ay,
                                0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
                const float c_tot = warp_sum_slots<kColorSlots>(cs, lane);
                g_tot = warp_sum_slots<16>(gs, lane);
                gi = lane >> 1;
                const uint32_t ci = (lane * (uint32_t)kColorSlots) >> 5;
                if ((lane & (32u / kColorSlots - 1u)) == 0u && ci < channels)
                    atomicAdd(v_colors + g * channels + ci, c_tot);
            }
            float *dst = nullptr;
            if (gi < 3u) dst = v_conics + 3 * g + gi;
            else if (gi < 5u) dst = v_means2d + 2 * g + (gi - 3u);
            else if (gi < 7u) dst = v_pix_vels + 2 * g + (gi - 5u);
            else if (gi == 7u) dst = v_opacities + g;
            else if (gi < 10u && v_means2d_abs != nullptr) dst = v_means2d_abs + 2 * g + (gi - 8u);
            if ((lane & 1u) == 0u && dst != nullptr) atomicAdd(dst, g_tot);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Lidar backward
// ---------------------------------------------------------------------------------------
template <int CDIM>
__global__ void rasterize_to_points_bwd_kernel(
    uint32_t C, int64_t n_isects, const float2 *__restrict__ means2d,
    const float *__restrict__ conics, const float *__restrict__ colors,
    const float *__restrict__ ranges, uint32_t channels,
    const float *__restrict__ opacities, const float *__restrict__ pix_vels,
    const float2 *__restrict__ depth_comps, const float *__restrict__ backgrounds,
    const float4 *__restrict__ raster_pts, uint32_t W, uint32_t H, uint32_t tile_width,
    uint32_t tile_height, uint32_t grid_w, uint32_t grid_h, int compute_alpha_sum,
    float alpha_sum_threshold, const int32_t *__restrict__ offsets,
    const int32_t *__restrict__ flatten_ids, uint32_t depth_idx,
    const float *__restrict__ render_alphas, const int32_t *__restrict__ last_ids,
    const float *__restrict__ v_render_colors, const float *__restrict__ v_render_alphas,
    const float *__restrict__ v_alpha_sum, float *__restrict__ v_means2d_abs,
    float *__restrict__ v_means2d, float *__restrict__ v_conics, float *__restrict__ v_colors,
    float *__restrict__ v_opacities, float *__restrict__ v_pix_vels,
    float *__restrict__ v_depth_comps, float *__restrict__ v_ranges) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int red[32];
    const uint32_t bs = blockDim.x;
    float4 *sA = reinterpret_cast<float4 *>(smem_raw);
    float4 *sB = sA + bs;
    float4 *sC = sB + bs;   // v_range, dc.x, dc.y, unused
    int32_t *sId = reinterpret_cast<int32_t *>(sC + bs);
    float *sRgb = reinterpret_cast<float *>(sId + bs);

    const uint32_t tiles_per_cam = grid_w * grid_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t ty = tile / grid_w, tx = tile - ty * grid_w;
    const uint32_t tr = threadIdx.x;
    const uint32_t i = ty * tile_height + tr / tile_width;
    const uint32_t j = tx * tile_width + tr % tile_width;
    bool inside = (tr < tile_width * tile_height) && (i < H && j < W);
    const size_t pix = ((size_t)cam * H + min(i, H - 1)) * W + min(j, W - 1);
    float px = 0.f, py = 0.f, pz = 0.f, roll = 0.f;
    if (inside) {
        const float4 rp = raster_pts[pix];
        px = rp.x; py = rp.y; pz = rp.z; roll = rp.w;
        if (pz <= 0.f) inside = false;
    }

    const TileRange range = tile_range(offsets, blockIdx.x, C * tiles_per_cam, n_isects);

    const uint32_t fstride = ranges ? channels - 1 : channels;
    const bool vec = (fstride % 4u == 0u) && ((reinterpret_cast<uintptr_t>(colors) & 15u) == 0u);
    const float T_final = 1.f - render_alphas[pix];
    float T = T_final;
    const int32_t bin_final = inside ? last_ids[pix] : 0;
    float buffer[CDIM], v_render_c[CDIM];
    float buffer_extra = 0.f;   // depth-compensation part of the depth channel's buffer
    float bg_dot = 0.f, v_depth_c = 0.f;
#pragma unroll
    for (int k = 0; k < CDIM; ++k) {
        buffer[k] = 0.f;
        v_render_c[k] = ((uint32_t)k < channels && inside) ? v_render_colors[pix * channels + k] : 0.f;
        if ((uint32_t)k == depth_idx) v_depth_c = v_render_c[k];
        if (backgrounds != nullptr && (uint32_t)k < channels)
            bg_dot += backgrounds[(size_t)cam * channels + k] * v_render_c[k];
    }
    const float v_render_a = inside ? v_render_alphas[pix] : 0.f;
    const float v_asum = (inside && v_alpha_sum != nullptr) ? v_alpha_sum[pix] : 0.f;

    const int32_t tile_last = block_max_int(bin_final, red);
    int32_t warp_bin_final = bin_final;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1)
        warp_bin_final = max(warp_bin_final, __shfl_xor_sync(0xffffffffu, warp_bin_final, off));
    const int32_t eff_end = min(range.end, tile_last + 1);
    if (eff_end <= range.start) return;
    const uint32_t num_batches = (uint32_t)(eff_end - range.start + bs - 1) / bs;
    const uint32_t lane = tr & 31;

    for (uint32_t b = 0; b < num_batches; ++b) {
        __syncthreads();
        const int32_t batch_end = eff_end - 1 - (int32_t)(bs * b);
        const int32_t batch_size = min((int32_t)bs, batch_end + 1 - range.start);
        const int32_t idx = batch_end - (int32_t)tr;
        if (idx >= range.start) {
            const int32_t g = flatten_ids[idx];
            const float2 xy = means2d[g];
            const float *v = pix_vels + 3 * (size_t)g;
            const float2 dc = depth_comps[g];
            sA[tr] = make_float4(xy.x, xy.y, v[0], v[1]);
            sB[tr] = make_float4(conics[3 * (size_t)g], conics[3 * (size_t)g + 1],
                                 conics[3 * (size_t)g + 2], opacities[g]);
            sC[tr] = make_float4(v[2], dc.x, dc.y, 0.f);
            sId[tr] = g;
            // rows of CDIM floats: the channels, then zeros, so that the channel loops below run in
            // packed pairs without tests
            float *row = sRgb + tr * CDIM;
            uint32_t filled = 0;
            if (fstride) {
                stage_row(row, colors, (size_t)g, fstride, vec);
                filled = (fstride + 3u) & ~3u;
            }
            if (ranges) {
                row[fstride] = ranges[g];
                filled = max(filled, fstride + 1u);
            }
            for (uint32_t k = filled; k < (uint32_t)CDIM; ++k) row[k] = 0.f;
        }
        __syncthreads();
        for (int32_t t = max(0, batch_end - warp_bin_final); t < batch_size; ++t) {
            bool valid = inside && (batch_end - t <= bin_final);
            float alpha = 0.f, opac = 0.f, vis = 0.f, dx = 0.f, dy = 0.f;
            float4 B = make_float4(0.f, 0.f, 0.f, 0.f), Cc = make_float4(0.f, 0.f, 0.f, 0.f);
            if (valid) {
                const float4 A = sA[t];
                B = sB[t];
                Cc = sC[t];
                opac = B.w;
                dx = angle_difference(A.x + roll * A.z, px);
                dy = angle_difference(A.y + roll * A.w, py);
                const float sigma = 0.5f * (B.x * dx * dx + B.z * dy * dy) + B.y * dx * dy;
                vis = __expf(-sigma);
                alpha = fminf(kAlphaMax, opac * vis);
                if (sigma < 0.f || alpha < kAlphaMin) valid = false;
            }
            if (!__any_sync(0xffffffffu, valid)) continue;
            float v_rgb[CDIM];
#pragma unroll
            for (int k = 0; k < CDIM; ++k) v_rgb[k] = 0.f;
            float v_conic_x = 0.f, v_conic_y = 0.f, v_conic_z = 0.f;
            float v_x = 0.f, v_y = 0.f, v_ax = 0.f, v_ay = 0.f, v_o = 0.f;
            float v_vx = 0.f, v_vy = 0.f, v_vz = 0.f, v_dcx = 0.f, v_dcy = 0.f;
            if (valid) {
                const float ra = 1.f / (1.f - alpha);
                T *= ra;
                const float fac = alpha * T;
                const float dterm = Cc.y * dx + Cc.z * dy + Cc.x * roll;
                // two channels per instruction (packed FP32 multiply-adds); channels beyond the
                // rendered ones have zero rows, zero cotangents and zero buffers
                const float *rgb = sRgb + (uint32_t)t * CDIM;
                const float2 fac2 = make_float2(fac, fac), T2 = make_float2(T, T), nra2 = make_float2(-ra, -ra);
                float2 va2 = make_float2(0.f, 0.f);
#pragma unroll
                for (int k = 0; k < CDIM; k += 4) {
                    const float4 c4 = *reinterpret_cast<const float4 *>(rgb + k);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int q = k + 2 * h;
                        const float2 c2 = h ? make_float2(c4.z, c4.w) : make_float2(c4.x, c4.y);
                        const float2 vr2 = make_float2(v_render_c[q], v_render_c[q + 1]);
                        const float2 b2 = make_float2(buffer[q], buffer[q + 1]);
                        const float2 g2 = __fmul2_rn(fac2, vr2);
                        v_rgb[q] = g2.x; v_rgb[q + 1] = g2.y;
                        const float2 u2 = __ffma2_rn(c2, T2, __fmul2_rn(b2, nra2));   // rgb T - buffer ra
                        va2 = __ffma2_rn(u2, vr2, va2);
                        const float2 nb2 = __ffma2_rn(c2, fac2, b2);
                        buffer[q] = nb2.x; buffer[q + 1] = nb2.y;
                    }
                }
                float v_alpha = va2.x + va2.y;
                v_alpha -= buffer_extra * ra * v_depth_c;   // the depth channel's buffer also holds the compensation terms
                const float v_rgb_depth = fac * v_depth_c;
                v_alpha += dterm * T * v_depth_c;
                v_alpha += T_final * ra * v_render_a;
                if (backgrounds != nullptr) v_alpha += -T_final * ra * bg_dot;
                if (opac * vis <= kAlphaMax) {
                    v_dcx = v_rgb_depth * dx;
                    v_dcy = v_rgb_depth * dy;
                    v_vz = v_rgb_depth * roll;
                    const float v_sigma = -opac * vis * v_alpha;
                    v_conic_x = 0.5f * v_sigma * dx * dx;
                    v_conic_y = v_sigma * dx * dy;
                    v_conic_z = 0.5f * v_sigma * dy * dy;
                    v_x = v_sigma * (B.x * dx + B.y * dy) + v_rgb_depth * Cc.y;
                    v_y = v_sigma * (B.y * dx + B.z * dy) + v_rgb_depth * Cc.z;
                    v_vx = v_x * roll;
                    v_vy = v_y * roll;
                    v_ax = fabsf(v_x);
                    v_ay = fabsf(v_y);
                    v_o = vis * v_alpha;
                }
                buffer_extra += dterm * fac;

                const float g_depth = rgb[depth_idx];
                if (compute_alpha_sum && g_depth < (pz - alpha_sum_threshold)) {
                    const float vs = v_asum * -opac * vis;
                    const float ux = vs * (B.x * dx + B.y * dy);
                    const float uy = vs * (B.y * dx + B.z * dy);
                    v_x += ux; v_y += uy;
                    v_vx += ux * roll; v_vy += uy * roll;
                    v_ax += fabsf(ux); v_ay += fabsf(uy);
                    v_conic_x += vs * 0.5f * dx * dx;
                    v_conic_y += vs * dx * dy;
                    v_conic_z += vs * 0.5f * dy * dy;
                    v_o += v_asum * vis;
                }
            }
            // warp totals: the feature gradients in one multi-value butterfly, the thirteen geometry
            // gradients in another; each total then sits on its own lane, which adds it in
            constexpr int kColorSlots = pow2_at_least(CDIM);
            float cs[kColorSlots];
#pragma unroll
            for (int k = 0; k < kColorSlots; ++k) cs[k] = k < CDIM ? v_rgb[k] : 0.f;
            float gs[16] = {v_conic_x, v_conic_y, v_conic_z, v_x, v_y, v_vx, v_vy, v_vz, v_dcx, v_dcy,
                            v_o, v_ax, v_ay, 0.f, 0.f, 0.f};
            const float c_tot = warp_sum_slots<kColorSlots>(cs, lane);
            const float g_tot = warp_sum_slots<16>(gs, lane);
            const size_t g = (size_t)sId[t];
            const uint32_t ci = (lane * (uint32_t)kColorSlots) >> 5;
            if ((lane & (32u / kColorSlots - 1u)) == 0u) {
                if (ci < fstride) atomicAdd(v_colors + g * fstride + ci, c_tot);
                else if (ci < channels) atomicAdd(v_ranges + g, c_tot);
            }
            const uint32_t gi = lane >> 1;
            float *dst = nullptr;
            if (gi < 3u) dst = v_conics + 3 * g + gi;
            else if (gi < 5u) dst = v_means2d + 2 * g + (gi - 3u);
            else if (gi < 8u) dst = v_pix_vels + 3 * g + (gi - 5u);
            else if (gi < 10u) dst = v_depth_comps + 2 * g + (gi - 8u);
            else if (gi == 10u) dst = v_opacities + g;
            else if (gi < 13u && v_means2d_abs != nullptr) dst = v_means2d_abs + 2 * g + (gi - 11u);
            if ((lane & 1u) == 0u && dst != nullptr) atomicAdd(dst, g_tot);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Dispatch on the channel count
// ---------------------------------------------------------------------------------------
#define SPL_DISPATCH_CDIM(channels, CALL)                                                        \
    do {                                                                                         \
        if ((channels) <= 4) { CALL(4); }                                                        \
        else if ((channels) <= 8) { CALL(8); }                                                   \
        else if ((channels) <= 16) { CALL(16); }                                                 \
        else if ((channels) <= 20) { CALL(20); }                                                 \
        else { CALL(32); }                                                                       \
    } while (0)

// A tile may have up to 1024 samples, one thread each; the backward kernels with many channels
// need more registers per thread than a block of that size can have. Said here, with the numbers,
// rather than by a failed launch.
template <typename K>
static int check_block_size(K kernel, uint32_t threads, uint32_t channels, const char *what) {
    if (threads <= 256) return SPLATAD_OK;
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kernel) != cudaSuccess) return check_launch(what);
    SPL_REQUIRE((uint32_t)fa.maxThreadsPerBlock >= threads, SPLATAD_ERR_BAD_ARG,
                "%s: a tile of %u samples with %u channels needs blocks of %u threads, this kernel runs at "
                "most %d (%d registers per thread): use a smaller tile or fewer channels per call",
                what, threads, channels, threads, fa.maxThreadsPerBlock, fa.numRegs);
    return SPLATAD_OK;
}

template <typename K>
static int set_smem(K kernel, size_t bytes, const char *what) {
    if (bytes > 32 * 1024) {   // the 48 KB default also has to hold the kernels' static shared memory
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            set_last_error("%s: cannot reserve %zu bytes of shared memory: %s", what, bytes,
                           cudaGetErrorString(e));
            return SPLATAD_ERR_CUDA;
        }
    }
    return SPLATAD_OK;
}

} // namespace splatad

using namespace splatad;

extern "C" int splatad_rasterize_to_pixels_fwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics, const float *colors,
    uint32_t channels, const float *opacities, const float *pix_vels,
    const float *rolling_shutter_time, const float *backgrounds, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, float *render_colors,
    float *render_alphas, int32_t *last_ids, void *stream) {
    SPL_REQUIRE(channels >= 1 && channels <= SPLATAD_MAX_CHANNELS, SPLATAD_ERR_CHANNELS,
                "rasterize_to_pixels_fwd: unsupported channel count %u (1..%d)", channels,
                SPLATAD_MAX_CHANNELS);
    SPL_REQUIRE(tile_size >= 1 && tile_size * tile_size <= 1024, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_pixels_fwd: tile_size^2 must be <= 1024");
    SPL_REQUIRE(render_colors && render_alphas && last_ids && tile_offsets && rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_pixels_fwd: null argument");
    SPL_REQUIRE(n_isects == 0 || (means2d && conics && colors && opacities && pix_vels && flatten_ids),
                SPLATAD_ERR_BAD_ARG, "rasterize_to_pixels_fwd: null input");
    const uint32_t blocks = C * tile_width * tile_height;
    if (blocks == 0 || image_width == 0 || image_height == 0) return SPLATAD_OK;
    const uint32_t bs = ((tile_size * tile_size + 31) / 32) * 32;   // whole warps
    size_t smem = (size_t)bs * (2 * sizeof(float4) + 2 * sizeof(int32_t));
    // the batch's colour rows ride along in shared memory while a block stays under 64 KB
    const size_t smem_colors = (size_t)bs * ((channels + 3u) & ~3u) * sizeof(float);
    const uint32_t stage_colors = (smem + smem_colors <= 64 * 1024) ? 1u : 0u;
    if (stage_colors) smem += smem_colors;
#define CALL(D)                                                                                   \
    {                                                                                             \
        int rc = set_smem(rasterize_to_pixels_fwd_kernel<D>, smem, "rasterize_to_pixels_fwd");    \
        if (rc != SPLATAD_OK) return rc;                                                          \
        launch_chained(rasterize_to_pixels_fwd_kernel<D>, blocks, bs, smem, (cudaStream_t)stream, \
            C, n_isects, (const float2 *)means2d, conics, colors, channels, opacities,            \
            (const float2 *)pix_vels, rolling_shutter_time, backgrounds, image_width,             \
            image_height, tile_size, tile_width, tile_height, tile_offsets, flatten_ids,          \
            render_colors, render_alphas, last_ids, stage_colors);                                \
    }
    {
        SPL_PROF("rasterize_to_pixels_fwd_kernel", (cudaStream_t)stream);
        SPL_DISPATCH_CDIM(channels, CALL);
    }
#undef CALL
    return check_launch("rasterize_to_pixels_fwd");
}

extern "C" int splatad_rasterize_to_pixels_bwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics, const float *colors,
    uint32_t channels, const float *opacities, const float *pix_vels,
    const float *rolling_shutter_time, const float *backgrounds, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const float *render_alphas,
    const int32_t *last_ids, const float *v_render_colors, const float *v_render_alphas,
    float *v_means2d_abs, float *v_means2d, float *v_conics, float *v_colors, float *v_opacities,
    float *v_pix_vels, void *stream) {
    SPL_REQUIRE(channels >= 1 && channels <= SPLATAD_MAX_CHANNELS, SPLATAD_ERR_CHANNELS,
                "rasterize_to_pixels_bwd: unsupported channel count %u (1..%d)", channels,
                SPLATAD_MAX_CHANNELS);
    SPL_REQUIRE(tile_size >= 1 && tile_size * tile_size <= 1024, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_pixels_bwd: tile_size^2 must be <= 1024");
    const uint32_t blocks = C * tile_width * tile_height;
    if (blocks == 0 || n_isects == 0 || image_width == 0 || image_height == 0) return SPLATAD_OK;
    SPL_REQUIRE(means2d && conics && colors && opacities && pix_vels && flatten_ids &&
                    tile_offsets && render_alphas && last_ids && v_render_colors &&
                    v_render_alphas && v_means2d && v_conics && v_colors && v_opacities &&
                    v_pix_vels && rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_pixels_bwd: null argument");
    const uint32_t bs = ((tile_size * tile_size + 31) / 32) * 32;   // whole warps
    const uint32_t cdim = channels <= 4 ? 4u : channels <= 8 ? 8u : channels <= 16 ? 16u : channels <= 20 ? 20u : 32u;
    const size_t smem = (size_t)bs * (2 * sizeof(float4) + 2 * sizeof(int32_t) + cdim * sizeof(float));   // rows of CDIM floats
#define CALL(D)                                                                                   \
    {                                                                                             \
        int rc = check_block_size(rasterize_to_pixels_bwd_kernel<D>, bs, channels, "rasterize_to_pixels_bwd"); \
        if (rc != SPLATAD_OK) return rc;                                                          \
        rc = set_smem(rasterize_to_pixels_bwd_kernel<D>, smem, "rasterize_to_pixels_bwd");    \
        if (rc != SPLATAD_OK) return rc;                                                          \
        rasterize_to_pixels_bwd_kernel<D><<<blocks, bs, smem, (cudaStream_t)stream>>>(            \
            C, n_isects, (const float2 *)means2d, conics, colors, channels, opacities,            \
            (const float2 *)pix_vels, rolling_shutter_time, backgrounds, image_width,             \
            image_height, tile_size, tile_width, tile_height, tile_offsets, flatten_ids,          \
            render_alphas, last_ids, v_render_colors, v_render_alphas, v_means2d_abs, v_means2d,  \
            v_conics, v_colors, v_opacities, v_pix_vels);                                         \
    }
    {
        SPL_PROF("rasterize_to_pixels_bwd_kernel", (cudaStream_t)stream);
        SPL_DISPATCH_CDIM(channels, CALL);
    }
#undef CALL
    return check_launch("rasterize_to_pixels_bwd");
}

extern "C" int splatad_rasterize_to_points_fwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics,
    const float *lidar_features, const float *gaussian_ranges, uint32_t channels,
    const float *opacities,
    const float *pix_vels, const float *depth_compensations, const float *backgrounds,
    const float *raster_pts, uint32_t image_width, uint32_t image_height, uint32_t tile_width,
    uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    int32_t compute_alpha_sum_until_points, float alpha_sum_threshold,
    const int32_t *tile_offsets, const int32_t *flatten_ids, uint32_t depth_channel_idx,
    float *render_features, float *render_alphas, float *alpha_sum_until_points,
    int32_t *last_ids, float *median_depths, void *stream) {
    SPL_REQUIRE(channels >= 1 && channels <= SPLATAD_MAX_CHANNELS, SPLATAD_ERR_CHANNELS,
                "rasterize_to_points_fwd: unsupported channel count %u (1..%d)", channels,
                SPLATAD_MAX_CHANNELS);
    SPL_REQUIRE(depth_channel_idx < channels, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_points_fwd: depth channel out of range");
    SPL_REQUIRE(!gaussian_ranges || depth_channel_idx == channels - 1, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_points_fwd: a separate range array is the last channel");
    SPL_REQUIRE(tile_width >= 1 && tile_height >= 1 && tile_width * tile_height <= 1024,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_fwd: tile must have <= 1024 points");
    SPL_REQUIRE(render_features && render_alphas && last_ids && median_depths && tile_offsets &&
                    raster_pts,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_fwd: null argument");
    SPL_REQUIRE(!compute_alpha_sum_until_points || alpha_sum_until_points, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_points_fwd: alpha-sum output missing");
    SPL_REQUIRE(n_isects == 0 || (means2d && conics && opacities && pix_vels &&
                                  depth_compensations && flatten_ids &&
                                  (lidar_features || (gaussian_ranges && channels == 1))),
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_fwd: null input");
    const uint32_t blocks = C * tile_grid_width * tile_grid_height;
    if (blocks == 0 || image_width == 0 || image_height == 0) return SPLATAD_OK;
    const uint32_t bs = ((tile_width * tile_height + 31) / 32) * 32;   // whole warps
    size_t smem = (size_t)bs * (3 * sizeof(float4) + sizeof(int32_t));
    // the batch's feature rows ride along in shared memory while a block stays under 64 KB
    const uint32_t cdim = channels <= 4 ? 4u : channels <= 8 ? 8u : channels <= 16 ? 16u : channels <= 20 ? 20u : 32u;
    const size_t smem_feat = (size_t)bs * cdim * sizeof(float);   // rows of CDIM floats, see SPL_DISPATCH_CDIM
    const uint32_t stage_features = (smem + smem_feat <= 64 * 1024) ? 1u : 0u;
    if (stage_features) smem += smem_feat;
#define CALL(D)                                                                                   \
    {                                                                                             \
        int rc = set_smem(rasterize_to_points_fwd_kernel<D>, smem, "rasterize_to_points_fwd");    \
        if (rc != SPLATAD_OK) return rc;                                                          \
        launch_chained(rasterize_to_points_fwd_kernel<D>, blocks, bs, smem, (cudaStream_t)stream, \
            C, n_isects, (const float2 *)means2d, conics, lidar_features, gaussian_ranges,        \
            channels, opacities,                                                                  \
            pix_vels, (const float2 *)depth_compensations, backgrounds,                           \
            (const float4 *)raster_pts, image_width, image_height, tile_width, tile_height,       \
            tile_grid_width, tile_grid_height, compute_alpha_sum_until_points,                    \
            alpha_sum_threshold, tile_offsets, flatten_ids, depth_channel_idx, render_features,   \
            render_alphas, alpha_sum_until_points, last_ids, median_depths, stage_features);      \
    }
    {
        SPL_PROF("rasterize_to_points_fwd_kernel", (cudaStream_t)stream);
        SPL_DISPATCH_CDIM(channels, CALL);
    }
#undef CALL
    return check_launch("rasterize_to_points_fwd");
}

extern "C" int splatad_rasterize_to_points_bwd(
    uint32_t C, int64_t n_isects, const float *means2d, const float *conics,
    const float *lidar_features, const float *gaussian_ranges, uint32_t channels,
    const float *opacities,
    const float *pix_vels, const float *depth_compensations, const float *backgrounds,
    const float *raster_pts, uint32_t image_width, uint32_t image_height, uint32_t tile_width,
    uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    int32_t compute_alpha_sum_until_points, float alpha_sum_threshold,
    const int32_t *tile_offsets, const int32_t *flatten_ids, uint32_t depth_channel_idx,
    const float *render_alphas, const int32_t *last_ids, const float *v_render_features,
    const float *v_render_alphas, const float *v_alpha_sum_until_points, float *v_means2d_abs,
    float *v_means2d, float *v_conics, float *v_features, float *v_opacities, float *v_pix_vels,
    float *v_depth_compensations, float *v_gaussian_ranges, void *stream) {
    SPL_REQUIRE(channels >= 1 && channels <= SPLATAD_MAX_CHANNELS, SPLATAD_ERR_CHANNELS,
                "rasterize_to_points_bwd: unsupported channel count %u (1..%d)", channels,
                SPLATAD_MAX_CHANNELS);
    SPL_REQUIRE(depth_channel_idx < channels, SPLATAD_ERR_BAD_ARG,
                "rasterize_to_points_bwd: depth channel out of range");
    SPL_REQUIRE(tile_width >= 1 && tile_height >= 1 && tile_width * tile_height <= 1024,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_bwd: tile must have <= 1024 points");
    const uint32_t blocks = C * tile_grid_width * tile_grid_height;
    if (blocks == 0 || n_isects == 0 || image_width == 0 || image_height == 0) return SPLATAD_OK;
    SPL_REQUIRE(means2d && conics && opacities && pix_vels &&
                    depth_compensations && flatten_ids && tile_offsets && raster_pts &&
                    render_alphas && last_ids && v_render_features && v_render_alphas &&
                    v_means2d && v_conics && v_opacities && v_pix_vels && v_depth_compensations,
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_bwd: null argument");
    SPL_REQUIRE((lidar_features && v_features) || (gaussian_ranges && channels == 1), SPLATAD_ERR_BAD_ARG,
                "rasterize_to_points_bwd: features / v_features missing");
    SPL_REQUIRE(!gaussian_ranges || (v_gaussian_ranges && depth_channel_idx == channels - 1),
                SPLATAD_ERR_BAD_ARG, "rasterize_to_points_bwd: range array needs v_gaussian_ranges");
    const uint32_t bs = ((tile_width * tile_height + 31) / 32) * 32;   // whole warps
    const uint32_t cdim = channels <= 4 ? 4u : channels <= 8 ? 8u : channels <= 16 ? 16u : channels <= 20 ? 20u : 32u;
    const size_t smem = (size_t)bs * (3 * sizeof(float4) + sizeof(int32_t) + cdim * sizeof(float));   // rows of CDIM floats
#define CALL(D)                                                                                   \
    {                                                                                             \
        int rc = check_block_size(rasterize_to_points_bwd_kernel<D>, bs, channels, "rasterize_to_points_bwd"); \
        if (rc != SPLATAD_OK) return rc;                                                          \
        rc = set_smem(rasterize_to_points_bwd_kernel<D>, smem, "rasterize_to_points_bwd");    \
        if (rc != SPLATAD_OK) return rc;                                                          \
        rasterize_to_points_bwd_kernel<D><<<blocks, bs, smem, (cudaStream_t)stream>>>(            \
            C, n_isects, (const float2 *)means2d, conics, lidar_features, gaussian_ranges,        \
            channels, opacities,                                                                  \
            pix_vels, (const float2 *)depth_compensations, backgrounds,                           \
            (const float4 *)raster_pts, image_width, image_height, tile_width, tile_height,       \
            tile_grid_width, tile_grid_height, compute_alpha_sum_until_points,                    \
            alpha_sum_threshold, tile_offsets, flatten_ids, depth_channel_idx, render_alphas,     \
            last_ids, v_render_features, v_render_alphas, v_alpha_sum_until_points,               \
            v_means2d_abs, v_means2d, v_conics, v_features, v_opacities, v_pix_vels,              \
            v_depth_compensations, v_gaussian_ranges);                                            \
    }
    {
        SPL_PROF("rasterize_to_points_bwd_kernel", (cudaStream_t)stream);
        SPL_DISPATCH_CDIM(channels, CALL);
    }
#undef CALL
    return check_launch("rasterize_to_points_bwd");
}
