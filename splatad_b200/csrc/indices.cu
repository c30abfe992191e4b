// Indices of the (Gaussian, pixel) pairs that contribute to an image within a range of list
// batches: rasterize_to_indices_in_range for camera pixels and its lidar twin. Integer outputs;
// the per-pair test is the FP32 arithmetic of the compositing kernels.
//
// Semantics follow the reference kernels
//   pixels  gsplat/cuda/csrc/rasterization.cu:839-990    host side 992-1090
//   points  gsplat/cuda/csrc/rasterization.cu:1092-1262  host side 1264-1358
// A batch is tile_w * tile_h consecutive entries of a tile's depth-ordered list; a call walks
// batches [range_start, range_end) of every tile starting from the caller's per-pixel
// transmittances, and lists, pixel after pixel (camera-major, row-major) and front to back inside
// a pixel, every Gaussian that passes the alpha >= 1/255, sigma >= 0 tests before the pixel stops
// at T * (1 - alpha) <= 1e-4.
//
// Two passes like the reference, with the prefix sum in between done here rather than by the
// caller: count per pixel -> exclusive scan over all pixels (three small kernels, 64-bit starts,
// the total behind the last start) -> write. One CTA per tile, one thread per pixel, the batch
// staged in shared memory as two float4 per Gaussian; a warp whose pixels have all stopped skips
// the batch body.
#include "common.cuh"
#include "composite_common.cuh"

namespace splatad {

struct IndicesArgs {
    uint32_t range_start, range_end, C, N;
    int64_t n_isects;
    const float2 *means2d;
    const float *conics, *opacities, *pix_vels, *rs_time;
    const float4 *raster_pts;
    uint32_t W, H, tile_w, tile_h, grid_w, grid_h;
    const int32_t *offsets, *flatten_ids;
    const float *transmittances;
    const int64_t *starts;    // write pass
    int32_t *cnts;            // count pass
    int64_t *gaussian_ids, *pixel_ids, *camera_ids;
    unsigned long long *pair_counters;   // count pass, optional: [0] += tested, [1] += contributing pairs
};

template <bool kLidar, bool kWrite>
__global__ void indices_in_range_kernel(const IndicesArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const uint32_t unit = a.tile_w * a.tile_h;           // entries per batch
    float4 *sA = reinterpret_cast<float4 *>(smem_raw);   // x, y, vx, vy
    float4 *sB = sA + unit;                              // conic a, b, c, opacity
    int32_t *sId = reinterpret_cast<int32_t *>(sB + unit);

    const uint32_t tiles_per_cam = a.grid_w * a.grid_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t ty = tile / a.grid_w, tx = tile - ty * a.grid_w;
    const uint32_t tr = threadIdx.x;
    const uint32_t i = ty * a.tile_h + tr / a.tile_w;
    const uint32_t j = tx * a.tile_w + tr % a.tile_w;
    const bool in_image = (tr < unit) && (i < a.H && j < a.W);
    const uint32_t pix_in_cam = i * a.W + j;
    const size_t pix = (size_t)cam * a.H * a.W + pix_in_cam;

    const TileRange range = tile_range(a.offsets, blockIdx.x, a.C * tiles_per_cam, a.n_isects);
    const uint32_t num_batches = (uint32_t)(range.end - range.start + unit - 1) / unit;
    if (a.range_start >= num_batches) {
        // nothing of this tile's list lies in the range
        if (!kWrite && in_image) a.cnts[pix] = 0;
        return;
    }

    bool inside = in_image;
    float px, py, roll = 0.f, T = 0.f;
    if (kLidar) {
        px = py = 0.f;
        if (inside) {
            const float4 rp = a.raster_pts[pix];
            px = rp.x; py = rp.y; roll = rp.w;
            if (rp.z <= 0.f) inside = false;   // not rendered
        }
    } else {
        px = (float)j + 0.5f;
        py = (float)i + 0.5f;
        roll = a.rs_time[cam] * ((py - 0.5f) / (float)(a.H - 1) - 0.5f);
    }
    int64_t base = 0;
    if (inside) {
        T = a.transmittances[pix];
        if (kWrite) base = a.starts[pix];
    }
    bool done = !inside;
    int32_t cnt = 0;
    uint32_t tested = 0;   // entries this pixel evaluated, the one it stops at included
    const uint32_t b_end = min(a.range_end, num_batches);
    for (uint32_t b = a.range_start; b < b_end; ++b) {
        if (__syncthreads_count(done) >= (int)blockDim.x) break;
        const uint32_t batch_start = (uint32_t)range.start + unit * b;
        const uint32_t idx = batch_start + tr;
        if (tr < unit && idx < (uint32_t)range.end) {
            const int32_t g = a.flatten_ids[idx];
            const float2 xy = a.means2d[g];
            const float *v = a.pix_vels + (kLidar ? 3 : 2) * (size_t)g;
            sA[tr] = make_float4(xy.x, xy.y, v[0], v[1]);
            sB[tr] = make_float4(a.conics[3 * (size_t)g], a.conics[3 * (size_t)g + 1],
                                 a.conics[3 * (size_t)g + 2], a.opacities[g]);
            if (kWrite) sId[tr] = g;
        }
        __syncthreads();
        if (__all_sync(0xffffffffu, done)) continue;
        const uint32_t batch_size = min(unit, (uint32_t)range.end - batch_start);
        for (uint32_t t = 0; t < batch_size && !done; ++t) {
            const float4 A = sA[t];
            const float4 B = sB[t];
            float dx, dy;
            if (kLidar) {
                dx = angle_difference(A.x + roll * A.z, px);
                dy = angle_difference(A.y + roll * A.w, py);
            } else {
                dx = A.x + roll * A.z - px;
                dy = A.y + roll * A.w - py;
            }
            const float sigma = 0.5f * (B.x * dx * dx + B.z * dy * dy) + B.y * dx * dy;
            const float alpha = fminf(kAlphaMax, B.w * __expf(-sigma));
            if (!kWrite) ++tested;
            if (sigma < 0.f || alpha < kAlphaMin) continue;
            const float next_T = T * (1.f - alpha);
            if (next_T <= kTStop) { done = true; break; }
            if (kWrite) {
                a.gaussian_ids[base + cnt] = (int64_t)((uint32_t)sId[t] % a.N);
                a.pixel_ids[base + cnt] = (int64_t)pix_in_cam;
                a.camera_ids[base + cnt] = (int64_t)cam;
            }
            ++cnt;
            T = next_T;
        }
    }
    if (!kWrite && in_image) a.cnts[pix] = cnt;
    if (!kWrite && a.pair_counters != nullptr) {
        unsigned long long t = tested, c = (unsigned long long)cnt;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            t += __shfl_xor_sync(0xffffffffu, t, off);
            c += __shfl_xor_sync(0xffffffffu, c, off);
        }
        if ((threadIdx.x & 31) == 0 && t) {
            atomicAdd(a.pair_counters, t);
            atomicAdd(a.pair_counters + 1, c);
        }
    }
}

// ---------------------------------------------------------------------------------------
// Exclusive prefix sum of the per-pixel counts: int32 counts -> int64 starts, total at the end
// ---------------------------------------------------------------------------------------
constexpr uint32_t kScanThreads = 1024;
constexpr uint32_t kScanItems = 4;
constexpr uint32_t kScanTile = kScanThreads * kScanItems;

// Exclusive scan of one value per thread over a block of kScanThreads; returns the thread's
// prefix, *total receives the block sum. red holds 32 values.
__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *red, int64_t *total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int64_t up = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= (uint32_t)off) inc += up;
    }
    __syncthreads();   // red may still be read from an earlier call
    if (lane == 31) red[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        int64_t w = red[lane];
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, w, off);
            if (lane >= (uint32_t)off) w += up;
        }
        red[lane] = w;
    }
    __syncthreads();
    *total = red[31];
    return inc - v + (warp ? red[warp - 1] : 0);
}

__global__ void __launch_bounds__(kScanThreads)
indices_tile_sums_kernel(const int32_t *__restrict__ cnts, uint64_t n, int64_t *__restrict__ sums) {
    __shared__ int64_t red[32];
    const uint64_t first = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
    int64_t v = 0;
#pragma unroll
    for (uint32_t k = 0; k < kScanItems; ++k)
        if (first + k < n) v += cnts[first + k];
    int64_t total;
    block_exclusive_scan(v, red, &total);
    if (threadIdx.x == 0) sums[blockIdx.x] = total;
}

// One block: sums[0 .. n_tiles) -> exclusive prefixes in place; the grand total goes behind the
// last start and to *total_out.
__global__ void __launch_bounds__(kScanThreads)
indices_spine_kernel(int64_t *__restrict__ sums, uint32_t n_tiles, int64_t *__restrict__ starts_end,
                     int64_t *__restrict__ total_out) {
    __shared__ int64_t red[32];
    int64_t carry = 0;
    for (uint32_t base = 0; base < n_tiles; base += kScanThreads) {
        const uint32_t k = base + threadIdx.x;
        const int64_t v = k < n_tiles ? sums[k] : 0;
        int64_t total;
        const int64_t ex = block_exclusive_scan(v, red, &total);
        if (k < n_tiles) sums[k] = carry + ex;
        carry += total;
    }
    if (threadIdx.x == 0) {
        *starts_end = carry;
        if (total_out) *total_out = carry;
    }
}

__global__ void __launch_bounds__(kScanThreads)
indices_starts_kernel(const int32_t *__restrict__ cnts, uint64_t n, const int64_t *__restrict__ sums,
                      int64_t *__restrict__ starts) {
    __shared__ int64_t red[32];
    const uint64_t first = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
    int32_t c[kScanItems];
    int64_t v = 0;
#pragma unroll
    for (uint32_t k = 0; k < kScanItems; ++k) {
        c[k] = first + k < n ? cnts[first + k] : 0;
        v += c[k];
    }
    int64_t total;
    int64_t run = block_exclusive_scan(v, red, &total) + sums[blockIdx.x];
#pragma unroll
    for (uint32_t k = 0; k < kScanItems; ++k) {
        if (first + k < n) starts[first + k] = run;
        run += c[k];
    }
}

struct IndicesWs {
    int32_t *cnts;
    int64_t *sums;
    size_t bytes;
};

static IndicesWs carve_indices(void *ws, uint64_t n_pix) {
    IndicesWs w;
    const size_t cnt_bytes = ((size_t)n_pix * sizeof(int32_t) + 255) & ~(size_t)255;
    const size_t n_tiles = (size_t)((n_pix + kScanTile - 1) / kScanTile);
    w.cnts = reinterpret_cast<int32_t *>(ws);
    w.sums = reinterpret_cast<int64_t *>(reinterpret_cast<unsigned char *>(ws) + cnt_bytes);
    w.bytes = cnt_bytes + ((n_tiles * sizeof(int64_t) + 255) & ~(size_t)255) + 256;
    return w;
}

template <typename K>
static int reserve_smem(K kernel, size_t bytes, const char *what) {
    if (bytes > 32 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
        if (e != cudaSuccess) {
            set_last_error("%s: cannot reserve %zu bytes of shared memory: %s", what, bytes,
                           cudaGetErrorString(e));
            return SPLATAD_ERR_CUDA;
        }
    }
    return SPLATAD_OK;
}

template <bool kLidar, bool kWrite>
static int launch_indices(const IndicesArgs &a, cudaStream_t st, const char *what) {
    const uint32_t unit = a.tile_w * a.tile_h;
    const uint32_t bs = ((unit + 31) / 32) * 32;   // whole warps
    const size_t smem = (size_t)unit * (2 * sizeof(float4) + sizeof(int32_t));
    const uint32_t blocks = a.C * a.grid_w * a.grid_h;
    int rc = reserve_smem(indices_in_range_kernel<kLidar, kWrite>, smem, what);
    if (rc != SPLATAD_OK) return rc;
    SPL_PROF(kWrite ? "indices_in_range_kernel<write>" : "indices_in_range_kernel<count>", st);
    indices_in_range_kernel<kLidar, kWrite><<<blocks, bs, smem, st>>>(a);
    return check_launch(what);
}

static int check_indices_args(const IndicesArgs &a, bool lidar, const char *what) {
    SPL_REQUIRE(a.tile_w >= 1 && a.tile_h >= 1 && a.tile_w * a.tile_h <= 1024, SPLATAD_ERR_BAD_ARG,
                "%s: a tile must have 1..1024 pixels", what);
    SPL_REQUIRE((uint64_t)a.grid_w * a.tile_w >= a.W && (uint64_t)a.grid_h * a.tile_h >= a.H,
                SPLATAD_ERR_BAD_ARG, "%s: the tile grid does not cover the image", what);
    SPL_REQUIRE(a.n_isects == 0 || (a.means2d && a.conics && a.opacities && a.pix_vels &&
                                    a.flatten_ids && a.N > 0),
                SPLATAD_ERR_BAD_ARG, "%s: null input", what);
    SPL_REQUIRE(a.offsets && a.transmittances && (lidar ? (const void *)a.raster_pts : (const void *)a.rs_time),
                SPLATAD_ERR_BAD_ARG, "%s: null argument", what);
    return SPLATAD_OK;
}

// count pass + prefix sum
template <bool kLidar>
static int indices_count(IndicesArgs a, void *workspace, size_t workspace_bytes, int64_t *chunk_starts,
                         int64_t *host_total, cudaStream_t st, const char *what) {
    int rc = check_indices_args(a, kLidar, what);
    if (rc != SPLATAD_OK) return rc;
    const uint64_t n_pix = (uint64_t)a.C * a.H * a.W;
    SPL_REQUIRE(chunk_starts, SPLATAD_ERR_BAD_ARG, "%s: chunk_starts missing", what);
    if (n_pix == 0 || a.n_isects == 0 || a.C * a.grid_w * a.grid_h == 0) {
        if (cudaMemsetAsync(chunk_starts, 0, (size_t)(n_pix + 1) * sizeof(int64_t), st) != cudaSuccess)
            return check_launch(what);
        if (host_total) *host_total = 0;
        return SPLATAD_OK;
    }
    const IndicesWs w = carve_indices(workspace, n_pix);
    SPL_REQUIRE(workspace && workspace_bytes >= w.bytes, SPLATAD_ERR_WORKSPACE,
                "%s: workspace of %zu bytes needed, %zu given", what, w.bytes, workspace_bytes);
    a.cnts = w.cnts;
    rc = launch_indices<kLidar, false>(a, st, what);
    if (rc != SPLATAD_OK) return rc;
    const uint32_t n_tiles = (uint32_t)((n_pix + kScanTile - 1) / kScanTile);
    {
        SPL_PROF("indices_scan", st);
        indices_tile_sums_kernel<<<n_tiles, kScanThreads, 0, st>>>(w.cnts, n_pix, w.sums);
        indices_spine_kernel<<<1, kScanThreads, 0, st>>>(w.sums, n_tiles, chunk_starts + n_pix, nullptr);
        indices_starts_kernel<<<n_tiles, kScanThreads, 0, st>>>(w.cnts, n_pix, w.sums, chunk_starts);
    }
    rc = check_launch(what);
    if (rc != SPLATAD_OK) return rc;
    if (host_total) {
        cudaError_t e = cudaMemcpyAsync(host_total, chunk_starts + n_pix, sizeof(int64_t),
                                        cudaMemcpyDeviceToHost, st);
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);
        if (e != cudaSuccess) {
            set_last_error("%s: reading the total failed: %s", what, cudaGetErrorString(e));
            return SPLATAD_ERR_CUDA;
        }
    }
    return SPLATAD_OK;
}

template <bool kLidar>
static int indices_write(IndicesArgs a, const int64_t *chunk_starts, cudaStream_t st, const char *what) {
    int rc = check_indices_args(a, kLidar, what);
    if (rc != SPLATAD_OK) return rc;
    if ((uint64_t)a.C * a.H * a.W == 0 || a.n_isects == 0 || a.C * a.grid_w * a.grid_h == 0) return SPLATAD_OK;
    SPL_REQUIRE(chunk_starts && a.gaussian_ids && a.pixel_ids && a.camera_ids, SPLATAD_ERR_BAD_ARG,
                "%s: null output", what);
    a.starts = chunk_starts;
    return launch_indices<kLidar, true>(a, st, what);
}

} // namespace splatad

using namespace splatad;

extern "C" size_t splatad_rasterize_to_indices_workspace_bytes(uint32_t C, uint32_t image_width,
                                                               uint32_t image_height) {
    return carve_indices(nullptr, (uint64_t)C * image_width * image_height).bytes;
}

static IndicesArgs camera_args(uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N,
                               int64_t n_isects, const float *transmittances, const float *means2d,
                               const float *conics, const float *opacities, const float *pix_vels,
                               const float *rolling_shutter_time, uint32_t image_width,
                               uint32_t image_height, uint32_t tile_size, uint32_t tile_width,
                               uint32_t tile_height, const int32_t *tile_offsets,
                               const int32_t *flatten_ids) {
    IndicesArgs a = {};
    a.range_start = range_start; a.range_end = range_end; a.C = C; a.N = N; a.n_isects = n_isects;
    a.means2d = (const float2 *)means2d; a.conics = conics; a.opacities = opacities;
    a.pix_vels = pix_vels; a.rs_time = rolling_shutter_time;
    a.W = image_width; a.H = image_height; a.tile_w = tile_size; a.tile_h = tile_size;
    a.grid_w = tile_width; a.grid_h = tile_height;
    a.offsets = tile_offsets; a.flatten_ids = flatten_ids; a.transmittances = transmittances;
    return a;
}

static IndicesArgs lidar_args(uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N,
                              int64_t n_isects, const float *transmittances, const float *means2d,
                              const float *conics, const float *opacities, const float *pix_vels,
                              const float *raster_pts, uint32_t image_width, uint32_t image_height,
                              uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width,
                              uint32_t tile_grid_height, const int32_t *tile_offsets,
                              const int32_t *flatten_ids) {
    IndicesArgs a = {};
    a.range_start = range_start; a.range_end = range_end; a.C = C; a.N = N; a.n_isects = n_isects;
    a.means2d = (const float2 *)means2d; a.conics = conics; a.opacities = opacities;
    a.pix_vels = pix_vels; a.raster_pts = (const float4 *)raster_pts;
    a.W = image_width; a.H = image_height; a.tile_w = tile_width; a.tile_h = tile_height;
    a.grid_w = tile_grid_width; a.grid_h = tile_grid_height;
    a.offsets = tile_offsets; a.flatten_ids = flatten_ids; a.transmittances = transmittances;
    return a;
}

extern "C" int splatad_rasterize_to_indices_in_range_count(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *rolling_shutter_time, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, void *workspace, size_t workspace_bytes,
    int64_t *chunk_starts, int64_t *host_total, void *stream) {
    return indices_count<false>(
        camera_args(range_start, range_end, C, N, n_isects, transmittances, means2d, conics, opacities,
                    pix_vels, rolling_shutter_time, image_width, image_height, tile_size, tile_width,
                    tile_height, tile_offsets, flatten_ids),
        workspace, workspace_bytes, chunk_starts, host_total, (cudaStream_t)stream,
        "rasterize_to_indices_in_range_count");
}

extern "C" int splatad_rasterize_to_indices_in_range_write(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *rolling_shutter_time, uint32_t image_width,
    uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const int64_t *chunk_starts,
    int64_t *gaussian_ids, int64_t *pixel_ids, int64_t *camera_ids, void *stream) {
    IndicesArgs a = camera_args(range_start, range_end, C, N, n_isects, transmittances, means2d, conics,
                                opacities, pix_vels, rolling_shutter_time, image_width, image_height,
                                tile_size, tile_width, tile_height, tile_offsets, flatten_ids);
    a.gaussian_ids = gaussian_ids; a.pixel_ids = pixel_ids; a.camera_ids = camera_ids;
    return indices_write<false>(a, chunk_starts, (cudaStream_t)stream,
                                "rasterize_to_indices_in_range_write");
}

extern "C" int splatad_rasterize_to_indices_in_range_lidar_count(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *raster_pts, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, void *workspace, size_t workspace_bytes,
    int64_t *chunk_starts, int64_t *host_total, void *stream) {
    return indices_count<true>(
        lidar_args(range_start, range_end, C, N, n_isects, transmittances, means2d, conics, opacities,
                   pix_vels, raster_pts, image_width, image_height, tile_width, tile_height,
                   tile_grid_width, tile_grid_height, tile_offsets, flatten_ids),
        workspace, workspace_bytes, chunk_starts, host_total, (cudaStream_t)stream,
        "rasterize_to_indices_in_range_lidar_count");
}

extern "C" int splatad_rasterize_to_indices_in_range_lidar_write(
    uint32_t range_start, uint32_t range_end, uint32_t C, uint32_t N, int64_t n_isects,
    const float *transmittances, const float *means2d, const float *conics, const float *opacities,
    const float *pix_vels, const float *raster_pts, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, const int64_t *chunk_starts,
    int64_t *gaussian_ids, int64_t *pixel_ids, int64_t *camera_ids, void *stream) {
    IndicesArgs a = lidar_args(range_start, range_end, C, N, n_isects, transmittances, means2d, conics,
                               opacities, pix_vels, raster_pts, image_width, image_height, tile_width,
                               tile_height, tile_grid_width, tile_grid_height, tile_offsets, flatten_ids);
    a.gaussian_ids = gaussian_ids; a.pixel_ids = pixel_ids; a.camera_ids = camera_ids;
    return indices_write<true>(a, chunk_starts, (cudaStream_t)stream,
                               "rasterize_to_indices_in_range_lidar_write");
}


// ---------------------------------------------------------------------------------------
// Pair counts of a whole frame (measurement aid)
// ---------------------------------------------------------------------------------------
template <bool kLidar>
static int count_pairs(IndicesArgs a, int32_t *pixel_counts, unsigned long long *counters, cudaStream_t st,
                       const char *what) {
    int rc = check_indices_args(a, kLidar, what);
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(pixel_counts && counters, SPLATAD_ERR_BAD_ARG, "%s: null output", what);
    if (cudaMemsetAsync(counters, 0, 2 * sizeof(unsigned long long), st) != cudaSuccess) return check_launch(what);
    if ((uint64_t)a.C * a.H * a.W == 0 || a.n_isects == 0 || a.C * a.grid_w * a.grid_h == 0) return SPLATAD_OK;
    a.cnts = pixel_counts;
    a.pair_counters = counters;
    return launch_indices<kLidar, false>(a, st, what);
}

extern "C" int splatad_count_composited_pairs(
    uint32_t C, uint32_t N, int64_t n_isects, const float *transmittances, const float *means2d,
    const float *conics, const float *opacities, const float *pix_vels, const float *rolling_shutter_time,
    uint32_t image_width, uint32_t image_height, uint32_t tile_size, uint32_t tile_width, uint32_t tile_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, int32_t *pixel_counts, uint64_t *counters,
    void *stream) {
    IndicesArgs a = {};
    a.range_start = 0; a.range_end = 0xffffffffu; a.C = C; a.N = N; a.n_isects = n_isects;
    a.means2d = (const float2 *)means2d; a.conics = conics; a.opacities = opacities; a.pix_vels = pix_vels;
    a.rs_time = rolling_shutter_time; a.W = image_width; a.H = image_height; a.tile_w = tile_size;
    a.tile_h = tile_size; a.grid_w = tile_width; a.grid_h = tile_height; a.offsets = tile_offsets;
    a.flatten_ids = flatten_ids; a.transmittances = transmittances;
    return count_pairs<false>(a, pixel_counts, (unsigned long long *)counters, (cudaStream_t)stream,
                              "count_composited_pairs");
}

extern "C" int splatad_count_composited_pairs_lidar(
    uint32_t C, uint32_t N, int64_t n_isects, const float *transmittances, const float *means2d,
    const float *conics, const float *opacities, const float *pix_vels, const float *raster_pts,
    uint32_t image_width, uint32_t image_height, uint32_t tile_width, uint32_t tile_height,
    uint32_t tile_grid_width, uint32_t tile_grid_height, const int32_t *tile_offsets,
    const int32_t *flatten_ids, int32_t *pixel_counts, uint64_t *counters, void *stream) {
    IndicesArgs a = {};
    a.range_start = 0; a.range_end = 0xffffffffu; a.C = C; a.N = N; a.n_isects = n_isects;
    a.means2d = (const float2 *)means2d; a.conics = conics; a.opacities = opacities; a.pix_vels = pix_vels;
    a.raster_pts = (const float4 *)raster_pts; a.W = image_width; a.H = image_height; a.tile_w = tile_width;
    a.tile_h = tile_height; a.grid_w = tile_grid_width; a.grid_h = tile_grid_height; a.offsets = tile_offsets;
    a.flatten_ids = flatten_ids; a.transmittances = transmittances;
    return count_pairs<true>(a, pixel_counts, (unsigned long long *)counters, (cudaStream_t)stream,
                             "count_composited_pairs_lidar");
}
