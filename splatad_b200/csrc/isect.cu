// Tile intersection: per-Gaussian tile rectangles, intersection counts, and the depth-ordered
// per-tile Gaussian lists (isect_ids / flatten_ids / isect_offsets).
//
// What the reference does (gsplat/cuda/csrc/rasterization.cu:15-216 camera, 287-529 lidar,
// 218-285 offsets): count tiles per Gaussian, cumsum, emit one 64-bit key
// (sensor | tile | depth bits) per intersection in flatten-index order, then a stable LSD
// radix sort of 12-byte pairs over 43-46 key bits, then a boundary scan for the offsets.
//
// What this file does instead, with bit-identical results: because a stable sort of the
// emitted keys orders each tile's list by (depth bits, flatten index), the same lists are
// obtained by
//   1. a stable radix sort of the *visible Gaussians* by their 32 depth bits (4 passes over
//      at most C*N 8-byte pairs - small, L2 resident),
//   2. emitting (sensor*n_tiles + tile, flatten index) pairs in that depth order, and
//   3. a stable radix split of those 8-byte pairs by the compact tile key only
//      (ceil(bits/8) passes: 2 for every configuration up to 65536 sensor-tiles),
// the last pass writing the 64-bit isect_ids and int32 flatten_ids directly. Offsets are a
// binary search per tile.
//
// All kernels run on a fixed grid (a multiple of the 148 SMs) and read problem sizes from
// device memory, so the whole sequence can be enqueued without a host round trip; the only
// device->host traffic is the (n_isects, n_visible, status) triple.
#include "common.cuh"

namespace splatad {

constexpr int kSortThreads = 256;
constexpr int kSortWarps = kSortThreads / 32;
constexpr int kItemsPerLane = 8;
constexpr int kWarpItems = 32 * kItemsPerLane;           // 256
constexpr int kTileItems = kSortWarps * kWarpItems;      // 2048
constexpr int kSortGrid = 4 * kNumSMs;                   // 592 persistent blocks
constexpr int kRadixBins = 256;
static_assert(kSortThreads == kRadixBins, "one thread per radix bin");
static_assert(kSortGrid <= 1024, "row scan and emit scan use one thread per sort block");

// counters[] slots (int64 each)
// The first CNT_SLOTS are what the plan copies to the host; the rest is device-side state.
enum { CNT_NISECT = 0, CNT_NVIS = 1, CNT_STATUS = 2, CNT_TICKET = 3, CNT_SLOTS = 4,
       CNT_DMIN = 4, CNT_DMAX = 5,   // depth range of the listed elements (float bit patterns)
       CNT_BLO = 6, CNT_BHI = 7,     // depth range the buckets span when the caller gave one (BHI < BLO: none)
       CNT_DEV_SLOTS = 8 };
enum { ST_OVERFLOW_CAPACITY = 1, ST_OVERFLOW_INT32 = 2, ST_DEPTH_BUCKETS = 4 };

// ---------------------------------------------------------------------------------------
// Block-wide exclusive scan for any blockDim.x that is a multiple of 32 (<= 1024).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t *warp_tot /*[33]*/,
                                                    uint32_t &total) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t nwarps = blockDim.x >> 5;
    uint32_t inc = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
        if (lane >= (uint32_t)off) inc += o;
    }
    if (lane == 31) warp_tot[warp] = inc;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = (lane < nwarps) ? warp_tot[lane] : 0u;
        uint32_t winc = w;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            uint32_t o = __shfl_up_sync(0xffffffffu, winc, off);
            if (lane >= (uint32_t)off) winc += o;
        }
        warp_tot[lane] = winc - w;   // exclusive warp offsets
        if (lane == 31) warp_tot[32] = winc;
    }
    __syncthreads();
    const uint32_t res = warp_tot[warp] + inc - v;
    total = warp_tot[32];
    __syncthreads();
    return res;
}

// ---------------------------------------------------------------------------------------
// Tile rectangles
// ---------------------------------------------------------------------------------------
struct Rect { int32_t x0, x1, y0, y1; };   // x: [x0, x1), y: [y0, y1)

struct CamGrid { uint32_t tile_size, tile_width, tile_height; };

__device__ __forceinline__ uint32_t clamp_tile(float v, uint32_t hi) {
    // float -> uint32 conversion that saturates negatives (and NaN) to 0, then min(hi)
    if (!(v > 0.f)) return 0u;
    if (v >= (float)hi) return hi;
    return (uint32_t)v;
}

__device__ __forceinline__ Rect cam_rect(float2 mean, int2 radius, CamGrid g) {
    const float ts = (float)g.tile_size;
    const float ex = (float)radius.x / ts, ey = (float)radius.y / ts;
    const float tx = mean.x / ts, ty = mean.y / ts;
    Rect r;
    r.x0 = (int32_t)clamp_tile(floorf(tx - ex), g.tile_width);
    r.y0 = (int32_t)clamp_tile(floorf(ty - ey), g.tile_height);
    r.x1 = (int32_t)clamp_tile(ceilf(tx + ex), g.tile_width);
    r.y1 = (int32_t)clamp_tile(ceilf(ty + ey), g.tile_height);
    return r;
}

struct LidarGrid {
    const float *elev_boundaries;   // [n_tiles_elev + 1], global or shared
    float tile_azim_res, min_azim;
    uint32_t n_tiles_azim, n_tiles_elev;
};

// Number of leading entries of the ascending array b[0 .. n) that are < v.
__device__ __forceinline__ int32_t lower_bound_f(const float *__restrict__ b, int32_t n, float v) {
    int32_t lo = 0, hi = n;
    while (lo < hi) {
        const int32_t m = (lo + hi) >> 1;
        if (b[m] < v) lo = m + 1; else hi = m;
    }
    return lo;
}

__device__ __forceinline__ Rect lidar_rect(float2 mean, float2 radius, const LidarGrid &g) {
    const float el_lo = mean.y - radius.y, el_hi = mean.y + radius.y;
    const float azim = mean.x - g.min_azim;
    const float az_lo = azim - radius.x, az_hi = azim + radius.x;
    const float azim_max = (float)g.n_tiles_azim * g.tile_azim_res;
    float t_lo, t_hi;
    if (az_lo >= 0.f) t_lo = az_lo / g.tile_azim_res;
    else t_lo = (fmodf(az_lo + 360.f, 360.f) - azim_max) / g.tile_azim_res;
    if (az_hi <= 360.f) t_hi = az_hi / g.tile_azim_res;
    else t_hi = (float)g.n_tiles_azim + fmodf(az_hi + 360.f, 360.f) / g.tile_azim_res;
    Rect r;
    r.x0 = (int32_t)floorf(t_lo);
    r.x1 = (int32_t)ceilf(t_hi);
    // first boundary not below the lower edge (minus one), first boundary not below the upper
    // edge: the reference walks the ascending boundaries one by one, a bisection finds the same
    // indices (a NaN edge compares false everywhere and leaves both at 0, as there)
    const int32_t ne = (int32_t)g.n_tiles_elev;
    const int32_t i = lower_bound_f(g.elev_boundaries, ne + 1, el_lo);
    r.y0 = max(i - 1, 0);
    r.y1 = min(max(i, lower_bound_f(g.elev_boundaries, ne + 1, el_hi)), ne);
    return r;
}

__device__ __forceinline__ int32_t rect_count(const Rect &r) {
    return (r.y1 - r.y0) * (r.x1 - r.x0);
}

constexpr int kMaxElevSmem = 1024;

template <bool kLidar>
struct GridArgs {
    CamGrid cam;
    LidarGrid lidar;
    const void *radii;      // int2 (camera) or float2 (lidar)
    const float2 *means2d;
};

template <bool kLidar>
__device__ __forceinline__ bool elem_rect(const GridArgs<kLidar> &a, uint32_t idx, Rect &r) {
    if (kLidar) {
        const float2 rad = reinterpret_cast<const float2 *>(a.radii)[idx];
        if (!(rad.x > 0.f)) return false;
        r = lidar_rect(a.means2d[idx], rad, a.lidar);
    } else {
        const int2 rad = reinterpret_cast<const int2 *>(a.radii)[idx];
        if (rad.x <= 0) return false;
        r = cam_rect(a.means2d[idx], rad, a.cam);
    }
    return true;
}

// Copies the elevation boundaries to shared memory when they fit and repoints the grid.
template <bool kLidar>
__device__ __forceinline__ void stage_boundaries(GridArgs<kLidar> &a, float *sb) {
    if (kLidar) {
        const uint32_t nb = a.lidar.n_tiles_elev + 1;
        if (nb <= kMaxElevSmem) {
            for (uint32_t i = threadIdx.x; i < nb; i += blockDim.x) sb[i] = a.lidar.elev_boundaries[i];
            __syncthreads();
            a.lidar.elev_boundaries = sb;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Depth order by buckets. The visible elements are ordered by (depth bits, flatten index) - what a
// stable radix sort of the depth bits from flatten order gives - in four short kernels instead of
// twelve. The depth range [dmin, dmax] of the listed elements comes with the rectangle count; an
// element's bucket is its depth's position in that range, in 262144 equal steps of depth (equal
// steps of the bit pattern would crowd the far half of the range into a few buckets): a weakly
// monotone function of the depth, so buckets are ordered like the keys. Count per bucket (global
// atomics), scan, scatter into bucket order with an atomic cursor per bucket (arbitrary order
// inside a bucket), then every element finds its rank inside its bucket by counting the bucket's
// elements that precede it in (bits, flatten index) order and is written to its final place: one
// thread per element, neighbours share their bucket. For a million depths between 0.3 and 113 m a
// bucket holds 4 elements on average and 17 where they are densest. Elements of a bucket with more than kBucketMax entries
// (depths that agree to within half a millimetre by the thousand) are passed through unordered and reported
// with status bit ST_DEPTH_BUCKETS: the caller repeats the plan with the radix sort (sort = 2).
// ---------------------------------------------------------------------------------------
constexpr uint32_t kDepthBuckets = 262144;
constexpr uint32_t kBucketMax = 1024;
constexpr uint32_t kBucketScanBlocks = kDepthBuckets / 1024;   // 256
static_assert(kBucketScanBlocks % 32 == 0 && kBucketScanBlocks <= 1024, "block totals are scanned by one warp");

struct DepthBuckets {
    float dmin, scale;
    __device__ __forceinline__ uint32_t operator()(uint32_t bits) const {
        const float d = __uint_as_float(bits);
        if (!(d == d)) return kDepthBuckets - 1;   // NaN patterns sort behind +infinity
        const float x = (d - dmin) * scale;        // weakly monotone in d for finite dmin, scale >= 0
        if (!(x > 0.f)) return 0u;                 // depths below a range given by the caller
        return x >= (float)(kDepthBuckets - 1) ? kDepthBuckets - 1 : (uint32_t)x;
    }
};

// The buckets span the range the caller gave for this frame (its last frame's, widened: depths
// outside it fall into the end buckets, which keeps the bucket index monotone in depth, and the
// ranks inside a bucket go by the full key) or, without one, the measured range of this frame.
__device__ __forceinline__ DepthBuckets depth_buckets(const int64_t *counters) {
    const bool given = (uint32_t)counters[CNT_BHI] >= (uint32_t)counters[CNT_BLO];
    const uint32_t lo = (uint32_t)counters[given ? CNT_BLO : CNT_DMIN];
    const uint32_t hi = min((uint32_t)counters[given ? CNT_BHI : CNT_DMAX], 0x7f800000u);   // a NaN maximum counts as +infinity
    DepthBuckets b;
    b.dmin = __uint_as_float(min(lo, hi));
    const float range = __uint_as_float(hi) - b.dmin;
    b.scale = (range > 0.f) ? (float)(kDepthBuckets - 1) / range : 0.f;   // infinite range: scale 0, one bucket
    return b;
}

// tiles_per_gauss[idx] for every (sensor, Gaussian) / packed row. With rect_xw / rect_yh the
// rectangle is also stored, packed into two words per element (x0 | width << 16, first grid row |
// height << 16 with grid row = sensor * tile rows + y; 16-bit fields, used only when
// the geometry is within its limits) for the row / column split, and the total is added to *n_isects.
// {count, sequence number, status bits} for a polling host, stored by whichever kernel knows them first
// into mapped pinned memory: count and status, a system-wide fence, then the sequence number.
__device__ __forceinline__ void tell_host(volatile int64_t *early_host, int64_t seq, int64_t n_isects,
                                          int64_t status, int64_t depth_range = 0) {
    early_host[0] = n_isects;
    early_host[2] = status;
    early_host[3] = depth_range;   // dmin bits | dmax bits << 32 of the listed elements, 0: not known here
    __threadfence_system();
    early_host[1] = seq;
    __threadfence_system();
}

constexpr int kCountThreads = 1024;   // few, large blocks: every block ends with a handful of same-address atomics

template <bool kLidar>
__global__ void __launch_bounds__(kCountThreads)
isect_count_kernel(GridArgs<kLidar> a, uint32_t total, int32_t *__restrict__ tiles_per_gauss,
                   const int64_t *__restrict__ camera_ids, uint32_t N, uint32_t *__restrict__ rect_xw,
                   uint32_t *__restrict__ rect_yh, int64_t *__restrict__ n_isects,
                   int64_t *__restrict__ ticket /* with early_host: a zeroed counter */,
                   volatile int64_t *early_host /* optional, host-mapped: {count, sequence number, status} */,
                   int64_t early_seq,
                   const uint32_t *__restrict__ depth_bits /* optional: depth range of the listed elements */,
                   int64_t *__restrict__ counters /* with depth_bits: CNT_DMIN / CNT_DMAX / CNT_NVIS */,
                   uint32_t *__restrict__ bcount /* optional, with a given bucket range: the bucket counts */) {
    chain_enter();
    DepthBuckets bucket{0.f, 0.f};
    if (bcount != nullptr) bucket = depth_buckets(counters);
    __shared__ float sb[kLidar ? kMaxElevSmem : 1];
    __shared__ unsigned long long wsum[kCountThreads / 32];
    stage_boundaries<kLidar>(a, sb);
    const uint32_t tile_rows = kLidar ? a.lidar.n_tiles_elev : a.cam.tile_height;
    unsigned long long sum = 0;
    uint32_t dmin = 0xffffffffu, dmax = 0u, nvis = 0u;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += gridDim.x * blockDim.x) {
        Rect r;
        int32_t cnt = 0;
        uint32_t xw = 0, yh = 0;
        if (elem_rect<kLidar>(a, idx, r)) {
            cnt = rect_count(r);
            if (rect_xw != nullptr && cnt > 0) {
                const uint32_t sensor = camera_ids ? (uint32_t)camera_ids[idx] : idx / N;
                xw = ((uint32_t)r.x0 & 0xffffu) | ((uint32_t)(r.x1 - r.x0) << 16);
                yh = (sensor * tile_rows + (uint32_t)r.y0) | ((uint32_t)(r.y1 - r.y0) << 16);
            }
        }
        tiles_per_gauss[idx] = cnt;
        if (rect_xw != nullptr) {
            rect_xw[idx] = xw;
            rect_yh[idx] = yh;
        }
        sum += (unsigned long long)(cnt > 0 ? cnt : 0);
        if (depth_bits != nullptr && cnt > 0) {
            const uint32_t d = __ldg(depth_bits + idx);
            dmin = min(dmin, d);
            dmax = max(dmax, d);
            ++nvis;
            if (bcount != nullptr) atomicAdd(&bcount[bucket(d)], 1u);
        }
    }
    if (depth_bits != nullptr) {
        __shared__ uint32_t s_rng[3];
        if (threadIdx.x == 0) { s_rng[0] = 0xffffffffu; s_rng[1] = 0u; s_rng[2] = 0u; }
        __syncthreads();
        dmin = __reduce_min_sync(0xffffffffu, dmin);
        dmax = __reduce_max_sync(0xffffffffu, dmax);
        nvis = __reduce_add_sync(0xffffffffu, nvis);
        if ((threadIdx.x & 31) == 0 && nvis) {
            atomicMin(&s_rng[0], dmin);
            atomicMax(&s_rng[1], dmax);
            atomicAdd(&s_rng[2], nvis);
        }
        __syncthreads();
        if (threadIdx.x == 0 && s_rng[2]) {
            atomicMin(reinterpret_cast<unsigned int *>(counters + CNT_DMIN), s_rng[0]);
            atomicMax(reinterpret_cast<unsigned int *>(counters + CNT_DMAX), s_rng[1]);
            atomicAdd(reinterpret_cast<unsigned long long *>(counters + CNT_NVIS), (unsigned long long)s_rng[2]);
        }
    }
    if (n_isects == nullptr) return;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (uint32_t w = 0; w < blockDim.x / 32; ++w) t += wsum[w];
        if (t) atomicAdd((unsigned long long *)n_isects, t);
        if (early_host != nullptr) {
            // the block that finishes last hands the total straight to the host (a store to mapped
            // pinned memory): nobody waits on anybody, and no copy sits between this kernel and the next
            __threadfence();
            if (atomicAdd((unsigned long long *)ticket, 1ull) + 1ull == (unsigned long long)gridDim.x) {
                __threadfence();
                const unsigned long long total_isects = atomicAdd((unsigned long long *)n_isects, 0ull);
                *ticket = 0;
                tell_host(early_host, early_seq, (int64_t)total_isects, 0);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// Radix sort passes (stable LSD, up to 8 bits per pass) on (uint32 key, uint32 value) pairs.
// Each of the kSortGrid blocks owns a contiguous run of 2048-item tiles.
//   upsweep:   per-block digit histogram            -> hist[digit][block]
//   rowscan:   exclusive scan of each digit's row   -> hist (in place), digit_totals
//   downsweep: stable rank + scatter (through shared memory so global writes are runs)
// Source of a pass is either a pair buffer with a device-side count, or (kGen) the implicit
// list idx = 0..total-1 with key = depth bits, value = idx, restricted to tiles_per_gauss>0.
// ---------------------------------------------------------------------------------------
struct PassSrc {
    const uint32_t *keys;            // pair source
    const uint32_t *vals;
    const int64_t *n_ptr;            // device count (pair source)
    const uint32_t *depth_bits;      // gen source
    const int32_t *tiles_per_gauss;  // gen source
    uint32_t total;                  // gen source length
    uint32_t n_cap;                  // pair source: upper bound on the count (buffer size); 0 = none
};

template <bool kGen>
__device__ __forceinline__ uint32_t src_count(const PassSrc &s) {
    if (kGen) return s.total;
    int64_t n = *s.n_ptr;
    if (s.n_cap != 0 && n > (int64_t)s.n_cap) n = (int64_t)s.n_cap;
    return (uint32_t)n;
}

__device__ __forceinline__ void block_range(uint32_t n, uint32_t &lo, uint32_t &hi) {
    const uint32_t tiles = (n + kTileItems - 1) / kTileItems;
    const uint32_t per = (tiles + gridDim.x - 1) / gridDim.x;
    const uint64_t l = (uint64_t)blockIdx.x * per * kTileItems;
    const uint64_t h = l + (uint64_t)per * kTileItems;
    lo = (uint32_t)(l < n ? l : n);
    hi = (uint32_t)(h < n ? h : n);
}

// Adds one key to the warp-private digit histogram (order is irrelevant for a histogram, so
// plain shared-memory atomics are used; a warp whose 32 keys share one digit - typical for the
// high tile-key digit - does a single add instead of a 32-way serialised atomic).
__device__ __forceinline__ void hist_add(uint32_t *wh_row, bool valid, uint32_t key, int shift,
                                         uint32_t mask, uint32_t lane) {
    const uint32_t digit = valid ? ((key >> shift) & mask) : 0xffffffffu;
    const uint32_t d0 = __shfl_sync(0xffffffffu, digit, 0);
    if (__all_sync(0xffffffffu, digit == d0)) {
        if (lane == 0 && valid) wh_row[d0] += 32u;
        __syncwarp();
    } else if (valid) {
        atomicAdd(&wh_row[digit], 1u);
    }
}

template <bool kGen>
__global__ void __launch_bounds__(kSortThreads)
radix_upsweep_kernel(PassSrc s, int shift, uint32_t mask, uint32_t *__restrict__ hist) {
    chain_enter();
    __shared__ uint32_t wh[kSortWarps][kRadixBins];
    for (uint32_t i = threadIdx.x; i < kSortWarps * kRadixBins; i += blockDim.x) (&wh[0][0])[i] = 0u;
    __syncthreads();
    const uint32_t n = src_count<kGen>(s);
    uint32_t lo, hi;
    block_range(n, lo, hi);   // lo is a multiple of 4096
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint32_t *row = wh[warp];
    const uint32_t *kp = kGen ? s.depth_bits : s.keys;
    const bool aligned = (reinterpret_cast<uintptr_t>(kp) & 15u) == 0 &&
                         (!kGen || (reinterpret_cast<uintptr_t>(s.tiles_per_gauss) & 15u) == 0);
    constexpr uint32_t kStep = kSortThreads * 8;   // two 128-bit loads per thread and iteration
    uint32_t base = lo;
    if (aligned) {
        for (; base + kStep <= hi; base += kStep) {
            const uint32_t i0 = base + threadIdx.x * 4, i1 = i0 + kSortThreads * 4;
            const uint4 k0 = __ldg(reinterpret_cast<const uint4 *>(kp + i0));
            const uint4 k1 = __ldg(reinterpret_cast<const uint4 *>(kp + i1));
            int4 c0 = make_int4(1, 1, 1, 1), c1 = c0;
            if (kGen) {
                c0 = __ldg(reinterpret_cast<const int4 *>(s.tiles_per_gauss + i0));
                c1 = __ldg(reinterpret_cast<const int4 *>(s.tiles_per_gauss + i1));
            }
            hist_add(row, c0.x > 0, k0.x, shift, mask, lane);
            hist_add(row, c0.y > 0, k0.y, shift, mask, lane);
            hist_add(row, c0.z > 0, k0.z, shift, mask, lane);
            hist_add(row, c0.w > 0, k0.w, shift, mask, lane);
            hist_add(row, c1.x > 0, k1.x, shift, mask, lane);
            hist_add(row, c1.y > 0, k1.y, shift, mask, lane);
            hist_add(row, c1.z > 0, k1.z, shift, mask, lane);
            hist_add(row, c1.w > 0, k1.w, shift, mask, lane);
        }
    }
    for (; base < hi; base += kSortThreads) {
        const uint32_t i = base + threadIdx.x;
        bool valid = i < hi;
        uint32_t key = 0;
        if (valid) {
            if (kGen) valid = s.tiles_per_gauss[i] > 0;
            if (valid) key = kp[i];
        }
        hist_add(row, valid, key, shift, mask, lane);
    }
    __syncthreads();
    for (uint32_t d = threadIdx.x; d < kRadixBins; d += blockDim.x) {
        uint32_t sum = 0;
#pragma unroll
        for (int w = 0; w < kSortWarps; ++w) sum += wh[w][d];
        hist[(size_t)d * gridDim.x + blockIdx.x] = sum;
    }
}

// One block per digit; blockDim.x >= grid size of the sort kernels (multiple of 32).
__global__ void radix_rowscan_kernel(uint32_t *__restrict__ hist, uint32_t nblocks,
                                     uint32_t *__restrict__ digit_totals) {
    chain_enter();
    __shared__ uint32_t wt[33];
    const uint32_t d = blockIdx.x;
    const uint32_t b = threadIdx.x;
    uint32_t v = (b < nblocks) ? hist[(size_t)d * nblocks + b] : 0u;
    uint32_t total;
    const uint32_t ex = block_excl_scan(v, wt, total);
    if (b < nblocks) hist[(size_t)d * nblocks + b] = ex;
    if (b == 0) digit_totals[d] = total;
}

struct FinalOut {
    int64_t *isect_ids;          // [capacity]
    int32_t *flatten_ids;        // [capacity]
    const uint32_t *depth_bits;  // [total elems]
    uint32_t n_tiles;            // tiles per sensor
    uint32_t tile_n_bits;
    int64_t capacity;
};

template <bool kGen, bool kFinal>
__global__ void __launch_bounds__(kSortThreads)
radix_downsweep_kernel(PassSrc s, int shift, int nbits, uint32_t mask, const uint32_t *__restrict__ hist,
                       const uint32_t *__restrict__ digit_totals, uint32_t *__restrict__ keys_out,
                       uint32_t *__restrict__ vals_out, FinalOut fin,
                       int64_t *__restrict__ n_out /* optional: total valid count */) {
    chain_enter();
    __shared__ uint32_t wh[kSortWarps][kRadixBins];
    __shared__ uint32_t digit_base[kRadixBins];
    __shared__ uint32_t tile_excl[kRadixBins];
    __shared__ uint32_t tile_cnt[kRadixBins];
    __shared__ uint32_t wt[33];
    __shared__ uint32_t st_keys[kTileItems];
    __shared__ uint32_t st_vals[kTileItems];

    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    {
        uint32_t tot;
        const uint32_t dt = digit_totals[tid];
        const uint32_t ex = block_excl_scan(dt, wt, tot);
        digit_base[tid] = ex + hist[(size_t)tid * gridDim.x + blockIdx.x];
        if (n_out != nullptr && blockIdx.x == 0 && tid == 0) *n_out = (int64_t)tot;
    }
    __syncthreads();

    const uint32_t n = src_count<kGen>(s);
    uint32_t lo, hi;
    block_range(n, lo, hi);

    for (uint32_t tile_lo = lo; tile_lo < hi; tile_lo += kTileItems) {
        for (uint32_t i = tid; i < kSortWarps * kRadixBins; i += kSortThreads) (&wh[0][0])[i] = 0u;
        __syncthreads();

        uint32_t keys[kItemsPerLane], vals[kItemsPerLane];
        uint16_t ranks[kItemsPerLane];
        uint32_t validmask = 0;
        const uint32_t wbase = tile_lo + warp * kWarpItems + lane;
#pragma unroll
        for (int r = 0; r < kItemsPerLane; ++r) {
            const uint32_t i = wbase + r * 32;
            bool valid = i < hi;
            uint32_t key = 0, val = 0;
            if (valid) {
                if (kGen) {
                    valid = s.tiles_per_gauss[i] > 0;
                    if (valid) { key = s.depth_bits[i]; val = i; }
                } else {
                    key = s.keys[i];
                    val = s.vals[i];
                }
            }
            keys[r] = key; vals[r] = val;
            if (valid) validmask |= (1u << r);
        }
#pragma unroll
        for (int r = 0; r < kItemsPerLane; ++r) {
            const bool valid = (validmask >> r) & 1u;
            const uint32_t digit = valid ? ((keys[r] >> shift) & mask) : kRadixBins;
            // lanes with the same digit: one ballot per digit bit (cheaper than match.any when
            // a warp holds many distinct digits)
            uint32_t peers = __ballot_sync(0xffffffffu, valid);
            for (int b = 0; b < nbits; ++b) {
                const uint32_t bal = __ballot_sync(0xffffffffu, (digit >> b) & 1u);
                peers &= ((digit >> b) & 1u) ? bal : ~bal;
            }
            if (!valid) peers = 1u << lane;
            const uint32_t leader = (uint32_t)(__ffs(peers) - 1);
            uint32_t old = 0;
            if (valid && lane == leader) {
                old = wh[warp][digit];
                wh[warp][digit] = old + __popc(peers);
            }
            old = __shfl_sync(0xffffffffu, old, leader);
            ranks[r] = (uint16_t)(old + __popc(peers & ((1u << lane) - 1u)));
            __syncwarp();
        }
        __syncthreads();
        // per digit: exclusive offsets of the warps, tile count, then exclusive scan over digits
        {
            uint32_t run = 0;
#pragma unroll
            for (int w = 0; w < kSortWarps; ++w) {
                const uint32_t c = wh[w][tid];
                wh[w][tid] = run;
                run += c;
            }
            tile_cnt[tid] = run;
            uint32_t tot;
            tile_excl[tid] = block_excl_scan(run, wt, tot);
        }
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kItemsPerLane; ++r) {
            if ((validmask >> r) & 1u) {
                const uint32_t digit = (keys[r] >> shift) & mask;
                const uint32_t pos = tile_excl[digit] + wh[warp][digit] + ranks[r];
                st_keys[pos] = keys[r];
                st_vals[pos] = vals[r];
            }
        }
        __syncthreads();
        const uint32_t tile_n = tile_excl[kRadixBins - 1] + tile_cnt[kRadixBins - 1];
        for (uint32_t j = tid; j < tile_n; j += kSortThreads) {
            const uint32_t k = st_keys[j];
            const uint32_t v = st_vals[j];
            const uint32_t digit = (k >> shift) & mask;
            const uint32_t gpos = digit_base[digit] + (j - tile_excl[digit]);
            if (kFinal) {
                if ((int64_t)gpos < fin.capacity) {
                    const uint32_t cid = k / fin.n_tiles;
                    const uint32_t tile = k - cid * fin.n_tiles;
                    const int64_t id = ((int64_t)cid << (32 + fin.tile_n_bits)) |
                                       ((int64_t)tile << 32) | (int64_t)fin.depth_bits[v];
                    fin.isect_ids[gpos] = id;
                    fin.flatten_ids[gpos] = (int32_t)v;
                }
            } else {
                keys_out[gpos] = k;
                vals_out[gpos] = v;
            }
        }
        __syncthreads();
        digit_base[tid] += tile_cnt[tid];
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kThreads)
depth_bucket_count_kernel(const uint32_t *__restrict__ depth_bits, const int32_t *__restrict__ tiles_per_gauss,
                          uint32_t total, const int64_t *__restrict__ counters, uint32_t *__restrict__ bcount) {
    chain_enter();
    const DepthBuckets bucket = depth_buckets(counters);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x)
        if (tiles_per_gauss[i] > 0) atomicAdd(&bcount[bucket(__ldg(depth_bits + i))], 1u);
}

// Blocks of 1024 threads, one bucket per thread: starts within the block's 1024 buckets, counts
// back to zero (they become the scatter's cursors), the block's total. The block that finishes
// last turns the block totals into block offsets (a bucket's start = bstart[b] + boff[b >> 10]), sets
// the status bit for oversized buckets and - when asked - tells the polling host.
__global__ void __launch_bounds__(1024)
depth_bucket_scan_kernel(uint32_t *__restrict__ bcount, uint32_t *__restrict__ bstart, uint32_t *__restrict__ boff,
                         int64_t *__restrict__ counters, volatile int64_t *early_host, int64_t early_seq) {
    chain_enter();
    __shared__ uint32_t wt[33];
    __shared__ bool s_last;
    const uint32_t b = blockIdx.x * 1024 + threadIdx.x;
    const uint32_t c = bcount[b];
    bcount[b] = 0u;
    uint32_t total;
    bstart[b] = block_excl_scan(c, wt, total);
    const bool big = __syncthreads_or(c > kBucketMax);
    if (threadIdx.x == 0) {
        boff[kBucketScanBlocks + 1 + blockIdx.x] = total;
        if (big) atomicOr((unsigned long long *)&counters[CNT_STATUS], (unsigned long long)ST_DEPTH_BUCKETS);
        __threadfence();
        s_last = atomicAdd((unsigned long long *)&counters[CNT_TICKET], 1ull) + 1ull == (unsigned long long)gridDim.x;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (threadIdx.x < 32) {
        // the block totals: kBucketScanBlocks / 32 consecutive ones per lane
        constexpr uint32_t per = kBucketScanBlocks / 32;
        const volatile uint32_t *tot = boff + kBucketScanBlocks + 1;
        uint32_t v[per], sum = 0;
#pragma unroll
        for (uint32_t k = 0; k < per; ++k) {
            v[k] = tot[per * threadIdx.x + k];
            sum += v[k];
        }
        uint32_t inc = sum;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
            if (threadIdx.x >= (uint32_t)off) inc += o;
        }
        uint32_t run = inc - sum;
#pragma unroll
        for (uint32_t k = 0; k < per; ++k) {
            boff[per * threadIdx.x + k] = run;
            run += v[k];
        }
        if (threadIdx.x == 31) {
            boff[kBucketScanBlocks] = inc;
            counters[CNT_TICKET] = 0;
            __threadfence();
            if (early_host != nullptr)
                tell_host(early_host, early_seq, counters[CNT_NISECT],
                          (int64_t)atomicOr((unsigned long long *)&counters[CNT_STATUS], 0ull),
                          (int64_t)(((unsigned long long)(uint32_t)counters[CNT_DMAX] << 32) |
                                    (unsigned long long)(uint32_t)counters[CNT_DMIN]));
        }
    }
}

__global__ void __launch_bounds__(kThreads)
depth_bucket_scatter_kernel(const uint32_t *__restrict__ depth_bits, const int32_t *__restrict__ tiles_per_gauss,
                            uint32_t total, const int64_t *__restrict__ counters,
                            const uint32_t *__restrict__ bstart, const uint32_t *__restrict__ boff,
                            uint32_t *__restrict__ bcursor, uint2 *__restrict__ pairs /* {bits, flatten index} */) {
    chain_enter();
    const DepthBuckets bucket = depth_buckets(counters);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        if (tiles_per_gauss[i] <= 0) continue;
        const uint32_t d = __ldg(depth_bits + i);
        const uint32_t b = bucket(d);
        const uint32_t pos = bstart[b] + boff[b >> 10] + atomicAdd(&bcursor[b], 1u);
        pairs[pos] = make_uint2(d, i);
    }
}

// One thread per scattered element: its rank among the elements of its bucket in (bits, flatten
// index) order, by counting, and the move to its final place. Neighbouring threads hold neighbouring
// elements, almost always of the same bucket: the loads of the loop are broadcasts.
__global__ void __launch_bounds__(kThreads)
depth_bucket_rank_kernel(const int64_t *__restrict__ counters, const uint32_t *__restrict__ bstart,
                         const uint32_t *__restrict__ boff, const uint2 *__restrict__ pairs,
                         uint32_t *__restrict__ keys_out, uint32_t *__restrict__ vals_out) {
    chain_enter();
    const DepthBuckets bucket = depth_buckets(counters);
    const uint32_t n = boff[kBucketScanBlocks];
    for (uint32_t p = blockIdx.x * blockDim.x + threadIdx.x; p < n; p += gridDim.x * blockDim.x) {
        const uint2 mine = __ldg(pairs + p);
        const uint32_t key = mine.x, val = mine.y;
        const uint32_t b = bucket(key);
        const uint32_t lo = bstart[b] + boff[b >> 10];
        const uint32_t hi = (b + 1 < kDepthBuckets && ((b + 1) & 1023u)) ? bstart[b + 1] + boff[b >> 10]
                            : (b + 1 < kDepthBuckets ? boff[(b + 1) >> 10] : n);
        uint32_t rank = p - lo;                      // crowded bucket: passed through as it is
        if (hi - lo <= kBucketMax) {
            rank = 0;
            const unsigned long long me = ((unsigned long long)key << 32) | val;
#pragma unroll 4
            for (uint32_t j = lo; j < hi; ++j) {
                const uint2 o = __ldg(pairs + j);
                rank += ((((unsigned long long)o.x << 32) | o.y) < me) ? 1u : 0u;
            }
        }
        keys_out[lo + rank] = key;
        vals_out[lo + rank] = val;
    }
}

// ---------------------------------------------------------------------------------------
// Emission of (compact tile key, flatten index) pairs in depth order.
// ---------------------------------------------------------------------------------------
struct EmitArgs {
    const uint32_t *order;           // [n_vis] flatten indices in depth order, or nullptr = identity
    const int64_t *n_order_ptr;      // device count of `order` (ignored for identity)
    uint32_t total;                  // identity length
    const int32_t *tiles_per_gauss;  // [total]
    const int64_t *camera_ids;       // packed: sensor of each row, else nullptr
    uint32_t N;                      // Gaussians per sensor ([C, N] layout)
    uint32_t n_tiles;                // tiles per sensor
    uint32_t tile_n_bits;
    const uint32_t *depth_bits;
    int64_t capacity;
};

__device__ __forceinline__ void emit_range(const EmitArgs &e, uint32_t &lo, uint32_t &hi) {
    const uint32_t n = e.order ? (uint32_t)(*e.n_order_ptr) : e.total;
    const uint32_t chunks = (n + kThreads - 1) / kThreads;
    const uint32_t per = (chunks + gridDim.x - 1) / gridDim.x;
    const uint64_t l = (uint64_t)blockIdx.x * per * kThreads;
    const uint64_t h = l + (uint64_t)per * kThreads;
    lo = (uint32_t)(l < n ? l : n);
    hi = (uint32_t)(h < n ? h : n);
}

__global__ void __launch_bounds__(kThreads)
emit_blocksum_kernel(EmitArgs e, unsigned long long *__restrict__ block_sums) {
    __shared__ unsigned long long ws[kThreads / 32];
    uint32_t lo, hi;
    emit_range(e, lo, hi);
    unsigned long long sum = 0;
    for (uint32_t p = lo + threadIdx.x; p < hi; p += kThreads) {
        const uint32_t idx = e.order ? e.order[p] : p;
        const int32_t c = e.tiles_per_gauss[idx];
        sum += (unsigned long long)(c > 0 ? c : 0);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < kThreads / 32; ++w) t += ws[w];
        block_sums[blockIdx.x] = t;
    }
}

// Single block (1024 threads): exclusive scan of the per-block sums; writes n_isects and the
// status word.
__global__ void __launch_bounds__(1024)
emit_scan_kernel(const unsigned long long *__restrict__ block_sums, uint32_t nblocks,
                 unsigned long long *__restrict__ block_offs, int64_t *__restrict__ counters) {
    __shared__ unsigned long long part[1024];
    const uint32_t t = threadIdx.x;
    const unsigned long long v = (t < nblocks) ? block_sums[t] : 0ull;
    part[t] = v;
    __syncthreads();
    for (uint32_t off = 1; off < 1024; off <<= 1) {
        const unsigned long long o = (t >= off) ? part[t - off] : 0ull;
        __syncthreads();
        part[t] += o;
        __syncthreads();
    }
    if (t < nblocks) block_offs[t] = part[t] - v;
    if (t == 1023) {
        const unsigned long long run = part[1023];
        counters[CNT_NISECT] = (int64_t)run;
        if (run > 0x7fffffffull) counters[CNT_STATUS] |= ST_OVERFLOW_INT32;
    }
}

// Exclusive offset of every entry of the emission order: eoff[p] = number of intersections
// emitted before entry p. Same block ranges as emit_blocksum_kernel.
__global__ void __launch_bounds__(kThreads)
emit_offsets_kernel(EmitArgs e, const unsigned long long *__restrict__ block_offs,
                    uint32_t *__restrict__ eoff) {
    __shared__ uint32_t wt[33];
    uint32_t lo, hi;
    emit_range(e, lo, hi);
    uint32_t running = (uint32_t)block_offs[blockIdx.x];
    for (uint32_t base = lo; base < hi; base += kThreads) {
        const uint32_t p = base + threadIdx.x;
        uint32_t cnt = 0;
        if (p < hi) {
            const uint32_t idx = e.order ? e.order[p] : p;
            const int32_t c = e.tiles_per_gauss[idx];
            cnt = (uint32_t)(c > 0 ? c : 0);
        }
        uint32_t chunk_total;
        const uint32_t ex = block_excl_scan(cnt, wt, chunk_total);
        if (p < hi) eoff[p] = running + ex;
        running += chunk_total;
    }
}

constexpr uint32_t kEmitPerThread = 16;
constexpr uint32_t kEmitUnit = kThreads * kEmitPerThread;   // 4096 intersections per work unit
constexpr uint32_t kEmitEntries = 1024;                     // entries staged per sub-chunk
constexpr uint32_t kEmitUnitsPerBatch = 64;                 // unit windows searched at once

// last p in [lo, hi] with eoff[p] <= q (eoff is non-decreasing, eoff[lo] <= q)
__device__ __forceinline__ uint32_t find_entry(const uint32_t *__restrict__ eoff, uint32_t lo,
                                               uint32_t hi, uint32_t q) {
    while (lo < hi) {
        const uint32_t m = (lo + hi + 1) >> 1;
        if (__ldg(eoff + m) <= q) lo = m; else hi = m - 1;
    }
    return lo;
}

// Writes the intersections in emission order, balanced by OUTPUT position: depth-sorted
// Gaussians have wildly different tile counts (the nearest ones cover thousands of tiles), so
// work is split into units of kEmitUnit consecutive outputs. The entries overlapping a unit are
// staged in shared memory (rectangle computed once per entry), every entry marks the first output
// it owns, and a prefix-max over the unit tells each output which entry it belongs to.
template <bool kLidar, bool kDirect64>
__global__ void __launch_bounds__(kThreads)
emit_kernel(GridArgs<kLidar> a, EmitArgs e, const uint32_t *__restrict__ eoff,
            const int64_t *__restrict__ counters_in, uint32_t *__restrict__ keys_out,
            uint32_t *__restrict__ vals_out, int64_t *__restrict__ ids64_out,
            int32_t *__restrict__ flat_out, int64_t *__restrict__ counters) {
    __shared__ float sb[kLidar ? kMaxElevSmem : 1];
    __shared__ uint32_t s_off[kEmitEntries + 1];
    __shared__ int4 s_rect[kEmitEntries];           // x0, width, y0, sensor
    __shared__ uint32_t s_idx[kEmitEntries];
    __shared__ uint32_t owner[kThreads * (kEmitPerThread + 1)];   // padded: 17 words per thread
    __shared__ uint32_t s_win[2 * kEmitUnitsPerBatch];
    __shared__ uint32_t wmax[kThreads / 32];
    stage_boundaries<kLidar>(a, sb);
    const uint32_t n_entries = e.order ? (uint32_t)(*e.n_order_ptr) : e.total;
    const int64_t m_total = counters_in[CNT_NISECT];
    int64_t m64 = m_total;
    bool overflow = false;
    if (m64 > e.capacity) { m64 = e.capacity; overflow = true; }
    const uint32_t M = (uint32_t)m64;
    if (n_entries == 0 || M == 0) return;
    const uint32_t n_units = (M + kEmitUnit - 1) / kEmitUnit;
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (uint32_t u0 = blockIdx.x; u0 < n_units; u0 += gridDim.x * kEmitUnitsPerBatch) {
        // entry windows of this block's next units, searched in parallel
        __syncthreads();
        if (tid < 2 * kEmitUnitsPerBatch) {
            const uint32_t u = u0 + (tid >> 1) * gridDim.x;
            if (u < n_units) {
                const uint32_t q_lo = u * kEmitUnit;
                const uint32_t q_last = min(M, q_lo + kEmitUnit) - 1;
                s_win[tid] = find_entry(eoff, 0, n_entries - 1, (tid & 1) ? q_last : q_lo);
            }
        }
        __syncthreads();
        for (uint32_t b = 0; b < kEmitUnitsPerBatch; ++b) {
            const uint32_t u = u0 + b * gridDim.x;
            if (u >= n_units) break;
            const uint32_t q_lo = u * kEmitUnit;
            const uint32_t q_hi = min(M, q_lo + kEmitUnit);   // exclusive
            const uint32_t p_lo = s_win[2 * b], p_hi = s_win[2 * b + 1];
            for (uint32_t c_lo = p_lo; c_lo <= p_hi; c_lo += kEmitEntries) {
                const uint32_t c_hi = min(p_hi, c_lo + kEmitEntries - 1);
                const uint32_t n_e = c_hi - c_lo + 1;
                __syncthreads();
                for (uint32_t i = tid; i < n_e; i += kThreads) {
                    const uint32_t p = c_lo + i;
                    const uint32_t idx = e.order ? __ldg(e.order + p) : p;
                    Rect r;
                    int4 packed = make_int4(0, 0, 0, 0);
                    if (elem_rect<kLidar>(a, idx, r)) {
                        packed.x = r.x0;
                        packed.y = r.x1 - r.x0;
                        packed.z = r.y0;
                        packed.w = (int32_t)(e.camera_ids ? (uint32_t)e.camera_ids[idx] : idx / e.N);
                    }
                    s_off[i] = __ldg(eoff + p);
                    s_rect[i] = packed;
                    s_idx[i] = idx;
                }
                if (tid == 0)
                    s_off[n_e] = (c_hi + 1 < n_entries) ? __ldg(eoff + c_hi + 1)
                                                        : (uint32_t)min(m_total, (int64_t)0xffffffffll);
                for (uint32_t i = tid; i < kThreads * (kEmitPerThread + 1); i += kThreads) owner[i] = 0u;
                __syncthreads();
                // outputs of this unit covered by the staged entries
                const uint32_t o_lo = max(q_lo, s_off[0]);
                const uint32_t o_hi = min(q_hi, s_off[n_e]);
                for (uint32_t i = tid; i < n_e; i += kThreads) {
                    const uint32_t s0 = s_off[i], s1 = s_off[i + 1];
                    if (s1 > s0 && s1 > o_lo && s0 < o_hi) {
                        const uint32_t j = max(s0, o_lo) - o_lo;
                        owner[j + j / kEmitPerThread] = i + 1;
                    }
                }
                __syncthreads();
                // inclusive prefix-max over owner: per-thread segment, then across threads
                uint32_t run = 0;
                uint32_t *seg = owner + tid * (kEmitPerThread + 1);
#pragma unroll
                for (uint32_t k = 0; k < kEmitPerThread; ++k) {
                    run = max(run, seg[k]);
                    seg[k] = run;
                }
                uint32_t inc = run;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
                    if (lane >= (uint32_t)off) inc = max(inc, o);
                }
                if (lane == 31) wmax[warp] = inc;
                __syncthreads();
                uint32_t prefix = __shfl_up_sync(0xffffffffu, inc, 1);
                if (lane == 0) prefix = 0;
                for (uint32_t w = 0; w < warp; ++w) prefix = max(prefix, wmax[w]);
#pragma unroll
                for (uint32_t k = 0; k < kEmitPerThread; ++k) seg[k] = max(seg[k], prefix);
                __syncthreads();
                // coalesced emission
                const uint32_t n_out = o_hi > o_lo ? o_hi - o_lo : 0u;
                for (uint32_t j = tid; j < n_out; j += kThreads) {
                    const uint32_t own = owner[j + j / kEmitPerThread];
                    if (own == 0) continue;   // cannot happen: every output has an owner
                    const uint32_t i = own - 1;
                    const int4 r = s_rect[i];
                    const uint32_t q = o_lo + j;
                    const uint32_t k = q - s_off[i];
                    const uint32_t w = (uint32_t)r.y;
                    const uint32_t dy = k / w;
                    const uint32_t dx = k - dy * w;
                    const int32_t ty = r.z + (int32_t)dy;
                    int32_t tx = r.x + (int32_t)dx;
                    uint32_t tile;
                    if (kLidar) {
                        const int32_t na = (int32_t)a.lidar.n_tiles_azim;
                        tx %= na;
                        if (tx < 0) tx += na;
                        tile = (uint32_t)ty * a.lidar.n_tiles_azim + (uint32_t)tx;
                    } else {
                        tile = (uint32_t)ty * a.cam.tile_width + (uint32_t)tx;
                    }
                    const uint32_t idx = s_idx[i];
                    if (kDirect64) {
                        ids64_out[q] = ((int64_t)(uint32_t)r.w << (32 + e.tile_n_bits)) |
                                       ((int64_t)tile << 32) | (int64_t)e.depth_bits[idx];
                        flat_out[q] = (int32_t)idx;
                    } else {
                        keys_out[q] = (uint32_t)r.w * e.n_tiles + tile;
                        vals_out[q] = idx;
                    }
                }
            }
        }
    }
    if (overflow && blockIdx.x == 0 && threadIdx.x == 0)
        atomicOr((unsigned long long *)&counters[CNT_STATUS], (unsigned long long)ST_OVERFLOW_CAPACITY);
}

// ---------------------------------------------------------------------------------------
// Row / column split (at most 128 tile rows and 16384 tiles over all sensors, rows of at most
// 1024 tiles: a lidar with 57 x 16 tiles, a 1920 x 1080 camera with 120 x 68): builds the
// per-tile lists without ever writing the emission out.
//
// A rectangle is a stack of `h` row runs, each `w` tiles wide. The tile lists of grid row r are
// made of the row runs of the rectangles that cover r, in depth order, so the split is done in
// two stable steps that both write long contiguous runs:
//   A. rows:    every depth-ordered entry appends one record (run start, width, flatten index,
//               depth bits, running output offset) to the bucket of each grid row it covers.
//               Ranks inside a bucket come from one ballot per (32 entries, row); the offsets
//               from a warp prefix sum of the widths. ~0.4 records per intersection.
//   B. columns: the records of a row, expanded to their `w` outputs, are cut into units of
//               4096 consecutive outputs (one block each, 512 per warp). The number of outputs
//               per column of a piece comes from +1 / -1 updates of a difference row; inside a
//               piece the warp walks 32 outputs at a time: the records that start inside the
//               32 outputs set one bit each, which tells every lane its record, and lanes that
//               hit the same column are ranked in lane order (one ballot per column bit). The
//               4096 outputs are put in tile order in shared memory and leave as ~70-entry
//               runs per tile.
// Positions are exclusive sums over (earlier tiles, earlier units, earlier warps), all of
// them plain scans: the result is the same for any scheduling.
// ---------------------------------------------------------------------------------------
constexpr uint32_t kSplitMaxRows = 128;                    // grid rows over all sensors
constexpr uint32_t kSplitMaxWidth = 1024;                  // tiles per row
constexpr uint32_t kSplitMaxTiles = 16384;
constexpr uint32_t kSplitMaxSlots = kSplitMaxTiles + kSplitMaxRows;   // rows * (row_width + 1)
constexpr uint32_t kSplitWarps = 8;
// Entries per warp in step A, chosen per call: 128 for grids of up to 32 rows, 32 above (a warp walks
// its entries 32 at a time and loops over the rows for each window: with many rows that chain gets
// long and short pieces keep more warps in flight; config 1, 68 rows: step A 119 -> 71 us).
constexpr uint32_t kSplitWarpEntriesMin = 32, kSplitWarpEntriesMax = 128;
constexpr uint32_t kSplitSub = 512;                        // outputs per warp in step B
constexpr uint32_t kSplitUnit = kSplitWarps * kSplitSub;   // outputs per block in step B
constexpr uint32_t kSplitColBits = 11;

struct SplitArgs {
    uint32_t warp_entries;       // step A: entries per warp (a multiple of 32)
    // entries: rectangles by flatten index, visited in depth order
    const uint32_t *rect_xw;     // [total] x0 | width << 16
    const uint32_t *rect_yh;     // [total] first grid row | height << 16
    const uint32_t *order;       // [n_entries] flatten index, depth order
    const uint32_t *depth_key;   // [n_entries] depth bits
    const int64_t *n_entries_ptr;
    const int64_t *counters;     // CNT_NISECT
    int64_t capacity;
    uint32_t rows;               // grid rows over all sensors
    uint32_t tile_rows;          // rows per sensor
    uint32_t row_width, stride;  // tiles per row, row_width + 1
    uint32_t tile_n_bits, col_bits, wrap;
    // workspace
    uint32_t *ha_cnt, *ha_out;   // [blocks][rows]: records / outputs per (1024 entries, row); scanned
    uint32_t *hw_cnt, *hw_out;   // [blocks][warps][rows]: the same per warp (128 entries), as counted
    uint32_t *row_rec, *row_out, *row_unit;   // [rows + 1] exclusive starts
    uint4 *rec;                  // records {run start | width << 16, output offset, flatten index,
                                 // depth bits}, row bucket after row bucket
    uint32_t *hb;                // [units_b][stride] outputs per (unit, column); after the scan:
                                 // outputs of the column in earlier units of the row
    uint32_t *hw;                // [units_b][warps][stride] outputs per (unit, warp, column)
    uint32_t *hb_first;          // [units_b][warps] record owning the first output of the warp
    uint32_t *slot_tot, *slot_base;           // [rows * stride]
};

// Warp-cooperative search: last record p in [lo, hi] whose output offset is <= q (offsets are
// non-decreasing, that of lo is <= q). 32 probes per round.
__device__ __forceinline__ uint32_t rec_off(const SplitArgs &a, uint32_t p) {
    return __ldg(reinterpret_cast<const uint32_t *>(a.rec + p) + 1);
}

// ---- step A: rows -----------------------------------------------------------------------
struct SplitEntry {
    uint32_t xw, row0, h, idx;
    bool valid;
};

__device__ __forceinline__ SplitEntry split_load_entry(const SplitArgs &a, uint32_t p, uint32_t n_entries) {
    SplitEntry e{0u, 0u, 0u, 0u, p < n_entries};
    if (e.valid) {
        e.idx = __ldg(a.order + p);
        e.xw = __ldg(a.rect_xw + e.idx);
        const uint32_t yh = __ldg(a.rect_yh + e.idx);
        e.row0 = yh & 0xffffu;
        e.h = yh >> 16;
    }
    return e;
}

// Records and outputs per grid row of the a.warp_entries entries starting at `first`, for the
// 32 rows starting at `row_lo`; lane l holds row row_lo + l.
__device__ __forceinline__ void split_rows_of_warp(const SplitArgs &a, uint32_t first, uint32_t n_entries,
                                                   uint32_t lane, uint32_t row_lo, uint32_t &cnt,
                                                   uint32_t &out) {
    cnt = 0;
    out = 0;
    const uint32_t row_hi = min(a.rows, row_lo + 32u);
    for (uint32_t win = 0; win < a.warp_entries / 32; ++win) {
        const uint32_t base = first + win * 32;
        if (base >= n_entries) break;
        const SplitEntry e = split_load_entry(a, base + lane, n_entries);
        const uint32_t w = e.xw >> 16;
        for (uint32_t r = row_lo; r < row_hi; ++r) {
            const bool hit = e.valid && (r - e.row0) < e.h;
            const uint32_t bal = __ballot_sync(0xffffffffu, hit);
            if (bal == 0u) continue;
            const uint32_t s = __reduce_add_sync(0xffffffffu, hit ? w : 0u);
            if (row_lo + lane == r) {
                cnt += __popc(bal);
                out += s;
            }
        }
    }
}

// More intersections than output slots: the split is skipped altogether (the record arrays are
// sized by the capacity) and only the status bit is raised.
__device__ __forceinline__ bool split_overflow(const SplitArgs &a) {
    return a.counters[CNT_NISECT] > a.capacity;
}

__global__ void __launch_bounds__(kSplitWarps * 32)
rowsplit_count_kernel(SplitArgs a) {
    chain_enter();
    __shared__ uint32_t s_cnt[kSplitMaxRows], s_out[kSplitMaxRows];
    if (split_overflow(a)) return;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t n_entries = (uint32_t)(*a.n_entries_ptr);
    const uint32_t first = blockIdx.x * kSplitWarps * a.warp_entries;
    if (first >= n_entries) return;
    if (threadIdx.x < kSplitMaxRows) {
        s_cnt[threadIdx.x] = 0;
        s_out[threadIdx.x] = 0;
    }
    __syncthreads();
    const uint32_t wu = blockIdx.x * kSplitWarps + warp;
    for (uint32_t row_lo = 0; row_lo < a.rows; row_lo += 32) {
        uint32_t cnt, out;
        split_rows_of_warp(a, first + warp * a.warp_entries, n_entries, lane, row_lo, cnt, out);
        const uint32_t r = row_lo + lane;
        if (r < a.rows) {
            // kept per warp too, so that the scatter does not have to count again
            a.hw_cnt[wu * a.rows + r] = cnt;
            a.hw_out[wu * a.rows + r] = out;
            if (cnt) {
                atomicAdd(&s_cnt[r], cnt);
                atomicAdd(&s_out[r], out);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x < a.rows) {
        a.ha_cnt[blockIdx.x * a.rows + threadIdx.x] = s_cnt[threadIdx.x];
        a.ha_out[blockIdx.x * a.rows + threadIdx.x] = s_out[threadIdx.x];
    }
}

// Block r: exclusive scan over the entry blocks of grid row r (in place). The block that
// finishes last turns the row totals into the row starts of records, outputs and step-B units.
__global__ void __launch_bounds__(1024)
rowsplit_scan_kernel(SplitArgs a, unsigned long long *__restrict__ ticket) {
    chain_enter();
    __shared__ uint32_t wt[33];
    __shared__ bool s_last;
    const uint32_t r = blockIdx.x, tid = threadIdx.x;
    if (split_overflow(a)) return;
    const uint32_t n_entries = (uint32_t)(*a.n_entries_ptr);
    const uint32_t block_entries = kSplitWarps * a.warp_entries;
    const uint32_t n_units = (n_entries + block_entries - 1) / block_entries;
    uint32_t carry_c = 0, carry_o = 0;
    for (uint32_t u0 = 0; u0 < n_units; u0 += 1024) {
        const uint32_t u = u0 + tid;
        const bool live = u < n_units;
        const uint32_t vc = live ? a.ha_cnt[u * a.rows + r] : 0u;
        const uint32_t vo = live ? a.ha_out[u * a.rows + r] : 0u;
        uint32_t tc, to;
        const uint32_t ec = block_excl_scan(vc, wt, tc);
        const uint32_t eo = block_excl_scan(vo, wt, to);
        if (live) {
            a.ha_cnt[u * a.rows + r] = carry_c + ec;
            a.ha_out[u * a.rows + r] = carry_o + eo;
        }
        carry_c += tc;
        carry_o += to;
    }
    // row totals, parked in the upper half of the row tables until the last block arrives
    if (tid == 0) {
        a.row_rec[kSplitMaxRows + 1 + r] = carry_c;
        a.row_out[kSplitMaxRows + 1 + r] = carry_o;
        __threadfence();
        s_last = atomicAdd(ticket, 1ull) + 1ull == (unsigned long long)gridDim.x;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // exclusive scans over the rows (rows <= 128 <= blockDim)
    const uint32_t vc = tid < a.rows ? a.row_rec[kSplitMaxRows + 1 + tid] : 0u;
    const uint32_t vo = tid < a.rows ? a.row_out[kSplitMaxRows + 1 + tid] : 0u;
    const uint32_t vu = (vo + kSplitUnit - 1) / kSplitUnit;
    uint32_t tc, to, tu;
    const uint32_t ec = block_excl_scan(vc, wt, tc);
    const uint32_t eo = block_excl_scan(vo, wt, to);
    const uint32_t eu = block_excl_scan(vu, wt, tu);
    if (tid < a.rows) {
        a.row_rec[tid] = ec;
        a.row_out[tid] = eo;
        a.row_unit[tid] = eu;
    }
    if (tid == 0) {
        a.row_rec[a.rows] = tc;
        a.row_out[a.rows] = to;
        a.row_unit[a.rows] = tu;
        *ticket = 0ull;
    }
}

// kOneGroup: at most 32 grid rows, so the loop over groups of 32 rows runs once from row 0.
template <bool kOneGroup>
__global__ void __launch_bounds__(kSplitWarps * 32)
rowsplit_scatter_kernel(SplitArgs a) {
    chain_enter();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t lt = (1u << lane) - 1u;
    if (split_overflow(a)) return;
    const uint32_t n_entries = (uint32_t)(*a.n_entries_ptr);
    const uint32_t wu = blockIdx.x * kSplitWarps + warp;
    const uint32_t first = wu * a.warp_entries;
    if (first >= n_entries) return;
    const uint32_t cap = (uint32_t)(a.capacity < 0x7fffffffll ? a.capacity : 0x7fffffffll);
    for (uint32_t row_lo = 0; row_lo < (kOneGroup ? 1u : a.rows); row_lo += 32) {
        // lane l: where this warp's records / outputs of row row_lo + l start: row start, earlier
        // blocks (scanned), earlier warps of this block (as counted)
        const uint32_t row_hi = min(a.rows, row_lo + 32u);
        const uint32_t my_row = row_lo + lane;
        uint32_t rec_at = 0, out_at = 0, row_start = 0, row_piece0 = 0;
        if (my_row < a.rows) {
            row_start = a.row_out[my_row];
            row_piece0 = a.row_unit[my_row] * kSplitWarps;   // first step-B piece of the row
            rec_at = a.row_rec[my_row] + a.ha_cnt[blockIdx.x * a.rows + my_row];
            out_at = row_start + a.ha_out[blockIdx.x * a.rows + my_row];
            for (uint32_t w2 = blockIdx.x * kSplitWarps; w2 < wu; ++w2) {
                rec_at += a.hw_cnt[w2 * a.rows + my_row];
                out_at += a.hw_out[w2 * a.rows + my_row];
            }
        }
        for (uint32_t win = 0; win < a.warp_entries / 32; ++win) {
            const uint32_t base = first + win * 32;
            if (base >= n_entries) break;
            const uint32_t p = base + lane;
            const SplitEntry e = split_load_entry(a, p, n_entries);
            const uint32_t w = e.xw >> 16;
            uint32_t xs = 0, idx = 0, depth = 0;
            if (e.valid) {
                int32_t x0 = (int32_t)(int16_t)(e.xw & 0xffffu);
                if (a.wrap) {
                    x0 %= (int32_t)a.row_width;
                    if (x0 < 0) x0 += (int32_t)a.row_width;
                }
                xs = (uint32_t)x0;
                idx = e.idx;
                depth = __ldg(a.depth_key + p);
            }
            for (uint32_t r = row_lo; r < row_hi; ++r) {
                const bool hit = e.valid && (r - e.row0) < e.h;
                const uint32_t bal = __ballot_sync(0xffffffffu, hit);
                if (bal == 0u) continue;
                // exclusive prefix of the widths of the hit lanes
                const uint32_t v = hit ? w : 0u;
                uint32_t inc = v;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const uint32_t o = __shfl_up_sync(0xffffffffu, inc, off);
                    if (lane >= (uint32_t)off) inc += o;
                }
                const uint32_t total = __shfl_sync(0xffffffffu, inc, 31);
                const uint32_t rbase = __shfl_sync(0xffffffffu, rec_at, r - row_lo);
                const uint32_t obase = __shfl_sync(0xffffffffu, out_at, r - row_lo);
                const uint32_t rstart = __shfl_sync(0xffffffffu, row_start, r - row_lo);
                const uint32_t rpiece0 = __shfl_sync(0xffffffffu, row_piece0, r - row_lo);
                if (hit) {
                    const uint32_t pos = rbase + __popc(bal & lt);
                    const uint32_t s0 = obase + inc - v;
                    if (pos < cap) {
                        a.rec[pos] = make_uint4(xs | (w << 16), s0, idx, depth);
                        // step B cuts the row's outputs into pieces of kSplitSub: the record that
                        // holds the first output of a piece is noted for it
                        const uint32_t rel = s0 - rstart;
                        for (uint32_t m = (rel + kSplitSub - 1) / kSplitSub; m * kSplitSub < rel + w; ++m)
                            a.hb_first[rpiece0 + m] = pos;
                    }
                }
                if (my_row == r) {
                    rec_at += __popc(bal);
                    out_at += total;
                }
            }
        }
    }
}

// ---- step B: columns --------------------------------------------------------------------
struct SplitUnit {
    uint32_t row, q_lo, q_hi;   // grid row and output range
    uint32_t n_rec, n_out;      // records / outputs in all rows
    bool live;
};

__device__ __forceinline__ SplitUnit split_unit(const SplitArgs &a, uint32_t u, uint32_t lane) {
    SplitUnit s{};
    const uint32_t n_units = a.row_unit[a.rows];
    s.n_rec = a.row_rec[a.rows];
    s.n_out = a.row_out[a.rows];
    s.live = u < n_units;
    if (!s.live) return s;
    // last row whose first unit is <= u (rows without outputs own no unit and are passed over)
    if (a.rows <= 32) {   // one probe per lane
        const uint32_t m = __ballot_sync(0xffffffffu, lane < a.rows && a.row_unit[lane] <= u);
        s.row = 31u - __clz(m);
    } else {
        uint32_t lo = 0, hi = a.rows - 1;
        while (lo < hi) {
            const uint32_t m = (lo + hi + 1) >> 1;
            if (a.row_unit[m] <= u) lo = m; else hi = m - 1;
        }
        s.row = lo;
    }
    const uint32_t k = u - a.row_unit[s.row];
    const uint32_t row_end = a.row_out[s.row + 1];
    s.q_lo = min(row_end, a.row_out[s.row] + k * kSplitUnit);
    s.q_hi = min(row_end, s.q_lo + kSplitUnit);
    return s;
}

// Adds the outputs [q_lo, q_hi) to a difference row (one record per lane), starting at the record
// `first` that owns output q_lo (noted by step A's scatter).
__device__ __forceinline__ void split_count_cols(int32_t *d, const SplitArgs &a, uint32_t q_lo,
                                                 uint32_t q_hi, uint32_t n_rec, uint32_t n_out,
                                                 uint32_t first, uint32_t lane) {
    if (q_lo >= q_hi || n_rec == 0) return;
    const uint32_t rw = a.row_width;
    uint32_t base = first;
    while (true) {
        const uint32_t p = base + lane;
        uint32_t s1 = 0u;
        if (p < n_rec) {
            const uint2 xo = __ldg(reinterpret_cast<const uint2 *>(a.rec + p));
            const uint32_t s0 = xo.y;
            s1 = (p + 1 < n_rec) ? rec_off(a, p + 1) : n_out;
            if (s0 < q_hi && s1 > q_lo) {
                const uint32_t xw = xo.x;
                const uint32_t k_lo = max(s0, q_lo) - s0, k_hi = min(s1, q_hi) - s0;
                uint32_t start = (xw & 0xffffu) + k_lo;
                uint32_t len = k_hi - k_lo;
                if (a.wrap) {
                    if (len >= rw) {   // the run covers every tile of the row `full` times
                        const int32_t full = (int32_t)(len / rw);
                        atomicAdd(d, full);
                        atomicAdd(d + rw, -full);
                        len -= (uint32_t)full * rw;
                    }
                    if (len) {
                        if (start >= rw) start %= rw;
                        const uint32_t end = start + len;
                        atomicAdd(d + start, 1);
                        if (end <= rw) {
                            atomicAdd(d + end, -1);
                        } else {
                            atomicAdd(d + rw, -1);
                            atomicAdd(d, 1);
                            atomicAdd(d + (end - rw), -1);
                        }
                    }
                } else if (start + len <= rw) {
                    atomicAdd(d + start, 1);
                    atomicAdd(d + start + len, -1);
                }
            }
        }
        const uint32_t last_s1 = __shfl_sync(0xffffffffu, s1, 31);
        if (base + 32 >= n_rec || last_s1 >= q_hi) break;
        base += 32;
    }
}

// In-place inclusive prefix sum of d[0 .. n) by one warp.
__device__ __forceinline__ void warp_prefix_inplace(int32_t *d, uint32_t n, uint32_t lane) {
    int32_t carry = 0;
    for (uint32_t i0 = 0; i0 < n; i0 += 32) {
        const uint32_t i = i0 + lane;
        int32_t v = i < n ? d[i] : 0;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int32_t o = __shfl_up_sync(0xffffffffu, v, off);
            if (lane >= (uint32_t)off) v += o;
        }
        v += carry;
        if (i < n) d[i] = v;
        carry = __shfl_sync(0xffffffffu, v, 31);
    }
}

__global__ void __launch_bounds__(kSplitWarps * 32)
colsplit_count_kernel(SplitArgs a) {
    chain_enter();
    extern __shared__ int32_t s_d[];   // [kSplitWarps][stride]
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (split_overflow(a)) return;
    const SplitUnit u = split_unit(a, blockIdx.x, lane);
    if (!u.live) return;
    int32_t *wd = s_d + warp * a.stride;
    for (uint32_t i = lane; i < a.stride; i += 32) wd[i] = 0;
    __syncwarp();
    const uint32_t q_lo = min(u.q_hi, u.q_lo + warp * kSplitSub);
    const uint32_t q_hi = min(u.q_hi, q_lo + kSplitSub);
    const size_t piece = (size_t)blockIdx.x * kSplitWarps + warp;
    const uint32_t first = q_lo < q_hi ? min(a.hb_first[piece], u.n_rec ? u.n_rec - 1 : 0u) : 0u;
    split_count_cols(wd, a, q_lo, q_hi, u.n_rec, u.n_out, first, lane);
    __syncwarp();
    warp_prefix_inplace(wd, a.stride, lane);
    __syncthreads();
    // per warp (so that the scatter does not have to count again) and per unit (to be scanned)
    uint32_t *prow = a.hw + piece * a.stride;
    for (uint32_t i = lane; i < a.stride; i += 32) prow[i] = (uint32_t)wd[i];
    uint32_t *row = a.hb + (size_t)blockIdx.x * a.stride;
    for (uint32_t i = tid; i < a.stride; i += blockDim.x) {
        uint32_t tot = 0;
#pragma unroll
        for (uint32_t w2 = 0; w2 < kSplitWarps; ++w2) tot += (uint32_t)s_d[w2 * a.stride + i];
        row[i] = tot;
    }
}

// One block per grid row and group of 32 columns: exclusive scan over the units of the row for
// those columns (in place); the column totals go to slot_tot[r][col]. The block that finishes last (an atomic ticket, nobody waits)
// scans the totals into slot_base and, when asked, writes the tile offsets - the slot starts
// without the closing column of every row - followed by the total.
__global__ void __launch_bounds__(1024)
colsplit_scan_kernel(SplitArgs a, unsigned long long *__restrict__ ticket, int32_t *__restrict__ offsets) {
    chain_enter();
    __shared__ uint32_t seg_sum[32][33];
    __shared__ uint32_t wt[33];
    __shared__ bool s_last;
    const uint32_t lane = threadIdx.x & 31, seg = threadIdx.x >> 5;
    // one block per (grid row, group of 32 columns)
    const uint32_t n_groups = (a.stride + 31) / 32;
    const uint32_t r = blockIdx.x / n_groups, c_first = (blockIdx.x - r * n_groups) * 32;
    const uint32_t n_tiles = a.rows * a.row_width;
    if (split_overflow(a)) {
        // the split is skipped for lack of room: every offset 0, so that compositing enqueued
        // behind it finds empty tiles instead of stale numbers
        if (offsets != nullptr)
            for (uint32_t t = blockIdx.x * 1024 + threadIdx.x; t <= n_tiles; t += gridDim.x * 1024) offsets[t] = 0;
        return;
    }
    const uint32_t ub0 = a.row_unit[r], n_units = a.row_unit[r + 1] - ub0;
    const uint32_t per = (n_units + 31) / 32;
    const uint32_t u_lo = min(n_units, seg * per), u_hi = min(n_units, u_lo + per);
    const size_t S = a.stride;
    {
        const uint32_t c = c_first + lane;
        const bool live = c < a.stride;
        uint32_t *col = a.hb + (size_t)ub0 * S + c;
        uint32_t sum = 0;
        if (live) {
            uint32_t u = u_lo;
            for (; u + 4 <= u_hi; u += 4) {
                const uint32_t *h = col + (size_t)u * S;
                const uint32_t v0 = h[0], v1 = h[S], v2 = h[2 * S], v3 = h[3 * S];
                sum += v0 + v1 + v2 + v3;
            }
            for (; u < u_hi; ++u) sum += col[(size_t)u * S];
        }
        __syncthreads();
        seg_sum[seg][lane] = sum;
        __syncthreads();
        uint32_t prefix = 0, total = 0;
        for (uint32_t s2 = 0; s2 < 32; ++s2) {
            const uint32_t v = seg_sum[s2][lane];
            if (s2 < seg) prefix += v;
            total += v;
        }
        if (live) {
            uint32_t run = prefix;
            for (uint32_t u = u_lo; u < u_hi; ++u) {
                uint32_t *h = col + (size_t)u * S;
                const uint32_t v = *h;
                *h = run;
                run += v;
            }
            if (seg == 0) a.slot_tot[r * a.stride + c] = total;
        }
    }
    __threadfence();   // the writers of slot_tot publish before the ticket is taken
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        s_last = atomicAdd(ticket, 1ull) + 1ull == (unsigned long long)gridDim.x;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // slot_base = exclusive scan of slot_tot, two slots per thread and 2048 per round
    const uint32_t n_slots = a.rows * a.stride;
    uint32_t total = 0;
    for (uint32_t s0 = 0; s0 < n_slots; s0 += 2048) {
        const uint32_t i0 = s0 + 2 * threadIdx.x, i1 = i0 + 1;
        const uint32_t v0 = i0 < n_slots ? a.slot_tot[i0] : 0u;
        const uint32_t v1 = i1 < n_slots ? a.slot_tot[i1] : 0u;
        uint32_t round_total;
        const uint32_t ex = block_excl_scan(v0 + v1, wt, round_total);
        if (i0 < n_slots) a.slot_base[i0] = total + ex;
        if (i1 < n_slots) a.slot_base[i1] = total + ex + v0;
        total += round_total;
    }
    if (threadIdx.x == 0) *ticket = 0ull;
    if (offsets == nullptr) return;
    __syncthreads();
    for (uint32_t t = threadIdx.x; t <= n_tiles; t += 1024) {
        const uint32_t rr = t / a.row_width, c = t - rr * a.row_width;
        offsets[t] = (t == n_tiles) ? (int32_t)total : (int32_t)a.slot_base[rr * a.stride + c];
    }
}

struct SplitWindow {
    uint32_t xw, s0, s1, idx, depth;
};

__device__ __forceinline__ SplitWindow split_load_window(const SplitArgs &a, uint32_t base, uint32_t lane,
                                                         uint32_t n_rec, uint32_t n_out) {
    SplitWindow win{0u, 0u, 0u, 0u, 0u};
    const uint32_t p = base + lane;
    if (p < n_rec) {
        const uint4 r = __ldg(a.rec + p);
        win.xw = r.x;
        win.s0 = r.y;
        win.s1 = (p + 1 < n_rec) ? rec_off(a, p + 1) : n_out;
        win.idx = r.z;
        win.depth = r.w;
    }
    return win;
}

__global__ void __launch_bounds__(kSplitWarps * 32)
colsplit_scatter_kernel(SplitArgs a, int64_t *__restrict__ isect_ids, int32_t *__restrict__ flatten_ids,
                        int64_t *__restrict__ counters) {
    chain_enter();
    extern __shared__ int32_t s_dyn[];
    // [kSplitWarps][stride] column tables, [stride] global - local start, staged outputs
    int32_t *s_tab = s_dyn;
    int32_t *s_shift = s_tab + kSplitWarps * a.stride;
    uint32_t *st_depth = reinterpret_cast<uint32_t *>(s_shift + a.stride);
    uint32_t *st_idx = st_depth + kSplitUnit;
    uint16_t *st_col = reinterpret_cast<uint16_t *>(st_idx + kSplitUnit);
    __shared__ uint32_t wt[33];
    const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t lt = (1u << lane) - 1u, le = 0xffffffffu >> (31 - lane);
    if (split_overflow(a)) {
        if (blockIdx.x == 0 && tid == 0)
            atomicOr((unsigned long long *)&counters[CNT_STATUS], (unsigned long long)ST_OVERFLOW_CAPACITY);
        return;
    }
    const SplitUnit u = split_unit(a, blockIdx.x, lane);
    if (!u.live) return;
    const uint32_t cap = (uint32_t)(a.capacity < 0x7fffffffll ? a.capacity : 0x7fffffffll);
    const uint32_t q_lo = min(u.q_hi, u.q_lo + warp * kSplitSub);
    const uint32_t q_hi = min(u.q_hi, q_lo + kSplitSub);
    int32_t *wd = s_tab + warp * a.stride;
    uint32_t *hist = reinterpret_cast<uint32_t *>(wd);

    // Local start of every (warp, column) inside the unit, and the shift to global positions: the
    // per-warp counts come from the count kernel, the unit's global starts from the scans.
    const size_t piece0 = (size_t)blockIdx.x * kSplitWarps;
    const uint32_t *hrow = a.hb + (size_t)blockIdx.x * a.stride;
    const uint32_t *sbase = a.slot_base + u.row * a.stride;
    uint32_t carry = 0;
    for (uint32_t c0 = 0; c0 < a.stride; c0 += blockDim.x) {
        const uint32_t c = c0 + tid;
        uint32_t cnt[kSplitWarps], tot = 0;
#pragma unroll
        for (uint32_t w2 = 0; w2 < kSplitWarps; ++w2) {
            cnt[w2] = c < a.stride ? a.hw[(piece0 + w2) * a.stride + c] : 0u;
            tot += cnt[w2];
        }
        uint32_t chunk_total;
        const uint32_t ex = block_excl_scan(tot, wt, chunk_total);
        if (c < a.stride) {
            uint32_t run = carry + ex;
            s_shift[c] = (int32_t)(hrow[c] + sbase[c] - run);
#pragma unroll
            for (uint32_t w2 = 0; w2 < kSplitWarps; ++w2) {
                s_tab[w2 * a.stride + c] = (int32_t)run;
                run += cnt[w2];
            }
        }
        carry += chunk_total;
    }
    const uint32_t first_rec = a.hb_first[piece0 + warp];
    __syncthreads();

    // walk the piece, 32 outputs at a time
    const uint32_t sensor = u.row / a.tile_rows, y = u.row - sensor * a.tile_rows;
    const uint32_t hi_row = (sensor << a.tile_n_bits) | (y * a.row_width);
    if (q_lo < q_hi && u.n_rec > 0) {
        uint32_t base = first_rec;
        uint32_t q = q_lo;
        SplitWindow win = split_load_window(a, base, lane, u.n_rec, u.n_out);
        while (q < q_hi && base < u.n_rec) {
            const SplitWindow nxt = split_load_window(a, base + 32, lane, u.n_rec, u.n_out);
            const uint32_t n_in = min(32u, u.n_rec - base);
            const uint32_t w_end = min(__shfl_sync(0xffffffffu, win.s1, n_in - 1), q_hi);
            uint32_t cur = 0;   // window lane of the record owning output q
            while (q < w_end) {
                // records after `cur` that start inside this chunk (one may start exactly at q)
                const bool starts = lane > cur && lane < n_in && win.s0 >= q && (win.s0 - q) < 32u;
                const uint32_t B = __reduce_or_sync(0xffffffffu, starts ? (1u << (win.s0 - q)) : 0u);
                const uint32_t o = q + lane;
                const uint32_t rel = __popc(B & le);
                const uint32_t own = (cur + rel) & 31u;
                const uint32_t jxw = __shfl_sync(0xffffffffu, win.xw, own);
                const uint32_t e0 = __shfl_sync(0xffffffffu, win.s0, own);
                const uint32_t idx = __shfl_sync(0xffffffffu, win.idx, own);
                const uint32_t depth = __shfl_sync(0xffffffffu, win.depth, own);
                uint32_t col = (jxw & 0xffffu) + (o - e0);
                if (a.wrap && col >= a.row_width) {
                    col -= a.row_width;
                    if (col >= a.row_width) col %= a.row_width;
                }
                // a column outside the row cannot come from a consistent record
                const bool active = o < w_end && col < a.row_width;
                if (!active) col = 0;
                // Rank among the outputs of this chunk in the same column: lanes with equal
                // columns are matched with one ballot per column bit and ranked in lane order.
                // (Letting the records of a chunk take turns instead - the columns of one run are
                // distinct - measured the same.)
                // (one match.any per step in place of the ballots measured 18 % slower for this kernel)
                uint32_t peers = __ballot_sync(0xffffffffu, active);
#pragma unroll
                for (uint32_t bit = 0; bit < kSplitColBits; ++bit) {
                    if (bit >= a.col_bits) break;
                    const bool one = (col >> bit) & 1u;
                    const uint32_t bal = __ballot_sync(0xffffffffu, one);
                    peers &= one ? bal : ~bal;
                }
                const uint32_t rank = __popc(peers & lt), cnt = __popc(peers);
                uint32_t v = 0;
                if (active) v = hist[col];
                __syncwarp();
                if (active && rank + 1 == cnt) hist[col] = v + cnt;   // one lane per column
                __syncwarp();
                const uint32_t lpos = v + rank;
                if (active && lpos < kSplitUnit) {
                    st_col[lpos] = (uint16_t)col;
                    st_depth[lpos] = depth;
                    st_idx[lpos] = idx;
                }
                cur += __popc(B);
                q = min(q + 32u, w_end);
            }
            base += 32;
            win = nxt;
        }
    }
    __syncthreads();
    // the unit's outputs now sit in tile order: consecutive threads write consecutive entries
    const uint32_t n_unit = u.q_hi - u.q_lo;
    for (uint32_t i = tid; i < n_unit; i += blockDim.x) {
        const uint32_t col = st_col[i];
        const uint32_t pos = i + (uint32_t)s_shift[col < a.stride ? col : 0];
        if (pos < cap) {
            isect_ids[pos] = ((int64_t)(hi_row + col) << 32) | (int64_t)st_depth[i];
            flatten_ids[pos] = (int32_t)st_idx[i];
        }
    }
}

// ---------------------------------------------------------------------------------------
// Offsets: offsets[c, tile] = first position whose (sensor, tile) >= (c, tile).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
offset_encode_kernel(const int64_t *__restrict__ isect_ids, const int64_t *n_ptr, int64_t n_imm,
                     uint32_t C, uint32_t n_tiles, uint32_t tile_n_bits,
                     int32_t *__restrict__ offsets) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t n = n_ptr ? (*n_ptr < n_imm ? *n_ptr : n_imm) : n_imm;
    if (t == C * n_tiles && n_ptr != nullptr) offsets[t] = (int32_t)n;   // fill only: the total
    if (t >= C * n_tiles) return;
    const int64_t cid = t / n_tiles, tile = t - (uint32_t)cid * n_tiles;
    const int64_t target = (cid << tile_n_bits) | tile;
    int64_t l = 0, h = n;   // first position with (id >> 32) >= target
    while (l < h) {
        const int64_t m = (l + h) >> 1;
        if ((isect_ids[m] >> 32) < target) l = m + 1; else h = m;
    }
    offsets[t] = (int32_t)l;
}

// counters back to zero (depth range: empty) and, for the bucket depth sort, its 65536 cursors
__global__ void init_counters_kernel(int64_t *counters, uint32_t *bcount, uint32_t bucket_lo, uint32_t bucket_hi) {
    chain_enter();
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < CNT_DEV_SLOTS)
        counters[t] = (t == CNT_DMIN) ? 0xffffffffll : (t == CNT_BLO) ? (int64_t)bucket_lo
                                                     : (t == CNT_BHI) ? (int64_t)bucket_hi : 0;
    if (bcount != nullptr)
        for (uint32_t i = t; i < kDepthBuckets; i += gridDim.x * blockDim.x) bcount[i] = 0u;
}

// ---------------------------------------------------------------------------------------
// Host orchestration
// ---------------------------------------------------------------------------------------
static inline size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

struct PlanWs {
    int64_t *counters;
    uint32_t *hist;
    uint32_t *digit_totals;
    unsigned long long *block_sums;
    unsigned long long *block_offs;
    uint32_t *keyA, *valA, *keyB, *valB;
    uint32_t *eoff;
    uint32_t *ha_cnt, *ha_out;   // row split: per (block of entries, grid row)
    uint32_t *hw_cnt, *hw_out;   // row split: per (warp of a block, grid row)
    uint32_t *rect_xw, *rect_yh; // row split: packed rectangles by flatten index
    uint32_t *bcount, *bstart;   // bucket depth sort: [65536] counts / cursors, [65536] starts in their scan block
    uint32_t *boff;              // [256] offsets of the scan blocks, [1] total, [256] block totals
    size_t bytes;
};

static PlanWs carve_plan(void *ws, uint64_t total) {
    PlanWs p;
    char *c = (char *)ws;
    size_t off = 0;
    auto take = [&](size_t b) { char *r = c ? c + off : nullptr; off += align256(b); return r; };
    p.counters = (int64_t *)take(sizeof(int64_t) * CNT_DEV_SLOTS);
    p.hist = (uint32_t *)take(sizeof(uint32_t) * kRadixBins * kSortGrid);
    p.digit_totals = (uint32_t *)take(sizeof(uint32_t) * kRadixBins);
    p.block_sums = (unsigned long long *)take(sizeof(unsigned long long) * kSortGrid);
    p.block_offs = (unsigned long long *)take(sizeof(unsigned long long) * kSortGrid);
    p.keyA = (uint32_t *)take(sizeof(uint32_t) * total);
    p.valA = (uint32_t *)take(sizeof(uint32_t) * total);
    p.keyB = (uint32_t *)take(sizeof(uint32_t) * total);
    p.valB = (uint32_t *)take(sizeof(uint32_t) * total);
    p.eoff = (uint32_t *)take(sizeof(uint32_t) * total);
    const uint64_t smallest_block = kSplitWarps * kSplitWarpEntriesMin;
    const size_t n_ha = (size_t)((total + smallest_block - 1) / smallest_block) * kSplitMaxRows;
    p.ha_cnt = (uint32_t *)take(sizeof(uint32_t) * n_ha);
    p.ha_out = (uint32_t *)take(sizeof(uint32_t) * n_ha);
    p.hw_cnt = (uint32_t *)take(sizeof(uint32_t) * n_ha * kSplitWarps);
    p.hw_out = (uint32_t *)take(sizeof(uint32_t) * n_ha * kSplitWarps);
    p.rect_xw = (uint32_t *)take(sizeof(uint32_t) * total);
    p.rect_yh = (uint32_t *)take(sizeof(uint32_t) * total);
    p.bcount = (uint32_t *)take(sizeof(uint32_t) * kDepthBuckets);
    p.bstart = (uint32_t *)take(sizeof(uint32_t) * kDepthBuckets);
    p.boff = (uint32_t *)take(sizeof(uint32_t) * (2 * kBucketScanBlocks + 1));
    p.bytes = off;
    return p;
}

struct FillWs {
    uint32_t *keyA, *valA, *keyB, *valB;
    size_t bytes;
};

static FillWs carve_fill(void *ws, uint64_t cap) {
    FillWs f;
    char *c = (char *)ws;
    size_t off = 0;
    auto take = [&](size_t b) { char *r = c ? c + off : nullptr; off += align256(b); return r; };
    f.keyA = (uint32_t *)take(sizeof(uint32_t) * cap);
    f.valA = (uint32_t *)take(sizeof(uint32_t) * cap);
    f.keyB = (uint32_t *)take(sizeof(uint32_t) * cap);
    f.valB = (uint32_t *)take(sizeof(uint32_t) * cap);
    f.bytes = off;
    return f;
}

struct SplitWs {
    uint32_t *row_rec, *row_out, *row_unit;
    uint4 *rec;
    uint32_t *hb, *hw, *hb_first, *slot_tot, *slot_base;
    uint32_t units_b_cap;
    size_t bytes;
};

static SplitWs carve_split(void *ws, uint64_t cap, uint32_t rows, uint32_t stride) {
    SplitWs w;
    char *c = (char *)ws;
    size_t off = 0;
    auto take = [&](size_t n) { char *r = c ? c + off : nullptr; off += align256(n); return r; };
    // [0 .. rows] exclusive starts; the second half parks the row totals during the scan
    w.row_rec = (uint32_t *)take(sizeof(uint32_t) * 2 * (kSplitMaxRows + 1));
    w.row_out = (uint32_t *)take(sizeof(uint32_t) * 2 * (kSplitMaxRows + 1));
    w.row_unit = (uint32_t *)take(sizeof(uint32_t) * (kSplitMaxRows + 1));
    w.rec = (uint4 *)take(sizeof(uint4) * cap);
    // every grid row rounds its outputs up to whole units
    w.units_b_cap = (uint32_t)((cap + kSplitUnit - 1) / kSplitUnit) + rows;
    w.hb = (uint32_t *)take(sizeof(uint32_t) * (size_t)w.units_b_cap * stride);
    w.hw = (uint32_t *)take(sizeof(uint32_t) * (size_t)w.units_b_cap * kSplitWarps * stride);
    w.hb_first = (uint32_t *)take(sizeof(uint32_t) * (size_t)w.units_b_cap * kSplitWarps);
    w.slot_tot = (uint32_t *)take(sizeof(uint32_t) * kSplitMaxSlots);
    w.slot_base = (uint32_t *)take(sizeof(uint32_t) * kSplitMaxSlots);
    w.bytes = off;
    return w;
}

static uint32_t bit_length(uint64_t v) {
    uint32_t b = 0;
    while (v) { ++b; v >>= 1; }
    return b;
}

struct IsectGeom {
    bool lidar;
    GridArgs<false> cam;
    GridArgs<true> lid;
    uint32_t C, N, total, n_tiles, tile_n_bits;
    const int64_t *camera_ids;
    const uint32_t *depth_bits;
};

// The row / column split applies to sorted output with at most 128 grid rows and 16384 tiles over
// all sensors and rows of at most 1024 tiles (every field of the packed rectangle record then fits
// 16 bits, the column tables fit shared memory).
static bool use_split(const IsectGeom &g, int sort) {
    if (!sort || (uint64_t)g.C * g.n_tiles > kSplitMaxTiles) return false;
    const uint64_t rw = g.lidar ? g.lid.lidar.n_tiles_azim : g.cam.cam.tile_width;
    const uint64_t rows = (uint64_t)g.C * (g.n_tiles / rw);
    return rows <= kSplitMaxRows && rw <= kSplitMaxWidth;
}

// One-shot request of the calling thread's next plan (splatad_isect_set_early_count): where the
// rectangle count kernel writes the intersection count for the host, and the number it tags it with.
static thread_local int64_t *t_early_host = nullptr;
static thread_local int64_t t_early_seq = 0;
static thread_local bool t_range_given = false;
static thread_local uint32_t t_range_lo = 0, t_range_hi = 0;

// plan: counts, depth order of visible Gaussians, n_isects.
static int isect_plan(const IsectGeom &g, int32_t *tiles_per_gauss, int sort, void *workspace,
                      size_t workspace_bytes, int64_t *host_counts, cudaStream_t st) {
    PlanWs p = carve_plan(workspace, g.total);
    SPL_REQUIRE(workspace != nullptr && workspace_bytes >= p.bytes, SPLATAD_ERR_WORKSPACE,
                "isect plan: workspace too small (%zu < %zu)", workspace_bytes, p.bytes);
    const uint32_t cam_n_bits = bit_length(g.C);   // floor(log2(C)) + 1
    SPL_REQUIRE(g.tile_n_bits + cam_n_bits <= 32, SPLATAD_ERR_KEY_BITS,
                "isect: tile bits (%u) + sensor bits (%u) exceed 32", g.tile_n_bits, cam_n_bits);
    SPL_REQUIRE((uint64_t)g.C * g.n_tiles <= 0xffffffffull, SPLATAD_ERR_KEY_BITS,
                "isect: sensors * tiles does not fit 32 bits");
    // sort: 0 = flatten order, 1 = sorted, depth order by buckets, 2 = sorted, depth order by radix passes
    const bool buckets = sort == 1;
    // a depth range handed over for this plan (splatad_isect_set_depth_range_hint): the rectangle count
    // fills the buckets itself and the separate bucket count is not launched
    const bool ranged = buckets && t_range_given && t_range_lo <= t_range_hi && t_range_hi < 0x7f800000u;
    const uint32_t range_lo = ranged ? t_range_lo : 1u, range_hi = ranged ? t_range_hi : 0u;
    t_range_given = false;
    {
        SPL_PROF("init_counters_kernel", st);
        if (buckets)
            launch_chained(init_counters_kernel, kDepthBuckets / 1024, 1024, 0, st, p.counters, p.bcount, range_lo, range_hi);
        else
            launch_chained(init_counters_kernel, 1, 32, 0, st, p.counters, (uint32_t *)nullptr, 1u, 0u);
    }
    // with few enough sensor-tiles the fill uses the row / column split: it wants the packed
    // rectangles and needs neither the emission offsets nor their block sums
    const bool split = use_split(g, sort);
    const uint32_t cgrid = min(div_up(g.total, kCountThreads), (uint32_t)(2 * kNumSMs));
    // the row / column split knows the intersection count when the rectangle count ends: a host that
    // has asked for it (to size or cut its lists) gets it from a kernel - the rectangle count itself,
    // or the bucket scan right behind it, which also knows whether the bucket sort applies - and need
    // not wait for the depth order
    int64_t *early = nullptr;
    if (split && t_early_host != nullptr) {
        void *dptr = nullptr;
        if (cudaHostGetDevicePointer(&dptr, t_early_host, 0) == cudaSuccess) early = (int64_t *)dptr;
        else (void)cudaGetLastError();   // not mapped for this device: the host falls back to the event
    }
    const int64_t seq = t_early_seq;
    t_early_host = nullptr;
    {
        SPL_PROF("isect_count_kernel", st);
        uint32_t *rx = split ? p.rect_xw : nullptr, *ry = split ? p.rect_yh : nullptr;
        int64_t *tot = split ? p.counters + CNT_NISECT : nullptr;
        int64_t *ticket = p.counters + CNT_TICKET;
        int64_t *early_here = buckets ? nullptr : early;
        const uint32_t *db = buckets ? g.depth_bits : nullptr;
        if (g.lidar)
            launch_chained(isect_count_kernel<true>, cgrid, kCountThreads, 0, st, g.lid, g.total, tiles_per_gauss,
                           g.camera_ids, g.N, rx, ry, tot, ticket, early_here, seq, db, p.counters,
                           ranged ? p.bcount : (uint32_t *)nullptr);
        else
            launch_chained(isect_count_kernel<false>, cgrid, kCountThreads, 0, st, g.cam, g.total, tiles_per_gauss,
                           g.camera_ids, g.N, rx, ry, tot, ticket, early_here, seq, db, p.counters,
                           ranged ? p.bcount : (uint32_t *)nullptr);
    }

    EmitArgs e{};
    e.total = g.total;
    e.tiles_per_gauss = tiles_per_gauss;
    e.camera_ids = g.camera_ids;
    e.N = g.N;
    if (buckets) {
        // depth order of the visible (count > 0) elements by buckets; result in keyB / valB
        const uint32_t bgrid = div_up(g.total, kThreads);   // one element per thread: the atomics' latency needs the parallelism
        // {bits, flatten index} pairs in bucket order: keyA and valA lie back to back in the workspace
        // (each g.total words, 256-byte aligned), together room for g.total 8-byte pairs
        uint2 *pairs = reinterpret_cast<uint2 *>(p.keyA);
        if (!ranged) {
            SPL_PROF("depth_bucket_count_kernel", st);
            launch_chained(depth_bucket_count_kernel, bgrid, kThreads, 0, st, g.depth_bits,
                           (const int32_t *)tiles_per_gauss, g.total, (const int64_t *)p.counters, p.bcount);
        }
        {
            SPL_PROF("depth_bucket_scan_kernel", st);
            launch_chained(depth_bucket_scan_kernel, kBucketScanBlocks, 1024, 0, st, p.bcount, p.bstart, p.boff,
                           p.counters, (volatile int64_t *)early, seq);
        }
        {
            SPL_PROF("depth_bucket_scatter_kernel", st);
            launch_chained(depth_bucket_scatter_kernel, bgrid, kThreads, 0, st, g.depth_bits,
                           (const int32_t *)tiles_per_gauss, g.total, (const int64_t *)p.counters,
                           (const uint32_t *)p.bstart, (const uint32_t *)p.boff, p.bcount, pairs);
        }
        {
            SPL_PROF("depth_bucket_rank_kernel", st);
            launch_chained(depth_bucket_rank_kernel, bgrid, kThreads, 0, st, (const int64_t *)p.counters,
                           (const uint32_t *)p.bstart, (const uint32_t *)p.boff, (const uint2 *)pairs, p.keyB, p.valB);
        }
        e.order = p.valB;
        e.n_order_ptr = p.counters + CNT_NVIS;
    } else if (sort) {
        // stable sort of the visible (count > 0) elements by depth bits: 4 passes of 8 bits
        uint32_t *ka = p.keyA, *va = p.valA, *kb = p.keyB, *vb = p.valB;
        FinalOut nofin{};
        for (int pass = 0; pass < 4; ++pass) {
            PassSrc s{};
            if (pass == 0) {
                s.depth_bits = g.depth_bits;
                s.tiles_per_gauss = tiles_per_gauss;
                s.total = g.total;
                {
                    SPL_PROF("depthsort_upsweep", st);
                    launch_chained(radix_upsweep_kernel<true>, kSortGrid, kSortThreads, 0, st, s, 0, 0xffu, p.hist);
                }
                {
                    SPL_PROF("depthsort_rowscan", st);
                    launch_chained(radix_rowscan_kernel, kRadixBins, ((kSortGrid + 31) / 32) * 32, 0, st,
                                   p.hist, (uint32_t)kSortGrid, p.digit_totals);
                }
                {
                    SPL_PROF("depthsort_downsweep", st);
                    launch_chained(radix_downsweep_kernel<true, false>, kSortGrid, kSortThreads, 0, st,
                                   s, 0, 8, 0xffu, p.hist, p.digit_totals, ka, va, nofin, p.counters + CNT_NVIS);
                }
            } else {
                s.keys = ka; s.vals = va; s.n_ptr = p.counters + CNT_NVIS;
                {
                    SPL_PROF("depthsort_upsweep", st);
                    launch_chained(radix_upsweep_kernel<false>, kSortGrid, kSortThreads, 0, st, s, 8 * pass, 0xffu, p.hist);
                }
                {
                    SPL_PROF("depthsort_rowscan", st);
                    launch_chained(radix_rowscan_kernel, kRadixBins, ((kSortGrid + 31) / 32) * 32, 0, st,
                                   p.hist, (uint32_t)kSortGrid, p.digit_totals);
                }
                {
                    SPL_PROF("depthsort_downsweep", st);
                    launch_chained(radix_downsweep_kernel<false, false>, kSortGrid, kSortThreads, 0, st,
                                   s, 8 * pass, 8, 0xffu, p.hist, p.digit_totals, kb, vb, nofin, nullptr);
                }
                uint32_t *t;
                t = ka; ka = kb; kb = t;
                t = va; va = vb; vb = t;
            }
        }
        // 4 passes: A -> (pass0 writes A) ... after pass 3 the result sits in `va`
        // pass0: gen->A ; pass1: A->B ; pass2: B->A ; pass3: A->B  => sorted order in valB
        e.order = va;
        e.n_order_ptr = p.counters + CNT_NVIS;
    }
    if (!split) {
        {
            SPL_PROF("emit_blocksum_kernel", st);
            emit_blocksum_kernel<<<kSortGrid, kThreads, 0, st>>>(e, p.block_sums);
        }
        {
            SPL_PROF("emit_scan_kernel", st);
            emit_scan_kernel<<<1, 1024, 0, st>>>(p.block_sums, kSortGrid, p.block_offs, p.counters);
        }
        {
            SPL_PROF("emit_offsets_kernel", st);
            emit_offsets_kernel<<<kSortGrid, kThreads, 0, st>>>(e, p.block_offs, p.eoff);
        }
    }
    if (host_counts != nullptr)
        cudaMemcpyAsync(host_counts, p.counters, sizeof(int64_t) * CNT_SLOTS, cudaMemcpyDeviceToHost, st);
    return check_launch("isect plan");
}

static int isect_fill(const IsectGeom &g, const int32_t *tiles_per_gauss, int sort,
                      void *plan_workspace, void *fill_workspace, size_t fill_workspace_bytes,
                      int64_t capacity, int64_t *isect_ids, int32_t *flatten_ids,
                      int32_t *tile_offsets, int64_t *host_counts, cudaStream_t st) {
    PlanWs p = carve_plan(plan_workspace, g.total);
    SPL_REQUIRE(plan_workspace != nullptr, SPLATAD_ERR_WORKSPACE, "isect fill: null plan workspace");
    if (capacity <= 0) return SPLATAD_OK;
    SPL_REQUIRE(isect_ids && flatten_ids, SPLATAD_ERR_BAD_ARG, "isect fill: null output");

    EmitArgs e{};
    e.total = g.total;
    e.tiles_per_gauss = tiles_per_gauss;
    e.camera_ids = g.camera_ids;
    e.N = g.N;
    e.n_tiles = g.n_tiles;
    e.tile_n_bits = g.tile_n_bits;
    e.depth_bits = g.depth_bits;
    e.capacity = capacity;

    if (!sort) {
        if (g.lidar) {
            {
                SPL_PROF("emit_kernel", st);
                emit_kernel<true, true><<<kSortGrid, kThreads, 0, st>>>(
                    g.lid, e, p.eoff, p.counters, nullptr, nullptr, isect_ids, flatten_ids, p.counters);
            }
        } else {
            {
                SPL_PROF("emit_kernel", st);
                emit_kernel<false, true><<<kSortGrid, kThreads, 0, st>>>(
                    g.cam, e, p.eoff, p.counters, nullptr, nullptr, isect_ids, flatten_ids, p.counters);
            }
        }
    } else if (use_split(g, sort)) {
        SplitArgs a{};
        a.rect_xw = p.rect_xw;
        a.rect_yh = p.rect_yh;
        a.order = p.valB;
        a.depth_key = p.keyB;
        a.n_entries_ptr = p.counters + CNT_NVIS;
        a.counters = p.counters;
        a.capacity = capacity;
        a.row_width = g.lidar ? g.lid.lidar.n_tiles_azim : g.cam.cam.tile_width;
        a.stride = a.row_width + 1;
        a.tile_rows = g.n_tiles / a.row_width;
        a.rows = g.C * a.tile_rows;
        a.tile_n_bits = g.tile_n_bits;
        a.col_bits = max(1u, bit_length((uint64_t)a.row_width - 1));
        a.wrap = g.lidar ? 1u : 0u;
        SplitWs w = carve_split(fill_workspace, (uint64_t)capacity, a.rows, a.stride);
        SPL_REQUIRE(fill_workspace != nullptr && fill_workspace_bytes >= w.bytes,
                    SPLATAD_ERR_WORKSPACE, "isect fill: workspace too small (%zu < %zu)",
                    fill_workspace_bytes, w.bytes);
        a.ha_cnt = p.ha_cnt;
        a.ha_out = p.ha_out;
        a.hw_cnt = p.hw_cnt;
        a.hw_out = p.hw_out;
        a.row_rec = w.row_rec; a.row_out = w.row_out; a.row_unit = w.row_unit;
        a.rec = w.rec;
        a.hb = w.hb; a.hw = w.hw; a.hb_first = w.hb_first; a.slot_tot = w.slot_tot; a.slot_base = w.slot_base;
        a.warp_entries = a.rows > 32 ? kSplitWarpEntriesMin : kSplitWarpEntriesMax;
        const uint32_t units_a = div_up(g.total, kSplitWarps * a.warp_entries);
        const size_t smem_count = sizeof(int32_t) * kSplitWarps * a.stride;
        const size_t smem_scatter = sizeof(int32_t) * ((kSplitWarps + 1) * a.stride + 2 * kSplitUnit) +
                                    sizeof(uint16_t) * kSplitUnit;
        if (smem_scatter > 32 * 1024)   // the 48 KB default also has to hold static shared memory
            cudaFuncSetAttribute(colsplit_scatter_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem_scatter);
        {
            SPL_PROF("rowsplit_count_kernel", st);
            launch_chained(rowsplit_count_kernel, units_a, kSplitWarps * 32, 0, st, a);
        }
        {
            SPL_PROF("rowsplit_scan_kernel", st);
            launch_chained(rowsplit_scan_kernel, a.rows, 1024, 0, st, a,
                           (unsigned long long *)(p.counters + CNT_TICKET));
        }
        {
            SPL_PROF("rowsplit_scatter_kernel", st);
            if (a.rows <= 32) launch_chained(rowsplit_scatter_kernel<true>, units_a, kSplitWarps * 32, 0, st, a);
            else launch_chained(rowsplit_scatter_kernel<false>, units_a, kSplitWarps * 32, 0, st, a);
        }
        {
            SPL_PROF("colsplit_count_kernel", st);
            launch_chained(colsplit_count_kernel, w.units_b_cap, kSplitWarps * 32, smem_count, st, a);
        }
        {
            SPL_PROF("colsplit_scan_kernel", st);
            launch_chained(colsplit_scan_kernel, a.rows * ((a.stride + 31) / 32), 1024, 0, st, a,
                           (unsigned long long *)(p.counters + CNT_TICKET), tile_offsets);
            tile_offsets = nullptr;   // done
        }
        {
            SPL_PROF("colsplit_scatter_kernel", st);
            launch_chained(colsplit_scatter_kernel, w.units_b_cap, kSplitWarps * 32, smem_scatter, st, a,
                           isect_ids, flatten_ids, p.counters);
        }
    } else {
        FillWs f = carve_fill(fill_workspace, (uint64_t)capacity);
        SPL_REQUIRE(fill_workspace != nullptr && fill_workspace_bytes >= f.bytes,
                    SPLATAD_ERR_WORKSPACE, "isect fill: workspace too small (%zu < %zu)",
                    fill_workspace_bytes, f.bytes);
        // depth order left by the plan in valB (see isect_plan)
        e.order = p.valB;
        e.n_order_ptr = p.counters + CNT_NVIS;
        if (g.lidar) {
            {
                SPL_PROF("emit_kernel", st);
                emit_kernel<true, false><<<kSortGrid, kThreads, 0, st>>>(
                    g.lid, e, p.eoff, p.counters, f.keyA, f.valA, nullptr, nullptr, p.counters);
            }
        } else {
            {
                SPL_PROF("emit_kernel", st);
                emit_kernel<false, false><<<kSortGrid, kThreads, 0, st>>>(
                    g.cam, e, p.eoff, p.counters, f.keyA, f.valA, nullptr, nullptr, p.counters);
            }
        }

        const uint64_t span = (uint64_t)g.C * g.n_tiles;
        const uint32_t key_bits = max(1u, bit_length(span - 1));
        const uint32_t npass = (key_bits + 7) / 8;
        const uint32_t bits_per = (key_bits + npass - 1) / npass;
        FinalOut fin{};
        fin.isect_ids = isect_ids;
        fin.flatten_ids = flatten_ids;
        fin.depth_bits = g.depth_bits;
        fin.n_tiles = g.n_tiles;
        fin.tile_n_bits = g.tile_n_bits;
        fin.capacity = capacity;
        uint32_t *ka = f.keyA, *va = f.valA, *kb = f.keyB, *vb = f.valB;
        for (uint32_t pass = 0; pass < npass; ++pass) {
            PassSrc s{};
            s.keys = ka; s.vals = va; s.n_ptr = p.counters + CNT_NISECT;
            s.n_cap = (uint32_t)(capacity < 0x7fffffffll ? capacity : 0x7fffffffll);
            const int shift = (int)(pass * bits_per);
            const uint32_t mask = (1u << bits_per) - 1u;
            {
                SPL_PROF("tilesort_upsweep", st);
                radix_upsweep_kernel<false><<<kSortGrid, kSortThreads, 0, st>>>(s, shift, mask, p.hist);
            }
            {
                SPL_PROF("tilesort_rowscan", st);
                radix_rowscan_kernel<<<kRadixBins, ((kSortGrid + 31) / 32) * 32, 0, st>>>(
                    p.hist, kSortGrid, p.digit_totals);
            }
            if (pass + 1 == npass) {
                {
                    SPL_PROF("tilesort_downsweep", st);
                    radix_downsweep_kernel<false, true><<<kSortGrid, kSortThreads, 0, st>>>(
                        s, shift, (int)bits_per, mask, p.hist, p.digit_totals, nullptr, nullptr, fin, nullptr);
                }
            } else {
                FinalOut nofin{};
                {
                    SPL_PROF("tilesort_downsweep", st);
                    radix_downsweep_kernel<false, false><<<kSortGrid, kSortThreads, 0, st>>>(
                        s, shift, (int)bits_per, mask, p.hist, p.digit_totals, kb, vb, nofin, nullptr);
                }
                uint32_t *t;
                t = ka; ka = kb; kb = t;
                t = va; va = vb; vb = t;
            }
        }
    }
    if (sort && tile_offsets != nullptr) {
        SPL_PROF("offset_encode_kernel", st);
        const uint32_t n_ct = g.C * g.n_tiles;
        offset_encode_kernel<<<div_up(n_ct + 1, kThreads), kThreads, 0, st>>>(
            isect_ids, p.counters + CNT_NISECT, capacity, g.C, g.n_tiles, g.tile_n_bits, tile_offsets);
    }
    if (host_counts != nullptr)
        cudaMemcpyAsync(host_counts, p.counters, sizeof(int64_t) * CNT_SLOTS, cudaMemcpyDeviceToHost, st);
    return check_launch("isect fill");
}

// ---------------------------------------------------------------------------------------
// Lidar points -> tiles (what prepares `raster_pts` from a point cloud before a lidar render;
// reference: gsplat/cuda/csrc/rasterization.cu:531-833). Same sort machinery as above on
// (sensor * n_tiles + tile, point index) pairs.
// ---------------------------------------------------------------------------------------
struct PointsWs {
    int64_t *count;
    uint32_t *hist, *digit_totals;
    uint32_t *keyA, *valA, *keyB, *valB;
    size_t bytes;
};

static PointsWs carve_points(void *ws, uint64_t total) {
    PointsWs p;
    char *c = (char *)ws;
    size_t off = 0;
    auto take = [&](size_t b) { char *r = c ? c + off : nullptr; off += align256(b); return r; };
    p.count = (int64_t *)take(sizeof(int64_t));
    p.hist = (uint32_t *)take(sizeof(uint32_t) * kRadixBins * kSortGrid);
    p.digit_totals = (uint32_t *)take(sizeof(uint32_t) * kRadixBins);
    p.keyA = (uint32_t *)take(sizeof(uint32_t) * total);
    p.valA = (uint32_t *)take(sizeof(uint32_t) * total);
    p.keyB = (uint32_t *)take(sizeof(uint32_t) * total);
    p.valB = (uint32_t *)take(sizeof(uint32_t) * total);
    p.bytes = off;
    return p;
}

// Tile of every point: azimuth tile by truncation (angles outside [0, 360) wrapped with fmodf),
// elevation tile = number of the first n_tiles_elev boundaries below the point, minus one.
__global__ void __launch_bounds__(kThreads)
points_tile_kernel(uint32_t total, uint32_t N, const int64_t *__restrict__ camera_ids,
                   const float2 *__restrict__ points2d, const float *__restrict__ elev_boundaries,
                   float tile_azim_resolution, float min_azim, uint32_t n_tiles_azim, uint32_t n_tiles_elev,
                   uint32_t *__restrict__ keys, uint32_t *__restrict__ vals, int64_t *__restrict__ tile_ids,
                   int32_t *__restrict__ flatten_ids, int64_t *__restrict__ count) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx == 0 && count != nullptr) *count = (int64_t)total;
    if (idx >= total) return;
    const float2 pt = points2d[idx];
    const float azim = pt.x - min_azim;
    float tile_azim;
    if (azim >= 0.f && azim < 360.f) tile_azim = azim / tile_azim_resolution;
    else tile_azim = fmodf(azim + 360.f, 360.f) / tile_azim_resolution;
    // float -> int conversion saturates (NaN -> 0); a point cannot land beyond the last tile of
    // its row, the clamp only keeps a malformed input inside the key range
    const uint32_t tx = min((uint32_t)max((int32_t)tile_azim, 0), n_tiles_azim - 1);
    int32_t i = 0;
    while (i < (int32_t)n_tiles_elev && elev_boundaries[i] < pt.y) ++i;
    const uint32_t ty = (uint32_t)max(i - 1, 0);
    const uint32_t cid = camera_ids ? (uint32_t)camera_ids[idx] : idx / N;
    const uint32_t tile = ty * n_tiles_azim + tx;
    if (keys != nullptr) {
        keys[idx] = cid * (n_tiles_azim * n_tiles_elev) + tile;
        vals[idx] = idx;
    } else {
        tile_ids[idx] = ((int64_t)cid << 32) | (int64_t)tile;
        flatten_ids[idx] = (int32_t)idx;
    }
}

__global__ void __launch_bounds__(kThreads)
points_ids_kernel(uint32_t total, uint32_t n_tiles, const uint32_t *__restrict__ keys,
                  const uint32_t *__restrict__ vals, int64_t *__restrict__ tile_ids,
                  int32_t *__restrict__ flatten_ids) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total) return;
    const uint32_t key = keys[idx];
    const uint32_t cid = key / n_tiles;
    tile_ids[idx] = ((int64_t)cid << 32) | (int64_t)(key - cid * n_tiles);
    flatten_ids[idx] = (int32_t)vals[idx];
}

// offsets[c, tile] = first position whose (sensor, tile) >= (c, tile); ids are sensor << 32 | tile.
__global__ void __launch_bounds__(kThreads)
points_offset_encode_kernel(const int64_t *__restrict__ point_ids, int64_t n, uint32_t C, uint32_t n_tiles,
                            int32_t *__restrict__ offsets) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= C * n_tiles) return;
    int64_t l = 0, h = n;
    while (l < h) {
        const int64_t m = (l + h) >> 1;
        const int64_t id = point_ids[m];
        const int64_t flat = (id >> 32) * (int64_t)n_tiles + (id & 0xffffffffll);
        if (flat < (int64_t)t) l = m + 1; else h = m;
    }
    offsets[t] = (int32_t)l;
}

// One block per tile, one thread per pixel of the tile: the thread of rank k takes the tile's
// k-th point (if there is one) and writes it at its own pixel.
__global__ void populate_image_kernel(uint32_t C, int64_t n_points, const float *__restrict__ points,
                                      uint32_t W, uint32_t H, uint32_t tile_width, uint32_t tile_height,
                                      uint32_t grid_w, uint32_t grid_h, const int32_t *__restrict__ offsets,
                                      const int32_t *__restrict__ flatten_ids, float *__restrict__ image) {
    const uint32_t tiles_per_cam = grid_w * grid_h;
    const uint32_t cam = blockIdx.x / tiles_per_cam;
    const uint32_t tile = blockIdx.x - cam * tiles_per_cam;
    const uint32_t by = tile / grid_w, bx = tile - by * grid_w;
    const uint32_t tr = threadIdx.x;
    if (tr >= tile_width * tile_height) return;
    const uint32_t i = by * tile_height + tr / tile_width;
    const uint32_t j = bx * tile_width + tr % tile_width;
    if (i >= H || j >= W) return;
    const int64_t start = offsets[blockIdx.x];
    int64_t end = (blockIdx.x + 1 == C * tiles_per_cam) ? n_points : (int64_t)offsets[blockIdx.x + 1];
    end = min(end, start + (int64_t)(tile_width * tile_height));
    const int64_t k = start + tr;
    if (k >= end) return;
    const float *src = points + (size_t)flatten_ids[k] * 5;
    float *dst = image + (((size_t)cam * H + i) * W + j) * 5;
#pragma unroll
    for (int c = 0; c < 5; ++c) dst[c] = src[c];
}

} // namespace splatad

using namespace splatad;

// =======================================================================================
// C-ABI
// =======================================================================================
extern "C" size_t splatad_isect_plan_workspace_bytes(uint64_t total_elems) {
    return carve_plan(nullptr, total_elems).bytes;
}

extern "C" size_t splatad_isect_fill_workspace_bytes(uint64_t capacity) {
    // the larger of the radix buffers and the split's records + tables; the widest rows and the
    // most rows together bound (units + rows) * stride of every geometry the split accepts
    const size_t a = carve_fill(nullptr, capacity).bytes;
    const size_t b = carve_split(nullptr, capacity, kSplitMaxRows, kSplitMaxWidth + 1).bytes;
    return a > b ? a : b;
}

static int make_cam_geom(IsectGeom &g, uint32_t C, uint32_t N, uint64_t total,
                         const float *means2d, const int32_t *radii, const float *depths,
                         const int64_t *camera_ids, uint32_t tile_size, uint32_t tile_width,
                         uint32_t tile_height) {
    SPL_REQUIRE(means2d && radii && depths, SPLATAD_ERR_BAD_ARG, "isect_tiles: null input");
    SPL_REQUIRE(C > 0 && tile_size > 0 && tile_width > 0 && tile_height > 0, SPLATAD_ERR_BAD_ARG,
                "isect_tiles: bad geometry");
    SPL_REQUIRE(total <= 0x7fffffffull, SPLATAD_ERR_BAD_ARG, "isect_tiles: too many elements");
    SPL_REQUIRE((uint64_t)tile_width * tile_height * C <= 0xffffffffull, SPLATAD_ERR_KEY_BITS,
                "isect_tiles: sensors * tiles does not fit 32 bits");
    g = IsectGeom{};
    g.lidar = false;
    g.cam.cam = CamGrid{tile_size, tile_width, tile_height};
    g.cam.radii = radii;
    g.cam.means2d = (const float2 *)means2d;
    g.C = C; g.N = N ? N : 1; g.total = (uint32_t)total;
    g.n_tiles = tile_width * tile_height;
    g.tile_n_bits = bit_length(g.n_tiles);
    g.camera_ids = camera_ids;
    g.depth_bits = (const uint32_t *)depths;
    return SPLATAD_OK;
}

static int make_lidar_geom(IsectGeom &g, uint32_t C, uint32_t N, uint64_t total,
                           const float *means2d, const float *radii, const float *depths,
                           const int64_t *camera_ids, const float *elev_boundaries,
                           uint32_t n_boundaries, float tile_azim_resolution, float min_azim) {
    SPL_REQUIRE(means2d && radii && depths && elev_boundaries, SPLATAD_ERR_BAD_ARG,
                "isect_lidar_tiles: null input");
    SPL_REQUIRE(C > 0 && n_boundaries >= 2 && tile_azim_resolution > 0.f, SPLATAD_ERR_BAD_ARG,
                "isect_lidar_tiles: bad geometry");
    SPL_REQUIRE(total <= 0x7fffffffull, SPLATAD_ERR_BAD_ARG, "isect_lidar_tiles: too many elements");
    g = IsectGeom{};
    g.lidar = true;
    g.lid.lidar.elev_boundaries = elev_boundaries;
    g.lid.lidar.tile_azim_res = tile_azim_resolution;
    g.lid.lidar.min_azim = min_azim;
    g.lid.lidar.n_tiles_azim = splatad_lidar_azimuth_tiles(tile_azim_resolution);
    g.lid.lidar.n_tiles_elev = n_boundaries - 1;
    g.lid.radii = radii;
    g.lid.means2d = (const float2 *)means2d;
    g.C = C; g.N = N ? N : 1; g.total = (uint32_t)total;
    g.n_tiles = g.lid.lidar.n_tiles_azim * g.lid.lidar.n_tiles_elev;
    g.tile_n_bits = bit_length(g.n_tiles);
    g.camera_ids = camera_ids;
    g.depth_bits = (const uint32_t *)depths;
    return SPLATAD_OK;
}

extern "C" int splatad_isect_tiles_plan(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const int32_t *radii,
    const float *depths, const int64_t *camera_ids, uint32_t tile_size, uint32_t tile_width,
    uint32_t tile_height, int32_t sort, int32_t *tiles_per_gauss, void *workspace,
    size_t workspace_bytes, int64_t *host_counts, void *stream) {
    if (total_elems == 0) {
        if (host_counts) for (int i = 0; i < CNT_SLOTS; ++i) host_counts[i] = 0;
        return SPLATAD_OK;
    }
    IsectGeom g;
    int rc = make_cam_geom(g, C, N, total_elems, means2d, radii, depths, camera_ids, tile_size,
                           tile_width, tile_height);
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(tiles_per_gauss, SPLATAD_ERR_BAD_ARG, "isect_tiles_plan: null tiles_per_gauss");
    return isect_plan(g, tiles_per_gauss, sort, workspace, workspace_bytes, host_counts,
                      (cudaStream_t)stream);
}

extern "C" int splatad_isect_tiles_fill(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const int32_t *radii,
    const float *depths, const int64_t *camera_ids, uint32_t tile_size, uint32_t tile_width,
    uint32_t tile_height, int32_t sort, const int32_t *tiles_per_gauss, void *plan_workspace,
    void *fill_workspace, size_t fill_workspace_bytes, int64_t capacity, int64_t *isect_ids,
    int32_t *flatten_ids, int32_t *tile_offsets, int64_t *host_counts, void *stream) {
    if (total_elems == 0 || capacity <= 0) return SPLATAD_OK;
    IsectGeom g;
    int rc = make_cam_geom(g, C, N, total_elems, means2d, radii, depths, camera_ids, tile_size,
                           tile_width, tile_height);
    if (rc != SPLATAD_OK) return rc;
    return isect_fill(g, tiles_per_gauss, sort, plan_workspace, fill_workspace,
                      fill_workspace_bytes, capacity, isect_ids, flatten_ids, tile_offsets, host_counts,
                      (cudaStream_t)stream);
}

extern "C" uint32_t splatad_lidar_azimuth_tiles(float tile_azim_resolution) {
    return tile_azim_resolution > 0.f ? (uint32_t)ceilf(360.f / tile_azim_resolution) : 0u;
}

extern "C" int splatad_isect_lidar_tiles_plan(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const float *radii,
    const float *depths, const int64_t *camera_ids, const float *elev_boundaries,
    uint32_t n_boundaries, float tile_azim_resolution, float min_azim, int32_t sort,
    int32_t *tiles_per_gauss, void *workspace, size_t workspace_bytes, int64_t *host_counts,
    void *stream) {
    if (total_elems == 0) {
        if (host_counts) for (int i = 0; i < CNT_SLOTS; ++i) host_counts[i] = 0;
        return SPLATAD_OK;
    }
    IsectGeom g;
    int rc = make_lidar_geom(g, C, N, total_elems, means2d, radii, depths, camera_ids,
                             elev_boundaries, n_boundaries, tile_azim_resolution, min_azim);
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(tiles_per_gauss, SPLATAD_ERR_BAD_ARG, "isect_lidar_tiles_plan: null tiles_per_gauss");
    return isect_plan(g, tiles_per_gauss, sort, workspace, workspace_bytes, host_counts,
                      (cudaStream_t)stream);
}

extern "C" int splatad_isect_lidar_tiles_fill(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *means2d, const float *radii,
    const float *depths, const int64_t *camera_ids, const float *elev_boundaries,
    uint32_t n_boundaries, float tile_azim_resolution, float min_azim, int32_t sort,
    const int32_t *tiles_per_gauss, void *plan_workspace, void *fill_workspace,
    size_t fill_workspace_bytes, int64_t capacity, int64_t *isect_ids, int32_t *flatten_ids,
    int32_t *tile_offsets, int64_t *host_counts, void *stream) {
    if (total_elems == 0 || capacity <= 0) return SPLATAD_OK;
    IsectGeom g;
    int rc = make_lidar_geom(g, C, N, total_elems, means2d, radii, depths, camera_ids,
                             elev_boundaries, n_boundaries, tile_azim_resolution, min_azim);
    if (rc != SPLATAD_OK) return rc;
    return isect_fill(g, tiles_per_gauss, sort, plan_workspace, fill_workspace,
                      fill_workspace_bytes, capacity, isect_ids, flatten_ids, tile_offsets, host_counts,
                      (cudaStream_t)stream);
}

extern "C" int splatad_isect_set_early_count(int64_t *host_pair, int64_t sequence) {
    t_early_host = host_pair;
    t_early_seq = sequence;
    return SPLATAD_OK;
}

extern "C" int splatad_isect_set_depth_range_hint(uint32_t depth_lo_bits, uint32_t depth_hi_bits) {
    t_range_given = true;
    t_range_lo = depth_lo_bits;
    t_range_hi = depth_hi_bits;
    return SPLATAD_OK;
}

extern "C" int splatad_isect_offset_encode(const int64_t *isect_ids, int64_t n_isects, uint32_t C,
                                           uint32_t tile_width, uint32_t tile_height,
                                           int32_t *offsets, void *stream) {
    SPL_REQUIRE(offsets, SPLATAD_ERR_BAD_ARG, "isect_offset_encode: null output");
    const uint64_t n_tiles = (uint64_t)tile_width * tile_height;
    SPL_REQUIRE(C > 0 && n_tiles > 0 && (uint64_t)C * n_tiles <= 0x7fffffffull, SPLATAD_ERR_BAD_ARG,
                "isect_offset_encode: bad geometry");
    SPL_REQUIRE(n_isects == 0 || isect_ids, SPLATAD_ERR_BAD_ARG, "isect_offset_encode: null input");
    const uint32_t tile_n_bits = bit_length(n_tiles);
    const uint32_t total = (uint32_t)(C * n_tiles);
    {
        SPL_PROF("offset_encode_kernel", (cudaStream_t)stream);
        offset_encode_kernel<<<div_up(total, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            isect_ids, nullptr, n_isects, C, (uint32_t)n_tiles, tile_n_bits, offsets);
    }
    return check_launch("isect_offset_encode");
}

// =======================================================================================
// Lidar points -> tiles -> raster image
// =======================================================================================
extern "C" size_t splatad_map_points_workspace_bytes(uint64_t total_elems) {
    return carve_points(nullptr, total_elems).bytes;
}

extern "C" int splatad_map_points_to_lidar_tiles(
    uint32_t C, uint32_t N, uint64_t total_elems, const float *points2d, const int64_t *camera_ids,
    const float *elev_boundaries, uint32_t n_boundaries, float tile_azim_resolution, float min_azim,
    int32_t sort, void *workspace, size_t workspace_bytes, int64_t *tile_ids, int32_t *flatten_ids,
    void *stream) {
    if (total_elems == 0) return SPLATAD_OK;
    cudaStream_t st = (cudaStream_t)stream;
    SPL_REQUIRE(points2d && elev_boundaries && tile_ids && flatten_ids, SPLATAD_ERR_BAD_ARG,
                "map_points_to_lidar_tiles: null argument");
    SPL_REQUIRE(C > 0 && n_boundaries >= 2 && tile_azim_resolution > 0.f, SPLATAD_ERR_BAD_ARG,
                "map_points_to_lidar_tiles: bad geometry");
    SPL_REQUIRE(total_elems <= 0x7fffffffull, SPLATAD_ERR_BAD_ARG, "map_points_to_lidar_tiles: too many points");
    const uint32_t total = (uint32_t)total_elems;
    const uint32_t n_az = splatad_lidar_azimuth_tiles(tile_azim_resolution), n_el = n_boundaries - 1;
    const uint64_t span = (uint64_t)C * n_az * n_el;
    SPL_REQUIRE(span <= 0xffffffffull, SPLATAD_ERR_KEY_BITS, "map_points_to_lidar_tiles: sensors * tiles does not fit 32 bits");
    const uint32_t n_per = N ? N : 1;
    const uint32_t grid = div_up(total, kThreads);
    if (!sort) {
        SPL_PROF("points_tile_kernel", st);
        points_tile_kernel<<<grid, kThreads, 0, st>>>(total, n_per, camera_ids, (const float2 *)points2d,
                                                     elev_boundaries, tile_azim_resolution, min_azim, n_az,
                                                     n_el, nullptr, nullptr, tile_ids, flatten_ids, nullptr);
        return check_launch("map_points_to_lidar_tiles");
    }
    PointsWs p = carve_points(workspace, total);
    SPL_REQUIRE(workspace != nullptr && workspace_bytes >= p.bytes, SPLATAD_ERR_WORKSPACE,
                "map_points_to_lidar_tiles: workspace too small (%zu < %zu)", workspace_bytes, p.bytes);
    {
        SPL_PROF("points_tile_kernel", st);
        points_tile_kernel<<<grid, kThreads, 0, st>>>(total, n_per, camera_ids, (const float2 *)points2d,
                                                     elev_boundaries, tile_azim_resolution, min_azim, n_az,
                                                     n_el, p.keyA, p.valA, nullptr, nullptr, p.count);
    }
    // stable LSD radix sort of the (key, index) pairs over the bits the keys use
    const uint32_t key_bits = max(1u, bit_length(span - 1));
    const uint32_t npass = (key_bits + 7) / 8;
    const uint32_t bits_per = (key_bits + npass - 1) / npass;
    uint32_t *ka = p.keyA, *va = p.valA, *kb = p.keyB, *vb = p.valB;
    FinalOut nofin{};
    for (uint32_t pass = 0; pass < npass; ++pass) {
        PassSrc s{};
        s.keys = ka; s.vals = va; s.n_ptr = p.count;
        s.n_cap = total;
        const int shift = (int)(pass * bits_per);
        const uint32_t mask = (1u << bits_per) - 1u;
        {
            SPL_PROF("points_sort_upsweep", st);
            radix_upsweep_kernel<false><<<kSortGrid, kSortThreads, 0, st>>>(s, shift, mask, p.hist);
        }
        {
            SPL_PROF("points_sort_rowscan", st);
            radix_rowscan_kernel<<<kRadixBins, ((kSortGrid + 31) / 32) * 32, 0, st>>>(p.hist, kSortGrid,
                                                                                    p.digit_totals);
        }
        {
            SPL_PROF("points_sort_downsweep", st);
            radix_downsweep_kernel<false, false><<<kSortGrid, kSortThreads, 0, st>>>(
                s, shift, (int)bits_per, mask, p.hist, p.digit_totals, kb, vb, nofin, nullptr);
        }
        uint32_t *t;
        t = ka; ka = kb; kb = t;
        t = va; va = vb; vb = t;
    }
    {
        SPL_PROF("points_ids_kernel", st);
        points_ids_kernel<<<grid, kThreads, 0, st>>>(total, n_az * n_el, ka, va, tile_ids, flatten_ids);
    }
    return check_launch("map_points_to_lidar_tiles");
}

extern "C" int splatad_points_mapping_offset_encode(const int64_t *point_ids, int64_t n_points, uint32_t C,
                                                    uint32_t tile_width, uint32_t tile_height,
                                                    int32_t *offsets, void *stream) {
    SPL_REQUIRE(offsets, SPLATAD_ERR_BAD_ARG, "points_mapping_offset_encode: null output");
    const uint64_t n_tiles = (uint64_t)tile_width * tile_height;
    SPL_REQUIRE(C > 0 && n_tiles > 0 && (uint64_t)C * n_tiles <= 0x7fffffffull, SPLATAD_ERR_BAD_ARG,
                "points_mapping_offset_encode: bad geometry");
    SPL_REQUIRE(n_points == 0 || point_ids, SPLATAD_ERR_BAD_ARG, "points_mapping_offset_encode: null input");
    const uint32_t total = (uint32_t)(C * n_tiles);
    {
        SPL_PROF("points_offset_encode_kernel", (cudaStream_t)stream);
        points_offset_encode_kernel<<<div_up(total, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            point_ids, n_points, C, (uint32_t)n_tiles, offsets);
    }
    return check_launch("points_mapping_offset_encode");
}

extern "C" int splatad_populate_image_from_points(
    uint32_t C, int64_t n_points, const float *points, uint32_t image_width, uint32_t image_height,
    uint32_t tile_width, uint32_t tile_height, uint32_t tile_grid_width, uint32_t tile_grid_height,
    const int32_t *tile_offsets, const int32_t *flatten_ids, float *image, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    SPL_REQUIRE(image && tile_offsets, SPLATAD_ERR_BAD_ARG, "populate_image_from_points: null argument");
    SPL_REQUIRE(tile_width >= 1 && tile_height >= 1 && tile_width * tile_height <= 1024, SPLATAD_ERR_BAD_ARG,
                "populate_image_from_points: tile_width * tile_height must be in 1..1024");
    SPL_REQUIRE(n_points == 0 || (points && flatten_ids), SPLATAD_ERR_BAD_ARG,
                "populate_image_from_points: null input");
    const size_t n_pix = (size_t)C * image_height * image_width;
    if (n_pix == 0) return SPLATAD_OK;
    cudaMemsetAsync(image, 0, n_pix * 5 * sizeof(float), st);
    const uint32_t blocks = C * tile_grid_width * tile_grid_height;
    if (blocks == 0 || n_points == 0) return check_launch("populate_image_from_points");
    const uint32_t bs = ((tile_width * tile_height + 31) / 32) * 32;
    {
        SPL_PROF("populate_image_kernel", st);
        populate_image_kernel<<<blocks, bs, 0, st>>>(C, n_points, points, image_width, image_height, tile_width,
                                                    tile_height, tile_grid_width, tile_grid_height, tile_offsets,
                                                    flatten_ids, image);
    }
    return check_launch("populate_image_from_points");
}
