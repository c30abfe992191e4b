// Device side of the Gaussian-sharded exchange: every rank projects its slice of the Gaussians for
// all sensors, the visible (sensor, Gaussian) records travel to the rank that owns the sensor, and
// arrive there in the order a single GPU would have produced them. The transport is the caller's
// (one all-to-all of fixed-width rows); these kernels build the send rows and place the received
// ones:
//   visible_rows_count / _fill   which (sensor, Gaussian) pairs travel, in (sensor, Gaussian) order
//   rows_gather                  out[i, :] = concat_k src_k[index[i], :]      (send rows; also the
//                                backward pass of rows_scatter)
//   rows_scatter                 dst_k[index[i], :] = in[i, columns of k]      (placing received rows;
//                                also the backward pass of rows_gather)
//   segment_row_map              received row -> final row, from a table of contiguous segments
// The pattern replaces the size exchange + row all-to-all helpers of gsplat/distributed.py:170-257
// (which leave packing and ordering to the caller's torch code).
#include "common.cuh"

namespace splatad {

constexpr int kMaxFields = 12;

struct RowFields {
    const uint32_t *src[kMaxFields];   // [rows_k, width_k] 32-bit words (floats or int32 bit patterns)
    uint32_t *dst[kMaxFields];
    int32_t col[kMaxFields + 1];       // first column of field k in the packed row; col[n] = row width
    int32_t n;
};

// Pairs with a positive first radius are the ones tile intersection lists (float radii in degrees
// for lidars, integer pixels for cameras: both are positive exactly when their bit pattern, read as
// a signed integer, is positive; patterns above +infinity are NaNs, which compare false).
__device__ __forceinline__ bool pair_visible(const int32_t *radii, uint64_t pair) {
    const int32_t bits = __ldg(radii + 2 * pair);
    return bits > 0 && bits <= 0x7f800000;
}

__global__ void __launch_bounds__(kThreads)
visible_rows_count_kernel(uint32_t C, uint32_t N, const int32_t *__restrict__ radii,
                          int32_t *__restrict__ counts) {
    const uint32_t nblocks = gridDim.x;
    const uint32_t n = blockIdx.x * kThreads + threadIdx.x;
    __shared__ int32_t warp_cnt[kThreads / 32];
    for (uint32_t c = 0; c < C; ++c) {
        const bool vis = n < N && pair_visible(radii, (uint64_t)c * N + n);
        const uint32_t m = __ballot_sync(0xffffffffu, vis);
        if ((threadIdx.x & 31) == 0) warp_cnt[threadIdx.x >> 5] = __popc(m);
        __syncthreads();
        if (threadIdx.x == 0) {
            int32_t s = 0;
#pragma unroll
            for (int w = 0; w < kThreads / 32; ++w) s += warp_cnt[w];
            counts[(size_t)c * nblocks + blockIdx.x] = s;
        }
        __syncthreads();
    }
}

// Exclusive scan of the [C * nblocks] block counts by one block; indptr[c] = first row of sensor c,
// indptr[C] = total (also written to *total_out and, if given, to pinned host memory later by a copy).
__global__ void __launch_bounds__(1024)
visible_rows_scan_kernel(const int32_t *__restrict__ counts, int32_t *__restrict__ offsets, uint32_t C,
                         uint32_t nblocks, int32_t *__restrict__ indptr, int64_t *__restrict__ total_out) {
    __shared__ int32_t part[1024];
    const uint32_t total = C * nblocks;
    const uint32_t t = threadIdx.x;
    const uint32_t per = (total + 1023) / 1024;
    const uint32_t lo = min(t * per, total), hi = min(lo + per, total);
    int32_t s = 0;
    for (uint32_t i = lo; i < hi; ++i) s += counts[i];
    part[t] = s;
    __syncthreads();
    for (uint32_t off = 1; off < 1024; off <<= 1) {
        int32_t v = (t >= off) ? part[t - off] : 0;
        __syncthreads();
        part[t] += v;
        __syncthreads();
    }
    int32_t run = (t == 0) ? 0 : part[t - 1];
    for (uint32_t i = lo; i < hi; ++i) {
        offsets[i] = run;
        if (i % nblocks == 0) indptr[i / nblocks] = run;
        run += counts[i];
    }
    if (t == 1023) {
        indptr[C] = part[1023];
        if (total_out) *total_out = (int64_t)part[1023];
    }
}

__global__ void __launch_bounds__(kThreads)
visible_rows_fill_kernel(uint32_t C, uint32_t N, const int32_t *__restrict__ radii,
                         const int32_t *__restrict__ offsets, int64_t capacity,
                         int32_t *__restrict__ row_index) {
    const uint32_t nblocks = gridDim.x;
    const uint32_t n = blockIdx.x * kThreads + threadIdx.x;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __shared__ int32_t warp_cnt[kThreads / 32];
    for (uint32_t c = 0; c < C; ++c) {
        const bool vis = n < N && pair_visible(radii, (uint64_t)c * N + n);
        const uint32_t m = __ballot_sync(0xffffffffu, vis);
        if (lane == 0) warp_cnt[warp] = __popc(m);
        __syncthreads();
        if (vis) {
            int32_t before = 0;
            for (uint32_t w = 0; w < warp; ++w) before += warp_cnt[w];
            const int64_t pos = (int64_t)offsets[(size_t)c * nblocks + blockIdx.x] + before +
                                __popc(m & ((1u << lane) - 1u));
            if (pos < capacity) row_index[pos] = (int32_t)(c * N + n);
        }
        __syncthreads();
    }
}

// Column of a packed row as seen by one lane: which field it belongs to and where inside it. A
// lane keeps the same columns for every row it visits (column = lane + 32 k), so the lookup happens
// once per kernel, not once per word.
constexpr int kMaxColsPerLane = 4;   // rows of up to 128 words
template <int kColsPerLane>
struct LaneCols {
    uint32_t *ptr[kColsPerLane];     // field base (source or destination); nullptr: no such field / column
    int32_t width[kColsPerLane];     // words per row of that field
    int32_t off[kColsPerLane];       // word inside the field's row
    int32_t kind[kColsPerLane];      // 0 data, 1 sensor id column, 2 Gaussian id column, -1 beyond the row
};

template <int kColsPerLane>
__device__ __forceinline__ LaneCols<kColsPerLane> lane_columns(const RowFields &f, int32_t id_cols, bool as_dst,
                                                                uint32_t lane) {
    LaneCols<kColsPerLane> lc;
    const int32_t W = f.col[f.n];
#pragma unroll
    for (int k = 0; k < kColsPerLane; ++k) {
        const int32_t c = (int32_t)lane + 32 * k;
        lc.ptr[k] = nullptr; lc.width[k] = 0; lc.off[k] = 0; lc.kind[k] = -1;
        if (c >= W + id_cols) continue;
        if (c < id_cols) { lc.kind[k] = 1 + c; continue; }
        const int32_t cc = c - id_cols;
        int q = 0;
        for (int t = 1; t < kMaxFields; ++t) q += (t < f.n && cc >= f.col[t]) ? 1 : 0;
        lc.kind[k] = 0;
        lc.ptr[k] = as_dst ? f.dst[q] : const_cast<uint32_t *>(f.src[q]);
        lc.width[k] = f.col[q + 1] - f.col[q];
        lc.off[k] = cc - f.col[q];
    }
    return lc;
}

// out[i, :] = fields gathered from row index[i] (or i): one warp per row, one lane per column. With
// `sensor_table`, the first two columns are ids instead of gathered data: the global sensor id of
// pair index[i] (sensor_table[index / N]) and its global Gaussian id (gaussian_start + index % N),
// as int32 bit patterns.
template <int kColsPerLane, int kRowsPerStep>
__global__ void __launch_bounds__(kThreads)
rows_gather_kernel(RowFields f, int64_t n_rows, const int32_t *__restrict__ index,
                   const int32_t *__restrict__ sensor_table, uint32_t N, int32_t gaussian_start,
                   uint32_t *__restrict__ out) {
    const uint32_t lane = threadIdx.x & 31;
    const int32_t id_cols = sensor_table ? 2 : 0;
    const int32_t Wt = f.col[f.n] + id_cols;
    const LaneCols<kColsPerLane> lc = lane_columns<kColsPerLane>(f, id_cols, false, lane);
    // kRowsPerStep consecutive rows per warp and step, all their loads issued before the first store:
    // with one row in flight per warp the kernel waited on its two dependent loads (index, then data)
    const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
    const int64_t w0 = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    for (int64_t i0 = w0 * kRowsPerStep; i0 < n_rows; i0 += n_warps * kRowsPerStep) {
        int64_t r[kRowsPerStep];
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j)
            r[j] = (i0 + j < n_rows) ? (index ? (int64_t)__ldg(index + i0 + j) : i0 + j) : -1;
        uint32_t v[kRowsPerStep][kColsPerLane];
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
#pragma unroll
            for (int k = 0; k < kColsPerLane; ++k) {
                v[j][k] = 0;
                if (lc.kind[k] < 0 || r[j] < 0) continue;
                if (lc.kind[k] == 1) v[j][k] = (uint32_t)__ldg(sensor_table + r[j] / N);
                else if (lc.kind[k] == 2) v[j][k] = (uint32_t)(gaussian_start + (int32_t)(r[j] % N));
                else if (lc.ptr[k]) v[j][k] = __ldg(lc.ptr[k] + r[j] * lc.width[k] + lc.off[k]);
            }
        }
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
#pragma unroll
            for (int k = 0; k < kColsPerLane; ++k)
                if (lc.kind[k] >= 0 && r[j] >= 0) out[(i0 + j) * Wt + lane + 32 * k] = v[j][k];
        }
    }
}

// dst_k[index[i] (or i), :] = in[i, columns of field k]: one warp per row; the two leading id
// columns of the rows (id_cols = 2) are widened to int64 into sensor_ids_out / gaussian_ids_out.
template <int kColsPerLane, int kRowsPerStep>
__global__ void __launch_bounds__(kThreads)
rows_scatter_kernel(RowFields f, int64_t n_rows, const int32_t *__restrict__ index, int32_t id_cols,
                    int64_t *__restrict__ sensor_ids_out, int64_t *__restrict__ gaussian_ids_out,
                    const uint32_t *__restrict__ in) {
    const uint32_t lane = threadIdx.x & 31;
    const int32_t Wt = f.col[f.n] + id_cols;
    const LaneCols<kColsPerLane> lc = lane_columns<kColsPerLane>(f, id_cols, true, lane);
    const int64_t n_warps = (int64_t)gridDim.x * (kThreads / 32);
    const int64_t w0 = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);
    for (int64_t i0 = w0 * kRowsPerStep; i0 < n_rows; i0 += n_warps * kRowsPerStep) {
        int64_t r[kRowsPerStep];
        uint32_t v[kRowsPerStep][kColsPerLane];
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
            const bool live = i0 + j < n_rows;
            r[j] = live ? (index ? (int64_t)__ldg(index + i0 + j) : i0 + j) : -1;
#pragma unroll
            for (int k = 0; k < kColsPerLane; ++k)
                v[j][k] = (live && lc.kind[k] >= 0) ? __ldg(in + (i0 + j) * Wt + lane + 32 * k) : 0u;
        }
#pragma unroll
        for (int j = 0; j < kRowsPerStep; ++j) {
            if (r[j] < 0) continue;
#pragma unroll
            for (int k = 0; k < kColsPerLane; ++k) {
                if (lc.kind[k] < 0) continue;
                if (lc.kind[k] == 1) { if (sensor_ids_out) sensor_ids_out[r[j]] = (int64_t)(int32_t)v[j][k]; }
                else if (lc.kind[k] == 2) { if (gaussian_ids_out) gaussian_ids_out[r[j]] = (int64_t)(int32_t)v[j][k]; }
                else if (lc.ptr[k]) lc.ptr[k][r[j] * lc.width[k] + lc.off[k]] = v[j][k];
            }
        }
    }
}

// Received rows come as S contiguous segments, one per (source rank, owned sensor) with the
// sensor index running fastest; segment s starts at src_start[s] in the receive buffer and at
// dst_start[s] in the final order. map[i] = final row of received row i; local_sensor[map[i]] =
// s % n_sensors, the index of the row's sensor among the sensors this rank owns. The table travels
// in the kernel's arguments (no copy to the device).
constexpr int kMaxSegments = 128;
struct SegmentTable {
    int64_t src_start[kMaxSegments];
    int64_t dst_start[kMaxSegments];
};

__global__ void __launch_bounds__(kThreads)
segment_row_map_kernel(const __grid_constant__ SegmentTable tab, int32_t S, int32_t n_sensors, int64_t n_rows,
                       int32_t *__restrict__ map, int64_t *__restrict__ local_sensor) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n_rows) return;
    int32_t lo = 0, hi = S - 1;   // last segment whose start is <= i
    while (lo < hi) {
        const int32_t mid = (lo + hi + 1) >> 1;
        if (tab.src_start[mid] <= i) lo = mid; else hi = mid - 1;
    }
    const int64_t r = tab.dst_start[lo] + (i - tab.src_start[lo]);
    map[i] = (int32_t)r;
    if (local_sensor) local_sensor[r] = (int64_t)(lo % n_sensors);
}

static int fill_fields(RowFields &f, int32_t n_fields, const void *const *ptrs, const int32_t *widths,
                       bool as_dst, const char *what) {
    SPL_REQUIRE(n_fields >= 0 && n_fields <= kMaxFields && (n_fields == 0 || (ptrs && widths)),
                SPLATAD_ERR_BAD_ARG, "%s: between 0 and %d fields with pointer and width tables", what, kMaxFields);
    f.n = n_fields;
    int32_t col = 0;
    for (int k = 0; k < kMaxFields; ++k) {
        f.src[k] = nullptr;
        f.dst[k] = nullptr;
        f.col[k] = col;
        if (k < n_fields) {
            SPL_REQUIRE(widths[k] > 0, SPLATAD_ERR_BAD_ARG, "%s: field %d has width %d", what, k, widths[k]);
            if (as_dst) f.dst[k] = (uint32_t *)ptrs[k]; else f.src[k] = (const uint32_t *)ptrs[k];
            col += widths[k];
        }
    }
    f.col[kMaxFields] = col;
    for (int k = n_fields; k <= kMaxFields; ++k) f.col[k] = col;
    return SPLATAD_OK;
}

static inline uint32_t grid_for(int64_t elems) {
    const int64_t want = (elems + kThreads - 1) / kThreads;
    const int64_t cap = (int64_t)kNumSMs * 32;
    return (uint32_t)(want < 1 ? 1 : (want > cap ? cap : want));
}

} // namespace splatad

using namespace splatad;

extern "C" size_t splatad_visible_rows_workspace_bytes(uint32_t C, uint32_t N) {
    return 2 * sizeof(int32_t) * (size_t)C * div_up(N, kThreads) + 256;
}

extern "C" int splatad_visible_rows_count(uint32_t C, uint32_t N, const void *radii, void *workspace,
                                          size_t workspace_bytes, int32_t *indptr, int64_t *total_device,
                                          void *stream) {
    SPL_REQUIRE(radii && workspace && indptr, SPLATAD_ERR_BAD_ARG, "visible_rows_count: null argument");
    SPL_REQUIRE(C > 0 && N > 0, SPLATAD_ERR_BAD_ARG, "visible_rows_count: empty input");
    SPL_REQUIRE((uint64_t)C * N <= 0x7FFFFFFFull, SPLATAD_ERR_OVERFLOW,
                "visible_rows_count: %llu (sensor, Gaussian) pairs do not fit int32 row indices",
                (unsigned long long)C * N);
    SPL_REQUIRE(workspace_bytes >= splatad_visible_rows_workspace_bytes(C, N), SPLATAD_ERR_WORKSPACE,
                "visible_rows_count: workspace too small");
    const uint32_t nblocks = div_up(N, kThreads);
    int32_t *counts = (int32_t *)workspace;
    int32_t *offsets = counts + (size_t)C * nblocks;
    cudaStream_t st = (cudaStream_t)stream;
    {
        SPL_PROF("visible_rows_count_kernel", st);
        visible_rows_count_kernel<<<nblocks, kThreads, 0, st>>>(C, N, (const int32_t *)radii, counts);
    }
    {
        SPL_PROF("visible_rows_scan_kernel", st);
        visible_rows_scan_kernel<<<1, 1024, 0, st>>>(counts, offsets, C, nblocks, indptr, total_device);
    }
    return check_launch("visible_rows_count");
}

extern "C" int splatad_visible_rows_fill(uint32_t C, uint32_t N, const void *radii, const void *workspace,
                                         int64_t capacity, int32_t *row_index, void *stream) {
    SPL_REQUIRE(radii && workspace && row_index, SPLATAD_ERR_BAD_ARG, "visible_rows_fill: null argument");
    SPL_REQUIRE(C > 0 && N > 0 && capacity >= 0, SPLATAD_ERR_BAD_ARG, "visible_rows_fill: empty input");
    const uint32_t nblocks = div_up(N, kThreads);
    const int32_t *offsets = (const int32_t *)workspace + (size_t)C * nblocks;
    {
        SPL_PROF("visible_rows_fill_kernel", (cudaStream_t)stream);
        visible_rows_fill_kernel<<<nblocks, kThreads, 0, (cudaStream_t)stream>>>(
            C, N, (const int32_t *)radii, offsets, capacity, row_index);
    }
    return check_launch("visible_rows_fill");
}

extern "C" int splatad_rows_gather(int64_t n_rows, const int32_t *index, int32_t n_fields,
                                   const void *const *field_ptrs, const int32_t *field_widths,
                                   const int32_t *sensor_table, uint32_t n_per_sensor,
                                   int32_t gaussian_start, void *out, void *stream) {
    RowFields f;
    const int rc = fill_fields(f, n_fields, field_ptrs, field_widths, false, "rows_gather");
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(n_rows >= 0 && (n_rows == 0 || out), SPLATAD_ERR_BAD_ARG, "rows_gather: null output");
    SPL_REQUIRE(!sensor_table || (index && n_per_sensor > 0), SPLATAD_ERR_BAD_ARG,
                "rows_gather: id columns need the pair index and the Gaussians per sensor");
    if (n_rows == 0) return SPLATAD_OK;
    SPL_REQUIRE(f.col[f.n] + (sensor_table ? 2 : 0) <= 32 * kMaxColsPerLane, SPLATAD_ERR_BAD_ARG,
                "rows_gather: rows of at most %d words", 32 * kMaxColsPerLane);
    // rows of up to 64 words (all the rows the renderer exchanges): two columns per lane, eight rows
    // in flight per warp; wider rows: four columns, four rows
    const bool narrow = f.col[f.n] + (sensor_table ? 2 : 0) <= 64;
    const int64_t per_warp = narrow ? 8 : 4;
    const int64_t elems = (n_rows + per_warp - 1) / per_warp * 32;
    {
        SPL_PROF("rows_gather_kernel", (cudaStream_t)stream);
        if (narrow)
            rows_gather_kernel<2, 8><<<grid_for(elems), kThreads, 0, (cudaStream_t)stream>>>(
                f, n_rows, index, sensor_table, n_per_sensor ? n_per_sensor : 1u, gaussian_start, (uint32_t *)out);
        else
            rows_gather_kernel<4, 4><<<grid_for(elems), kThreads, 0, (cudaStream_t)stream>>>(
                f, n_rows, index, sensor_table, n_per_sensor ? n_per_sensor : 1u, gaussian_start, (uint32_t *)out);
    }
    return check_launch("rows_gather");
}

extern "C" int splatad_rows_scatter(int64_t n_rows, const int32_t *index, int32_t n_fields,
                                    void *const *field_ptrs, const int32_t *field_widths, int32_t id_cols,
                                    int64_t *sensor_ids_out, int64_t *gaussian_ids_out, const void *in,
                                    void *stream) {
    RowFields f;
    const int rc = fill_fields(f, n_fields, (const void *const *)field_ptrs, field_widths, true, "rows_scatter");
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(id_cols == 0 || id_cols == 2, SPLATAD_ERR_BAD_ARG, "rows_scatter: id_cols must be 0 or 2");
    SPL_REQUIRE(n_rows >= 0 && (n_rows == 0 || in), SPLATAD_ERR_BAD_ARG, "rows_scatter: null input");
    if (n_rows == 0) return SPLATAD_OK;
    SPL_REQUIRE(f.col[f.n] + id_cols <= 32 * kMaxColsPerLane, SPLATAD_ERR_BAD_ARG,
                "rows_scatter: rows of at most %d words", 32 * kMaxColsPerLane);
    const bool narrow = f.col[f.n] + id_cols <= 64;
    const int64_t per_warp = narrow ? 8 : 4;
    const int64_t elems = (n_rows + per_warp - 1) / per_warp * 32;
    {
        SPL_PROF("rows_scatter_kernel", (cudaStream_t)stream);
        if (narrow)
            rows_scatter_kernel<2, 8><<<grid_for(elems), kThreads, 0, (cudaStream_t)stream>>>(
                f, n_rows, index, id_cols, sensor_ids_out, gaussian_ids_out, (const uint32_t *)in);
        else
            rows_scatter_kernel<4, 4><<<grid_for(elems), kThreads, 0, (cudaStream_t)stream>>>(
                f, n_rows, index, id_cols, sensor_ids_out, gaussian_ids_out, (const uint32_t *)in);
    }
    return check_launch("rows_scatter");
}

extern "C" int splatad_segment_row_map(int32_t n_segments, int32_t n_sensors, const int64_t *src_start,
                                       const int64_t *dst_start, int64_t n_rows, int32_t *row_map,
                                       int64_t *local_sensor_ids, void *stream) {
    SPL_REQUIRE(n_rows >= 0 && n_rows <= 0x7FFFFFFFll, SPLATAD_ERR_OVERFLOW,
                "segment_row_map: %lld rows do not fit int32", (long long)n_rows);
    if (n_rows == 0) return SPLATAD_OK;
    SPL_REQUIRE(n_segments > 0 && n_segments <= kMaxSegments && n_sensors > 0 && src_start && dst_start && row_map,
                SPLATAD_ERR_BAD_ARG, "segment_row_map: 1..%d segments and their tables are required", kMaxSegments);
    SegmentTable tab;
    for (int s = 0; s < kMaxSegments; ++s) {
        tab.src_start[s] = s < n_segments ? src_start[s] : 0x7FFFFFFFFFFFFFFFll;
        tab.dst_start[s] = s < n_segments ? dst_start[s] : 0;
    }
    {
        SPL_PROF("segment_row_map_kernel", (cudaStream_t)stream);
        segment_row_map_kernel<<<div_up(n_rows, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            tab, n_segments, n_sensors, n_rows, row_map, local_sensor_ids);
    }
    return check_launch("segment_row_map");
}
