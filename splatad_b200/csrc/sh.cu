// Real spherical-harmonics colour evaluation (degree 0..4) and its VJP.
//
// One thread per element evaluates all three colour channels; a block's contiguous slab of
// coefficients ([128, K, 3] floats) is moved global <-> shared with 128-bit accesses and read
// from shared memory with a padded row stride so the per-thread rows do not bank-conflict.
//
// Basis polynomials follow Sloan, "Efficient Spherical Harmonic Evaluation" (JCGT 2013), in
// the same arrangement as the reference: gsplat/cuda/csrc/sh.cu:13-93 (forward), 95-353 (VJP),
// kernels 355-406. Masked-out elements are written as zeros (the reference leaves them
// uninitialised).
#include "common.cuh"

namespace splatad {

constexpr int kShThreads = 128;
constexpr int kShMaxBases = 25;

// Fills b[0 .. (deg+1)^2) for a unit direction.
__device__ __forceinline__ void sh_bases(int deg, float x, float y, float z, float *b) {
    b[0] = 0.2820947917738781f;
    if (deg < 1) return;
    b[1] = -0.48860251190292f * y;
    b[2] = 0.48860251190292f * z;
    b[3] = -0.48860251190292f * x;
    if (deg < 2) return;
    const float z2 = z * z;
    const float fTmp0B = -1.092548430592079f * z;
    const float fC1 = x * x - y * y;
    const float fS1 = 2.f * x * y;
    b[4] = 0.5462742152960395f * fS1;
    b[5] = fTmp0B * y;
    b[6] = 0.9461746957575601f * z2 - 0.3153915652525201f;
    b[7] = fTmp0B * x;
    b[8] = 0.5462742152960395f * fC1;
    if (deg < 3) return;
    const float fTmp0C = -2.285228997322329f * z2 + 0.4570457994644658f;
    const float fTmp1B = 1.445305721320277f * z;
    const float fC2 = x * fC1 - y * fS1;
    const float fS2 = x * fS1 + y * fC1;
    b[9] = -0.5900435899266435f * fS2;
    b[10] = fTmp1B * fS1;
    b[11] = fTmp0C * y;
    b[12] = z * (1.865881662950577f * z2 - 1.119528997770346f);
    b[13] = fTmp0C * x;
    b[14] = fTmp1B * fC1;
    b[15] = -0.5900435899266435f * fC2;
    if (deg < 4) return;
    const float fTmp0D = z * (-4.683325804901025f * z2 + 2.007139630671868f);
    const float fTmp1C = 3.31161143515146f * z2 - 0.47308734787878f;
    const float fTmp2B = -1.770130769779931f * z;
    const float fC3 = x * fC2 - y * fS2;
    const float fS3 = x * fS2 + y * fC2;
    b[16] = 0.6258357354491763f * fS3;
    b[17] = fTmp2B * fS2;
    b[18] = fTmp1C * fS1;
    b[19] = fTmp0D * y;
    b[20] = 1.984313483298443f * z * b[12] - 1.006230589874905f * b[6];
    b[21] = fTmp0D * x;
    b[22] = fTmp1C * fC1;
    b[23] = fTmp2B * fC2;
    b[24] = 0.6258357354491763f * fC3;
}

// Partial derivatives of the bases with respect to the (unit) direction components.
__device__ __forceinline__ void sh_bases_grad(int deg, float x, float y, float z, float *bx,
                                              float *by, float *bz) {
    bx[0] = by[0] = bz[0] = 0.f;
    if (deg < 1) return;
    bx[1] = 0.f; by[1] = -0.48860251190292f; bz[1] = 0.f;
    bx[2] = 0.f; by[2] = 0.f; bz[2] = 0.48860251190292f;
    bx[3] = -0.48860251190292f; by[3] = 0.f; bz[3] = 0.f;
    if (deg < 2) return;
    const float z2 = z * z;
    const float fTmp0B = -1.092548430592079f * z, fTmp0B_z = -1.092548430592079f;
    const float fC1 = x * x - y * y, fC1_x = 2.f * x, fC1_y = -2.f * y;
    const float fS1 = 2.f * x * y, fS1_x = 2.f * y, fS1_y = 2.f * x;
    bx[4] = 0.5462742152960395f * fS1_x; by[4] = 0.5462742152960395f * fS1_y; bz[4] = 0.f;
    bx[5] = 0.f; by[5] = fTmp0B; bz[5] = fTmp0B_z * y;
    bx[6] = 0.f; by[6] = 0.f; bz[6] = 2.f * 0.9461746957575601f * z;
    bx[7] = fTmp0B; by[7] = 0.f; bz[7] = fTmp0B_z * x;
    bx[8] = 0.5462742152960395f * fC1_x; by[8] = 0.5462742152960395f * fC1_y; bz[8] = 0.f;
    if (deg < 3) return;
    const float fTmp0C = -2.285228997322329f * z2 + 0.4570457994644658f;
    const float fTmp0C_z = -2.285228997322329f * 2.f * z;
    const float fTmp1B = 1.445305721320277f * z, fTmp1B_z = 1.445305721320277f;
    const float fC2 = x * fC1 - y * fS1, fS2 = x * fS1 + y * fC1;
    const float fC2_x = fC1 + x * fC1_x - y * fS1_x;
    const float fC2_y = x * fC1_y - fS1 - y * fS1_y;
    const float fS2_x = fS1 + x * fS1_x + y * fC1_x;
    const float fS2_y = x * fS1_y + fC1 + y * fC1_y;
    const float pSH12 = z * (1.865881662950577f * z2 - 1.119528997770346f);
    const float pSH12_z = 3.f * 1.865881662950577f * z2 - 1.119528997770346f;
    bx[9] = -0.5900435899266435f * fS2_x; by[9] = -0.5900435899266435f * fS2_y; bz[9] = 0.f;
    bx[10] = fTmp1B * fS1_x; by[10] = fTmp1B * fS1_y; bz[10] = fTmp1B_z * fS1;
    bx[11] = 0.f; by[11] = fTmp0C; bz[11] = fTmp0C_z * y;
    bx[12] = 0.f; by[12] = 0.f; bz[12] = pSH12_z;
    bx[13] = fTmp0C; by[13] = 0.f; bz[13] = fTmp0C_z * x;
    bx[14] = fTmp1B * fC1_x; by[14] = fTmp1B * fC1_y; bz[14] = fTmp1B_z * fC1;
    bx[15] = -0.5900435899266435f * fC2_x; by[15] = -0.5900435899266435f * fC2_y; bz[15] = 0.f;
    if (deg < 4) return;
    const float fTmp0D = z * (-4.683325804901025f * z2 + 2.007139630671868f);
    const float fTmp0D_z = 3.f * -4.683325804901025f * z2 + 2.007139630671868f;
    const float fTmp1C = 3.31161143515146f * z2 - 0.47308734787878f;
    const float fTmp1C_z = 2.f * 3.31161143515146f * z;
    const float fTmp2B = -1.770130769779931f * z, fTmp2B_z = -1.770130769779931f;
    const float fC3_x = fC2 + x * fC2_x - y * fS2_x;
    const float fC3_y = x * fC2_y - fS2 - y * fS2_y;
    const float fS3_x = fS2 + y * fC2_x + x * fS2_x;
    const float fS3_y = x * fS2_y + fC2 + y * fC2_y;
    const float pSH6_z = 2.f * 0.9461746957575601f * z;
    bx[16] = 0.6258357354491763f * fS3_x; by[16] = 0.6258357354491763f * fS3_y; bz[16] = 0.f;
    bx[17] = fTmp2B * fS2_x; by[17] = fTmp2B * fS2_y; bz[17] = fTmp2B_z * fS2;
    bx[18] = fTmp1C * fS1_x; by[18] = fTmp1C * fS1_y; bz[18] = fTmp1C_z * fS1;
    bx[19] = 0.f; by[19] = fTmp0D; bz[19] = fTmp0D_z * y;
    bx[20] = 0.f; by[20] = 0.f;
    bz[20] = 1.984313483298443f * (pSH12 + z * pSH12_z) - 1.006230589874905f * pSH6_z;
    bx[21] = fTmp0D; by[21] = 0.f; bz[21] = fTmp0D_z * x;
    bx[22] = fTmp1C * fC1_x; by[22] = fTmp1C * fC1_y; bz[22] = fTmp1C_z * fC1;
    bx[23] = fTmp2B * fC2_x; by[23] = fTmp2B * fC2_y; bz[23] = fTmp2B_z * fC2;
    bx[24] = 0.6258357354491763f * fC3_x; by[24] = 0.6258357354491763f * fC3_y; bz[24] = 0.f;
}

// global [n, row] floats -> shared with row stride row+1
__device__ __forceinline__ void stage_rows_in(const float *__restrict__ src, float *smem,
                                              uint32_t n, uint32_t row) {
    const uint32_t nfl = n * row;
    if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
        const uint32_t nvec = nfl >> 2;
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x) {
            const float4 v = __ldg(s4 + i);
            const float vv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t f = 4 * i + k;
                smem[(f / row) * (row + 1) + f % row] = vv[k];
            }
        }
        for (uint32_t f = (nvec << 2) + threadIdx.x; f < nfl; f += blockDim.x)
            smem[(f / row) * (row + 1) + f % row] = __ldg(src + f);
    } else {
        for (uint32_t f = threadIdx.x; f < nfl; f += blockDim.x)
            smem[(f / row) * (row + 1) + f % row] = __ldg(src + f);
    }
}

__device__ __forceinline__ void stage_rows_out(float *__restrict__ dst, const float *smem,
                                               uint32_t n, uint32_t row) {
    const uint32_t nfl = n * row;
    if ((reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        const uint32_t nvec = nfl >> 2;
        float4 *d4 = reinterpret_cast<float4 *>(dst);
        for (uint32_t i = threadIdx.x; i < nvec; i += blockDim.x) {
            float vv[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t f = 4 * i + k;
                vv[k] = smem[(f / row) * (row + 1) + f % row];
            }
            d4[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
        }
        for (uint32_t f = (nvec << 2) + threadIdx.x; f < nfl; f += blockDim.x)
            dst[f] = smem[(f / row) * (row + 1) + f % row];
    } else {
        for (uint32_t f = threadIdx.x; f < nfl; f += blockDim.x)
            dst[f] = smem[(f / row) * (row + 1) + f % row];
    }
}

__global__ void __launch_bounds__(kShThreads)
sh_fwd_kernel(uint32_t n_elems, uint32_t K, int degree, const float *__restrict__ dirs,
              const float *__restrict__ coeffs, const uint8_t *__restrict__ masks,
              float *__restrict__ colors) {
    extern __shared__ __align__(16) float sm[];   // [kShThreads][3K+1]
    const uint32_t e0 = blockIdx.x * kShThreads;
    const uint32_t n = min((uint32_t)kShThreads, n_elems - e0);
    const uint32_t row = 3 * K;
    stage_rows_in(coeffs + (size_t)e0 * row, sm, n, row);
    __syncthreads();
    const uint32_t t = threadIdx.x;
    if (t >= n) return;
    const size_t e = (size_t)e0 + t;
    float r = 0.f, g = 0.f, bl = 0.f;
    if (masks == nullptr || masks[e]) {
        const float dx = dirs[3 * e], dy = dirs[3 * e + 1], dz = dirs[3 * e + 2];
        const float inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
        float b[kShMaxBases];
        sh_bases(degree, dx * inorm, dy * inorm, dz * inorm, b);
        const float *c = sm + t * (row + 1);
        const int nb = (degree + 1) * (degree + 1);
#pragma unroll
        for (int i = 0; i < kShMaxBases; ++i)
            if (i < nb) {
                r += b[i] * c[3 * i];
                g += b[i] * c[3 * i + 1];
                bl += b[i] * c[3 * i + 2];
            }
    }
    colors[3 * e] = r;
    colors[3 * e + 1] = g;
    colors[3 * e + 2] = bl;
}

__global__ void __launch_bounds__(kShThreads)
sh_bwd_kernel(uint32_t n_elems, uint32_t K, int degree, const float *__restrict__ dirs,
              const float *__restrict__ coeffs, const uint8_t *__restrict__ masks,
              const float *__restrict__ v_colors, float *__restrict__ v_coeffs,
              float *__restrict__ v_dirs) {
    extern __shared__ __align__(16) float sm[];   // [kShThreads][3K+1]
    const uint32_t e0 = blockIdx.x * kShThreads;
    const uint32_t n = min((uint32_t)kShThreads, n_elems - e0);
    const uint32_t row = 3 * K;
    const uint32_t t = threadIdx.x;
    const size_t e = (size_t)e0 + t;
    const bool live = t < n;
    const bool active = live && (masks == nullptr || masks[e]);
    const int nb = (degree + 1) * (degree + 1);
    float x = 0.f, y = 0.f, z = 1.f, inorm = 1.f;
    float vr = 0.f, vg = 0.f, vb = 0.f;
    if (active) {
        const float dx = dirs[3 * e], dy = dirs[3 * e + 1], dz = dirs[3 * e + 2];
        inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
        x = dx * inorm; y = dy * inorm; z = dz * inorm;
        vr = v_colors[3 * e]; vg = v_colors[3 * e + 1]; vb = v_colors[3 * e + 2];
    }
    if (v_dirs != nullptr) {
        stage_rows_in(coeffs + (size_t)e0 * row, sm, n, row);
        __syncthreads();
        if (live) {
            float gx = 0.f, gy = 0.f, gz = 0.f;
            if (active) {
                float bx[kShMaxBases], by[kShMaxBases], bz[kShMaxBases];
                sh_bases_grad(degree, x, y, z, bx, by, bz);
                const float *c = sm + t * (row + 1);
#pragma unroll
                for (int i = 0; i < kShMaxBases; ++i)
                    if (i < nb) {
                        const float w = vr * c[3 * i] + vg * c[3 * i + 1] + vb * c[3 * i + 2];
                        gx += bx[i] * w; gy += by[i] * w; gz += bz[i] * w;
                    }
                const float d = gx * x + gy * y + gz * z;
                gx = (gx - d * x) * inorm;
                gy = (gy - d * y) * inorm;
                gz = (gz - d * z) * inorm;
            }
            v_dirs[3 * e] = gx; v_dirs[3 * e + 1] = gy; v_dirs[3 * e + 2] = gz;
        }
        __syncthreads();
    }
    if (live) {
        float b[kShMaxBases];
        sh_bases(degree, x, y, z, b);
        float *c = sm + t * (row + 1);
#pragma unroll
        for (int i = 0; i < kShMaxBases; ++i)
            if ((uint32_t)i < K) {
                const float bi = (active && i < nb) ? b[i] : 0.f;
                c[3 * i] = bi * vr;
                c[3 * i + 1] = bi * vg;
                c[3 * i + 2] = bi * vb;
            }
        for (uint32_t i = kShMaxBases; i < K; ++i) {
            c[3 * i] = 0.f; c[3 * i + 1] = 0.f; c[3 * i + 2] = 0.f;
        }
    }
    __syncthreads();
    stage_rows_out(v_coeffs + (size_t)e0 * row, sm, n, row);
}

// ---------------------------------------------------------------------------------------
// View-dependent colours of the projected Gaussians in one pass: what the reference's
// rasterization() builds from a chain of torch ops around its SH kernel
// (gsplat/rendering.py:345-373: gather means / camera centres / coefficients by the packed ids,
// directions, spherical_harmonics, + 0.5, clamp at 0, concatenation of the depth channel).
// Entry e is (camera_ids[e], gaussian_ids[e]) in the packed layout and (e / N, e % N) in the
// dense one; entries with radii[e][0] <= 0 produce zeros and read no coefficients.
// ---------------------------------------------------------------------------------------
struct ShColorArgs {
    uint32_t n_elems, N, K;
    int degree;
    const float *means;         // [N, 3]
    const float *campos;        // [C, 3]
    const float *coeffs;        // [N, K, 3] or [C, N, K, 3]
    uint32_t coeffs_per_camera;
    const int64_t *camera_ids, *gaussian_ids;   // packed layout, else null
    const int32_t *radii;       // [n_elems, 2]
    const float *depths;        // [n_elems] or null
    uint32_t out_channels;      // 3, or 4 with the depth as last channel
};

__device__ __forceinline__ void sh_entry(const ShColorArgs &a, size_t e, uint32_t &cam, uint32_t &g) {
    if (a.gaussian_ids) {
        cam = (uint32_t)a.camera_ids[e];
        g = (uint32_t)a.gaussian_ids[e];
    } else {
        cam = (uint32_t)(e / a.N);
        g = (uint32_t)(e - (size_t)cam * a.N);
    }
}

// Gathers the first nfl floats of the coefficient rows listed in rows[0 .. n) (negative = skip)
// into shared memory with row stride row + 1.
__device__ __forceinline__ void stage_rows_gather(const float *__restrict__ coeffs, const int64_t *rows,
                                                  float *smem, uint32_t n, uint32_t row, uint32_t nfl) {
    if ((row & 3u) == 0 && (nfl & 3u) == 0 && (reinterpret_cast<uintptr_t>(coeffs) & 15u) == 0) {
        // four 16-byte loads in flight per thread before the first of them is stored: with a load and
        // its store in one loop iteration every thread waited out the memory latency twelve times
        const uint32_t per_row = nfl >> 2, total = n * per_row;
        constexpr int kInFlight = 4;
        for (uint32_t i0 = threadIdx.x; i0 < total; i0 += kInFlight * blockDim.x) {
            float4 v[kInFlight];
            uint32_t at[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const uint32_t i = i0 + u * blockDim.x;
                at[u] = 0xffffffffu;
                if (i >= total) continue;
                const uint32_t r = i / per_row, q = i - r * per_row;
                const int64_t src = rows[r];
                if (src < 0) continue;
                v[u] = __ldg(reinterpret_cast<const float4 *>(coeffs + (size_t)src * row) + q);
                at[u] = r * (row + 1) + 4 * q;
            }
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                if (at[u] == 0xffffffffu) continue;
                float *d = smem + at[u];
                d[0] = v[u].x; d[1] = v[u].y; d[2] = v[u].z; d[3] = v[u].w;
            }
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n * nfl; i += blockDim.x) {
            const uint32_t r = i / nfl, q = i - r * nfl;
            const int64_t src = rows[r];
            if (src < 0) continue;
            smem[r * (row + 1) + q] = __ldg(coeffs + (size_t)src * row + q);
        }
    }
}

// Adds the first nfl floats of the staged rows (row stride row + 1) to the rows of dst listed in
// rows[0 .. n) (negative = skip): consecutive threads add consecutive words of a row, four at a
// time where the alignment allows, instead of every thread walking its own row with scalar atomics.
__device__ __forceinline__ void scatter_rows_add(float *__restrict__ dst, const int64_t *rows, const float *smem,
                                                 uint32_t n, uint32_t row, uint32_t nfl) {
    if ((row & 3u) == 0 && (nfl & 3u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
        const uint32_t per_row = nfl >> 2;
        for (uint32_t i = threadIdx.x; i < n * per_row; i += blockDim.x) {
            const uint32_t r = i / per_row, q = i - r * per_row;
            const int64_t to = rows[r];
            if (to < 0) continue;
            const float *v = smem + r * (row + 1) + 4 * q;
            atomicAdd(reinterpret_cast<float4 *>(dst + (size_t)to * row) + q, make_float4(v[0], v[1], v[2], v[3]));
        }
    } else {
        for (uint32_t i = threadIdx.x; i < n * nfl; i += blockDim.x) {
            const uint32_t r = i / nfl, q = i - r * nfl;
            const int64_t to = rows[r];
            if (to < 0) continue;
            atomicAdd(dst + (size_t)to * row + q, smem[r * (row + 1) + q]);
        }
    }
}

__global__ void __launch_bounds__(kShThreads)
sh_colors_fwd_kernel(const ShColorArgs a, float *__restrict__ colors) {
    extern __shared__ __align__(16) float sm[];   // [kShThreads][3K+1] floats, then the row indices
    const uint32_t row = 3 * a.K;
    int64_t *rows = reinterpret_cast<int64_t *>(sm + ((kShThreads * (row + 1) + 1) & ~1u));
    const uint32_t e0 = blockIdx.x * kShThreads;
    const uint32_t n = min((uint32_t)kShThreads, a.n_elems - e0);
    const uint32_t t = threadIdx.x;
    const size_t e = (size_t)e0 + t;
    const int nb = (a.degree + 1) * (a.degree + 1);
    bool active = false;
    float dx = 0.f, dy = 0.f, dz = 1.f;
    if (t < n) {
        uint32_t cam, g;
        sh_entry(a, e, cam, g);
        active = a.radii[2 * e] > 0;
        rows[t] = active ? (int64_t)(a.coeffs_per_camera ? (size_t)cam * a.N + g : g) : -1;
        if (active) {
            dx = a.means[3 * (size_t)g] - a.campos[3 * cam];
            dy = a.means[3 * (size_t)g + 1] - a.campos[3 * cam + 1];
            dz = a.means[3 * (size_t)g + 2] - a.campos[3 * cam + 2];
        }
    }
    __syncthreads();
    stage_rows_gather(a.coeffs, rows, sm, n, row, 3 * nb);
    __syncthreads();
    if (t >= n) return;
    float r = 0.f, gg = 0.f, bl = 0.f;
    if (active) {
        const float inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
        float b[kShMaxBases];
        sh_bases(a.degree, dx * inorm, dy * inorm, dz * inorm, b);
        const float *c = sm + t * (row + 1);
#pragma unroll
        for (int i = 0; i < kShMaxBases; ++i)
            if (i < nb) {
                r += b[i] * c[3 * i];
                gg += b[i] * c[3 * i + 1];
                bl += b[i] * c[3 * i + 2];
            }
    }
    // + 0.5 and the clamp at zero apply to every entry, culled ones included (they hold 0 + 0.5)
    float *o = colors + e * a.out_channels;
    o[0] = fmaxf(r + 0.5f, 0.f);
    o[1] = fmaxf(gg + 0.5f, 0.f);
    o[2] = fmaxf(bl + 0.5f, 0.f);
    if (a.out_channels == 4) o[3] = a.depths[e];
}

// VJP of the above. v_coeffs / v_means / v_campos are accumulated with atomics (zero-initialise);
// v_depths [n_elems] is overwritten. Any of them may be null.
__global__ void __launch_bounds__(kShThreads)
sh_colors_bwd_kernel(const ShColorArgs a, const float *__restrict__ v_colors, float *__restrict__ v_coeffs,
                     float *__restrict__ v_means, float *__restrict__ v_campos, float *__restrict__ v_depths) {
    extern __shared__ __align__(16) float sm[];
    const uint32_t row = 3 * a.K;
    int64_t *rows = reinterpret_cast<int64_t *>(sm + ((kShThreads * (row + 1) + 1) & ~1u));
    const uint32_t e0 = blockIdx.x * kShThreads;
    const uint32_t n = min((uint32_t)kShThreads, a.n_elems - e0);
    const uint32_t t = threadIdx.x;
    const size_t e = (size_t)e0 + t;
    const int nb = (a.degree + 1) * (a.degree + 1);
    bool active = false;
    uint32_t cam = 0, g = 0;
    float dx = 0.f, dy = 0.f, dz = 1.f;
    if (t < n) {
        sh_entry(a, e, cam, g);
        active = a.radii[2 * e] > 0;
        rows[t] = active ? (int64_t)(a.coeffs_per_camera ? (size_t)cam * a.N + g : g) : -1;
        if (active) {
            dx = a.means[3 * (size_t)g] - a.campos[3 * cam];
            dy = a.means[3 * (size_t)g + 1] - a.campos[3 * cam + 1];
            dz = a.means[3 * (size_t)g + 2] - a.campos[3 * cam + 2];
        }
        if (v_depths) v_depths[e] = a.out_channels == 4 ? v_colors[e * a.out_channels + 3] : 0.f;
    }
    __syncthreads();
    stage_rows_gather(a.coeffs, rows, sm, n, row, 3 * nb);
    __syncthreads();
    float gx = 0.f, gy = 0.f, gz = 0.f;
    if (active) {
        const float inorm = rsqrtf(dx * dx + dy * dy + dz * dz);
        const float x = dx * inorm, y = dy * inorm, z = dz * inorm;
        float b[kShMaxBases];
        sh_bases(a.degree, x, y, z, b);
        const float *c = sm + t * (row + 1);
        float r = 0.f, gg = 0.f, bl = 0.f;
#pragma unroll
        for (int i = 0; i < kShMaxBases; ++i)
            if (i < nb) {
                r += b[i] * c[3 * i];
                gg += b[i] * c[3 * i + 1];
                bl += b[i] * c[3 * i + 2];
            }
        // the clamp passes the gradient where its input is >= 0, like torch.clamp_min
        const float *vc = v_colors + e * a.out_channels;
        const float vr = (r + 0.5f >= 0.f) ? vc[0] : 0.f;
        const float vg = (gg + 0.5f >= 0.f) ? vc[1] : 0.f;
        const float vb = (bl + 0.5f >= 0.f) ? vc[2] : 0.f;
        if (v_means || v_campos) {
            float bx[kShMaxBases], by[kShMaxBases], bz[kShMaxBases];
            sh_bases_grad(a.degree, x, y, z, bx, by, bz);
#pragma unroll
            for (int i = 0; i < kShMaxBases; ++i)
                if (i < nb) {
                    const float w = vr * c[3 * i] + vg * c[3 * i + 1] + vb * c[3 * i + 2];
                    gx += bx[i] * w; gy += by[i] * w; gz += bz[i] * w;
                }
            const float d = gx * x + gy * y + gz * z;
            gx = (gx - d * x) * inorm;
            gy = (gy - d * y) * inorm;
            gz = (gz - d * z) * inorm;
            if (v_means) {
                atomicAdd(v_means + 3 * (size_t)g, gx);
                atomicAdd(v_means + 3 * (size_t)g + 1, gy);
                atomicAdd(v_means + 3 * (size_t)g + 2, gz);
            }
        }
        if (v_coeffs) {
            // the coefficient row of this thread is no longer needed: its gradient takes its place
            // and leaves with the block's cooperative scatter below
            float *vrow = sm + t * (row + 1);
#pragma unroll
            for (int i = 0; i < kShMaxBases; ++i)
                if (i < nb) {
                    vrow[3 * i] = b[i] * vr;
                    vrow[3 * i + 1] = b[i] * vg;
                    vrow[3 * i + 2] = b[i] * vb;
                }
        }
    }
    if (v_coeffs) {
        __syncthreads();
        scatter_rows_add(v_coeffs, rows, sm, n, row, 3 * nb);
    }
    if (v_campos) {
        // d dirs / d campos = -1: one atomic per warp when its lanes share a camera
        const uint32_t cam0 = __shfl_sync(0xffffffffu, cam, 0);
        if (__all_sync(0xffffffffu, cam == cam0 || !active)) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                gx += __shfl_xor_sync(0xffffffffu, gx, off);
                gy += __shfl_xor_sync(0xffffffffu, gy, off);
                gz += __shfl_xor_sync(0xffffffffu, gz, off);
            }
            // lane 0 may be inactive with cam = 0: take the camera of any active lane
            const uint32_t act = __ballot_sync(0xffffffffu, active);
            if (act) {
                const uint32_t camw = __shfl_sync(0xffffffffu, cam, __ffs(act) - 1);
                if ((threadIdx.x & 31) == 0) {
                    atomicAdd(v_campos + 3 * camw, -gx);
                    atomicAdd(v_campos + 3 * camw + 1, -gy);
                    atomicAdd(v_campos + 3 * camw + 2, -gz);
                }
            }
        } else if (active) {
            atomicAdd(v_campos + 3 * cam, -gx);
            atomicAdd(v_campos + 3 * cam + 1, -gy);
            atomicAdd(v_campos + 3 * cam + 2, -gz);
        }
    }
}

// Camera centres in world coordinates, the translation column of inverse(viewmat), by cofactors
// in double precision (the general 4 x 4 inverse: the last row need not be 0 0 0 1).
__global__ void camera_centers_kernel(uint32_t C, const float *__restrict__ viewmats, float *__restrict__ campos) {
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    double m[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) m[i][j] = (double)viewmats[16 * (size_t)c + 4 * i + j];
    // cof[j] = cofactor of m[3][j]: (-1)^(3 + j) times the minor of the first three rows without column j
    double cof[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int c0 = j == 0 ? 1 : 0, c1 = j <= 1 ? 2 : 1, c2 = j <= 2 ? 3 : 2;
        const double minor = m[0][c0] * (m[1][c1] * m[2][c2] - m[1][c2] * m[2][c1]) -
                             m[0][c1] * (m[1][c0] * m[2][c2] - m[1][c2] * m[2][c0]) +
                             m[0][c2] * (m[1][c0] * m[2][c1] - m[1][c1] * m[2][c0]);
        cof[j] = ((3 + j) & 1) ? -minor : minor;
    }
    const double det = m[3][0] * cof[0] + m[3][1] * cof[1] + m[3][2] * cof[2] + m[3][3] * cof[3];
    // inverse[i][3] = cofactor(3, i) / det
#pragma unroll
    for (int i = 0; i < 3; ++i) campos[3 * (size_t)c + i] = (float)(cof[i] / det);
}

static size_t sh_colors_smem(uint32_t K) {
    return sizeof(float) * ((kShThreads * (3 * K + 1) + 1) & ~1u) + sizeof(int64_t) * kShThreads;
}

static int sh_colors_check(const ShColorArgs &a, const char *what) {
    SPL_REQUIRE(a.degree >= 0 && a.degree <= 4, SPLATAD_ERR_BAD_ARG, "%s: degree must be <= 4", what);
    SPL_REQUIRE((uint32_t)((a.degree + 1) * (a.degree + 1)) <= a.K, SPLATAD_ERR_BAD_ARG,
                "%s: K too small for the degree", what);
    SPL_REQUIRE(a.out_channels == 3 || (a.out_channels == 4 && a.depths), SPLATAD_ERR_BAD_ARG,
                "%s: 3 channels, or 4 with depths", what);
    SPL_REQUIRE(a.means && a.campos && a.coeffs && a.radii && a.N > 0, SPLATAD_ERR_BAD_ARG,
                "%s: null argument", what);
    SPL_REQUIRE((a.camera_ids == nullptr) == (a.gaussian_ids == nullptr), SPLATAD_ERR_BAD_ARG,
                "%s: camera_ids and gaussian_ids go together", what);
    SPL_REQUIRE(sh_colors_smem(a.K) <= 200 * 1024, SPLATAD_ERR_BAD_ARG, "%s: K too large", what);
    return SPLATAD_OK;
}

} // namespace splatad

using namespace splatad;
extern "C" int splatad_sh_colors_fwd(uint32_t n_elems, uint32_t N, uint32_t K, uint32_t degrees_to_use,
                                     const float *means, const float *campos, const float *coeffs,
                                     uint32_t coeffs_per_camera, const int64_t *camera_ids,
                                     const int64_t *gaussian_ids, const int32_t *radii, const float *depths,
                                     uint32_t out_channels, float *colors, void *stream) {
    if (n_elems == 0) return SPLATAD_OK;
    const ShColorArgs a = {n_elems, N, K, (int)degrees_to_use, means, campos, coeffs, coeffs_per_camera,
                           camera_ids, gaussian_ids, radii, depths, out_channels};
    int rc = sh_colors_check(a, "sh_colors_fwd");
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(colors, SPLATAD_ERR_BAD_ARG, "sh_colors_fwd: null output");
    const size_t smem = sh_colors_smem(K);
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(sh_colors_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    {
        SPL_PROF("sh_colors_fwd_kernel", (cudaStream_t)stream);
        sh_colors_fwd_kernel<<<div_up(n_elems, kShThreads), kShThreads, smem, (cudaStream_t)stream>>>(a, colors);
    }
    return check_launch("sh_colors_fwd");
}

extern "C" int splatad_sh_colors_bwd(uint32_t n_elems, uint32_t N, uint32_t K, uint32_t degrees_to_use,
                                     const float *means, const float *campos, const float *coeffs,
                                     uint32_t coeffs_per_camera, const int64_t *camera_ids,
                                     const int64_t *gaussian_ids, const int32_t *radii,
                                     uint32_t out_channels, const float *v_colors, float *v_coeffs,
                                     float *v_means, float *v_campos, float *v_depths, void *stream) {
    if (n_elems == 0) return SPLATAD_OK;
    // the depth values are not needed for the VJP: any non-null pointer satisfies the check
    const ShColorArgs a = {n_elems, N, K, (int)degrees_to_use, means, campos, coeffs, coeffs_per_camera,
                           camera_ids, gaussian_ids, radii, out_channels == 4 ? means : nullptr, out_channels};
    int rc = sh_colors_check(a, "sh_colors_bwd");
    if (rc != SPLATAD_OK) return rc;
    SPL_REQUIRE(v_colors, SPLATAD_ERR_BAD_ARG, "sh_colors_bwd: null argument");
    const size_t smem = sh_colors_smem(K);
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(sh_colors_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    {
        SPL_PROF("sh_colors_bwd_kernel", (cudaStream_t)stream);
        sh_colors_bwd_kernel<<<div_up(n_elems, kShThreads), kShThreads, smem, (cudaStream_t)stream>>>(
            a, v_colors, v_coeffs, v_means, v_campos, v_depths);
    }
    return check_launch("sh_colors_bwd");
}


extern "C" int splatad_sh_fwd(uint32_t n_elems, uint32_t K, uint32_t degrees_to_use,
                              const float *dirs, const float *coeffs, const uint8_t *masks,
                              float *colors, void *stream) {
    SPL_REQUIRE(degrees_to_use <= 4, SPLATAD_ERR_BAD_ARG, "sh_fwd: degree must be <= 4");
    SPL_REQUIRE((degrees_to_use + 1) * (degrees_to_use + 1) <= K, SPLATAD_ERR_BAD_ARG,
                "sh_fwd: K too small for the degree");
    if (n_elems == 0) return SPLATAD_OK;
    SPL_REQUIRE(dirs && coeffs && colors, SPLATAD_ERR_BAD_ARG, "sh_fwd: null argument");
    const size_t smem = sizeof(float) * kShThreads * (3 * K + 1);
    SPL_REQUIRE(smem <= 200 * 1024, SPLATAD_ERR_BAD_ARG, "sh_fwd: K too large");
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(sh_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    {
        SPL_PROF("sh_fwd_kernel", (cudaStream_t)stream);
        sh_fwd_kernel<<<div_up(n_elems, kShThreads), kShThreads, smem, (cudaStream_t)stream>>>(
            n_elems, K, (int)degrees_to_use, dirs, coeffs, masks, colors);
    }
    return check_launch("sh_fwd");
}

extern "C" int splatad_sh_bwd(uint32_t n_elems, uint32_t K, uint32_t degrees_to_use,
                              const float *dirs, const float *coeffs, const uint8_t *masks,
                              const float *v_colors, float *v_coeffs, float *v_dirs,
                              void *stream) {
    SPL_REQUIRE(degrees_to_use <= 4, SPLATAD_ERR_BAD_ARG, "sh_bwd: degree must be <= 4");
    SPL_REQUIRE((degrees_to_use + 1) * (degrees_to_use + 1) <= K, SPLATAD_ERR_BAD_ARG,
                "sh_bwd: K too small for the degree");
    if (n_elems == 0) return SPLATAD_OK;
    SPL_REQUIRE(dirs && coeffs && v_colors && v_coeffs, SPLATAD_ERR_BAD_ARG, "sh_bwd: null argument");
    const size_t smem = sizeof(float) * kShThreads * (3 * K + 1);
    SPL_REQUIRE(smem <= 200 * 1024, SPLATAD_ERR_BAD_ARG, "sh_bwd: K too large");
    if (smem > 32 * 1024)
        cudaFuncSetAttribute(sh_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    {
        SPL_PROF("sh_bwd_kernel", (cudaStream_t)stream);
        sh_bwd_kernel<<<div_up(n_elems, kShThreads), kShThreads, smem, (cudaStream_t)stream>>>(
            n_elems, K, (int)degrees_to_use, dirs, coeffs, masks, v_colors, v_coeffs, v_dirs);
    }
    return check_launch("sh_bwd");
}

extern "C" int splatad_camera_centers(uint32_t C, const float *viewmats, float *campos, void *stream) {
    if (C == 0) return SPLATAD_OK;
    SPL_REQUIRE(viewmats && campos, SPLATAD_ERR_BAD_ARG, "camera_centers: null argument");
    camera_centers_kernel<<<div_up(C, 64), 64, 0, (cudaStream_t)stream>>>(C, viewmats, campos);
    return check_launch("camera_centers");
}
