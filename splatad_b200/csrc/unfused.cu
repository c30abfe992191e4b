// The unfused building blocks of the projection, exported by the reference as separate ops
// (gsplat/__init__.py:4-18; kernels in gsplat/cuda/csrc/projection.cu:18-599, 1841-2266):
// quat_scale_to_covar_preci, world_to_cam, persp_proj, compute_pix_velocity, lidar_proj and
// compute_lidar_velocity, each with its backward. They are plain maps over Gaussians or
// (sensor, Gaussian) pairs built from the same device math as the fused kernels
// (splat_math.cuh); one thread per element, no shared state except the pose gradient.
#include "common.cuh"
#include "splat_math.cuh"

namespace splatad {

__device__ __forceinline__ V3 ld3g(const float *p) { return v3(p[0], p[1], p[2]); }
__device__ __forceinline__ void st3g(float *p, V3 v) { p[0] = v.x; p[1] = v.y; p[2] = v.z; }

__device__ __forceinline__ M3 ld_m3(const float *p) {
    M3 m;
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
        for (int j = 0; j < 3; ++j) m.m[i][j] = p[3 * i + j];
    return m;
}

__device__ __forceinline__ void st_m3(float *p, const M3 &m) {
#pragma unroll
    for (int i = 0; i < 3; ++i)
#pragma unroll
        for (int j = 0; j < 3; ++j) p[3 * i + j] = m.m[i][j];
}

__device__ __forceinline__ void st_triu(float *p, const M3 &m) {
    p[0] = m.m[0][0]; p[1] = m.m[0][1]; p[2] = m.m[0][2];
    p[3] = m.m[1][1]; p[4] = m.m[1][2]; p[5] = m.m[2][2];
}

// Gradient of a matrix given through its upper triangle: off-diagonal entries are shared by
// the two symmetric positions (gsplat/cuda/csrc/projection.cu:116-121).
__device__ __forceinline__ M3 ld_triu_grad(const float *p) {
    M3 m;
    m.m[0][0] = p[0]; m.m[1][1] = p[3]; m.m[2][2] = p[5];
    m.m[0][1] = m.m[1][0] = 0.5f * p[1];
    m.m[0][2] = m.m[2][0] = 0.5f * p[2];
    m.m[1][2] = m.m[2][1] = 0.5f * p[4];
    return m;
}

__device__ __forceinline__ Intrin ld_intrin(const float *K /* 3x3 row-major */) {
    Intrin k;
    k.fx = K[0]; k.fy = K[4]; k.cx = K[2]; k.cy = K[5];
    return k;
}

// ---------------------------------------------------------------------------------------
// quats, scales -> covariance (R S)(R S)^T and precision (R S^-1)(R S^-1)^T
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
quat_scale_fwd_kernel(uint32_t N, const float *__restrict__ quats, const float *__restrict__ scales,
                      int triu, float *__restrict__ covars, float *__restrict__ precis) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const float4 q4 = reinterpret_cast<const float4 *>(quats)[i];
    V4 q; q.x = q4.x; q.y = q4.y; q.z = q4.z; q.w = q4.w;
    const V3 s = ld3g(scales + 3 * (size_t)i);
    if (covars != nullptr) {
        const M3 c = quat_scale_to_covar(q, s);
        if (triu) st_triu(covars + 6 * (size_t)i, c); else st_m3(covars + 9 * (size_t)i, c);
    }
    if (precis != nullptr) {
        const M3 p = quat_scale_to_covar(q, v3(1.f / s.x, 1.f / s.y, 1.f / s.z));
        if (triu) st_triu(precis + 6 * (size_t)i, p); else st_m3(precis + 9 * (size_t)i, p);
    }
}

__global__ void __launch_bounds__(kThreads)
quat_scale_bwd_kernel(uint32_t N, const float *__restrict__ quats, const float *__restrict__ scales,
                      const float *__restrict__ v_covars, const float *__restrict__ v_precis, int triu,
                      float *__restrict__ v_quats, float *__restrict__ v_scales) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    const float4 q4 = reinterpret_cast<const float4 *>(quats)[i];
    V4 q; q.x = q4.x; q.y = q4.y; q.z = q4.z; q.w = q4.w;
    const V3 s = ld3g(scales + 3 * (size_t)i);
    const M3 R = quat_to_rotmat(q);
    V4 vq; vq.x = vq.y = vq.z = vq.w = 0.f;
    V3 vs = v3(0.f, 0.f, 0.f);
    if (v_covars != nullptr) {
        const M3 g = triu ? ld_triu_grad(v_covars + 6 * (size_t)i) : ld_m3(v_covars + 9 * (size_t)i);
        quat_scale_to_covar_vjp(q, s, R, g, vq, vs);
    }
    if (v_precis != nullptr) {
        const M3 g = triu ? ld_triu_grad(v_precis + 6 * (size_t)i) : ld_m3(v_precis + 9 * (size_t)i);
        const V3 is = v3(1.f / s.x, 1.f / s.y, 1.f / s.z);
        V3 v_is = v3(0.f, 0.f, 0.f);
        quat_scale_to_covar_vjp(q, is, R, g, vq, v_is);
        vs.x -= v_is.x * is.x * is.x;
        vs.y -= v_is.y * is.y * is.y;
        vs.z -= v_is.z * is.z * is.z;
    }
    reinterpret_cast<float4 *>(v_quats)[i] = make_float4(vq.x, vq.y, vq.z, vq.w);
    st3g(v_scales + 3 * (size_t)i, vs);
}

// ---------------------------------------------------------------------------------------
// world -> sensor frame
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
world_to_cam_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                        const float *__restrict__ covars, const float *__restrict__ viewmats,
                        float *__restrict__ means_c, float *__restrict__ covars_c) {
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    if (n >= N) return;
    const V3 m = ld3g(means + 3 * (size_t)n);
    const M3 cov = ld_m3(covars + 9 * (size_t)n);
    for (uint32_t c = 0; c < C; ++c) {
        const Pose p = load_pose(viewmats + 16 * c);
        const size_t o = (size_t)c * N + n;
        st3g(means_c + 3 * o, mul(p.R, m) + p.t);
        st_m3(covars_c + 9 * o, covar_world_to_cam(p.R, cov));
    }
}

// v_means / v_covars (may be NULL) are written, v_viewmats (may be NULL) is accumulated.
__global__ void __launch_bounds__(kThreads)
world_to_cam_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                        const float *__restrict__ covars, const float *__restrict__ viewmats,
                        const float *__restrict__ v_means_c, const float *__restrict__ v_covars_c,
                        float *__restrict__ v_means, float *__restrict__ v_covars,
                        float *__restrict__ v_viewmats) {
    __shared__ float red[(kThreads / 32) * 12];
    const uint32_t n = blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = n < N;
    const V3 m = live ? ld3g(means + 3 * (size_t)n) : v3(0.f, 0.f, 0.f);
    const M3 cov = live ? ld_m3(covars + 9 * (size_t)n) : m3_zero();
    V3 vm = v3(0.f, 0.f, 0.f);
    M3 vcov = m3_zero();
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t c = 0; c < C; ++c) {
        const Pose p = load_pose(viewmats + 16 * c);
        M3 vR = m3_zero();
        V3 vt = v3(0.f, 0.f, 0.f);
        if (live) {
            const size_t o = (size_t)c * N + n;
            const V3 g = ld3g(v_means_c + 3 * o);
            const M3 G = ld_m3(v_covars_c + 9 * o);
            // mean_c = R m + t
            vR = outer(g, m);
            vt = g;
            const V3 back = mul_t(p.R, g);
            vm = vm + back;
            covar_world_to_cam_vjp(p.R, cov, G, vR, vcov);
        }
        if (v_viewmats != nullptr) {
            const float vals[12] = {vR.m[0][0], vR.m[0][1], vR.m[0][2], vt.x, vR.m[1][0], vR.m[1][1],
                                    vR.m[1][2], vt.y, vR.m[2][0], vR.m[2][1], vR.m[2][2], vt.z};
#pragma unroll
            for (int k = 0; k < 12; ++k) {
                float v = vals[k];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                if (lane == 0) red[warp * 12 + k] = v;
            }
            __syncthreads();
            if (threadIdx.x < 12) {
                float s = 0.f;
#pragma unroll
                for (int w = 0; w < kThreads / 32; ++w) s += red[w * 12 + threadIdx.x];
                if (s != 0.f) atomicAdd(v_viewmats + 16 * c + threadIdx.x, s);   // rows 0..2 of the 4x4
            }
            __syncthreads();
        }
    }
    if (live) {
        if (v_means != nullptr) st3g(v_means + 3 * (size_t)n, vm);
        if (v_covars != nullptr) st_m3(v_covars + 9 * (size_t)n, vcov);
    }
}

// ---------------------------------------------------------------------------------------
// pinhole projection of sensor-frame Gaussians and their pixel velocity
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
persp_proj_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                      const float *__restrict__ covars, const float *__restrict__ Ks, int width, int height,
                      float *__restrict__ means2d, float *__restrict__ covars2d) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const Intrin K = ld_intrin(Ks + 9 * (i / N));
    M2 c2; V2 m2; PerspJ J;
    persp_proj(ld3g(means + 3 * i), ld_m3(covars + 9 * i), K, width, height, c2, m2, J);
    reinterpret_cast<float2 *>(means2d)[i] = make_float2(m2.x, m2.y);
    reinterpret_cast<float4 *>(covars2d)[i] = make_float4(c2.m[0][0], c2.m[0][1], c2.m[1][0], c2.m[1][1]);
}

__global__ void __launch_bounds__(kThreads)
persp_proj_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                      const float *__restrict__ covars, const float *__restrict__ Ks, int width, int height,
                      const float *__restrict__ v_means2d, const float *__restrict__ v_covars2d,
                      float *__restrict__ v_means, float *__restrict__ v_covars) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const Intrin K = ld_intrin(Ks + 9 * (i / N));
    const float2 g2 = reinterpret_cast<const float2 *>(v_means2d)[i];
    const float4 g4 = reinterpret_cast<const float4 *>(v_covars2d)[i];
    M2 G; G.m[0][0] = g4.x; G.m[0][1] = g4.y; G.m[1][0] = g4.z; G.m[1][1] = g4.w;
    V3 vm = v3(0.f, 0.f, 0.f);
    M3 vc = m3_zero();
    persp_proj_vjp(ld3g(means + 3 * i), ld_m3(covars + 9 * i), K, width, height, G, v2(g2.x, g2.y), vm, vc);
    st3g(v_means + 3 * i, vm);
    st_m3(v_covars + 9 * i, vc);
}

__global__ void __launch_bounds__(kThreads)
pix_velocity_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ p_view,
                        const float *__restrict__ lin, const float *__restrict__ ang,
                        const float *__restrict__ velocities, const float *__restrict__ Ks, int width,
                        int height, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const size_t c = i / N;
    const V3 p = ld3g(p_view + 3 * i);
    const PerspJ J = persp_jacobian(p, ld_intrin(Ks + 9 * c), width, height);
    const V2 v = compute_pix_velocity(p, ld3g(lin + 3 * c), ld3g(ang + 3 * c), ld3g(velocities + 3 * i), J);
    reinterpret_cast<float2 *>(out)[i] = make_float2(v.x, v.y);
}

__global__ void __launch_bounds__(kThreads)
pix_velocity_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ p_view,
                        const float *__restrict__ lin, const float *__restrict__ ang,
                        const float *__restrict__ velocities, const float *__restrict__ Ks, int width,
                        int height, const float *__restrict__ v_out, float *__restrict__ v_p_view,
                        float *__restrict__ v_velocities) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const size_t c = i / N;
    const float2 g = reinterpret_cast<const float2 *>(v_out)[i];
    V3 vp = v3(0.f, 0.f, 0.f), vv = v3(0.f, 0.f, 0.f);
    pix_velocity_vjp(ld3g(p_view + 3 * i), ld3g(lin + 3 * c), ld3g(ang + 3 * c), ld3g(velocities + 3 * i),
                     ld_intrin(Ks + 9 * c), width, height, v2(g.x, g.y), vp, vv);
    st3g(v_p_view + 3 * i, vp);
    st3g(v_velocities + 3 * i, vv);
}

// ---------------------------------------------------------------------------------------
// spherical projection of sensor-frame Gaussians and their (azimuth, elevation, range) velocity
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
lidar_proj_fwd_kernel(size_t total, const float *__restrict__ means, const float *__restrict__ covars,
                      float eps2d, float *__restrict__ means2d, float *__restrict__ covars2d,
                      float *__restrict__ depth_comps) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    V2 m2, dc; M2 c2; M3 J;
    lidar_proj(ld3g(means + 3 * i), ld_m3(covars + 9 * i), eps2d, m2, c2, dc, J);
    reinterpret_cast<float2 *>(means2d)[i] = make_float2(m2.x, m2.y);
    reinterpret_cast<float4 *>(covars2d)[i] = make_float4(c2.m[0][0], c2.m[0][1], c2.m[1][0], c2.m[1][1]);
    reinterpret_cast<float2 *>(depth_comps)[i] = make_float2(dc.x, dc.y);
}

__global__ void __launch_bounds__(kThreads)
lidar_proj_bwd_kernel(size_t total, const float *__restrict__ means, const float *__restrict__ covars,
                      float eps2d, const float *__restrict__ v_means2d, const float *__restrict__ v_covars2d,
                      const float *__restrict__ v_depth_comps, float *__restrict__ v_means,
                      float *__restrict__ v_covars) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float2 g2 = reinterpret_cast<const float2 *>(v_means2d)[i];
    const float4 g4 = reinterpret_cast<const float4 *>(v_covars2d)[i];
    const float2 gd = reinterpret_cast<const float2 *>(v_depth_comps)[i];
    M2 G; G.m[0][0] = g4.x; G.m[0][1] = g4.y; G.m[1][0] = g4.z; G.m[1][1] = g4.w;
    V3 vm = v3(0.f, 0.f, 0.f);
    M3 vc = m3_zero();
    lidar_proj_vjp(ld3g(means + 3 * i), ld_m3(covars + 9 * i), eps2d, v2(g2.x, g2.y), G, v2(gd.x, gd.y), vm, vc);
    st3g(v_means + 3 * i, vm);
    st_m3(v_covars + 9 * i, vc);
}

__global__ void __launch_bounds__(kThreads)
lidar_velocity_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ p_view,
                          const float *__restrict__ lin, const float *__restrict__ ang,
                          const float *__restrict__ velocities, float *__restrict__ out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const size_t c = i / N;
    const V3 p = ld3g(p_view + 3 * i);
    st3g(out + 3 * i, compute_lidar_velocity(p, ld3g(lin + 3 * c), ld3g(ang + 3 * c), ld3g(velocities + 3 * i),
                                             lidar_jacobian(p)));
}

__global__ void __launch_bounds__(kThreads)
lidar_velocity_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ p_view,
                          const float *__restrict__ lin, const float *__restrict__ ang,
                          const float *__restrict__ velocities, const float *__restrict__ v_out,
                          float *__restrict__ v_p_view, float *__restrict__ v_velocities) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)C * N) return;
    const size_t c = i / N;
    V3 vp = v3(0.f, 0.f, 0.f), vv = v3(0.f, 0.f, 0.f);
    lidar_velocity_vjp(ld3g(p_view + 3 * i), ld3g(lin + 3 * c), ld3g(ang + 3 * c), ld3g(velocities + 3 * i),
                       ld3g(v_out + 3 * i), vp, vv);
    st3g(v_p_view + 3 * i, vp);
    st3g(v_velocities + 3 * i, vv);
}

static inline uint32_t blocks_for(size_t n) { return (uint32_t)((n + kThreads - 1) / kThreads); }

} // namespace splatad

using namespace splatad;

#define SPL_LAUNCH(name, n, st, ...)                                                              \
    do {                                                                                          \
        SPL_PROF(#name, st);                                                                      \
        name<<<blocks_for(n), kThreads, 0, st>>>(__VA_ARGS__);                                    \
    } while (0)

extern "C" int splatad_quat_scale_to_covar_preci_fwd(uint32_t N, const float *quats, const float *scales,
                                                     int32_t triu, float *covars, float *precis,
                                                     void *stream) {
    if (N == 0) return SPLATAD_OK;
    SPL_REQUIRE(quats && scales && (covars || precis), SPLATAD_ERR_BAD_ARG,
                "quat_scale_to_covar_preci_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(quat_scale_fwd_kernel, N, st, N, quats, scales, triu, covars, precis);
    return check_launch("quat_scale_to_covar_preci_fwd");
}

extern "C" int splatad_quat_scale_to_covar_preci_bwd(uint32_t N, const float *quats, const float *scales,
                                                     const float *v_covars, const float *v_precis,
                                                     int32_t triu, float *v_quats, float *v_scales,
                                                     void *stream) {
    if (N == 0) return SPLATAD_OK;
    SPL_REQUIRE(quats && scales && v_quats && v_scales, SPLATAD_ERR_BAD_ARG,
                "quat_scale_to_covar_preci_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(quat_scale_bwd_kernel, N, st, N, quats, scales, v_covars, v_precis, triu, v_quats, v_scales);
    return check_launch("quat_scale_to_covar_preci_bwd");
}

extern "C" int splatad_world_to_cam_fwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                        const float *viewmats, float *means_c, float *covars_c,
                                        void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && viewmats && means_c && covars_c, SPLATAD_ERR_BAD_ARG,
                "world_to_cam_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(world_to_cam_fwd_kernel, N, st, C, N, means, covars, viewmats, means_c, covars_c);
    return check_launch("world_to_cam_fwd");
}

extern "C" int splatad_world_to_cam_bwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                        const float *viewmats, const float *v_means_c,
                                        const float *v_covars_c, float *v_means, float *v_covars,
                                        float *v_viewmats, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && viewmats && v_means_c && v_covars_c, SPLATAD_ERR_BAD_ARG,
                "world_to_cam_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(world_to_cam_bwd_kernel, N, st, C, N, means, covars, viewmats, v_means_c, v_covars_c, v_means,
               v_covars, v_viewmats);
    return check_launch("world_to_cam_bwd");
}

extern "C" int splatad_persp_proj_fwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                      const float *Ks, uint32_t width, uint32_t height, float *means2d,
                                      float *covars2d, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && Ks && means2d && covars2d, SPLATAD_ERR_BAD_ARG, "persp_proj_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(persp_proj_fwd_kernel, (size_t)C * N, st, C, N, means, covars, Ks, (int)width, (int)height,
               means2d, covars2d);
    return check_launch("persp_proj_fwd");
}

extern "C" int splatad_persp_proj_bwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                      const float *Ks, uint32_t width, uint32_t height,
                                      const float *v_means2d, const float *v_covars2d, float *v_means,
                                      float *v_covars, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && Ks && v_means2d && v_covars2d && v_means && v_covars, SPLATAD_ERR_BAD_ARG,
                "persp_proj_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(persp_proj_bwd_kernel, (size_t)C * N, st, C, N, means, covars, Ks, (int)width, (int)height,
               v_means2d, v_covars2d, v_means, v_covars);
    return check_launch("persp_proj_bwd");
}

extern "C" int splatad_compute_pix_velocity_fwd(uint32_t C, uint32_t N, const float *p_view,
                                                const float *lin_vel, const float *ang_vel,
                                                const float *velocities, const float *Ks, uint32_t width,
                                                uint32_t height, float *pix_vels, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(p_view && lin_vel && ang_vel && velocities && Ks && pix_vels, SPLATAD_ERR_BAD_ARG,
                "compute_pix_velocity_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(pix_velocity_fwd_kernel, (size_t)C * N, st, C, N, p_view, lin_vel, ang_vel, velocities, Ks,
               (int)width, (int)height, pix_vels);
    return check_launch("compute_pix_velocity_fwd");
}

extern "C" int splatad_compute_pix_velocity_bwd(uint32_t C, uint32_t N, const float *p_view,
                                                const float *lin_vel, const float *ang_vel,
                                                const float *velocities, const float *Ks, uint32_t width,
                                                uint32_t height, const float *v_pix_vels, float *v_p_view,
                                                float *v_velocities, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(p_view && lin_vel && ang_vel && velocities && Ks && v_pix_vels && v_p_view && v_velocities,
                SPLATAD_ERR_BAD_ARG, "compute_pix_velocity_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(pix_velocity_bwd_kernel, (size_t)C * N, st, C, N, p_view, lin_vel, ang_vel, velocities, Ks,
               (int)width, (int)height, v_pix_vels, v_p_view, v_velocities);
    return check_launch("compute_pix_velocity_bwd");
}

extern "C" int splatad_lidar_proj_fwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                      float eps2d, float *means2d, float *covars2d,
                                      float *depth_compensations, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && means2d && covars2d && depth_compensations, SPLATAD_ERR_BAD_ARG,
                "lidar_proj_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(lidar_proj_fwd_kernel, (size_t)C * N, st, (size_t)C * N, means, covars, eps2d, means2d, covars2d,
               depth_compensations);
    return check_launch("lidar_proj_fwd");
}

extern "C" int splatad_lidar_proj_bwd(uint32_t C, uint32_t N, const float *means, const float *covars,
                                      float eps2d, const float *v_means2d, const float *v_covars2d,
                                      const float *v_depth_compensations, float *v_means, float *v_covars,
                                      void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(means && covars && v_means2d && v_covars2d && v_depth_compensations && v_means && v_covars,
                SPLATAD_ERR_BAD_ARG, "lidar_proj_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(lidar_proj_bwd_kernel, (size_t)C * N, st, (size_t)C * N, means, covars, eps2d, v_means2d,
               v_covars2d, v_depth_compensations, v_means, v_covars);
    return check_launch("lidar_proj_bwd");
}

extern "C" int splatad_compute_lidar_velocity_fwd(uint32_t C, uint32_t N, const float *p_view,
                                                  const float *lin_vel, const float *ang_vel,
                                                  const float *velocities, float *lidar_vels, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(p_view && lin_vel && ang_vel && velocities && lidar_vels, SPLATAD_ERR_BAD_ARG,
                "compute_lidar_velocity_fwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(lidar_velocity_fwd_kernel, (size_t)C * N, st, C, N, p_view, lin_vel, ang_vel, velocities,
               lidar_vels);
    return check_launch("compute_lidar_velocity_fwd");
}

extern "C" int splatad_compute_lidar_velocity_bwd(uint32_t C, uint32_t N, const float *p_view,
                                                  const float *lin_vel, const float *ang_vel,
                                                  const float *velocities, const float *v_lidar_vels,
                                                  float *v_p_view, float *v_velocities, void *stream) {
    if (N == 0 || C == 0) return SPLATAD_OK;
    SPL_REQUIRE(p_view && lin_vel && ang_vel && velocities && v_lidar_vels && v_p_view && v_velocities,
                SPLATAD_ERR_BAD_ARG, "compute_lidar_velocity_bwd: null argument");
    cudaStream_t st = (cudaStream_t)stream;
    SPL_LAUNCH(lidar_velocity_bwd_kernel, (size_t)C * N, st, C, N, p_view, lin_vel, ang_vel, velocities,
               v_lidar_vels, v_p_view, v_velocities);
    return check_launch("compute_lidar_velocity_bwd");
}
