// Projection of 3-D Gaussians to a pinhole camera image or a spherical lidar range image,
// both with rolling-shutter velocities, forward and backward.
//
// Layout and parallelisation (B200): one thread per Gaussian, looping over the C sensors of
// the call, so the Gaussian's parameters are read from HBM once for all sensors and the
// parameter gradients of the backward pass are accumulated in registers and written with
// plain stores (no atomics for means / quats / scales / covars in the [C, N] layout). The
// 3-wide AoS arrays (means, scales, velocities, conics, lidar velocities) move through
// shared memory so that global traffic is 128-bit.
//
// Behaviour follows the reference kernels
//   camera fwd/bwd   gsplat/cuda/csrc/projection.cu:605-751 / 753-964
//   packed fwd/bwd   gsplat/cuda/csrc/projection.cu:1157-1353 / 1466-1716
//   lidar fwd/bwd    gsplat/cuda/csrc/projection.cu:2268-2417 / 2419-2629
// except that entries of culled (sensor, Gaussian) pairs are written as zeros instead of
// being left uninitialised.
#include "common.cuh"
#include "splat_math.cuh"

namespace splatad {

struct SensorCam {
    Pose pose;
    Intrin K;
    V3 lin, ang;
    float rs_time;
};

struct SensorLidar {
    Pose pose;
    V3 lin, ang;
    float rs_time;
};

__device__ __forceinline__ V3 ld3(const float *p) { return v3(p[0], p[1], p[2]); }

__device__ __forceinline__ SensorCam load_cam(const float *viewmats, const float *Ks,
                                              const float *lin, const float *ang,
                                              const float *rs, uint32_t c) {
    SensorCam s;
    s.pose = load_pose(viewmats + 16 * c);
    const float *K = Ks + 9 * c;
    s.K.fx = K[0]; s.K.fy = K[4]; s.K.cx = K[2]; s.K.cy = K[5];
    s.lin = ld3(lin + 3 * c);
    s.ang = ld3(ang + 3 * c);
    s.rs_time = rs[c];
    return s;
}

__device__ __forceinline__ SensorLidar load_lidar(const float *viewmats, const float *lin,
                                                  const float *ang, const float *rs, uint32_t c) {
    SensorLidar s;
    s.pose = load_pose(viewmats + 16 * c);
    s.lin = ld3(lin + 3 * c);
    s.ang = ld3(ang + 3 * c);
    s.rs_time = rs[c];
    return s;
}

// Symmetric 3x3 (upper triangle). The forward kernels carry covariances in this form: only six
// entries are ever computed, and the congruences A S A^T below produce only the entries their
// callers read.
struct Sym3 { float xx, xy, xz, yy, yz, zz; };

__device__ __forceinline__ Sym3 to_sym(const M3 &m) {
    Sym3 s;
    s.xx = m.m[0][0]; s.xy = m.m[0][1]; s.xz = m.m[0][2];
    s.yy = m.m[1][1]; s.yz = m.m[1][2]; s.zz = m.m[2][2];
    return s;
}

// row^T S for a symmetric S
__device__ __forceinline__ V3 row_times_sym(V3 r, const Sym3 &S) {
    return v3(r.x * S.xx + r.y * S.xy + r.z * S.xz, r.x * S.xy + r.y * S.yy + r.z * S.yz,
              r.x * S.xz + r.y * S.yz + r.z * S.zz);
}

// R S R^T (sensor-frame covariance), upper triangle
__device__ __forceinline__ Sym3 rotate_sym(const M3 &R, const Sym3 &S) {
    const V3 r0 = v3(R.m[0][0], R.m[0][1], R.m[0][2]);
    const V3 r1 = v3(R.m[1][0], R.m[1][1], R.m[1][2]);
    const V3 r2 = v3(R.m[2][0], R.m[2][1], R.m[2][2]);
    const V3 t0 = row_times_sym(r0, S), t1 = row_times_sym(r1, S), t2 = row_times_sym(r2, S);
    Sym3 o;
    o.xx = dot(t0, r0); o.xy = dot(t0, r1); o.xz = dot(t0, r2);
    o.yy = dot(t1, r1); o.yz = dot(t1, r2); o.zz = dot(t2, r2);
    return o;
}

// One reciprocal (two units in the last place) where the result scales an output that is compared
// with a tolerance, never a quantity that decides culling or a tile rectangle.
__device__ __forceinline__ float fast_rcp(float x) { return __fdividef(1.f, x); }

struct CamProj {
    bool valid;
    float ex, ey;   // extents (float, before int truncation)
    V2 mean2d;
    float depth;
    float conic[3];
    float comp;
    V2 pix_vel;
};

// Per-sensor constants of the pinhole projection (the clamp limits of x/z, y/z need 1/fx, 1/fy).
struct CamLimits { float x_pos, x_neg, y_pos, y_neg; };

__device__ __forceinline__ CamLimits cam_limits(const Intrin &K, int width, int height) {
    const float rfx = 1.f / K.fx, rfy = 1.f / K.fy;
    const float tan_fovx = 0.5f * (float)width * rfx, tan_fovy = 0.5f * (float)height * rfy;
    CamLimits l;
    l.x_pos = ((float)width - K.cx) * rfx + 0.3f * tan_fovx;
    l.x_neg = K.cx * rfx + 0.3f * tan_fovx;
    l.y_pos = ((float)height - K.cy) * rfy + 0.3f * tan_fovy;
    l.y_neg = K.cy * rfy + 0.3f * tan_fovy;
    return l;
}

// Forward pinhole projection of one Gaussian. Same steps as persp_proj / add_blur / inverse2 of
// splat_math.cuh (gsplat/cuda/csrc/utils.cuh:190-279, 491-550), written for the forward kernels:
// symmetric covariances, the Jacobian's zeros never multiplied, one reciprocal of the blurred
// determinant shared by the conic and the compensation, one of the depth shared by mean and
// Jacobian. Radii and the culling comparisons keep correctly rounded sqrt / reciprocal.
__device__ __forceinline__ CamProj project_cam(const SensorCam &s, const CamLimits &lim, V3 mean,
                                               const Sym3 &covar, bool has_vel, V3 vel_w, int width,
                                               int height, float eps2d, float near_plane,
                                               float far_plane, float radius_clip) {
    CamProj o;
    o.valid = false;
    o.ex = o.ey = 0.f; o.mean2d = v2(0.f, 0.f); o.depth = 0.f;
    o.conic[0] = o.conic[1] = o.conic[2] = 0.f; o.comp = 0.f; o.pix_vel = v2(0.f, 0.f);

    const V3 p = mul(s.pose.R, mean) + s.pose.t;
    if (p.z < near_plane || p.z > far_plane) return o;
    // everything that needs the sensor's pose and motion first, so that they are dead below
    const bool rolling = s.rs_time > 0.f;
    V3 tv = v3(0.f, 0.f, 0.f);   // velocity of the point relative to the sensor, sensor frame
    if (rolling) {
        tv = s.lin + cross(s.ang, p);
        if (has_vel) tv = tv - mul(s.pose.R, vel_w);
    }
    const Sym3 S = rotate_sym(s.pose.R, covar);
    const float rz = __frcp_rn(p.z);
    const float xr = p.x * rz, yr = p.y * rz;
    const float tx = p.z * fminf(lim.x_pos, fmaxf(-lim.x_neg, xr));
    const float ty = p.z * fminf(lim.y_pos, fmaxf(-lim.y_neg, yr));
    const float rz2 = rz * rz;
    const float j00 = s.K.fx * rz, j11 = s.K.fy * rz;
    const float j02 = -s.K.fx * tx * rz2, j12 = -s.K.fy * ty * rz2;
    // rows of J: [j00 0 j02], [0 j11 j12]
    const float a0 = j00 * S.xx + j02 * S.xz, a1 = j00 * S.xy + j02 * S.yz, a2 = j00 * S.xz + j02 * S.zz;
    const float b1 = j11 * S.yy + j12 * S.yz, b2 = j11 * S.yz + j12 * S.zz;
    const float c00 = a0 * j00 + a2 * j02;
    const float c01 = a1 * j11 + a2 * j12;
    const float c11 = b1 * j11 + b2 * j12;
    const float det_orig = c00 * c11 - c01 * c01;
    const float A = c00 + eps2d, B = c11 + eps2d;
    const float det = A * B - c01 * c01;
    if (!(det > 0.f)) return o;
    float ex = 3.f * sqrtf(A);
    float ey = 3.f * sqrtf(B);
    if (ex <= radius_clip && ey <= radius_clip) return o;
    const V2 m2d = v2(s.K.fx * xr + s.K.cx, s.K.fy * yr + s.K.cy);
    V2 pv = v2(0.f, 0.f);
    if (rolling) {
        pv = v2(-(j00 * tv.x + j02 * tv.z), -(j11 * tv.y + j12 * tv.z));
        ex += fabsf(pv.x) * 0.5f * s.rs_time;
        ey += fabsf(pv.y) * 0.5f * s.rs_time;
    }
    if (m2d.x + ex <= 0.f || m2d.x - ex >= (float)width || m2d.y + ey <= 0.f ||
        m2d.y - ey >= (float)height)
        return o;
    const float inv_det = fast_rcp(det);
    o.valid = true;
    o.ex = ex; o.ey = ey; o.mean2d = m2d; o.depth = p.z;
    o.conic[0] = B * inv_det; o.conic[1] = -c01 * inv_det; o.conic[2] = A * inv_det;
    o.comp = sqrtf(fmaxf(0.f, det_orig * inv_det));
    o.pix_vel = pv;
    return o;
}

struct LidarProj {
    bool valid;
    float ex, ey;
    V2 mean2d;
    float depth;
    float conic[3];
    float comp;
    V3 pix_vel;
    V2 depth_comp;
};

// Forward spherical projection of one Gaussian: the steps of lidar_proj / lidar_jacobian /
// depth_compensation_from_cov3d / add_blur / inverse2 of splat_math.cuh
// (gsplat/cuda/csrc/utils.cuh:12-31, 281-318, 491-550) with the work that only the forward pass
// allows taken out: two reciprocal square roots (1/r, 1/sqrt(x^2 + y^2)) give every quotient of
// the Jacobian; of J Sigma J^T only the 2x2 angular block and the two range-angle entries are
// formed (the range row of J Sigma is never needed: by symmetry both entries are products of the
// angular rows of J Sigma with the range row of J); the blurred determinant's reciprocal is shared
// by the conic, the compensation and the depth compensation. Range, radii and every culling
// comparison keep correctly rounded arithmetic.
__device__ __forceinline__ LidarProj project_lidar(const SensorLidar &s, V3 mean, const Sym3 &covar,
                                                   bool has_vel, V3 vel_w, float min_el,
                                                   float max_el, float min_az, float max_az,
                                                   float eps2d, float near_plane, float far_plane,
                                                   float radius_clip) {
    LidarProj o;
    o.valid = false;
    o.ex = o.ey = 0.f; o.mean2d = v2(0.f, 0.f); o.depth = 0.f;
    o.conic[0] = o.conic[1] = o.conic[2] = 0.f; o.comp = 0.f;
    o.pix_vel = v3(0.f, 0.f, 0.f); o.depth_comp = v2(0.f, 0.f);

    const V3 p = mul(s.pose.R, mean) + s.pose.t;
    const float s2 = p.x * p.x + p.y * p.y;
    const float r2 = s2 + p.z * p.z;
    const float dist = sqrtf(r2);
    if (dist < near_plane || dist > far_plane) return o;
    // everything that needs the sensor's pose and motion first, so that they are dead below
    const bool rolling = s.rs_time > 0.f;
    V3 tv = v3(0.f, 0.f, 0.f);   // velocity of the point relative to the sensor, sensor frame
    if (rolling) {
        tv = s.lin + cross(s.ang, p);
        if (has_vel) tv = tv - mul(s.pose.R, vel_w);
    }
    const Sym3 S = rotate_sym(s.pose.R, covar);
    const float rinv = rsqrtf(r2), sinv = rsqrtf(s2);
    const float inv_s2 = sinv * sinv, inv_r2 = rinv * rinv, sxy = s2 * sinv;
    // rows of J (degrees): azimuth [ja0 ja1 0], elevation [jb0 jb1 jb2], range c = p / r
    const float ka = inv_s2 * kRadToDeg;
    const float ja0 = -p.y * ka, ja1 = p.x * ka;
    const float kb = inv_r2 * sinv * kRadToDeg;
    const float jb0 = -p.x * p.z * kb, jb1 = -p.y * p.z * kb, jb2 = sxy * inv_r2 * kRadToDeg;
    const V3 c = v3(p.x * rinv, p.y * rinv, p.z * rinv);
    const V3 ta = v3(ja0 * S.xx + ja1 * S.xy, ja0 * S.xy + ja1 * S.yy, ja0 * S.xz + ja1 * S.yz);
    const V3 tb = row_times_sym(v3(jb0, jb1, jb2), S);
    const float c00 = ta.x * ja0 + ta.y * ja1;
    const float c01 = ta.x * jb0 + ta.y * jb1 + ta.z * jb2;
    const float c11 = tb.x * jb0 + tb.y * jb1 + tb.z * jb2;
    const float cr0 = dot(ta, c), cr1 = dot(tb, c);   // range-azimuth, range-elevation covariance
    const float det_orig = c00 * c11 - c01 * c01;
    const float A = c00 + eps2d, B = c11 + eps2d;
    const float det = A * B - c01 * c01;
    if (!(det > 0.f)) return o;
    float ex = 3.f * sqrtf(fmaxf(0.f, A));
    float ey = 3.f * sqrtf(fmaxf(0.f, B));
    if (ex <= radius_clip && ey <= radius_clip) return o;
    V3 pv = v3(0.f, 0.f, 0.f);
    if (rolling) {
        pv = v3(-(ja0 * tv.x + ja1 * tv.y), -(jb0 * tv.x + jb1 * tv.y + jb2 * tv.z), -dot(c, tv));
        ex += fabsf(pv.x) * 0.5f * s.rs_time;
        ey += fabsf(pv.y) * 0.5f * s.rs_time;
    }
    const V2 m2d = v2(atan2f(p.y, p.x) * kRadToDeg, asinf(p.z * rinv) * kRadToDeg);
    if (m2d.y + ey <= min_el || m2d.y - ey >= max_el || m2d.x + ex <= min_az || m2d.x - ex >= max_az)
        return o;
    const float inv_det = fast_rcp(det);
    o.valid = true;
    o.ex = ex; o.ey = ey; o.mean2d = m2d; o.depth = dist;
    o.conic[0] = B * inv_det; o.conic[1] = -c01 * inv_det; o.conic[2] = A * inv_det;
    o.comp = sqrtf(fmaxf(0.f, det_orig * inv_det));
    o.pix_vel = pv;
    o.depth_comp = v2((c01 * cr1 - B * cr0) * inv_det, (c01 * cr0 - A * cr1) * inv_det);
    return o;
}

// Shared-memory slab loader for this block's Gaussians. Returns through references.
struct GaussIn {
    V3 mean;
    M3 covar;
    V4 quat;
    V3 scale;
    V3 vel;
};

// Shared-memory staging buffer of the projection kernels: means [256*3] | velocities [256*3] |
// scales [256*3] or covars [256*6]; the same memory is reused for the 3-wide outputs.
constexpr int kStageFloats = kThreads * 12;

// Issues every global->shared copy of this block's slab first and synchronises once, so the
// loads of all arrays are in flight together.
template <bool kNeedQS>
__device__ __forceinline__ GaussIn load_gaussian(const float *__restrict__ means,
                                                 const float *__restrict__ covars,
                                                 const float *__restrict__ quats,
                                                 const float *__restrict__ scales,
                                                 const float *__restrict__ velocities, uint32_t N,
                                                 uint32_t g0, float *smem /* kStageFloats */) {
    GaussIn in;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    in.mean = v3(0.f, 0.f, 1.f); in.scale = v3(1.f, 1.f, 1.f); in.vel = v3(0.f, 0.f, 0.f);
    in.quat.x = 1.f; in.quat.y = in.quat.z = in.quat.w = 0.f;
    float *s_mean = smem, *s_vel = smem + kThreads * 3, *s_cov = smem + kThreads * 6;

    float4 q = make_float4(1.f, 0.f, 0.f, 0.f);
    if (covars == nullptr && live) q = __ldg(reinterpret_cast<const float4 *>(quats) + g0 + t);
    stage_in(means + (size_t)g0 * 3, s_mean, n * 3);
    if (velocities != nullptr) stage_in(velocities + (size_t)g0 * 3, s_vel, n * 3);
    if (covars != nullptr) stage_in(covars + (size_t)g0 * 6, s_cov, n * 6);
    else stage_in(scales + (size_t)g0 * 3, s_cov, n * 3);
    __syncthreads();
    if (live) {
        in.mean = ld3(s_mean + 3 * t);
        if (velocities != nullptr) in.vel = ld3(s_vel + 3 * t);
        if (covars != nullptr) in.covar = covar_from_triu(s_cov + 6 * t);
        else in.scale = ld3(s_cov + 3 * t);
    }
    if (covars == nullptr) {
        in.quat.x = q.x; in.quat.y = q.y; in.quat.z = q.z; in.quat.w = q.w;
        in.covar = quat_scale_to_covar(in.quat, in.scale);
    } else if (!live) {
        in.covar = m3_zero();
    }
    __syncthreads();   // the staging buffer is reused for outputs
    return in;
}

// ---------------------------------------------------------------------------------------
// Lidar forward
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads, 4)
lidar_projection_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                            const float *__restrict__ covars, const float *__restrict__ quats,
                            const float *__restrict__ scales, const float *__restrict__ velocities,
                            const float *__restrict__ viewmats, float min_el, float max_el,
                            float min_az, float max_az, const float *__restrict__ lin_vel,
                            const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                            float eps2d, float near_plane, float far_plane, float radius_clip,
                            float *__restrict__ radii, float *__restrict__ means2d,
                            float *__restrict__ depths, float *__restrict__ conics,
                            float *__restrict__ compensations, float *__restrict__ pix_vels,
                            float *__restrict__ depth_comps) {
    __shared__ __align__(16) float smem[kStageFloats];
    const uint32_t g0 = blockIdx.x * kThreads;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    GaussIn in = load_gaussian<false>(means, covars, quats, scales, velocities, N, g0, smem);
    const Sym3 covar = to_sym(in.covar);

    for (uint32_t c = 0; c < C; ++c) {
        SensorLidar s = load_lidar(viewmats, lin_vel, ang_vel, rs_time, c);
        LidarProj o = project_lidar(s, in.mean, covar, velocities != nullptr, in.vel, min_el,
                                    max_el, min_az, max_az, eps2d, near_plane, far_plane,
                                    radius_clip);
        const size_t base = (size_t)c * N + g0;
        if (live) {
            const size_t i = base + t;
            reinterpret_cast<float2 *>(radii)[i] = make_float2(o.ex, o.ey);
            reinterpret_cast<float2 *>(means2d)[i] = make_float2(o.mean2d.x, o.mean2d.y);
            reinterpret_cast<float2 *>(depth_comps)[i] = make_float2(o.depth_comp.x, o.depth_comp.y);
            depths[i] = o.depth;
            if (compensations != nullptr) compensations[i] = o.comp;
            smem[3 * t + 0] = o.conic[0]; smem[3 * t + 1] = o.conic[1]; smem[3 * t + 2] = o.conic[2];
            smem[kThreads * 3 + 3 * t + 0] = o.pix_vel.x;
            smem[kThreads * 3 + 3 * t + 1] = o.pix_vel.y;
            smem[kThreads * 3 + 3 * t + 2] = o.pix_vel.z;
        }
        __syncthreads();
        stage_out(conics + base * 3, smem, n * 3);
        stage_out(pix_vels + base * 3, smem + kThreads * 3, n * 3);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// Lidar forward, pipelined: a persistent grid (four CTAs per SM) walks the full slabs of 256
// Gaussians; while a CTA computes on one slab, the bulk-copy engine fetches its next one (means,
// quats, scales, velocities: four one-dimensional bulk copies completing on an mbarrier) into the
// other half of a double buffer. The profile of the one-slab-per-CTA kernel showed its largest
// stalls at the slab loads and the barriers around them. Same arithmetic, same outputs; a ragged
// last slab is one more round filled with plain loads (a second launch for it cost as much as a
// fifth of the whole projection). Inputs that are not 16-byte aligned, covariance inputs and scenes
// of fewer than 256 Gaussians go through that kernel.
// ---------------------------------------------------------------------------------------
struct __align__(128) ProjSlab {
    float mean[kThreads * 3];
    float quat[kThreads * 4];
    float scale[kThreads * 3];
    float vel[kThreads * 3];
};

static __device__ unsigned long long g_async_copy_timeouts = 0ull;

__global__ void __launch_bounds__(kThreads, 4)
lidar_projection_fwd_pipelined_kernel(uint32_t C, uint32_t N, uint32_t n_slabs, const float *__restrict__ means,
                                      const float *__restrict__ quats, const float *__restrict__ scales,
                                      const float *__restrict__ velocities, const float *__restrict__ viewmats,
                                      float min_el, float max_el, float min_az, float max_az,
                                      const float *__restrict__ lin_vel, const float *__restrict__ ang_vel,
                                      const float *__restrict__ rs_time, float eps2d, float near_plane,
                                      float far_plane, float radius_clip, float *__restrict__ radii,
                                      float *__restrict__ means2d, float *__restrict__ depths,
                                      float *__restrict__ conics, float *__restrict__ compensations,
                                      float *__restrict__ pix_vels, float *__restrict__ depth_comps) {
    __shared__ ProjSlab slab[2];
    __shared__ __align__(16) float s_out[kThreads * 6];
    __shared__ __align__(8) unsigned long long bar[2];
    const uint32_t t = threadIdx.x;
    const bool has_vel = velocities != nullptr;
    const uint32_t slab_bytes = (uint32_t)sizeof(float) * kThreads * (has_vel ? 13u : 10u);
    if (t == 0) {
        mbar_init(&bar[0], 1);
        mbar_init(&bar[1], 1);
        mbar_init_fence();
    }
    __syncthreads();

    auto fetch = [&](uint32_t s, uint32_t b) {   // thread 0: slab s into buffer b
        mbar_arrive_expect_tx(&bar[b], slab_bytes);
        bulk_copy_g2s(slab[b].mean, means + (size_t)s * kThreads * 3, sizeof(float) * kThreads * 3, &bar[b]);
        bulk_copy_g2s(slab[b].quat, quats + (size_t)s * kThreads * 4, sizeof(float) * kThreads * 4, &bar[b]);
        bulk_copy_g2s(slab[b].scale, scales + (size_t)s * kThreads * 3, sizeof(float) * kThreads * 3, &bar[b]);
        if (has_vel)
            bulk_copy_g2s(slab[b].vel, velocities + (size_t)s * kThreads * 3, sizeof(float) * kThreads * 3, &bar[b]);
    };

    // n_slabs counts the full slabs; a ragged last slab (N not a multiple of 256) is one more round
    // for the CTA whose turn it is, filled with plain loads
    const uint32_t n_rounds = n_slabs + ((uint64_t)n_slabs * kThreads < N ? 1u : 0u);
    uint32_t parity[2] = {0u, 0u};
    uint32_t b = 0;
    if (t == 0 && blockIdx.x < n_slabs) fetch(blockIdx.x, 0);
    for (uint32_t s = blockIdx.x; s < n_rounds; s += gridDim.x, b ^= 1u) {
        const uint32_t next = s + gridDim.x;
        const uint32_t n = min((uint32_t)kThreads, N - s * kThreads);
        const bool live = t < n;
        // buffer b ^ 1 was read in the previous round, which ended with a barrier
        if (t == 0 && next < n_slabs) fetch(next, b ^ 1u);
        if (s < n_slabs) {
            const bool arrived = mbar_wait_bounded(&bar[b], parity[b]);
            if (!__syncthreads_and(arrived)) {
                // a copy did not complete within the limit: count it, give the copies in flight one more
                // bounded chance to land (their target is this CTA's shared memory), and leave
                if (t == 0) atomicAdd(&g_async_copy_timeouts, 1ull);
                mbar_wait_bounded(&bar[b], parity[b]);
                if (next < n_slabs) mbar_wait_bounded(&bar[b ^ 1u], parity[b ^ 1u]);
                return;
            }
            parity[b] ^= 1u;
        } else {
            // no copy was issued into this buffer for the ragged slab
            const size_t g = (size_t)s * kThreads;
            for (uint32_t i = t; i < n * 3; i += kThreads) {
                slab[b].mean[i] = means[g * 3 + i];
                slab[b].scale[i] = scales[g * 3 + i];
                if (has_vel) slab[b].vel[i] = velocities[g * 3 + i];
            }
            for (uint32_t i = t; i < n * 4; i += kThreads) slab[b].quat[i] = quats[g * 4 + i];
            __syncthreads();
        }
        const ProjSlab &in = slab[b];
        // threads beyond a ragged slab's end compute on whatever the buffer holds and store nothing
        const V3 mean = ld3(in.mean + 3 * t);
        const V3 scale = ld3(in.scale + 3 * t);
        const float4 q = reinterpret_cast<const float4 *>(in.quat)[t];
        const V3 vel = has_vel ? ld3(in.vel + 3 * t) : v3(0.f, 0.f, 0.f);
        __syncthreads();   // every thread has its inputs: the buffer may be refilled next round
        V4 quat;
        quat.x = q.x; quat.y = q.y; quat.z = q.z; quat.w = q.w;
        const Sym3 covar = to_sym(quat_scale_to_covar(quat, scale));
        const uint32_t g0 = s * kThreads;
        for (uint32_t c = 0; c < C; ++c) {
            SensorLidar sen = load_lidar(viewmats, lin_vel, ang_vel, rs_time, c);
            LidarProj o = project_lidar(sen, mean, covar, has_vel, vel, min_el, max_el, min_az, max_az, eps2d,
                                        near_plane, far_plane, radius_clip);
            const size_t base = (size_t)c * N + g0;
            const size_t i = base + t;
            if (live) {
                reinterpret_cast<float2 *>(radii)[i] = make_float2(o.ex, o.ey);
                reinterpret_cast<float2 *>(means2d)[i] = make_float2(o.mean2d.x, o.mean2d.y);
                reinterpret_cast<float2 *>(depth_comps)[i] = make_float2(o.depth_comp.x, o.depth_comp.y);
                depths[i] = o.depth;
                if (compensations != nullptr) compensations[i] = o.comp;
            }
            s_out[3 * t + 0] = o.conic[0]; s_out[3 * t + 1] = o.conic[1]; s_out[3 * t + 2] = o.conic[2];
            s_out[kThreads * 3 + 3 * t + 0] = o.pix_vel.x;
            s_out[kThreads * 3 + 3 * t + 1] = o.pix_vel.y;
            s_out[kThreads * 3 + 3 * t + 2] = o.pix_vel.z;
            __syncthreads();
            stage_out(conics + base * 3, s_out, n * 3);
            stage_out(pix_vels + base * 3, s_out + kThreads * 3, n * 3);
            __syncthreads();
        }
    }
}

// ---------------------------------------------------------------------------------------
// Camera forward, [C, N] layout
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
projection_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                      const float *__restrict__ covars, const float *__restrict__ quats,
                      const float *__restrict__ scales, const float *__restrict__ velocities,
                      const float *__restrict__ viewmats, const float *__restrict__ Ks, int width,
                      int height, const float *__restrict__ lin_vel,
                      const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                      float eps2d, float near_plane, float far_plane, float radius_clip,
                      int32_t *__restrict__ radii, float *__restrict__ means2d,
                      float *__restrict__ depths, float *__restrict__ conics,
                      float *__restrict__ compensations, float *__restrict__ pix_vels) {
    __shared__ __align__(16) float smem[kStageFloats];
    const uint32_t g0 = blockIdx.x * kThreads;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    GaussIn in = load_gaussian<false>(means, covars, quats, scales, velocities, N, g0, smem);
    const Sym3 covar = to_sym(in.covar);

    for (uint32_t c = 0; c < C; ++c) {
        SensorCam s = load_cam(viewmats, Ks, lin_vel, ang_vel, rs_time, c);
        CamProj o = project_cam(s, cam_limits(s.K, width, height), in.mean, covar, velocities != nullptr, in.vel,
                                width, height, eps2d, near_plane, far_plane, radius_clip);
        const size_t base = (size_t)c * N + g0;
        if (live) {
            const size_t i = base + t;
            int2 r = make_int2((int32_t)o.ex, (int32_t)o.ey);
            reinterpret_cast<int2 *>(radii)[i] = r;
            reinterpret_cast<float2 *>(means2d)[i] = make_float2(o.mean2d.x, o.mean2d.y);
            reinterpret_cast<float2 *>(pix_vels)[i] = make_float2(o.pix_vel.x, o.pix_vel.y);
            depths[i] = o.depth;
            if (compensations != nullptr) compensations[i] = o.comp;
            smem[3 * t + 0] = o.conic[0]; smem[3 * t + 1] = o.conic[1]; smem[3 * t + 2] = o.conic[2];
        }
        __syncthreads();
        stage_out(conics + base * 3, smem, n * 3);
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------
// Camera forward, packed (COO) layout: rows ordered camera-major, Gaussian-minor.
// Pass 1 (block_counts != nullptr) counts the visible Gaussians of each (camera, block);
// pass 2 (block_offsets != nullptr) recomputes and writes rows at the scanned offsets.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
projection_packed_fwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                             const float *__restrict__ covars, const float *__restrict__ quats,
                             const float *__restrict__ scales, const float *__restrict__ velocities,
                             const float *__restrict__ viewmats, const float *__restrict__ Ks,
                             int width, int height, const float *__restrict__ lin_vel,
                             const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                             float eps2d, float near_plane, float far_plane, float radius_clip,
                             int32_t *__restrict__ block_counts,        // [C, nblocks] pass 1
                             const int32_t *__restrict__ block_offsets, // [C, nblocks] pass 2 (exclusive)
                             int64_t capacity /* rows the outputs hold; < 0: as many as needed */,
                             const int32_t *__restrict__ counts_ro /* pass 2, capacity >= 0: pass 1's counts */,
                             int64_t *__restrict__ camera_ids, int64_t *__restrict__ gaussian_ids,
                             int32_t *__restrict__ radii, float *__restrict__ means2d,
                             float *__restrict__ depths, float *__restrict__ conics,
                             float *__restrict__ compensations, float *__restrict__ pix_vels) {
    __shared__ __align__(16) float smem[kStageFloats];
    __shared__ int32_t warp_counts[kThreads / 32];
    const uint32_t g0 = blockIdx.x * kThreads;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    const uint32_t lane = t & 31, warp = t >> 5;
    GaussIn in = load_gaussian<false>(means, covars, quats, scales, velocities, N, g0, smem);
    const Sym3 covar = to_sym(in.covar);

    for (uint32_t c = 0; c < C; ++c) {
        SensorCam s = load_cam(viewmats, Ks, lin_vel, ang_vel, rs_time, c);
        CamProj o = project_cam(s, cam_limits(s.K, width, height), in.mean, covar, velocities != nullptr, in.vel,
                                width, height, eps2d, near_plane, far_plane, radius_clip);
        const bool vis = live && o.valid;
        const uint32_t ballot = __ballot_sync(0xffffffffu, vis);
        if (lane == 0) warp_counts[warp] = __popc(ballot);
        __syncthreads();
        int32_t before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < kThreads / 32; ++w) {
            const int32_t cw = warp_counts[w];
            if (w < (int)warp) before += cw;
            total += cw;
        }
        __syncthreads();
        if (block_counts != nullptr) {
            if (t == 0) block_counts[(size_t)c * gridDim.x + blockIdx.x] = total;
            continue;
        }
        if (vis) {
            const int64_t row = (int64_t)block_offsets[(size_t)c * gridDim.x + blockIdx.x] + before +
                                __popc(ballot & ((1u << lane) - 1u));
            if (capacity >= 0 && row >= capacity) continue;   // the caller sees nnz > capacity and refills
            camera_ids[row] = (int64_t)c;
            gaussian_ids[row] = (int64_t)(g0 + t);
            radii[2 * row] = (int32_t)o.ex;
            radii[2 * row + 1] = (int32_t)o.ey;
            means2d[2 * row] = o.mean2d.x;
            means2d[2 * row + 1] = o.mean2d.y;
            depths[row] = o.depth;
            conics[3 * row] = o.conic[0];
            conics[3 * row + 1] = o.conic[1];
            conics[3 * row + 2] = o.conic[2];
            pix_vels[2 * row] = o.pix_vel.x;
            pix_vels[2 * row + 1] = o.pix_vel.y;
            if (compensations != nullptr) compensations[row] = o.comp;
        }
    }
    // Outputs with room to spare (written before the host knows the row count): the rows behind the
    // last packed one get ids 0 and radii 0, which every consumer skips.
    if (block_counts == nullptr && capacity >= 0 && counts_ro != nullptr) {
        const size_t last = (size_t)C * gridDim.x - 1;
        const int64_t nnz = (int64_t)block_offsets[last] + counts_ro[last];
        for (int64_t r = nnz + (int64_t)blockIdx.x * kThreads + t; r < capacity; r += (int64_t)gridDim.x * kThreads) {
            camera_ids[r] = 0;
            gaussian_ids[r] = 0;
            radii[2 * r] = 0;
            radii[2 * r + 1] = 0;
        }
    }
}

// Exclusive scan of the [C * nblocks] block counts (single block), total -> *nnz and
// indptr[c] = offset of camera c's first row, indptr[C] = nnz.
__global__ void __launch_bounds__(1024)
packed_scan_kernel(const int32_t *__restrict__ counts, int32_t *__restrict__ offsets, uint32_t C,
                   uint32_t nblocks, int32_t *__restrict__ indptr, int64_t *__restrict__ nnz_out) {
    __shared__ int32_t part[1024];
    const uint32_t total = C * nblocks;
    const uint32_t t = threadIdx.x;
    const uint32_t per = (total + 1023) / 1024;
    const uint32_t lo = min(t * per, total), hi = min(lo + per, total);
    int32_t s = 0;
    for (uint32_t i = lo; i < hi; ++i) s += counts[i];
    part[t] = s;
    __syncthreads();
    // Hillis-Steele inclusive scan over 1024 partials
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
        *nnz_out = (int64_t)part[1023];
    }
}

// ---------------------------------------------------------------------------------------
// Backward helpers
// ---------------------------------------------------------------------------------------
struct ParamGrads {
    V3 v_mean;
    M3 v_covar;   // full 3x3 gradient of the world covariance
};

// Block-level reduction of 12 floats (v_R 9 + v_t 3) followed by one atomicAdd set per block.
__device__ __forceinline__ void block_reduce_viewmat(const M3 &v_R, V3 v_t, float *v_viewmat,
                                                     float *red /* [kThreads/32][12] */) {
    float vals[12] = {v_R.m[0][0], v_R.m[0][1], v_R.m[0][2], v_t.x,
                      v_R.m[1][0], v_R.m[1][1], v_R.m[1][2], v_t.y,
                      v_R.m[2][0], v_R.m[2][1], v_R.m[2][2], v_t.z};
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
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
        if (s != 0.f) atomicAdd(v_viewmat + threadIdx.x, s);   // rows 0..2 of the 4x4
    }
    __syncthreads();
}

// Camera backward for one (sensor, Gaussian) pair. Returns the world-space mean gradient and
// covariance gradient, accumulates v_R / v_t.
__device__ __forceinline__ void cam_pair_bwd(const SensorCam &s, const GaussIn &in, bool has_vel,
                                             int width, int height, float eps2d,
                                             const float *conic3, float comp, bool has_comp,
                                             V2 v_mean2d, float v_depth, const float *v_conic3,
                                             float v_comp, V2 v_pix_vel, V3 &v_mean, M3 &v_covar,
                                             M3 &v_R, V3 &v_t, V3 &v_vel_w) {
    M2 cinv;
    cinv.m[0][0] = conic3[0]; cinv.m[0][1] = conic3[1]; cinv.m[1][0] = conic3[1]; cinv.m[1][1] = conic3[2];
    M2 v_cinv;
    v_cinv.m[0][0] = v_conic3[0]; v_cinv.m[0][1] = v_conic3[1] * 0.5f;
    v_cinv.m[1][0] = v_conic3[1] * 0.5f; v_cinv.m[1][1] = v_conic3[2];
    M2 v_cov2d = m2_zero();
    inverse2_vjp(cinv, v_cinv, v_cov2d);
    if (has_comp) add_blur_vjp(eps2d, cinv, comp, v_comp, v_cov2d);

    V3 p = mul(s.pose.R, in.mean) + s.pose.t;
    M3 covar_c = covar_world_to_cam(s.pose.R, in.covar);

    V3 v_p = v3(0.f, 0.f, 0.f);
    if (s.rs_time > 0.f) {
        V3 vel_c = has_vel ? mul(s.pose.R, in.vel) : v3(0.f, 0.f, 0.f);
        V3 v_vel_c = v3(0.f, 0.f, 0.f);
        pix_velocity_vjp(p, s.lin, s.ang, vel_c, s.K, width, height, v_pix_vel, v_p, v_vel_c);
        if (has_vel) {
            v_R = add(v_R, outer(v_vel_c, in.vel));
            v_vel_w = v_vel_w + mul_t(s.pose.R, v_vel_c);
        }
    }
    M3 v_covar_c = m3_zero();
    persp_proj_vjp(p, covar_c, s.K, width, height, v_cov2d, v_mean2d, v_p, v_covar_c);
    v_p.z += v_depth;
    // p = R mean + t
    v_R = add(v_R, outer(v_p, in.mean));
    v_t = v_t + v_p;
    v_mean = v_mean + mul_t(s.pose.R, v_p);
    covar_world_to_cam_vjp(s.pose.R, in.covar, v_covar_c, v_R, v_covar);
}

__device__ __forceinline__ void lidar_pair_bwd(const SensorLidar &s, const GaussIn &in,
                                               bool has_vel, float eps2d, const float *conic3,
                                               float comp, bool has_comp, V2 v_mean2d,
                                               float v_depth, const float *v_conic3, float v_comp,
                                               V3 v_pix_vel, V2 v_depth_comp, V3 &v_mean,
                                               M3 &v_covar, M3 &v_R, V3 &v_t, V3 &v_vel_w) {
    M2 cinv;
    cinv.m[0][0] = conic3[0]; cinv.m[0][1] = conic3[1]; cinv.m[1][0] = conic3[1]; cinv.m[1][1] = conic3[2];
    M2 v_cinv;
    v_cinv.m[0][0] = v_conic3[0]; v_cinv.m[0][1] = v_conic3[1] * 0.5f;
    v_cinv.m[1][0] = v_conic3[1] * 0.5f; v_cinv.m[1][1] = v_conic3[2];
    M2 v_cov2d = m2_zero();
    inverse2_vjp(cinv, v_cinv, v_cov2d);
    if (has_comp) add_blur_vjp(eps2d, cinv, comp, v_comp, v_cov2d);

    V3 p = mul(s.pose.R, in.mean) + s.pose.t;
    M3 covar_c = covar_world_to_cam(s.pose.R, in.covar);

    V3 v_p = v3(0.f, 0.f, 0.f);
    if (s.rs_time > 0.f) {
        V3 vel_c = has_vel ? mul(s.pose.R, in.vel) : v3(0.f, 0.f, 0.f);
        V3 v_vel_c = v3(0.f, 0.f, 0.f);
        lidar_velocity_vjp(p, s.lin, s.ang, vel_c, v_pix_vel, v_p, v_vel_c);
        if (has_vel) {
            v_R = add(v_R, outer(v_vel_c, in.vel));
            v_vel_w = v_vel_w + mul_t(s.pose.R, v_vel_c);
        }
    }
    M3 v_covar_c = m3_zero();
    lidar_proj_vjp(p, covar_c, eps2d, v_mean2d, v_cov2d, v_depth_comp, v_p, v_covar_c);
    const float rinv = spl_rnorm3(p.x, p.y, p.z);
    v_p.x += p.x * rinv * v_depth;
    v_p.y += p.y * rinv * v_depth;
    v_p.z += p.z * rinv * v_depth;
    v_R = add(v_R, outer(v_p, in.mean));
    v_t = v_t + v_p;
    v_mean = v_mean + mul_t(s.pose.R, v_p);
    covar_world_to_cam_vjp(s.pose.R, in.covar, v_covar_c, v_R, v_covar);
}

__device__ __forceinline__ void covar_grad_to_triu(const M3 &g, float *o) {
    o[0] = g.m[0][0];
    o[1] = g.m[0][1] + g.m[1][0];
    o[2] = g.m[0][2] + g.m[2][0];
    o[3] = g.m[1][1];
    o[4] = g.m[1][2] + g.m[2][1];
    o[5] = g.m[2][2];
}

// Writes the per-Gaussian parameter gradients of this block (means, and covars or
// quats+scales, optionally velocities) through shared memory.
__device__ __forceinline__ void store_param_grads(const GaussIn &in, bool use_covars, V3 v_mean,
                                                  const M3 &v_covar, V3 v_vel_w, uint32_t g0,
                                                  uint32_t n, float *smem, float *v_means,
                                                  float *v_covars, float *v_quats, float *v_scales,
                                                  float *v_velocities) {
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    if (v_means != nullptr) {
        if (live) { smem[3 * t] = v_mean.x; smem[3 * t + 1] = v_mean.y; smem[3 * t + 2] = v_mean.z; }
        __syncthreads();
        stage_out(v_means + (size_t)g0 * 3, smem, n * 3);
        __syncthreads();
    }
    if (v_velocities != nullptr) {
        if (live) { smem[3 * t] = v_vel_w.x; smem[3 * t + 1] = v_vel_w.y; smem[3 * t + 2] = v_vel_w.z; }
        __syncthreads();
        stage_out(v_velocities + (size_t)g0 * 3, smem, n * 3);
        __syncthreads();
    }
    if (use_covars) {
        if (v_covars != nullptr) {
            if (live) covar_grad_to_triu(v_covar, smem + 6 * t);
            __syncthreads();
            stage_out(v_covars + (size_t)g0 * 6, smem, n * 6);
            __syncthreads();
        }
    } else {
        V4 v_quat; v_quat.x = v_quat.y = v_quat.z = v_quat.w = 0.f;
        V3 v_scale = v3(0.f, 0.f, 0.f);
        M3 R = quat_to_rotmat(in.quat);
        quat_scale_to_covar_vjp(in.quat, in.scale, R, v_covar, v_quat, v_scale);
        if (v_quats != nullptr && live)
            reinterpret_cast<float4 *>(v_quats)[g0 + t] = make_float4(v_quat.x, v_quat.y, v_quat.z, v_quat.w);
        if (v_scales != nullptr) {
            if (live) { smem[3 * t] = v_scale.x; smem[3 * t + 1] = v_scale.y; smem[3 * t + 2] = v_scale.z; }
            __syncthreads();
            stage_out(v_scales + (size_t)g0 * 3, smem, n * 3);
            __syncthreads();
        }
    }
}

// ---------------------------------------------------------------------------------------
// Camera backward, [C, N] layout
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
projection_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                      const float *__restrict__ covars, const float *__restrict__ quats,
                      const float *__restrict__ scales, const float *__restrict__ velocities,
                      const float *__restrict__ viewmats, const float *__restrict__ Ks, int width,
                      int height, const float *__restrict__ lin_vel,
                      const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                      float eps2d, const int32_t *__restrict__ radii,
                      const float *__restrict__ conics, const float *__restrict__ compensations,
                      const float *__restrict__ v_means2d, const float *__restrict__ v_depths,
                      const float *__restrict__ v_conics, const float *__restrict__ v_compensations,
                      const float *__restrict__ v_pix_vels, float *__restrict__ v_means,
                      float *__restrict__ v_covars, float *__restrict__ v_quats,
                      float *__restrict__ v_scales, float *__restrict__ v_viewmats,
                      float *__restrict__ v_velocities) {
    __shared__ __align__(16) float smem[kStageFloats];
    __shared__ float red[(kThreads / 32) * 12];
    const uint32_t g0 = blockIdx.x * kThreads;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    GaussIn in = load_gaussian<true>(means, covars, quats, scales, velocities, N, g0, smem);

    V3 v_mean = v3(0.f, 0.f, 0.f), v_vel_w = v3(0.f, 0.f, 0.f);
    M3 v_covar = m3_zero();
    for (uint32_t c = 0; c < C; ++c) {
        SensorCam s = load_cam(viewmats, Ks, lin_vel, ang_vel, rs_time, c);
        const size_t i = (size_t)c * N + g0 + t;
        M3 v_R = m3_zero();
        V3 v_t = v3(0.f, 0.f, 0.f);
        if (live && radii[2 * i] > 0) {
            const float cn[3] = {conics[3 * i], conics[3 * i + 1], conics[3 * i + 2]};
            const float vcn[3] = {v_conics[3 * i], v_conics[3 * i + 1], v_conics[3 * i + 2]};
            const bool has_comp = v_compensations != nullptr;
            cam_pair_bwd(s, in, velocities != nullptr, width, height, eps2d, cn,
                         has_comp ? compensations[i] : 0.f, has_comp,
                         v2(v_means2d[2 * i], v_means2d[2 * i + 1]), v_depths[i], vcn,
                         has_comp ? v_compensations[i] : 0.f,
                         v2(v_pix_vels[2 * i], v_pix_vels[2 * i + 1]), v_mean, v_covar, v_R, v_t,
                         v_vel_w);
        }
        if (v_viewmats != nullptr) block_reduce_viewmat(v_R, v_t, v_viewmats + 16 * c, red);
    }
    store_param_grads(in, covars != nullptr, v_mean, v_covar, v_vel_w, g0, n, smem, v_means,
                      v_covars, v_quats, v_scales, v_velocities);
}

// ---------------------------------------------------------------------------------------
// Lidar backward, [C, N] layout
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
lidar_projection_bwd_kernel(uint32_t C, uint32_t N, const float *__restrict__ means,
                            const float *__restrict__ covars, const float *__restrict__ quats,
                            const float *__restrict__ scales, const float *__restrict__ velocities,
                            const float *__restrict__ viewmats, const float *__restrict__ lin_vel,
                            const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                            float eps2d, const float *__restrict__ radii,
                            const float *__restrict__ conics,
                            const float *__restrict__ compensations,
                            const float *__restrict__ v_means2d, const float *__restrict__ v_depths,
                            const float *__restrict__ v_conics,
                            const float *__restrict__ v_compensations,
                            const float *__restrict__ v_pix_vels,
                            const float *__restrict__ v_depth_comps, float *__restrict__ v_means,
                            float *__restrict__ v_covars, float *__restrict__ v_quats,
                            float *__restrict__ v_scales, float *__restrict__ v_viewmats,
                            float *__restrict__ v_velocities) {
    __shared__ __align__(16) float smem[kStageFloats];
    __shared__ float red[(kThreads / 32) * 12];
    const uint32_t g0 = blockIdx.x * kThreads;
    const uint32_t n = min((uint32_t)kThreads, N - g0);
    const uint32_t t = threadIdx.x;
    const bool live = t < n;
    GaussIn in = load_gaussian<true>(means, covars, quats, scales, velocities, N, g0, smem);

    V3 v_mean = v3(0.f, 0.f, 0.f), v_vel_w = v3(0.f, 0.f, 0.f);
    M3 v_covar = m3_zero();
    for (uint32_t c = 0; c < C; ++c) {
        SensorLidar s = load_lidar(viewmats, lin_vel, ang_vel, rs_time, c);
        const size_t i = (size_t)c * N + g0 + t;
        M3 v_R = m3_zero();
        V3 v_t = v3(0.f, 0.f, 0.f);
        if (live && radii[2 * i] > 0.f) {
            const float cn[3] = {conics[3 * i], conics[3 * i + 1], conics[3 * i + 2]};
            const float vcn[3] = {v_conics[3 * i], v_conics[3 * i + 1], v_conics[3 * i + 2]};
            const bool has_comp = v_compensations != nullptr;
            lidar_pair_bwd(s, in, velocities != nullptr, eps2d, cn,
                           has_comp ? compensations[i] : 0.f, has_comp,
                           v2(v_means2d[2 * i], v_means2d[2 * i + 1]), v_depths[i], vcn,
                           has_comp ? v_compensations[i] : 0.f,
                           v3(v_pix_vels[3 * i], v_pix_vels[3 * i + 1], v_pix_vels[3 * i + 2]),
                           v2(v_depth_comps[2 * i], v_depth_comps[2 * i + 1]), v_mean, v_covar,
                           v_R, v_t, v_vel_w);
        }
        if (v_viewmats != nullptr) block_reduce_viewmat(v_R, v_t, v_viewmats + 16 * c, red);
    }
    store_param_grads(in, covars != nullptr, v_mean, v_covar, v_vel_w, g0, n, smem, v_means,
                      v_covars, v_quats, v_scales, v_velocities);
}

// ---------------------------------------------------------------------------------------
// Camera backward, packed layout: one thread per packed row. Rows of one Gaussian (one per
// camera that sees it) are far apart, so parameter gradients use atomics (dense outputs) or
// are written per row (sparse_grad).
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
projection_packed_bwd_kernel(uint32_t C, uint32_t N, uint32_t nnz, const float *__restrict__ means,
                             const float *__restrict__ covars, const float *__restrict__ quats,
                             const float *__restrict__ scales, const float *__restrict__ velocities,
                             const float *__restrict__ viewmats, const float *__restrict__ Ks,
                             int width, int height, const float *__restrict__ lin_vel,
                             const float *__restrict__ ang_vel, const float *__restrict__ rs_time,
                             float eps2d, const int64_t *__restrict__ camera_ids,
                             const int64_t *__restrict__ gaussian_ids,
                             const float *__restrict__ conics,
                             const float *__restrict__ compensations,
                             const float *__restrict__ v_means2d, const float *__restrict__ v_depths,
                             const float *__restrict__ v_conics,
                             const float *__restrict__ v_compensations,
                             const float *__restrict__ v_pix_vels, int sparse_grad,
                             float *__restrict__ v_means, float *__restrict__ v_covars,
                             float *__restrict__ v_quats, float *__restrict__ v_scales,
                             float *__restrict__ v_viewmats, float *__restrict__ v_velocities) {
    const uint32_t idx = blockIdx.x * kThreads + threadIdx.x;
    if (idx >= nnz) return;
    const uint32_t c = (uint32_t)camera_ids[idx];
    const uint32_t g = (uint32_t)gaussian_ids[idx];
    GaussIn in;
    in.mean = ld3(means + 3 * (size_t)g);
    in.vel = velocities != nullptr ? ld3(velocities + 3 * (size_t)g) : v3(0.f, 0.f, 0.f);
    if (covars != nullptr) {
        in.covar = covar_from_triu(covars + 6 * (size_t)g);
    } else {
        const float4 q = __ldg(reinterpret_cast<const float4 *>(quats) + g);
        in.quat.x = q.x; in.quat.y = q.y; in.quat.z = q.z; in.quat.w = q.w;
        in.scale = ld3(scales + 3 * (size_t)g);
        in.covar = quat_scale_to_covar(in.quat, in.scale);
    }
    SensorCam s = load_cam(viewmats, Ks, lin_vel, ang_vel, rs_time, c);
    const size_t i = idx;
    const float cn[3] = {conics[3 * i], conics[3 * i + 1], conics[3 * i + 2]};
    const float vcn[3] = {v_conics[3 * i], v_conics[3 * i + 1], v_conics[3 * i + 2]};
    const bool has_comp = v_compensations != nullptr;
    V3 v_mean = v3(0.f, 0.f, 0.f), v_vel_w = v3(0.f, 0.f, 0.f), v_t = v3(0.f, 0.f, 0.f);
    M3 v_covar = m3_zero(), v_R = m3_zero();
    cam_pair_bwd(s, in, velocities != nullptr, width, height, eps2d, cn,
                 has_comp ? compensations[i] : 0.f, has_comp,
                 v2(v_means2d[2 * i], v_means2d[2 * i + 1]), v_depths[i], vcn,
                 has_comp ? v_compensations[i] : 0.f, v2(v_pix_vels[2 * i], v_pix_vels[2 * i + 1]),
                 v_mean, v_covar, v_R, v_t, v_vel_w);

    const size_t row = sparse_grad ? (size_t)idx : (size_t)g;
    auto put = [&](float *base, size_t off, float v) {
        if (sparse_grad) base[off] = v; else atomicAdd(base + off, v);
    };
    if (v_means != nullptr) {
        put(v_means, 3 * row, v_mean.x); put(v_means, 3 * row + 1, v_mean.y); put(v_means, 3 * row + 2, v_mean.z);
    }
    if (v_velocities != nullptr) {
        put(v_velocities, 3 * row, v_vel_w.x); put(v_velocities, 3 * row + 1, v_vel_w.y);
        put(v_velocities, 3 * row + 2, v_vel_w.z);
    }
    if (covars != nullptr) {
        if (v_covars != nullptr) {
            float o[6];
            covar_grad_to_triu(v_covar, o);
            for (int k = 0; k < 6; ++k) put(v_covars, 6 * row + k, o[k]);
        }
    } else {
        V4 v_quat; v_quat.x = v_quat.y = v_quat.z = v_quat.w = 0.f;
        V3 v_scale = v3(0.f, 0.f, 0.f);
        M3 R = quat_to_rotmat(in.quat);
        quat_scale_to_covar_vjp(in.quat, in.scale, R, v_covar, v_quat, v_scale);
        if (v_quats != nullptr) {
            put(v_quats, 4 * row, v_quat.x); put(v_quats, 4 * row + 1, v_quat.y);
            put(v_quats, 4 * row + 2, v_quat.z); put(v_quats, 4 * row + 3, v_quat.w);
        }
        if (v_scales != nullptr) {
            put(v_scales, 3 * row, v_scale.x); put(v_scales, 3 * row + 1, v_scale.y);
            put(v_scales, 3 * row + 2, v_scale.z);
        }
    }
    if (v_viewmats != nullptr) {
        float *vm = v_viewmats + 16 * (size_t)c;
        for (int r = 0; r < 3; ++r) {
            for (int k = 0; k < 3; ++k) atomicAdd(vm + 4 * r + k, v_R.m[r][k]);
        }
        atomicAdd(vm + 3, v_t.x); atomicAdd(vm + 7, v_t.y); atomicAdd(vm + 11, v_t.z);
    }
}

} // namespace splatad

using namespace splatad;

// =======================================================================================
// C-ABI
// =======================================================================================
extern "C" int splatad_lidar_projection_fwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, float min_elevation,
    float max_elevation, float min_azimuth, float max_azimuth, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, float *radii, float *means2d,
    float *depths, float *conics, float *compensations, float *pix_vels,
    float *depth_compensations, void *stream) {
    SPL_REQUIRE(means && viewmats && linear_velocity && angular_velocity && rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "lidar_projection_fwd: null input");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "lidar_projection_fwd: covars or (quats, scales) required");
    SPL_REQUIRE(radii && means2d && depths && conics && pix_vels && depth_compensations,
                SPLATAD_ERR_BAD_ARG, "lidar_projection_fwd: null output");
    if (C == 0 || N == 0) return SPLATAD_OK;
    cudaStream_t st = (cudaStream_t)stream;
    // the pipelined kernel when the bulk copies' 16-byte rule holds for every input; covariance
    // inputs, odd alignments and scenes of fewer than 256 Gaussians through the plain kernel
    auto aligned16 = [](const void *ptr) { return (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0; };
    uint32_t n_slabs = 0;
    if (covars == nullptr && aligned16(means) && aligned16(quats) && aligned16(scales) &&
        (velocities == nullptr || aligned16(velocities)))
        n_slabs = N / kThreads;
    if (n_slabs > 0) {
        SPL_PROF("lidar_projection_fwd_kernel", st);
        const uint32_t n_rounds = div_up(N, kThreads);   // the ragged last slab rides along
        const uint32_t grid = n_rounds < (uint32_t)(4 * kNumSMs) ? n_rounds : (uint32_t)(4 * kNumSMs);
        lidar_projection_fwd_pipelined_kernel<<<grid, kThreads, 0, st>>>(
            C, N, n_slabs, means, quats, scales, velocities, viewmats, min_elevation, max_elevation, min_azimuth,
            max_azimuth, linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
            radius_clip, radii, means2d, depths, conics, compensations, pix_vels, depth_compensations);
    } else {
        SPL_PROF("lidar_projection_fwd_kernel", st);
        lidar_projection_fwd_kernel<<<div_up(N, kThreads), kThreads, 0, st>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, min_elevation, max_elevation,
            min_azimuth, max_azimuth, linear_velocity, angular_velocity, rolling_shutter_time, eps2d,
            near_plane, far_plane, radius_clip, radii, means2d, depths, conics, compensations,
            pix_vels, depth_compensations);
    }
    return check_launch("lidar_projection_fwd");
}

// Number of bulk-copy waits that ran into their limit since the last call (then reset); the kernels
// that use such copies leave their outputs unwritten when it happens. Synchronises the device.
extern "C" int splatad_async_copy_timeouts(int64_t *count) {
    SPL_REQUIRE(count != nullptr, SPLATAD_ERR_BAD_ARG, "async_copy_timeouts: null output");
    unsigned long long v = 0ull;
    const unsigned long long zero = 0ull;
    cudaError_t e = cudaMemcpyFromSymbol(&v, g_async_copy_timeouts, sizeof(v));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_async_copy_timeouts, &zero, sizeof(zero));
    if (e != cudaSuccess) {
        set_last_error("async_copy_timeouts: %s", cudaGetErrorString(e));
        return SPLATAD_ERR_CUDA;
    }
    *count = (int64_t)v;
    return SPLATAD_OK;
}

extern "C" int splatad_lidar_projection_bwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats,
    const float *linear_velocity, const float *angular_velocity,
    const float *rolling_shutter_time, float eps2d, const float *radii, const float *conics,
    const float *compensations, const float *v_means2d, const float *v_depths,
    const float *v_conics, const float *v_compensations, const float *v_pix_vels,
    const float *v_depth_compensations, float *v_means, float *v_covars, float *v_quats,
    float *v_scales, float *v_viewmats, float *v_velocities, void *stream) {
    SPL_REQUIRE(means && viewmats && linear_velocity && angular_velocity && rolling_shutter_time &&
                    radii && conics && v_means2d && v_depths && v_conics && v_pix_vels &&
                    v_depth_compensations,
                SPLATAD_ERR_BAD_ARG, "lidar_projection_bwd: null input");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "lidar_projection_bwd: covars or (quats, scales) required");
    SPL_REQUIRE(!v_compensations || compensations, SPLATAD_ERR_BAD_ARG,
                "lidar_projection_bwd: v_compensations given without compensations");
    if (C == 0 || N == 0) return SPLATAD_OK;
    {
        SPL_PROF("lidar_projection_bwd_kernel", (cudaStream_t)stream);
        lidar_projection_bwd_kernel<<<div_up(N, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, linear_velocity,
            angular_velocity, rolling_shutter_time, eps2d, radii, conics, compensations, v_means2d,
            v_depths, v_conics, v_compensations, v_pix_vels, v_depth_compensations, v_means, v_covars,
            v_quats, v_scales, v_viewmats, v_velocities);
    }
    return check_launch("lidar_projection_bwd");
}

extern "C" int splatad_projection_fwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, int32_t *radii, float *means2d,
    float *depths, float *conics, float *compensations, float *pix_vels, void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && linear_velocity && angular_velocity &&
                    rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "projection_fwd: null input");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_fwd: covars or (quats, scales) required");
    SPL_REQUIRE(radii && means2d && depths && conics && pix_vels, SPLATAD_ERR_BAD_ARG,
                "projection_fwd: null output");
    if (C == 0 || N == 0) return SPLATAD_OK;
    {
        SPL_PROF("projection_fwd_kernel", (cudaStream_t)stream);
        projection_fwd_kernel<<<div_up(N, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, Ks, image_width, image_height,
            linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
            radius_clip, radii, means2d, depths, conics, compensations, pix_vels);
    }
    return check_launch("projection_fwd");
}

extern "C" int splatad_projection_bwd(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    const int32_t *radii, const float *conics, const float *compensations,
    const float *v_means2d, const float *v_depths, const float *v_conics,
    const float *v_compensations, const float *v_pix_vels, float *v_means, float *v_covars,
    float *v_quats, float *v_scales, float *v_viewmats, float *v_velocities, void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && linear_velocity && angular_velocity &&
                    rolling_shutter_time && radii && conics && v_means2d && v_depths && v_conics &&
                    v_pix_vels,
                SPLATAD_ERR_BAD_ARG, "projection_bwd: null input");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_bwd: covars or (quats, scales) required");
    SPL_REQUIRE(!v_compensations || compensations, SPLATAD_ERR_BAD_ARG,
                "projection_bwd: v_compensations given without compensations");
    if (C == 0 || N == 0) return SPLATAD_OK;
    {
        SPL_PROF("projection_bwd_kernel", (cudaStream_t)stream);
        projection_bwd_kernel<<<div_up(N, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, Ks, image_width, image_height,
            linear_velocity, angular_velocity, rolling_shutter_time, eps2d, radii, conics,
            compensations, v_means2d, v_depths, v_conics, v_compensations, v_pix_vels, v_means,
            v_covars, v_quats, v_scales, v_viewmats, v_velocities);
    }
    return check_launch("projection_bwd");
}

extern "C" size_t splatad_projection_packed_workspace_bytes(uint32_t C, uint32_t N) {
    // block counts + block offsets
    return 2 * sizeof(int32_t) * (size_t)C * div_up(N, kThreads) + 256;
}

extern "C" int splatad_projection_packed_count(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, void *workspace,
    size_t workspace_bytes, int32_t *indptr, int64_t *nnz_device, void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && linear_velocity && angular_velocity &&
                    rolling_shutter_time && indptr && nnz_device && workspace,
                SPLATAD_ERR_BAD_ARG, "projection_packed_count: null argument");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_packed_count: covars or (quats, scales) required");
    SPL_REQUIRE(workspace_bytes >= splatad_projection_packed_workspace_bytes(C, N),
                SPLATAD_ERR_WORKSPACE, "projection_packed_count: workspace too small");
    SPL_REQUIRE(C > 0 && N > 0, SPLATAD_ERR_BAD_ARG, "projection_packed_count: empty input");
    const uint32_t nblocks = div_up(N, kThreads);
    int32_t *counts = (int32_t *)workspace;
    int32_t *offsets = counts + (size_t)C * nblocks;
    cudaStream_t st = (cudaStream_t)stream;
    {
        SPL_PROF("projection_packed_fwd_kernel", st);
        projection_packed_fwd_kernel<<<nblocks, kThreads, 0, st>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, Ks, image_width, image_height,
            linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
            radius_clip, counts, nullptr, (int64_t)-1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
            nullptr, nullptr, nullptr);
    }
    {
        SPL_PROF("packed_scan_kernel", st);
        packed_scan_kernel<<<1, 1024, 0, st>>>(counts, offsets, C, nblocks, indptr, nnz_device);
    }
    return check_launch("projection_packed_count");
}

extern "C" int splatad_projection_packed_fill(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, const void *workspace, int64_t capacity,
    int64_t *camera_ids, int64_t *gaussian_ids, int32_t *radii, float *means2d, float *depths,
    float *conics, float *compensations, float *pix_vels, void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && linear_velocity && angular_velocity &&
                    rolling_shutter_time && workspace && camera_ids && gaussian_ids && radii &&
                    means2d && depths && conics && pix_vels,
                SPLATAD_ERR_BAD_ARG, "projection_packed_fill: null argument");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_packed_fill: covars or (quats, scales) required");
    SPL_REQUIRE(C > 0 && N > 0, SPLATAD_ERR_BAD_ARG, "projection_packed_fill: empty input");
    const uint32_t nblocks = div_up(N, kThreads);
    const int32_t *offsets = (const int32_t *)workspace + (size_t)C * nblocks;
    {
        SPL_PROF("projection_packed_fwd_kernel", (cudaStream_t)stream);
        projection_packed_fwd_kernel<<<nblocks, kThreads, 0, (cudaStream_t)stream>>>(
            C, N, means, covars, quats, scales, velocities, viewmats, Ks, image_width, image_height,
            linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
            radius_clip, nullptr, offsets, capacity, (const int32_t *)workspace, camera_ids, gaussian_ids, radii,
            means2d, depths, conics, compensations, pix_vels);
    }
    return check_launch("projection_packed_fill");
}

extern "C" int splatad_projection_packed_bwd(
    uint32_t C, uint32_t N, uint32_t nnz, const float *means, const float *covars,
    const float *quats, const float *scales, const float *velocities, const float *viewmats,
    const float *Ks, int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    const int64_t *camera_ids, const int64_t *gaussian_ids, const float *conics,
    const float *compensations, const float *v_means2d, const float *v_depths,
    const float *v_conics, const float *v_compensations, const float *v_pix_vels,
    int32_t sparse_grad, float *v_means, float *v_covars, float *v_quats, float *v_scales,
    float *v_viewmats, float *v_velocities, void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && linear_velocity && angular_velocity &&
                    rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "projection_packed_bwd: null input");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_packed_bwd: covars or (quats, scales) required");
    SPL_REQUIRE(!v_compensations || compensations, SPLATAD_ERR_BAD_ARG,
                "projection_packed_bwd: v_compensations given without compensations");
    if (nnz == 0) return SPLATAD_OK;
    SPL_REQUIRE(camera_ids && gaussian_ids && conics && v_means2d && v_depths && v_conics &&
                    v_pix_vels,
                SPLATAD_ERR_BAD_ARG, "projection_packed_bwd: null input");
    {
        SPL_PROF("projection_packed_bwd_kernel", (cudaStream_t)stream);
        projection_packed_bwd_kernel<<<div_up(nnz, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
            C, N, nnz, means, covars, quats, scales, velocities, viewmats, Ks, image_width,
            image_height, linear_velocity, angular_velocity, rolling_shutter_time, eps2d, camera_ids,
            gaussian_ids, conics, compensations, v_means2d, v_depths, v_conics, v_compensations,
            v_pix_vels, sparse_grad, v_means, v_covars, v_quats, v_scales, v_viewmats, v_velocities);
    }
    return check_launch("projection_packed_bwd");
}

// =======================================================================================
// Allocation-free variant of the packed count
// =======================================================================================
namespace splatad {

// Scratch of splatad_projection_packed_count_noalloc: per-(camera, block) visible counts followed
// by their exclusive offsets. 2 x 65536 int32 = 512 KiB, resident on every GPU that loads the
// library until the process exits.
constexpr uint32_t kNoAllocMaxBlockRows = 65536;
static __device__ __align__(256) int32_t g_packed_count_scratch[2 * kNoAllocMaxBlockRows];

// Device address of the scratch array on the CURRENT device, looked up once per device. In host
// code the array's name is only a handle for the runtime, not a device address, so the address
// must come from cudaGetSymbolAddress.
static int packed_count_scratch(int32_t **out) {
    constexpr int kMaxDevices = 64;
    static int32_t *cached[kMaxDevices] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        set_last_error("projection_packed_count_noalloc: cudaGetDevice failed or device index %d unsupported", dev);
        return SPLATAD_ERR_CUDA;
    }
    int32_t *p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        void *addr = nullptr;
        e = cudaGetSymbolAddress(&addr, g_packed_count_scratch);
        if (e != cudaSuccess || addr == nullptr) {
            set_last_error("projection_packed_count_noalloc: cudaGetSymbolAddress failed: %s",
                           cudaGetErrorString(e));
            return SPLATAD_ERR_CUDA;
        }
        p = (int32_t *)addr;
        __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);
    }
    *out = p;
    return SPLATAD_OK;
}

} // namespace splatad

extern "C" int splatad_projection_packed_count_noalloc(
    uint32_t C, uint32_t N, const float *means, const float *covars, const float *quats,
    const float *scales, const float *velocities, const float *viewmats, const float *Ks,
    int32_t image_width, int32_t image_height, const float *linear_velocity,
    const float *angular_velocity, const float *rolling_shutter_time, float eps2d,
    float near_plane, float far_plane, float radius_clip, int32_t *indptr, int64_t *nnz_device,
    void *stream) {
    SPL_REQUIRE(means && viewmats && Ks && indptr && nnz_device && linear_velocity &&
                    angular_velocity && rolling_shutter_time,
                SPLATAD_ERR_BAD_ARG, "projection_packed_count_noalloc: null argument");
    SPL_REQUIRE(covars || (quats && scales), SPLATAD_ERR_BAD_ARG,
                "projection_packed_count_noalloc: covars or (quats, scales) required");
    SPL_REQUIRE(C > 0 && N > 0, SPLATAD_ERR_BAD_ARG, "projection_packed_count_noalloc: empty input");
    const uint64_t nblocks = div_up(N, kThreads);
    const uint64_t rows = (uint64_t)C * nblocks;
    SPL_REQUIRE(rows <= kNoAllocMaxBlockRows, SPLATAD_ERR_WORKSPACE,
                "projection_packed_count_noalloc: C * ceil(N / 256) = %llu exceeds the built-in scratch of "
                "%u rows; use splatad_projection_packed_count with a caller workspace",
                (unsigned long long)rows, kNoAllocMaxBlockRows);
    int32_t *scratch = nullptr;
    const int rc = packed_count_scratch(&scratch);
    if (rc != SPLATAD_OK) return rc;
    int32_t *counts = scratch;
    int32_t *offsets = scratch + rows;
    cudaStream_t st = (cudaStream_t)stream;
    // every slot the scan reads is written by the count pass of this same call: nothing in the
    // scratch needs clearing, and what earlier (larger) calls left behind is never read
    projection_packed_fwd_kernel<<<(uint32_t)nblocks, kThreads, 0, st>>>(
        C, N, means, covars, quats, scales, velocities, viewmats, Ks, image_width, image_height,
        linear_velocity, angular_velocity, rolling_shutter_time, eps2d, near_plane, far_plane,
        radius_clip, counts, nullptr, (int64_t)-1, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
        nullptr, nullptr);
    packed_scan_kernel<<<1, 1024, 0, st>>>(counts, offsets, C, (uint32_t)nblocks, indptr, nnz_device);
    return check_launch("projection_packed_count_noalloc");
}
