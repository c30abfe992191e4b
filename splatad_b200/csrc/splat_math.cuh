// Small fixed-size linear algebra and the per-Gaussian projection math (forward and VJP)
// shared by the projection kernels. Everything is FP32 and row-major: m[i][j] is row i,
// column j. All functions are usable from host code too (SPL_HD), which lets the CPU test
// harness run exactly the arithmetic the kernels run.
//
// Reference maths being restated (file:line in carlinds/splatad):
//   quaternion -> rotation, R S S^T R^T        gsplat/cuda/csrc/utils.cuh:57-119
//   pinhole EWA projection + clamp             gsplat/cuda/csrc/utils.cuh:190-279
//   spherical (lidar) projection + Jacobian    gsplat/cuda/csrc/utils.cuh:281-426
//   depth compensation from 3x3 spherical cov  gsplat/cuda/csrc/utils.cuh:12-55
//   blur / inverse / their VJPs                gsplat/cuda/csrc/utils.cuh:491-550
//   rolling-shutter velocities                 gsplat/cuda/csrc/helpers.cuh:80-309
#pragma once

#include <math.h>
#include <stdint.h>

#if defined(__CUDACC__)
#define SPL_HD __host__ __device__ __forceinline__
#else
#define SPL_HD inline
#endif

namespace splatad {

constexpr float kRadToDeg = 57.2957795131f;

struct V2 { float x, y; };
struct V3 { float x, y, z; };
struct V4 { float x, y, z, w; };
struct M2 { float m[2][2]; };
struct M3 { float m[3][3]; };

SPL_HD V3 v3(float x, float y, float z) { V3 r; r.x = x; r.y = y; r.z = z; return r; }
SPL_HD V2 v2(float x, float y) { V2 r; r.x = x; r.y = y; return r; }
SPL_HD V3 operator+(V3 a, V3 b) { return v3(a.x + b.x, a.y + b.y, a.z + b.z); }
SPL_HD V3 operator-(V3 a, V3 b) { return v3(a.x - b.x, a.y - b.y, a.z - b.z); }
SPL_HD V3 operator*(float s, V3 a) { return v3(s * a.x, s * a.y, s * a.z); }
SPL_HD float dot(V3 a, V3 b) { return a.x * b.x + a.y * b.y + a.z * b.z; }
SPL_HD V3 cross(V3 a, V3 b) {
    return v3(a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x);
}

SPL_HD M3 m3_zero() {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) r.m[i][j] = 0.f;
    return r;
}
SPL_HD M2 m2_zero() {
    M2 r;
    r.m[0][0] = r.m[0][1] = r.m[1][0] = r.m[1][1] = 0.f;
    return r;
}
SPL_HD M3 mul(const M3 &a, const M3 &b) {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j)
            r.m[i][j] = a.m[i][0] * b.m[0][j] + a.m[i][1] * b.m[1][j] + a.m[i][2] * b.m[2][j];
    return r;
}
// a * b^T
SPL_HD M3 mul_nt(const M3 &a, const M3 &b) {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j)
            r.m[i][j] = a.m[i][0] * b.m[j][0] + a.m[i][1] * b.m[j][1] + a.m[i][2] * b.m[j][2];
    return r;
}
// a^T * b
SPL_HD M3 mul_tn(const M3 &a, const M3 &b) {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j)
            r.m[i][j] = a.m[0][i] * b.m[0][j] + a.m[1][i] * b.m[1][j] + a.m[2][i] * b.m[2][j];
    return r;
}
SPL_HD M3 transpose(const M3 &a) {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) r.m[i][j] = a.m[j][i];
    return r;
}
SPL_HD M3 add(const M3 &a, const M3 &b) {
    M3 r;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) r.m[i][j] = a.m[i][j] + b.m[i][j];
    return r;
}
SPL_HD V3 mul(const M3 &a, V3 v) {
    return v3(a.m[0][0] * v.x + a.m[0][1] * v.y + a.m[0][2] * v.z,
              a.m[1][0] * v.x + a.m[1][1] * v.y + a.m[1][2] * v.z,
              a.m[2][0] * v.x + a.m[2][1] * v.y + a.m[2][2] * v.z);
}
// a^T * v
SPL_HD V3 mul_t(const M3 &a, V3 v) {
    return v3(a.m[0][0] * v.x + a.m[1][0] * v.y + a.m[2][0] * v.z,
              a.m[0][1] * v.x + a.m[1][1] * v.y + a.m[2][1] * v.z,
              a.m[0][2] * v.x + a.m[1][2] * v.y + a.m[2][2] * v.z);
}
SPL_HD M3 outer(V3 a, V3 b) {
    M3 r;
    r.m[0][0] = a.x * b.x; r.m[0][1] = a.x * b.y; r.m[0][2] = a.x * b.z;
    r.m[1][0] = a.y * b.x; r.m[1][1] = a.y * b.y; r.m[1][2] = a.y * b.z;
    r.m[2][0] = a.z * b.x; r.m[2][1] = a.z * b.y; r.m[2][2] = a.z * b.z;
    return r;
}

SPL_HD float spl_rsqrt(float x) {
#if defined(__CUDA_ARCH__)
    return rsqrtf(x);
#else
    return 1.0f / sqrtf(x);
#endif
}

// ---------------------------------------------------------------------------------------
// Sensor pose: rotation R and translation t of a row-major 4x4 world->sensor matrix.
// ---------------------------------------------------------------------------------------
struct Pose { M3 R; V3 t; };

SPL_HD Pose load_pose(const float *vm /* 16 floats */) {
    Pose p;
    p.R.m[0][0] = vm[0]; p.R.m[0][1] = vm[1]; p.R.m[0][2] = vm[2];  p.t.x = vm[3];
    p.R.m[1][0] = vm[4]; p.R.m[1][1] = vm[5]; p.R.m[1][2] = vm[6];  p.t.y = vm[7];
    p.R.m[2][0] = vm[8]; p.R.m[2][1] = vm[9]; p.R.m[2][2] = vm[10]; p.t.z = vm[11];
    return p;
}

// ---------------------------------------------------------------------------------------
// Quaternion (w, x, y, z; need not be normalised) -> rotation matrix, and covariance
// Sigma = (R S)(R S)^T.
// ---------------------------------------------------------------------------------------
SPL_HD M3 quat_to_rotmat(V4 q /* x=w, y=x, z=y, w=z in storage order */) {
    float w = q.x, x = q.y, y = q.z, z = q.w;
    float inv_norm = spl_rsqrt(x * x + y * y + z * z + w * w);
    x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
    float x2 = x * x, y2 = y * y, z2 = z * z;
    float xy = x * y, xz = x * z, yz = y * z;
    float wx = w * x, wy = w * y, wz = w * z;
    M3 R;
    R.m[0][0] = 1.f - 2.f * (y2 + z2); R.m[0][1] = 2.f * (xy - wz);       R.m[0][2] = 2.f * (xz + wy);
    R.m[1][0] = 2.f * (xy + wz);       R.m[1][1] = 1.f - 2.f * (x2 + z2); R.m[1][2] = 2.f * (yz - wx);
    R.m[2][0] = 2.f * (xz - wy);       R.m[2][1] = 2.f * (yz + wx);       R.m[2][2] = 1.f - 2.f * (x2 + y2);
    return R;
}

SPL_HD M3 quat_scale_to_covar(V4 quat, V3 scale) {
    M3 R = quat_to_rotmat(quat);
    M3 M;
    for (int i = 0; i < 3; ++i) {
        M.m[i][0] = R.m[i][0] * scale.x;
        M.m[i][1] = R.m[i][1] * scale.y;
        M.m[i][2] = R.m[i][2] * scale.z;
    }
    return mul_nt(M, M);
}

// VJP of quat -> R. v_R is dL/dR (row-major). Accumulates into v_quat (storage order w,x,y,z).
SPL_HD void quat_to_rotmat_vjp(V4 q, const M3 &vR, V4 &v_quat) {
    float w = q.x, x = q.y, y = q.z, z = q.w;
    float inv_norm = spl_rsqrt(x * x + y * y + z * z + w * w);
    x *= inv_norm; y *= inv_norm; z *= inv_norm; w *= inv_norm;
    // G(i,j) = dL/dR(i,j)
    const float (*G)[3] = vR.m;
    float vw = 2.f * (x * (G[2][1] - G[1][2]) + y * (G[0][2] - G[2][0]) + z * (G[1][0] - G[0][1]));
    float vx = 2.f * (-2.f * x * (G[1][1] + G[2][2]) + y * (G[1][0] + G[0][1]) +
                      z * (G[2][0] + G[0][2]) + w * (G[2][1] - G[1][2]));
    float vy = 2.f * (x * (G[1][0] + G[0][1]) - 2.f * y * (G[0][0] + G[2][2]) +
                      z * (G[2][1] + G[1][2]) + w * (G[0][2] - G[2][0]));
    float vz = 2.f * (x * (G[2][0] + G[0][2]) + y * (G[2][1] + G[1][2]) -
                      2.f * z * (G[0][0] + G[1][1]) + w * (G[1][0] - G[0][1]));
    float d = vw * w + vx * x + vy * y + vz * z;
    v_quat.x += (vw - d * w) * inv_norm;
    v_quat.y += (vx - d * x) * inv_norm;
    v_quat.z += (vy - d * y) * inv_norm;
    v_quat.w += (vz - d * z) * inv_norm;
}

// VJP of Sigma = (R S)(R S)^T with respect to quat and scale.
SPL_HD void quat_scale_to_covar_vjp(V4 quat, V3 scale, const M3 &R, const M3 &v_covar,
                                    V4 &v_quat, V3 &v_scale) {
    M3 M;
    for (int i = 0; i < 3; ++i) {
        M.m[i][0] = R.m[i][0] * scale.x;
        M.m[i][1] = R.m[i][1] * scale.y;
        M.m[i][2] = R.m[i][2] * scale.z;
    }
    // dL/dM = (G + G^T) M
    M3 Gs = add(v_covar, transpose(v_covar));
    M3 vM = mul(Gs, M);
    M3 vR;
    for (int i = 0; i < 3; ++i) {
        vR.m[i][0] = vM.m[i][0] * scale.x;
        vR.m[i][1] = vM.m[i][1] * scale.y;
        vR.m[i][2] = vM.m[i][2] * scale.z;
    }
    quat_to_rotmat_vjp(quat, vR, v_quat);
    v_scale.x += R.m[0][0] * vM.m[0][0] + R.m[1][0] * vM.m[1][0] + R.m[2][0] * vM.m[2][0];
    v_scale.y += R.m[0][1] * vM.m[0][1] + R.m[1][1] * vM.m[1][1] + R.m[2][1] * vM.m[2][1];
    v_scale.z += R.m[0][2] * vM.m[0][2] + R.m[1][2] * vM.m[1][2] + R.m[2][2] * vM.m[2][2];
}

SPL_HD M3 covar_from_triu(const float *c /* 6 */) {
    M3 S;
    S.m[0][0] = c[0]; S.m[0][1] = c[1]; S.m[0][2] = c[2];
    S.m[1][0] = c[1]; S.m[1][1] = c[3]; S.m[1][2] = c[4];
    S.m[2][0] = c[2]; S.m[2][1] = c[4]; S.m[2][2] = c[5];
    return S;
}

// Sigma_c = R Sigma R^T and its VJP.
SPL_HD M3 covar_world_to_cam(const M3 &R, const M3 &covar) { return mul_nt(mul(R, covar), R); }

SPL_HD void covar_world_to_cam_vjp(const M3 &R, const M3 &covar, const M3 &v_covar_c, M3 &v_R,
                                   M3 &v_covar) {
    // dL/dR = G R Sigma^T + G^T R Sigma ; dL/dSigma = R^T G R
    M3 a = mul_nt(mul(v_covar_c, R), covar);
    M3 b = mul(mul_tn(v_covar_c, R), covar);
    v_R = add(v_R, add(a, b));
    v_covar = add(v_covar, mul(mul_tn(R, v_covar_c), R));
}

// ---------------------------------------------------------------------------------------
// 2x2 helpers: blur, inverse and VJPs (symmetric 2x2 stored as full M2).
// ---------------------------------------------------------------------------------------
SPL_HD float add_blur(float eps2d, M2 &covar, float &compensation) {
    float det_orig = covar.m[0][0] * covar.m[1][1] - covar.m[0][1] * covar.m[1][0];
    covar.m[0][0] += eps2d;
    covar.m[1][1] += eps2d;
    float det_blur = covar.m[0][0] * covar.m[1][1] - covar.m[0][1] * covar.m[1][0];
    compensation = sqrtf(fmaxf(0.f, det_orig / det_blur));
    return det_blur;
}

SPL_HD void inverse2(const M2 &M, float det, M2 &Minv) {
    float inv_det = 1.f / det;
    Minv.m[0][0] = M.m[1][1] * inv_det;
    Minv.m[0][1] = -M.m[0][1] * inv_det;
    Minv.m[1][0] = Minv.m[0][1];
    Minv.m[1][1] = M.m[0][0] * inv_det;
}

// P = M^-1 ; dL/dM += -P (dL/dP) P
SPL_HD void inverse2_vjp(const M2 &P, const M2 &vP, M2 &vM) {
    M2 t;
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 2; ++j) t.m[i][j] = P.m[i][0] * vP.m[0][j] + P.m[i][1] * vP.m[1][j];
    for (int i = 0; i < 2; ++i)
        for (int j = 0; j < 2; ++j)
            vM.m[i][j] += -(t.m[i][0] * P.m[0][j] + t.m[i][1] * P.m[1][j]);
}

SPL_HD void add_blur_vjp(float eps2d, const M2 &conic_blur, float compensation,
                         float v_compensation, M2 &v_covar) {
    float det_conic_blur =
        conic_blur.m[0][0] * conic_blur.m[1][1] - conic_blur.m[0][1] * conic_blur.m[1][0];
    float v_sqr_comp = v_compensation * 0.5f / (compensation + 1e-6f);
    float one_minus_sqr_comp = 1.f - compensation * compensation;
    v_covar.m[0][0] += v_sqr_comp * (one_minus_sqr_comp * conic_blur.m[0][0] - eps2d * det_conic_blur);
    v_covar.m[0][1] += v_sqr_comp * (one_minus_sqr_comp * conic_blur.m[0][1]);
    v_covar.m[1][0] += v_sqr_comp * (one_minus_sqr_comp * conic_blur.m[1][0]);
    v_covar.m[1][1] += v_sqr_comp * (one_minus_sqr_comp * conic_blur.m[1][1] - eps2d * det_conic_blur);
}

// ---------------------------------------------------------------------------------------
// Pinhole projection (EWA with the 0.3*tan(fov) clamp of x/z, y/z).
// ---------------------------------------------------------------------------------------
struct Intrin { float fx, fy, cx, cy; };

struct PerspJ { float j00, j11, j02, j12; float tx, ty, rz; bool x_in, y_in; };

SPL_HD PerspJ persp_jacobian(V3 p, Intrin K, int width, int height) {
    PerspJ o;
    float tan_fovx = 0.5f * (float)width / K.fx;
    float tan_fovy = 0.5f * (float)height / K.fy;
    float lim_x_pos = ((float)width - K.cx) / K.fx + 0.3f * tan_fovx;
    float lim_x_neg = K.cx / K.fx + 0.3f * tan_fovx;
    float lim_y_pos = ((float)height - K.cy) / K.fy + 0.3f * tan_fovy;
    float lim_y_neg = K.cy / K.fy + 0.3f * tan_fovy;
    float rz = 1.f / p.z;
    float rz2 = rz * rz;
    float xr = p.x * rz, yr = p.y * rz;
    o.x_in = (xr <= lim_x_pos) && (xr >= -lim_x_neg);
    o.y_in = (yr <= lim_y_pos) && (yr >= -lim_y_neg);
    o.tx = p.z * fminf(lim_x_pos, fmaxf(-lim_x_neg, xr));
    o.ty = p.z * fminf(lim_y_pos, fmaxf(-lim_y_neg, yr));
    o.rz = rz;
    o.j00 = K.fx * rz;
    o.j11 = K.fy * rz;
    o.j02 = -K.fx * o.tx * rz2;
    o.j12 = -K.fy * o.ty * rz2;
    return o;
}

SPL_HD void persp_proj(V3 p, const M3 &cov3d, Intrin K, int width, int height, M2 &cov2d,
                       V2 &mean2d, PerspJ &J) {
    J = persp_jacobian(p, K, width, height);
    // rows of J: [j00 0 j02], [0 j11 j12]
    const float (*S)[3] = cov3d.m;
    float a0 = J.j00 * S[0][0] + J.j02 * S[2][0];
    float a1 = J.j00 * S[0][1] + J.j02 * S[2][1];
    float a2 = J.j00 * S[0][2] + J.j02 * S[2][2];
    float b0 = J.j11 * S[1][0] + J.j12 * S[2][0];
    float b1 = J.j11 * S[1][1] + J.j12 * S[2][1];
    float b2 = J.j11 * S[1][2] + J.j12 * S[2][2];
    cov2d.m[0][0] = a0 * J.j00 + a2 * J.j02;
    cov2d.m[0][1] = a1 * J.j11 + a2 * J.j12;
    cov2d.m[1][0] = b0 * J.j00 + b2 * J.j02;
    cov2d.m[1][1] = b1 * J.j11 + b2 * J.j12;
    mean2d.x = K.fx * p.x * J.rz + K.cx;
    mean2d.y = K.fy * p.y * J.rz + K.cy;
}

// pixel velocity = -J (lin + ang x p - vel_c)
SPL_HD V2 compute_pix_velocity(V3 p, V3 lin, V3 ang, V3 vel_c, const PerspJ &J) {
    V3 tv = lin + cross(ang, p) - vel_c;
    return v2(-(J.j00 * tv.x + J.j02 * tv.z), -(J.j11 * tv.y + J.j12 * tv.z));
}

SPL_HD void persp_proj_vjp(V3 p, const M3 &cov3d, Intrin K, int width, int height,
                           const M2 &v_cov2d, V2 v_mean2d, V3 &v_mean3d, M3 &v_cov3d) {
    PerspJ J = persp_jacobian(p, K, width, height);
    float rz = J.rz, rz2 = rz * rz, rz3 = rz2 * rz;
    // Jm: 2x3
    float Jm[2][3] = {{J.j00, 0.f, J.j02}, {0.f, J.j11, J.j12}};
    // dL/dSigma += J^T G J
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) {
            float s = 0.f;
            for (int a = 0; a < 2; ++a)
                for (int b = 0; b < 2; ++b) s += Jm[a][i] * v_cov2d.m[a][b] * Jm[b][j];
            v_cov3d.m[i][j] += s;
        }
    v_mean3d.x += K.fx * rz * v_mean2d.x;
    v_mean3d.y += K.fy * rz * v_mean2d.y;
    v_mean3d.z += -(K.fx * p.x * v_mean2d.x + K.fy * p.y * v_mean2d.y) * rz2;

    // dL/dJ = G J Sigma^T + G^T J Sigma   (2x3)
    float vJ[2][3];
    for (int a = 0; a < 2; ++a)
        for (int j = 0; j < 3; ++j) {
            float s = 0.f;
            for (int b = 0; b < 2; ++b)
                for (int k = 0; k < 3; ++k)
                    s += v_cov2d.m[a][b] * Jm[b][k] * cov3d.m[j][k] +
                         v_cov2d.m[b][a] * Jm[b][k] * cov3d.m[k][j];
            vJ[a][j] = s;
        }
    if (J.x_in) v_mean3d.x += -K.fx * rz2 * vJ[0][2];
    else        v_mean3d.z += -K.fx * rz3 * vJ[0][2] * J.tx;
    if (J.y_in) v_mean3d.y += -K.fy * rz2 * vJ[1][2];
    else        v_mean3d.z += -K.fy * rz3 * vJ[1][2] * J.ty;
    v_mean3d.z += -K.fx * rz2 * vJ[0][0] - K.fy * rz2 * vJ[1][1] +
                  2.f * K.fx * J.tx * rz3 * vJ[0][2] + 2.f * K.fy * J.ty * rz3 * vJ[1][2];
}

// VJP of the pixel velocity w.r.t. the camera-space point and the camera-space Gaussian velocity.
SPL_HD void pix_velocity_vjp(V3 p, V3 lin, V3 ang, V3 vel_c, Intrin K, int width, int height,
                             V2 v_pv, V3 &v_p, V3 &v_vel_c) {
    PerspJ J = persp_jacobian(p, K, width, height);
    float rz = J.rz, rz2 = rz * rz;
    V3 tv = lin + cross(ang, p) - vel_c;
    if (J.x_in) v_p.x += v_pv.x * K.fx * rz2 * tv.z;
    else        v_p.z += v_pv.x * K.fx * rz2 * rz * J.tx * tv.z;
    if (J.y_in) v_p.y += v_pv.y * K.fy * rz2 * tv.z;
    else        v_p.z += v_pv.y * K.fy * rz2 * rz * J.ty * tv.z;
    // dJ/dz applied to tv
    float dx = -K.fx * rz2 * tv.x + 2.f * K.fx * J.tx * rz2 * rz * tv.z;
    float dy = -K.fy * rz2 * tv.y + 2.f * K.fy * J.ty * rz2 * rz * tv.z;
    v_p.z -= v_pv.x * dx + v_pv.y * dy;
    // v_total_vel = -J^T v_pv
    V3 v_tv = v3(-(J.j00 * v_pv.x), -(J.j11 * v_pv.y), -(J.j02 * v_pv.x + J.j12 * v_pv.y));
    V3 v_rot = cross(ang, v_tv);
    v_p.x -= v_rot.x; v_p.y -= v_rot.y; v_p.z -= v_rot.z;
    v_vel_c.x -= v_tv.x; v_vel_c.y -= v_tv.y; v_vel_c.z -= v_tv.z;
}

// ---------------------------------------------------------------------------------------
// Spherical (lidar) projection. Angles in degrees. Jacobian rows: azimuth, elevation, range.
// ---------------------------------------------------------------------------------------
SPL_HD float spl_rnorm3(float x, float y, float z) {
#if defined(__CUDA_ARCH__)
    return rnorm3df(x, y, z);
#else
    return 1.0f / sqrtf(x * x + y * y + z * z);
#endif
}
SPL_HD float spl_norm3(float x, float y, float z) {
#if defined(__CUDA_ARCH__)
    return norm3df(x, y, z);
#else
    return sqrtf(x * x + y * y + z * z);
#endif
}

SPL_HD M3 lidar_jacobian(V3 p) {
    float x2 = p.x * p.x, y2 = p.y * p.y, z2 = p.z * p.z;
    float xz = p.x * p.z, yz = p.y * p.z;
    float r2 = x2 + y2 + z2;
    float rinv = spl_rnorm3(p.x, p.y, p.z);
    float sxy = hypotf(p.x, p.y);
    float sxy_inv = 1.f / sxy;
    float k = 1.f / r2 * sxy_inv;
    M3 J;
    J.m[0][0] = -p.y / (x2 + y2) * kRadToDeg; J.m[0][1] = p.x / (x2 + y2) * kRadToDeg; J.m[0][2] = 0.f;
    J.m[1][0] = -xz * k * kRadToDeg;          J.m[1][1] = -yz * k * kRadToDeg;         J.m[1][2] = sxy / r2 * kRadToDeg;
    J.m[2][0] = p.x * rinv;                   J.m[2][1] = p.y * rinv;                  J.m[2][2] = p.z * rinv;
    return J;
}

SPL_HD V2 depth_compensation_from_cov3d(const M3 &c, float eps2d) {
    float a1 = c.m[0][0] + eps2d, a2 = c.m[0][1];
    float b1 = c.m[1][0], b2 = c.m[1][1] + eps2d;
    float c1 = c.m[2][0], c2 = c.m[2][1];
    float invD = 1.f / (a1 * b2 - a2 * b1);
    return v2((b1 * c2 - b2 * c1) * invD, (a2 * c1 - a1 * c2) * invD);
}

SPL_HD void depth_compensation_from_cov3d_vjp(const M3 &c, float eps2d, V2 v_dc, M3 &v_c) {
    float a1 = c.m[0][0] + eps2d, a2 = c.m[0][1];
    float b1 = c.m[1][0], b2 = c.m[1][1] + eps2d;
    float c1 = c.m[2][0], c2 = c.m[2][1];
    float invD = 1.f / (a1 * b2 - a2 * b1);
    float dc1 = (b1 * c2 - b2 * c1) * invD;
    float dc2 = (a2 * c1 - a1 * c2) * invD;
    v_c.m[0][0] += (v_dc.x * (-dc1 * b2) + v_dc.y * (-c2 - dc2 * b2)) * invD;   // d/da1
    v_c.m[0][1] += (v_dc.x * (dc1 * b1) + v_dc.y * (c1 + dc2 * b1)) * invD;     // d/da2
    v_c.m[1][0] += (v_dc.x * (c2 + dc1 * a2) + v_dc.y * (dc2 * a2)) * invD;     // d/db1
    v_c.m[1][1] += (v_dc.x * (-c1 - dc1 * a1) + v_dc.y * (-dc2 * a1)) * invD;   // d/db2
    v_c.m[2][0] += (v_dc.x * (-b2) + v_dc.y * (a2)) * invD;                     // d/dc1
    v_c.m[2][1] += (v_dc.x * (b1) + v_dc.y * (-a1)) * invD;                     // d/dc2
}

SPL_HD void lidar_proj(V3 p, const M3 &cov3d, float eps2d, V2 &mean2d, M2 &cov2d, V2 &depth_comp,
                       M3 &J) {
    J = lidar_jacobian(p);
    M3 cs = mul_nt(mul(J, cov3d), J);
    cov2d.m[0][0] = cs.m[0][0]; cov2d.m[0][1] = cs.m[0][1];
    cov2d.m[1][0] = cs.m[1][0]; cov2d.m[1][1] = cs.m[1][1];
    float rinv = spl_rnorm3(p.x, p.y, p.z);
    mean2d.x = atan2f(p.y, p.x) * kRadToDeg;
    mean2d.y = asinf(p.z * rinv) * kRadToDeg;
    depth_comp = depth_compensation_from_cov3d(cs, eps2d);
}

// (azimuth, elevation, range) velocity = -J (lin + ang x p - vel_c)
SPL_HD V3 compute_lidar_velocity(V3 p, V3 lin, V3 ang, V3 vel_c, const M3 &J) {
    V3 tv = lin + cross(ang, p) - vel_c;
    V3 r = mul(J, tv);
    return v3(-r.x, -r.y, -r.z);
}

// Derivatives of the 3x3 spherical Jacobian with respect to x, y, z (each a 3x3, row-major,
// rows az / el / range), used by both lidar VJPs below.
SPL_HD void lidar_jacobian_derivs(V3 p, M3 &dJdx, M3 &dJdy, M3 &dJdz) {
    const float x = p.x, y = p.y, z = p.z;
    const float x2 = x * x, y2 = y * y, z2 = z * z;
    const float x4 = x2 * x2, y4 = y2 * y2;
    const float s2 = x2 + y2;
    const float sxy = hypotf(x, y);
    const float sxy_inv = 1.f / sxy;
    const float s2sq = s2 * s2;
    const float s3 = sxy * s2;
    const float r2 = s2 + z2;
    const float r4 = r2 * r2;
    const float rinv = spl_rsqrt(r2);
    const float r3_inv = 1.f / r2 * rinv;
    const float xy = x * y, xz = x * z, yz = y * z, xyz = x * y * z;
    const float den1 = 1.f / (s3 * r4);
    const float den2 = 1.f / r4 * sxy_inv;
    const float D = kRadToDeg;

    dJdx.m[0][0] = 2.f * xy / s2sq * D;
    dJdx.m[0][1] = (y2 - x2) / s2sq * D;
    dJdx.m[0][2] = 0.f;
    dJdx.m[1][0] = z * (2.f * x4 + x2 * y2 - y2 * (y2 + z2)) * den1 * D;
    dJdx.m[1][1] = xyz * (3.f * x2 + 3.f * y2 + z2) * den1 * D;
    dJdx.m[1][2] = -x * (s2 - z2) * den2 * D;
    dJdx.m[2][0] = (y2 + z2) * r3_inv;
    dJdx.m[2][1] = -xy * r3_inv;
    dJdx.m[2][2] = -xz * r3_inv;

    dJdy.m[0][0] = (y2 - x2) / s2sq * D;
    dJdy.m[0][1] = -2.f * xy / s2sq * D;
    dJdy.m[0][2] = 0.f;
    dJdy.m[1][0] = xyz * (3.f * x2 + 3.f * y2 + z2) * den1 * D;
    dJdy.m[1][1] = -z * (x4 + x2 * (z2 - y2) - 2.f * y4) * den1 * D;
    dJdy.m[1][2] = -y * (s2 - z2) * den2 * D;
    dJdy.m[2][0] = -xy * r3_inv;
    dJdy.m[2][1] = (x2 + z2) * r3_inv;
    dJdy.m[2][2] = -yz * r3_inv;

    dJdz.m[0][0] = 0.f;
    dJdz.m[0][1] = 0.f;
    dJdz.m[0][2] = 0.f;
    dJdz.m[1][0] = -x * (s2 - z2) * den2 * D;
    dJdz.m[1][1] = -y * (s2 - z2) * den2 * D;
    dJdz.m[1][2] = -2.f * z * sxy / r4 * D;
    dJdz.m[2][0] = -xz * r3_inv;
    dJdz.m[2][1] = -yz * r3_inv;
    dJdz.m[2][2] = s2 * r3_inv;
}

SPL_HD float frob(const M3 &a, const M3 &b) {
    float s = 0.f;
    for (int i = 0; i < 3; ++i)
        for (int j = 0; j < 3; ++j) s += a.m[i][j] * b.m[i][j];
    return s;
}

// VJP of lidar_proj: gradients of (mean2d, blurred-cov2d, depth_comp) back to the
// sensor-space mean and covariance.
SPL_HD void lidar_proj_vjp(V3 p, const M3 &cov3d, float eps2d, V2 v_mean2d, const M2 &v_cov2d,
                           V2 v_depth_comp, V3 &v_mean3d, M3 &v_cov3d) {
    M3 J = lidar_jacobian(p);
    M3 cs = mul_nt(mul(J, cov3d), J);
    // gradient on the full 3x3 spherical covariance: depth-compensation part + top-left 2x2
    M3 v_cs = m3_zero();
    depth_compensation_from_cov3d_vjp(cs, eps2d, v_depth_comp, v_cs);
    v_cs.m[0][0] += v_cov2d.m[0][0]; v_cs.m[0][1] += v_cov2d.m[0][1];
    v_cs.m[1][0] += v_cov2d.m[1][0]; v_cs.m[1][1] += v_cov2d.m[1][1];
    // dL/dSigma_c = J^T G J
    v_cov3d = add(v_cov3d, mul(mul_tn(J, v_cs), J));
    // mean2d gradient through the first two rows of J
    v_mean3d.x += v_mean2d.x * J.m[0][0] + v_mean2d.y * J.m[1][0];
    v_mean3d.y += v_mean2d.x * J.m[0][1] + v_mean2d.y * J.m[1][1];
    v_mean3d.z += v_mean2d.x * J.m[0][2] + v_mean2d.y * J.m[1][2];
    // dL/dJ = G J Sigma^T + G^T J Sigma
    M3 vJ = add(mul_nt(mul(v_cs, J), cov3d), mul(mul_tn(v_cs, J), cov3d));
    M3 dx, dy, dz;
    lidar_jacobian_derivs(p, dx, dy, dz);
    v_mean3d.x += frob(vJ, dx);
    v_mean3d.y += frob(vJ, dy);
    v_mean3d.z += frob(vJ, dz);
}

// VJP of the lidar velocity w.r.t. the sensor-space point and sensor-space Gaussian velocity.
SPL_HD void lidar_velocity_vjp(V3 p, V3 lin, V3 ang, V3 vel_c, V3 v_pv, V3 &v_p, V3 &v_vel_c) {
    V3 tv = lin + cross(ang, p) - vel_c;
    M3 J = lidar_jacobian(p);
    M3 dx, dy, dz;
    lidar_jacobian_derivs(p, dx, dy, dz);
    v_p.x -= dot(v_pv, mul(dx, tv));
    v_p.y -= dot(v_pv, mul(dy, tv));
    v_p.z -= dot(v_pv, mul(dz, tv));
    V3 v_tv = mul_t(J, v_pv);
    v_tv = v3(-v_tv.x, -v_tv.y, -v_tv.z);
    V3 v_rot = cross(ang, v_tv);
    v_p.x -= v_rot.x; v_p.y -= v_rot.y; v_p.z -= v_rot.z;
    v_vel_c.x -= v_tv.x; v_vel_c.y -= v_tv.y; v_vel_c.z -= v_tv.z;
}

} // namespace splatad
