// The two device-side pieces of the densification strategies that consume the render path's
// outputs during training:
//   * the running statistics update of the default strategy, one fused kernel in place of the
//     chain of torch ops in gsplat/strategy/default.py:203-258 (clone, two scalings, mask,
//     where, norm, two index_add_, gather / maximum / scatter);
//   * compute_relocation, equation (9) of "3D Gaussian Splatting as Markov Chain Monte Carlo":
//     gsplat/cuda/csrc/relocation.cu:4-31 (host side 33-53, wrapper gsplat/relocation.py:10-49).
#include "common.cuh"

namespace splatad {

// One thread per (sensor, Gaussian) entry of the projection outputs.
//   unpacked (gaussian_ids == nullptr): entry e belongs to Gaussian e % N and takes part when
//     radii[e][0] > 0;
//   packed: every entry takes part, Gaussian gaussian_ids[e].
// grad2d[g] += |(gx * sx, gy * sy)|, count[g] += 1, radii_state[g] = max(., max(radii[e]) * inv_extent).
// The maximum is a true scatter-max (the reference's indexed assignment keeps an arbitrary one of
// the candidates when a Gaussian is seen by several sensors).
__global__ void densify_update_state_kernel(uint64_t total, uint32_t N, const float2 *__restrict__ grads,
                                            const int32_t *__restrict__ radii,
                                            const int64_t *__restrict__ gaussian_ids, float sx, float sy,
                                            float inv_extent, float *__restrict__ grad2d,
                                            float *__restrict__ count, float *__restrict__ radii_state) {
    const uint64_t e = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= total) return;
    const int32_t rx = radii[2 * e], ry = radii[2 * e + 1];
    uint64_t g;
    if (gaussian_ids) {
        g = (uint64_t)gaussian_ids[e];
        if (g >= N) return;
    } else {
        if (rx <= 0) return;
        g = e % N;
    }
    const float2 v = grads[e];
    const float gx = v.x * sx, gy = v.y * sy;
    atomicAdd(grad2d + g, sqrtf(gx * gx + gy * gy));
    atomicAdd(count + g, 1.f);
    if (radii_state) {
        const float r = (float)max(rx, ry) * inv_extent;
        // non-negative floats order like their bit patterns
        if (r > 0.f) atomicMax(reinterpret_cast<int *>(radii_state + g), __float_as_int(r));
    }
}

// One thread per Gaussian. The double sum keeps the reference's order (i outer, k inner, float
// accumulation); powers of the new opacity are built by repeated multiplication.
__global__ void compute_relocation_kernel(uint32_t N, const float *__restrict__ opacities,
                                          const float *__restrict__ scales, const int32_t *__restrict__ ratios,
                                          const float *__restrict__ binoms, int32_t n_max,
                                          float *__restrict__ new_opacities, float *__restrict__ new_scales) {
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= N) return;
    const int32_t n_idx = min(max(ratios[idx], 1), n_max);
    const float op = opacities[idx];
    const float new_op = 1.f - powf(1.f - op, 1.f / (float)n_idx);
    new_opacities[idx] = new_op;
    float denom_sum = 0.f;
    for (int32_t i = 1; i <= n_idx; ++i) {
        float xp = new_op;   // new_op^(k + 1)
        float sign = 1.f;
        const float *row = binoms + (size_t)(i - 1) * n_max;
        for (int32_t k = 0; k <= i - 1; ++k) {
            denom_sum += row[k] * ((sign / sqrtf((float)(k + 1))) * xp);
            xp *= new_op;
            sign = -sign;
        }
    }
    const float coeff = op / denom_sum;
#pragma unroll
    for (int c = 0; c < 3; ++c) new_scales[3 * (size_t)idx + c] = coeff * scales[3 * (size_t)idx + c];
}

} // namespace splatad

using namespace splatad;

extern "C" int splatad_densify_update_state(
    uint64_t total, uint32_t N, const float *grads, const int32_t *radii, const int64_t *gaussian_ids,
    uint32_t image_width, uint32_t image_height, uint32_t n_cameras, float *grad2d, float *count,
    float *radii_state, void *stream) {
    if (total == 0) return SPLATAD_OK;
    SPL_REQUIRE(grads && radii && grad2d && count && N > 0, SPLATAD_ERR_BAD_ARG,
                "densify_update_state: null argument");
    SPL_REQUIRE(total <= (uint64_t)0x7fffffff * kThreads, SPLATAD_ERR_BAD_ARG,
                "densify_update_state: too many entries");
    const float sx = (float)image_width / 2.f * (float)n_cameras;
    const float sy = (float)image_height / 2.f * (float)n_cameras;
    const uint32_t extent = image_width > image_height ? image_width : image_height;
    SPL_REQUIRE(extent > 0, SPLATAD_ERR_BAD_ARG, "densify_update_state: empty image");
    SPL_PROF("densify_update_state_kernel", (cudaStream_t)stream);
    densify_update_state_kernel<<<div_up(total, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
        total, N, (const float2 *)grads, radii, gaussian_ids, sx, sy, 1.f / (float)extent, grad2d, count,
        radii_state);
    return check_launch("densify_update_state");
}

extern "C" int splatad_compute_relocation(uint32_t N, const float *opacities, const float *scales,
                                          const int32_t *ratios, const float *binoms, int32_t n_max,
                                          float *new_opacities, float *new_scales, void *stream) {
    if (N == 0) return SPLATAD_OK;
    SPL_REQUIRE(opacities && scales && ratios && binoms && new_opacities && new_scales && n_max >= 1,
                SPLATAD_ERR_BAD_ARG, "compute_relocation: null argument");
    SPL_PROF("compute_relocation_kernel", (cudaStream_t)stream);
    compute_relocation_kernel<<<div_up(N, kThreads), kThreads, 0, (cudaStream_t)stream>>>(
        N, opacities, scales, ratios, binoms, n_max, new_opacities, new_scales);
    return check_launch("compute_relocation");
}
