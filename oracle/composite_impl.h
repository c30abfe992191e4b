/*
 * CPU restatement of the compositing kernels. TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).
 * Included twice by composite.c with REAL = float (suffix _f32) and REAL = double (suffix _f64).
 *
 * Follows, per pixel and in list order,
 *   pixels forward   gsplat/cuda/csrc/rasterization.cu:1398-1401, 1466-1517
 *   points forward   gsplat/cuda/csrc/rasterization.cu:2082-2091, 2154-2218
 *   pixels backward  gsplat/cuda/csrc/rasterization.cu:2909-2923, 2960-3087
 *   points backward  gsplat/cuda/csrc/rasterization.cu:3826-3845, 3884-4052
 *   angle wrap       gsplat/cuda/csrc/utils.cuh:552-555
 * (per-pair maths also at gsplat/cuda/_torch_impl.py:670-683 and 765-807).
 *
 * `ambiguous[pix]` is set when a threshold decision of that pixel (alpha >= 1/255, the
 * transmittance stop at 1e-4, the alpha cap at 0.999, the median crossing at 0.5, the
 * alpha-sum range test) is within a relative `amb_tol` of flipping, so that a comparison
 * against another floating-point evaluation order can set those pixels aside.
 * `counters[0]` += tested pairs, `counters[1]` += contributing pairs (for the flop model).
 */

#define ALPHA_MAX ((REAL)0.999f)
#define ALPHA_MIN ((REAL)(1.f / 255.f))
#define T_STOP ((REAL)1e-4f)

static inline REAL FN(angle_difference)(REAL a, REAL b) {
    REAL diff = FMOD((a - b + (REAL)180), (REAL)360) - (REAL)180;
    return diff < (REAL)-180 ? diff + (REAL)360 : diff;
}

static inline int FN(near)(REAL v, REAL ref, REAL tol) {
    REAL d = v - ref;
    if (d < 0) d = -d;
    REAL s = ref < 0 ? -ref : ref;
    return d <= tol * s;
}

void FN(rasterize_to_pixels_fwd)(
    int C, long n_isects, const REAL *means2d, const REAL *conics, const REAL *colors, int channels,
    const REAL *opacities, const REAL *pix_vels, const REAL *rs_time, const REAL *backgrounds, int W,
    int H, int tile_size, int tile_w, int tile_h, const int *offsets, const int *flatten_ids,
    REAL *render_colors, REAL *render_alphas, int *last_ids, unsigned char *ambiguous, REAL amb_tol,
    long *counters) {
    const long n_tiles_total = (long)C * tile_w * tile_h;
    long tested_total = 0, contrib_total = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : tested_total, contrib_total)
    for (long tile = 0; tile < n_tiles_total; ++tile) {
        const int cam = (int)(tile / ((long)tile_w * tile_h));
        const int t = (int)(tile % ((long)tile_w * tile_h));
        const int ty = t / tile_w, tx = t % tile_w;
        const int start = offsets[tile];
        const int end = (tile + 1 == n_tiles_total) ? (int)n_isects : offsets[tile + 1];
        for (int li = 0; li < tile_size; ++li)
            for (int lj = 0; lj < tile_size; ++lj) {
                const int i = ty * tile_size + li, j = tx * tile_size + lj;
                if (i >= H || j >= W) continue;
                const long pix = ((long)cam * H + i) * W + j;
                const REAL px = (REAL)j + (REAL)0.5, py = (REAL)i + (REAL)0.5;
                const REAL roll = rs_time[cam] * ((py - (REAL)0.5) / (REAL)(H - 1) - (REAL)0.5);
                REAL T = 1;
                int cur_idx = 0;
                unsigned char amb = 0;
                REAL *out = render_colors + pix * channels;
                for (int k = 0; k < channels; ++k) out[k] = 0;
                for (int idx = start; idx < end; ++idx) {
                    const long g = flatten_ids[idx];
                    const REAL dx = means2d[2 * g] + roll * pix_vels[2 * g] - px;
                    const REAL dy = means2d[2 * g + 1] + roll * pix_vels[2 * g + 1] - py;
                    const REAL ca = conics[3 * g], cb = conics[3 * g + 1], cc = conics[3 * g + 2];
                    const REAL sigma = (REAL)0.5 * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    const REAL raw = opacities[g] * EXP(-sigma);
                    const REAL alpha = raw < ALPHA_MAX ? raw : ALPHA_MAX;
                    ++tested_total;
                    if (FN(near)(raw, ALPHA_MIN, amb_tol)) amb = 1;
                    if (sigma < 0 || alpha < ALPHA_MIN) continue;
                    const REAL next_T = T * ((REAL)1 - alpha);
                    if (FN(near)(next_T, T_STOP, amb_tol)) amb = 1;
                    if (next_T <= T_STOP) break;
                    ++contrib_total;
                    const REAL vis = alpha * T;
                    const REAL *c = colors + g * channels;
                    for (int k = 0; k < channels; ++k) out[k] += c[k] * vis;
                    cur_idx = idx;
                    T = next_T;
                }
                render_alphas[pix] = (REAL)1 - T;
                if (backgrounds)
                    for (int k = 0; k < channels; ++k) out[k] += T * backgrounds[(long)cam * channels + k];
                last_ids[pix] = cur_idx;
                if (ambiguous) ambiguous[pix] = amb;
            }
    }
    if (counters) { counters[0] += tested_total; counters[1] += contrib_total; }
}

void FN(rasterize_to_points_fwd)(
    int C, long n_isects, const REAL *means2d, const REAL *conics, const REAL *colors, int channels,
    const REAL *opacities, const REAL *pix_vels, const REAL *depth_comps, const REAL *backgrounds,
    const REAL *raster_pts, int W, int H, int tile_width, int tile_height, int grid_w, int grid_h,
    int compute_alpha_sum, REAL alpha_sum_threshold, const int *offsets, const int *flatten_ids,
    int depth_idx, REAL *render_colors, REAL *render_alphas, REAL *alpha_sum_out, int *last_ids,
    REAL *median_depths, unsigned char *ambiguous, REAL amb_tol, long *counters) {
    const long n_tiles_total = (long)C * grid_w * grid_h;
    long tested_total = 0, contrib_total = 0;
#pragma omp parallel for schedule(dynamic, 4) reduction(+ : tested_total, contrib_total)
    for (long tile = 0; tile < n_tiles_total; ++tile) {
        const int cam = (int)(tile / ((long)grid_w * grid_h));
        const int t = (int)(tile % ((long)grid_w * grid_h));
        const int ty = t / grid_w, tx = t % grid_w;
        const int start = offsets[tile];
        const int end = (tile + 1 == n_tiles_total) ? (int)n_isects : offsets[tile + 1];
        for (int li = 0; li < tile_height; ++li)
            for (int lj = 0; lj < tile_width; ++lj) {
                const int i = ty * tile_height + li, j = tx * tile_width + lj;
                if (i >= H || j >= W) continue;
                const long pix = ((long)cam * H + i) * W + j;
                REAL *out = render_colors + pix * channels;
                for (int k = 0; k < channels; ++k) out[k] = 0;
                render_alphas[pix] = 0;
                last_ids[pix] = 0;
                median_depths[pix] = 0;
                if (alpha_sum_out) alpha_sum_out[pix] = 0;
                if (ambiguous) ambiguous[pix] = 0;
                const REAL px = raster_pts[4 * pix], py = raster_pts[4 * pix + 1];
                const REAL pz = raster_pts[4 * pix + 2], roll = raster_pts[4 * pix + 3];
                if (pz <= 0) continue;
                REAL T = 1, asum = 0, median = 0;
                int cur_idx = 0;
                unsigned char amb = 0;
                for (int idx = start; idx < end; ++idx) {
                    const long g = flatten_ids[idx];
                    const REAL dx = FN(angle_difference)(means2d[2 * g] + roll * pix_vels[3 * g], px);
                    const REAL dy = FN(angle_difference)(means2d[2 * g + 1] + roll * pix_vels[3 * g + 1], py);
                    const REAL ca = conics[3 * g], cb = conics[3 * g + 1], cc = conics[3 * g + 2];
                    const REAL sigma = (REAL)0.5 * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    const REAL raw = opacities[g] * EXP(-sigma);
                    const REAL alpha = raw < ALPHA_MAX ? raw : ALPHA_MAX;
                    ++tested_total;
                    if (FN(near)(raw, ALPHA_MIN, amb_tol)) amb = 1;
                    if (sigma < 0 || alpha < ALPHA_MIN) continue;
                    const REAL next_T = T * ((REAL)1 - alpha);
                    if (FN(near)(next_T, T_STOP, amb_tol)) amb = 1;
                    if (next_T <= T_STOP) break;
                    ++contrib_total;
                    const REAL vis = alpha * T;
                    const REAL *c = colors + g * channels;
                    for (int k = 0; k < channels; ++k) out[k] += c[k] * vis;
                    const REAL dterm = depth_comps[2 * g] * dx + depth_comps[2 * g + 1] * dy +
                                       pix_vels[3 * g + 2] * roll;
                    out[depth_idx] += dterm * vis;
                    if (FN(near)(next_T, (REAL)0.5, amb_tol) || FN(near)(T, (REAL)0.5, amb_tol)) amb = 1;
                    if (T > (REAL)0.5 && next_T <= (REAL)0.5) median = c[depth_idx] + dterm;
                    if (compute_alpha_sum) {
                        const REAL lim = pz - alpha_sum_threshold;
                        if (FN(near)(c[depth_idx], lim, amb_tol)) amb = 1;
                        if (c[depth_idx] < lim) asum += alpha;
                    }
                    cur_idx = idx;
                    T = next_T;
                }
                render_alphas[pix] = (REAL)1 - T;
                if (backgrounds)
                    for (int k = 0; k < channels; ++k) out[k] += T * backgrounds[(long)cam * channels + k];
                last_ids[pix] = cur_idx;
                median_depths[pix] = median;
                if (alpha_sum_out) alpha_sum_out[pix] = asum;
                if (ambiguous) ambiguous[pix] = amb;
            }
    }
    if (counters) { counters[0] += tested_total; counters[1] += contrib_total; }
}

static inline void FN(atomic_add)(double *p, double v) {
#pragma omp atomic
    *p += v;
}

/* Backward. Gradient outputs are double regardless of REAL (they accumulate across pixels). */
void FN(rasterize_to_pixels_bwd)(
    int C, long n_isects, const REAL *means2d, const REAL *conics, const REAL *colors, int channels,
    const REAL *opacities, const REAL *pix_vels, const REAL *rs_time, const REAL *backgrounds, int W,
    int H, int tile_size, int tile_w, int tile_h, const int *offsets, const int *flatten_ids,
    const REAL *render_alphas, const int *last_ids, const REAL *v_render_colors,
    const REAL *v_render_alphas, double *v_means2d_abs, double *v_means2d, double *v_conics,
    double *v_colors, double *v_opacities, double *v_pix_vels) {
    const long n_tiles_total = (long)C * tile_w * tile_h;
#pragma omp parallel for schedule(dynamic, 4)
    for (long tile = 0; tile < n_tiles_total; ++tile) {
        const int cam = (int)(tile / ((long)tile_w * tile_h));
        const int t = (int)(tile % ((long)tile_w * tile_h));
        const int ty = t / tile_w, tx = t % tile_w;
        const int start = offsets[tile];
        const int end = (tile + 1 == n_tiles_total) ? (int)n_isects : offsets[tile + 1];
        REAL buffer[512];
        for (int li = 0; li < tile_size; ++li)
            for (int lj = 0; lj < tile_size; ++lj) {
                const int i = ty * tile_size + li, j = tx * tile_size + lj;
                if (i >= H || j >= W) continue;
                const long pix = ((long)cam * H + i) * W + j;
                const REAL px = (REAL)j + (REAL)0.5, py = (REAL)i + (REAL)0.5;
                const REAL roll = rs_time[cam] * ((py - (REAL)0.5) / (REAL)(H - 1) - (REAL)0.5);
                const REAL T_final = (REAL)1 - render_alphas[pix];
                REAL T = T_final;
                const int bin_final = last_ids[pix];
                const REAL *v_c = v_render_colors + pix * channels;
                const REAL v_a = v_render_alphas[pix];
                for (int k = 0; k < channels; ++k) buffer[k] = 0;
                int top = bin_final < end - 1 ? bin_final : end - 1;
                for (int idx = top; idx >= start; --idx) {
                    const long g = flatten_ids[idx];
                    const REAL dx = means2d[2 * g] + roll * pix_vels[2 * g] - px;
                    const REAL dy = means2d[2 * g + 1] + roll * pix_vels[2 * g + 1] - py;
                    const REAL ca = conics[3 * g], cb = conics[3 * g + 1], cc = conics[3 * g + 2];
                    const REAL sigma = (REAL)0.5 * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    const REAL vis = EXP(-sigma);
                    const REAL opac = opacities[g];
                    const REAL raw = opac * vis;
                    const REAL alpha = raw < ALPHA_MAX ? raw : ALPHA_MAX;
                    if (sigma < 0 || alpha < ALPHA_MIN) continue;
                    const REAL ra = (REAL)1 / ((REAL)1 - alpha);
                    T *= ra;
                    const REAL fac = alpha * T;
                    const REAL *c = colors + g * channels;
                    REAL v_alpha = 0;
                    for (int k = 0; k < channels; ++k) {
                        FN(atomic_add)(v_colors + g * channels + k, (double)(fac * v_c[k]));
                        v_alpha += (c[k] * T - buffer[k] * ra) * v_c[k];
                    }
                    v_alpha += T_final * ra * v_a;
                    if (backgrounds) {
                        REAL accum = 0;
                        for (int k = 0; k < channels; ++k) accum += backgrounds[(long)cam * channels + k] * v_c[k];
                        v_alpha += -T_final * ra * accum;
                    }
                    if (raw <= ALPHA_MAX) {
                        const REAL v_sigma = -opac * vis * v_alpha;
                        FN(atomic_add)(v_conics + 3 * g, (double)((REAL)0.5 * v_sigma * dx * dx));
                        FN(atomic_add)(v_conics + 3 * g + 1, (double)(v_sigma * dx * dy));
                        FN(atomic_add)(v_conics + 3 * g + 2, (double)((REAL)0.5 * v_sigma * dy * dy));
                        const REAL vx = v_sigma * (ca * dx + cb * dy);
                        const REAL vy = v_sigma * (cb * dx + cc * dy);
                        FN(atomic_add)(v_means2d + 2 * g, (double)vx);
                        FN(atomic_add)(v_means2d + 2 * g + 1, (double)vy);
                        FN(atomic_add)(v_pix_vels + 2 * g, (double)(vx * roll));
                        FN(atomic_add)(v_pix_vels + 2 * g + 1, (double)(vy * roll));
                        if (v_means2d_abs) {
                            FN(atomic_add)(v_means2d_abs + 2 * g, (double)(vx < 0 ? -vx : vx));
                            FN(atomic_add)(v_means2d_abs + 2 * g + 1, (double)(vy < 0 ? -vy : vy));
                        }
                        FN(atomic_add)(v_opacities + g, (double)(vis * v_alpha));
                    }
                    for (int k = 0; k < channels; ++k) buffer[k] += c[k] * fac;
                }
            }
    }
}

void FN(rasterize_to_points_bwd)(
    int C, long n_isects, const REAL *means2d, const REAL *conics, const REAL *colors, int channels,
    const REAL *opacities, const REAL *pix_vels, const REAL *depth_comps, const REAL *backgrounds,
    const REAL *raster_pts, int W, int H, int tile_width, int tile_height, int grid_w, int grid_h,
    int compute_alpha_sum, REAL alpha_sum_threshold, const int *offsets, const int *flatten_ids,
    int depth_idx, const REAL *render_alphas, const int *last_ids, const REAL *v_render_colors,
    const REAL *v_render_alphas, const REAL *v_alpha_sum, double *v_means2d_abs, double *v_means2d,
    double *v_conics, double *v_colors, double *v_opacities, double *v_pix_vels,
    double *v_depth_comps) {
    const long n_tiles_total = (long)C * grid_w * grid_h;
#pragma omp parallel for schedule(dynamic, 4)
    for (long tile = 0; tile < n_tiles_total; ++tile) {
        const int cam = (int)(tile / ((long)grid_w * grid_h));
        const int t = (int)(tile % ((long)grid_w * grid_h));
        const int ty = t / grid_w, tx = t % grid_w;
        const int start = offsets[tile];
        const int end = (tile + 1 == n_tiles_total) ? (int)n_isects : offsets[tile + 1];
        REAL buffer[512];
        for (int li = 0; li < tile_height; ++li)
            for (int lj = 0; lj < tile_width; ++lj) {
                const int i = ty * tile_height + li, j = tx * tile_width + lj;
                if (i >= H || j >= W) continue;
                const long pix = ((long)cam * H + i) * W + j;
                const REAL px = raster_pts[4 * pix], py = raster_pts[4 * pix + 1];
                const REAL pz = raster_pts[4 * pix + 2], roll = raster_pts[4 * pix + 3];
                if (pz <= 0) continue;
                const REAL T_final = (REAL)1 - render_alphas[pix];
                REAL T = T_final;
                const int bin_final = last_ids[pix];
                const REAL *v_c = v_render_colors + pix * channels;
                const REAL v_a = v_render_alphas[pix];
                const REAL v_as = v_alpha_sum ? v_alpha_sum[pix] : 0;
                for (int k = 0; k < channels; ++k) buffer[k] = 0;
                int top = bin_final < end - 1 ? bin_final : end - 1;
                for (int idx = top; idx >= start; --idx) {
                    const long g = flatten_ids[idx];
                    const REAL dx = FN(angle_difference)(means2d[2 * g] + roll * pix_vels[3 * g], px);
                    const REAL dy = FN(angle_difference)(means2d[2 * g + 1] + roll * pix_vels[3 * g + 1], py);
                    const REAL ca = conics[3 * g], cb = conics[3 * g + 1], cc = conics[3 * g + 2];
                    const REAL sigma = (REAL)0.5 * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    const REAL vis = EXP(-sigma);
                    const REAL opac = opacities[g];
                    const REAL raw = opac * vis;
                    const REAL alpha = raw < ALPHA_MAX ? raw : ALPHA_MAX;
                    if (sigma < 0 || alpha < ALPHA_MIN) continue;
                    const REAL ra = (REAL)1 / ((REAL)1 - alpha);
                    T *= ra;
                    const REAL fac = alpha * T;
                    const REAL *c = colors + g * channels;
                    const REAL dcx = depth_comps[2 * g], dcy = depth_comps[2 * g + 1];
                    const REAL dterm = dcx * dx + dcy * dy + pix_vels[3 * g + 2] * roll;
                    REAL v_alpha = 0;
                    for (int k = 0; k < channels; ++k) {
                        FN(atomic_add)(v_colors + g * channels + k, (double)(fac * v_c[k]));
                        v_alpha += (c[k] * T - buffer[k] * ra) * v_c[k];
                    }
                    const REAL v_rgb_depth = fac * v_c[depth_idx];
                    v_alpha += dterm * T * v_c[depth_idx];
                    v_alpha += T_final * ra * v_a;
                    if (backgrounds) {
                        REAL accum = 0;
                        for (int k = 0; k < channels; ++k) accum += backgrounds[(long)cam * channels + k] * v_c[k];
                        v_alpha += -T_final * ra * accum;
                    }
                    REAL vx = 0, vy = 0, vax = 0, vay = 0, vvx = 0, vvy = 0, vvz = 0, vo = 0;
                    REAL vca = 0, vcb = 0, vcc = 0, vdx = 0, vdy = 0;
                    if (raw <= ALPHA_MAX) {
                        vdx = v_rgb_depth * dx;
                        vdy = v_rgb_depth * dy;
                        vvz = v_rgb_depth * roll;
                        const REAL v_sigma = -opac * vis * v_alpha;
                        vca = (REAL)0.5 * v_sigma * dx * dx;
                        vcb = v_sigma * dx * dy;
                        vcc = (REAL)0.5 * v_sigma * dy * dy;
                        vx = v_sigma * (ca * dx + cb * dy) + v_rgb_depth * dcx;
                        vy = v_sigma * (cb * dx + cc * dy) + v_rgb_depth * dcy;
                        vvx = vx * roll;
                        vvy = vy * roll;
                        vax = vx < 0 ? -vx : vx;
                        vay = vy < 0 ? -vy : vy;
                        vo = vis * v_alpha;
                    }
                    for (int k = 0; k < channels; ++k) buffer[k] += c[k] * fac;
                    buffer[depth_idx] += dterm * fac;
                    if (compute_alpha_sum && c[depth_idx] < (pz - alpha_sum_threshold)) {
                        const REAL vs = v_as * -opac * vis;
                        const REAL ux = vs * (ca * dx + cb * dy);
                        const REAL uy = vs * (cb * dx + cc * dy);
                        vx += ux; vy += uy;
                        vvx += ux * roll; vvy += uy * roll;
                        vax += ux < 0 ? -ux : ux; vay += uy < 0 ? -uy : uy;
                        vca += vs * (REAL)0.5 * dx * dx;
                        vcb += vs * dx * dy;
                        vcc += vs * (REAL)0.5 * dy * dy;
                        vo += v_as * vis;
                    }
                    FN(atomic_add)(v_conics + 3 * g, (double)vca);
                    FN(atomic_add)(v_conics + 3 * g + 1, (double)vcb);
                    FN(atomic_add)(v_conics + 3 * g + 2, (double)vcc);
                    FN(atomic_add)(v_means2d + 2 * g, (double)vx);
                    FN(atomic_add)(v_means2d + 2 * g + 1, (double)vy);
                    if (v_means2d_abs) {
                        FN(atomic_add)(v_means2d_abs + 2 * g, (double)vax);
                        FN(atomic_add)(v_means2d_abs + 2 * g + 1, (double)vay);
                    }
                    FN(atomic_add)(v_pix_vels + 3 * g, (double)vvx);
                    FN(atomic_add)(v_pix_vels + 3 * g + 1, (double)vvy);
                    FN(atomic_add)(v_pix_vels + 3 * g + 2, (double)vvz);
                    FN(atomic_add)(v_depth_comps + 2 * g, (double)vdx);
                    FN(atomic_add)(v_depth_comps + 2 * g + 1, (double)vdy);
                    FN(atomic_add)(v_opacities + g, (double)vo);
                }
            }
    }
}

/*
 * Indices of the (Gaussian, pixel) pairs that contribute within batches [range_start, range_end)
 * of every tile's list, a batch being tile_w * tile_h list entries, starting from the given
 * per-pixel transmittances. Follows gsplat/cuda/csrc/rasterization.cu:839-990 (camera) and
 * 1092-1262 (lidar). Called twice like the reference's kernel: with chunk_starts == NULL it
 * counts per pixel into chunk_cnts, otherwise it writes gaussian_ids (index % N) and pixel_ids
 * (camera * H * W + row-major pixel) at chunk_starts[pixel] + k in list order.
 */
void FN(rasterize_to_indices_in_range)(
    int lidar, long range_start, long range_end, int C, long N, long n_isects, const REAL *means2d,
    const REAL *conics, const REAL *opacities, const REAL *pix_vels, const REAL *rs_time,
    const REAL *raster_pts, int W, int H, int tile_w, int tile_h, int grid_w, int grid_h,
    const int *offsets, const int *flatten_ids, const REAL *transmittances, const long *chunk_starts,
    int *chunk_cnts, long *gaussian_ids, long *pixel_ids, unsigned char *ambiguous, REAL amb_tol) {
    const long n_tiles_total = (long)C * grid_w * grid_h;
    const long block_size = (long)tile_w * tile_h;
    const int vstride = lidar ? 3 : 2;
#pragma omp parallel for schedule(dynamic, 4)
    for (long tile = 0; tile < n_tiles_total; ++tile) {
        const int cam = (int)(tile / ((long)grid_w * grid_h));
        const int t = (int)(tile % ((long)grid_w * grid_h));
        const int ty = t / grid_w, tx = t % grid_w;
        const long start = offsets[tile];
        const long end = (tile + 1 == n_tiles_total) ? n_isects : offsets[tile + 1];
        const long num_batches = (end - start + block_size - 1) / block_size;
        if (range_start >= num_batches) continue;
        const long b_end = range_end < num_batches ? range_end : num_batches;
        const long lo = start + block_size * range_start;
        const long hi = (start + block_size * b_end) < end ? (start + block_size * b_end) : end;
        for (int li = 0; li < tile_h; ++li)
            for (int lj = 0; lj < tile_w; ++lj) {
                const int i = ty * tile_h + li, j = tx * tile_w + lj;
                if (i >= H || j >= W) continue;
                const long pix = ((long)cam * H + i) * W + j;
                REAL px, py, roll;
                if (lidar) {
                    px = raster_pts[4 * pix];
                    py = raster_pts[4 * pix + 1];
                    roll = raster_pts[4 * pix + 3];
                    if (raster_pts[4 * pix + 2] <= 0) continue;
                } else {
                    px = (REAL)j + (REAL)0.5;
                    py = (REAL)i + (REAL)0.5;
                    roll = rs_time[cam] * ((py - (REAL)0.5) / (REAL)(H - 1) - (REAL)0.5);
                }
                REAL T = transmittances[pix];
                int cnt = 0;
                unsigned char amb = 0;
                for (long idx = lo; idx < hi; ++idx) {
                    const long g = flatten_ids[idx];
                    REAL dx = means2d[2 * g] + roll * pix_vels[vstride * g];
                    REAL dy = means2d[2 * g + 1] + roll * pix_vels[vstride * g + 1];
                    if (lidar) {
                        dx = FN(angle_difference)(dx, px);
                        dy = FN(angle_difference)(dy, py);
                    } else {
                        dx -= px;
                        dy -= py;
                    }
                    const REAL ca = conics[3 * g], cb = conics[3 * g + 1], cc = conics[3 * g + 2];
                    const REAL sigma = (REAL)0.5 * (ca * dx * dx + cc * dy * dy) + cb * dx * dy;
                    const REAL raw = opacities[g] * EXP(-sigma);
                    const REAL alpha = raw < ALPHA_MAX ? raw : ALPHA_MAX;
                    if (FN(near)(raw, ALPHA_MIN, amb_tol)) amb = 1;
                    if (sigma < 0 || alpha < ALPHA_MIN) continue;
                    const REAL next_T = T * ((REAL)1 - alpha);
                    if (FN(near)(next_T, T_STOP, amb_tol)) amb = 1;
                    if (next_T <= T_STOP) break;
                    if (chunk_starts) {
                        gaussian_ids[chunk_starts[pix] + cnt] = g % N;
                        pixel_ids[chunk_starts[pix] + cnt] = pix;
                    }
                    ++cnt;
                    T = next_T;
                }
                if (!chunk_starts) chunk_cnts[pix] = cnt;
                if (ambiguous) ambiguous[pix] = amb;
            }
    }
}

#undef ALPHA_MAX
#undef ALPHA_MIN
#undef T_STOP
