/*
 * srf_oracle.cpp -- CPU oracle for the render hot path and the density-grid refresh of
 * SphericalRF.  TEST INFRASTRUCTURE: loaded only by tests, the smoke check and the
 * benchmark's CPU-baseline leg.  PARITY UNPINNED (see srf_oracle.h).
 *
 * Citations are file:line inside the reference project.  One scalar function per reference
 * function, one ray at a time, in the reference's statement order.  Where the reference
 * leans on code that is not in its tree, the oracle fixes a definition and says so:
 *
 *   [M] CUDA math library (atan2f, asinf, cosf, sinf, __expf, __logf, powf): replaced by the
 *       correctly-rounded-primitive definitions of include/srf_canon_math.h.
 *   [E] Eigen (version unpinned): dot/norm/matrix-vector products of three terms reduce as
 *       Eigen's unrolled scalar reduction does, t0 + (t1 + t2), with the additions fused into
 *       multiply-adds (what nvcc's default contraction makes of them):
 *       a*b + (c*d + e*f)  ->  fma(a,b, fma(c,d, e*f))   (srf_dot3f).
 *   [T] tiny-cuda-nn (revision unpinned): multiresolution hash encoding, spherical harmonics
 *       and the fully fused MLP are restated from the Instant-NGP paper (Mueller et al. 2022):
 *       fp16 parameters and activations, fp32 accumulation in index order, one rounding to
 *       fp16 at every layer boundary; PCG32 (O'Neill 2014) with Jakob's float conversion;
 *       the grid mean is a fixed binary-tree sum.
 *
 * Build: make -C oracle   (g++ -O2 -ffp-contract=off -fopenmp)
 */
#include "srf_oracle.h"
#include "../include/srf_canon_math.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

const double kInvPi = 0.318309886183790671537767526745028724;   /* M_1_PI */
const double kPi    = 3.14159265358979323846;                   /* M_PI   */

struct V3 { float x, y, z; };
struct Box { V3 mn, mx; };

inline V3 v3(float x, float y, float z) { V3 r = {x, y, z}; return r; }

/* ---- fp16 ------------------------------------------------------------------------------- */
inline float h2f(uint16_t h) { _Float16 v; memcpy(&v, &h, 2); return (float)v; }
inline uint16_t f2h(float f) { _Float16 v = (_Float16)f; uint16_t h; memcpy(&h, &v, 2); return h; }

/* ---- resolved configuration --------------------------------------------------------------- */
struct Cfg {
    srf_config_t c;
    Box box;
    float min_step, max_step;
    uint32_t cells;       /* grid_size^3 */
    float per_level_scale;
};

/* internal/sampler/occupancy_sampler.cu:909-944 */
Cfg resolve(const srf_config_t* in) {
    Cfg r;
    r.c = *in;
    const float amount = 0.5f * (float)in->aabb_scale;               /* :915 */
    r.box.mn = v3(0.5f - amount, 0.5f - amount, 0.5f - amount);
    r.box.mx = v3(0.5f + amount, 0.5f + amount, 0.5f + amount);
    const float sqrt3 = 1.73205080757f;                              /* :10 */
    r.min_step = in->min_cone_stepsize > 0.f ? in->min_cone_stepsize
                                             : sqrt3 / (float)in->maximum_marching_steps;   /* :936 */
    r.max_step = in->max_cone_stepsize > 0.f ? in->max_cone_stepsize
               : (in->use_grid ? (sqrt3 * (float)(1u << (in->num_cascades - 1)) / (float)in->grid_size)
                               : r.min_step);                        /* :937 */
    r.cells = in->grid_size * in->grid_size * in->grid_size;
    float pls = in->per_level_scale;
    if (pls <= 0.f && in->n_levels > 1) {                            /* ngp_network.h:620-625 */
        pls = std::exp(std::log(in->desired_resolution / (float)in->base_resolution) / (float)(in->n_levels - 1));
    }
    r.per_level_scale = pls;
    return r;
}

/* ---- Morton code (tiny-cuda-nn morton3D: x -> bit 0, y -> bit 1, z -> bit 2) [T] ---------- */
inline uint32_t expand_bits(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}
inline uint32_t morton3D(uint32_t x, uint32_t y, uint32_t z) {
    return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2);
}
inline uint32_t morton3D_invert(uint32_t x) {
    x = x & 0x49249249u;
    x = (x | (x >> 2)) & 0xc30c30c3u;
    x = (x | (x >> 4)) & 0x0f00f00fu;
    x = (x | (x >> 8)) & 0xff0000ffu;
    x = (x | (x >> 16)) & 0x0000ffffu;
    return x;
}

/* ---- low-discrepancy sequence: internal/utils/random_val.cuh:137-273 ---------------------- */
/* Sobol direction numbers of dimensions 0 and 1 (the only ones the render path draws):
   dimension 0 is the bit-reversal sequence, dimension 1 follows v[k] = v[k-1] ^ (v[k-1] >> 1). */
inline uint32_t sobol(uint32_t index, uint32_t dim) {                /* :137-194 */
    uint32_t X = 0, v = 0x80000000u;
    for (uint32_t bit = 0; bit < 32; ++bit) {
        if ((index >> bit) & 1u) X ^= v;
        v = dim == 0 ? (v >> 1) : (v ^ (v >> 1));
    }
    return X;
}
inline uint32_t hash_combine(uint32_t seed, uint32_t v) { return seed ^ (v + (seed << 6) + (seed >> 2)); }   /* :204 */
inline uint32_t reverse_bits(uint32_t x) {                           /* :208-214 */
    x = (((x & 0xaaaaaaaau) >> 1) | ((x & 0x55555555u) << 1));
    x = (((x & 0xccccccccu) >> 2) | ((x & 0x33333333u) << 2));
    x = (((x & 0xf0f0f0f0u) >> 4) | ((x & 0x0f0f0f0fu) << 4));
    x = (((x & 0xff00ff00u) >> 8) | ((x & 0x00ff00ffu) << 8));
    return ((x >> 16) | (x << 16));
}
inline uint32_t laine_karras_permutation(uint32_t x, uint32_t seed) {   /* :216-223 */
    x += seed;
    x ^= x * 0x6c50b47cu;
    x ^= x * 0xb82f1e52u;
    x ^= x * 0xc7afe638u;
    x ^= x * 0x8d22f6e6u;
    return x;
}
inline uint32_t nested_uniform_scramble_base2(uint32_t x, uint32_t seed) {   /* :225-230 */
    return reverse_bits(laine_karras_permutation(reverse_bits(x), seed));
}
const float kS32 = 2.3283064365386963e-10f;                          /* float(1.0/(1ull<<32)) */
inline float ld_random_val(uint32_t index, uint32_t seed, uint32_t dim) {   /* :262-266 */
    index = nested_uniform_scramble_base2(index, seed);
    return (float)nested_uniform_scramble_base2(sobol(index, dim), hash_combine(seed, dim)) * kS32;
}
inline void ld_random_val_2d(uint32_t index, uint32_t seed, float* a, float* b) {   /* :256-260, :241-248 */
    index = nested_uniform_scramble_base2(index, seed);
    *a = (float)nested_uniform_scramble_base2(sobol(index, 0), hash_combine(seed, 0)) * kS32;
    *b = (float)nested_uniform_scramble_base2(sobol(index, 1), hash_combine(seed, 1)) * kS32;
}
inline float fractf(float x) { return x - floorf(x); }              /* :54 */
inline void ld_random_pixel_offset(uint32_t spp, float* ox, float* oy) {   /* :268-273 */
    float a0, b0, a1, b1;
    ld_random_val_2d(0, 0xdeadbeefu, &a0, &b0);
    ld_random_val_2d(spp, 0xdeadbeefu, &a1, &b1);
    *ox = fractf((0.5f - a0) + a1);
    *oy = fractf((0.5f - b0) + b1);
}

/* ---- bounding box: internal/sampler/bounding_box.h:145-191 -------------------------------- */
inline bool box_contains(const Box& b, const V3& p) {                /* :185-190 */
    return p.x >= b.mn.x && p.x <= b.mx.x && p.y >= b.mn.y && p.y <= b.mx.y && p.z >= b.mn.z && p.z <= b.mx.z;
}
inline float box_ray_tmin(const Box& b, const V3& pos, const V3& dir) {   /* :145-179, .x() of the result */
    float tmin = (b.mn.x - pos.x) / dir.x;
    float tmax = (b.mx.x - pos.x) / dir.x;
    if (tmin > tmax) std::swap(tmin, tmax);
    float tymin = (b.mn.y - pos.y) / dir.y;
    float tymax = (b.mx.y - pos.y) / dir.y;
    if (tymin > tymax) std::swap(tymin, tymax);
    if ((tmin > tymax) || (tymin > tmax)) return 100000.0f;
    if (tymin > tmin) tmin = tymin;
    if (tymax < tmax) tmax = tymax;
    float tzmin = (b.mn.z - pos.z) / dir.z;
    float tzmax = (b.mx.z - pos.z) / dir.z;
    if (tzmin > tzmax) std::swap(tzmin, tzmax);
    if ((tmin > tzmax) || (tzmin > tmax)) return 100000.0f;
    if (tzmin > tmin) tmin = tzmin;
    return tmin;
}

/* ---- camera: internal/utils/common_device.h:143-165 --------------------------------------- */
inline void pixel_to_ray(const srf_view_t& v, bool snap, uint32_t px, uint32_t py, V3* o, V3* d) {
    float ox, oy;
    ld_random_pixel_offset(snap ? 0u : v.spp_index, &ox, &oy);       /* :152 */
    const float rw = (float)v.width, rh = (float)v.height;
    const float xx = ((float)px + ox) / rw;                          /* :153 */
    const float yy = ((float)py + oy) / rh;
    const float fx = rw * v.relative_focal_length[0];                /* testbed.cu:483 */
    const float fy = rh * v.relative_focal_length[1];
    const float dx = (xx - v.principal_point[0]) * rw / fx;          /* :157 */
    const float dy = (yy - v.principal_point[1]) * rh / fy;          /* :158 */
    const float dz = 1.0f;
    const float* m = v.camera;                                       /* row-major 3x4 */
    *o = v3(m[3], m[7], m[11]);                                      /* :155 */
    const float rx = srf_dot3f(m[0], dx, m[1], dy, m[2], dz);        /* :161 [E] */
    const float ry = srf_dot3f(m[4], dx, m[5], dy, m[6], dz);
    const float rz = srf_dot3f(m[8], dx, m[9], dy, m[10], dz);
    const float n = srf_norm3f(rx, ry, rz);                          /* :162 [E] */
    *d = v3(rx / n, ry / n, rz / n);
}

/* ---- step size: internal/sampler/occupancy_sampler.cu:287-331 ----------------------------- */
inline float clampf(float v, float lo, float hi) { return fminf(fmaxf(v, lo), hi); }
inline float calc_dt(const Cfg& g, float t) {
    float dt = 0.f;
    const float ds = 1.f / (float)g.c.maximum_marching_steps;        /* :299 */
    switch (g.c.sampling_type) {
    case SRF_SAMPLING_ORIGINAL:
        dt = clampf(t * g.c.cone_angle_constant, g.min_step, g.max_step);   /* :304 */
        break;
    case SRF_SAMPLING_DISPARITY: {
        const float g_tfar = 1.f / g.c.far_distance, g_tnear = 1.f / g.c.near_distance, g_t0 = 1.f / t;   /* :309 */
        const float g_t1 = fmaf(ds, g_tfar - g_tnear, g_t0);         /* :310 */
        const float t1 = 1.f / g_t1;
        dt = t1 - t;
        if (dt < 0.f) dt = t >= g.c.far_distance ? 0.f : g.c.far_distance - t;   /* :313-315 */
    } break;
    case SRF_SAMPLING_LOG: {
        const float g_tfar = srf_logf(g.c.far_distance), g_tnear = srf_logf(g.c.near_distance), g_t0 = srf_logf(t);   /* :320 [M] */
        const float g_t1 = fmaf(ds, g_tfar - g_tnear, g_t0);
        float t1 = srf_expf(g_t1);
        t1 = t1 < g.c.far_distance ? t1 : g.c.far_distance;
        dt = t1 - t;
    } break;
    default: break;
    }
    return dt;
}

/* ---- warps: internal/utils/common_device.h:375-526 ---------------------------------------- */
inline V3 box_diag(const Box& b) { return v3(b.mx.x - b.mn.x, b.mx.y - b.mn.y, b.mx.z - b.mn.z); }

V3 warp_position(const Cfg& g, const V3& pos) {
    V3 z = v3(0.f, 0.f, 0.f);
    switch (g.c.warping_type) {
    case SRF_WARP_NGP: {                                             /* :380-384 */
        const V3 dg = box_diag(g.box);
        z = v3((pos.x - g.box.mn.x) / dg.x, (pos.y - g.box.mn.y) / dg.y, (pos.z - g.box.mn.z) / dg.z);
    } break;
    case SRF_WARP_MIPNERF360: {                                      /* :385-395 */
        const V3 x = v3((pos.x - 0.5f) * 2.f, (pos.y - 0.5f) * 2.f, (pos.z - 0.5f) * 2.f);
        const float mag = srf_norm3f(x.x, x.y, x.z);
        const float inv = 1.f / mag;
        if (mag <= 1.f) z = x;
        else { const float s = (2.f - inv) * inv; z = v3(s * x.x, s * x.y, s * x.z); }
        z = v3(fmaf(z.x, 0.25f, 0.5f), fmaf(z.y, 0.25f, 0.5f), fmaf(z.z, 0.25f, 0.5f));
    } break;
    case SRF_WARP_DONERF: {                                          /* :396-406 */
        const V3 dg = box_diag(g.box);
        const float dmax = srf_norm3f(dg.x, dg.y, dg.z);
        const V3 x = v3(pos.x - 0.5f, pos.y - 0.5f, pos.z - 0.5f);
        const float mag = srf_norm3f(x.x, x.y, x.z);
        if (mag == 0.f) z = x;
        else { const float q = sqrtf(mag * dmax); z = v3(x.x / q, x.y / q, x.z / q); }
        z = v3(fmaf(z.x, 0.5f, 0.5f), fmaf(z.y, 0.5f, 0.5f), fmaf(z.z, 0.5f, 0.5f));
    } break;
    case SRF_WARP_SIGMOID:                                           /* :407-411 [M] */
        z = v3(srf_logisticf(pos.x - 0.5f), srf_logisticf(pos.y - 0.5f), srf_logisticf(pos.z - 0.5f));
        break;
    case SRF_WARP_ERP:            /* :412-431 has no break: its result is overwritten by the next case */
    case SRF_WARP_SINUSOIDAL: {                                      /* :432-447 */
        const V3 p = v3(pos.x - 0.5f, pos.y - 0.5f, pos.z - 0.5f);
        float p_mag = srf_norm3f(p.x, p.y, p.z);
        const float p_mag_inv = 1.f / p_mag;
        const float theta = srf_atan2f(p.y, p.x);                    /* [M] */
        const float phi = srf_asinf(p.z * p_mag_inv);                /* [M] */
        p_mag = (p_mag <= 1.f) ? p_mag : (2.f - p_mag_inv);
        p_mag *= 0.5f;
        /* M_1_PI is a double: these two expressions are evaluated in fp64 (:443-444) */
        const double tx = (double)(theta * srf_cosf(phi)) * kInvPi;
        z.x = (float)fma(tx, 0.5, 0.5);
        z.y = (float)fma((double)phi, kInvPi, 0.5);
        z.z = p_mag;
    } break;
    default: break;
    }
    return z;
}

V3 unwarp_position(const Cfg& g, const V3& pos) {
    V3 x = v3(0.f, 0.f, 0.f);
    switch (g.c.warping_type) {
    case SRF_WARP_NGP: {                                             /* :460-464 */
        const V3 dg = box_diag(g.box);
        x = v3(fmaf(pos.x, dg.x, g.box.mn.x), fmaf(pos.y, dg.y, g.box.mn.y), fmaf(pos.z, dg.z, g.box.mn.z));
    } break;
    case SRF_WARP_MIPNERF360: {                                      /* :465-476 */
        const V3 z = v3((pos.x - 0.5f) * 4.f, (pos.y - 0.5f) * 4.f, (pos.z - 0.5f) * 4.f);
        const float mag = srf_norm3f(z.x, z.y, z.z);
        const float inv = 1.f / mag;
        if (mag <= 1.f) x = z;
        else { const float s = 1.f / (2.f - mag) * inv; x = v3(s * z.x, s * z.y, s * z.z); }
        x = v3(fmaf(x.x, 0.5f, 0.5f), fmaf(x.y, 0.5f, 0.5f), fmaf(x.z, 0.5f, 0.5f));
    } break;
    case SRF_WARP_DONERF: {                                          /* :477-488 */
        const V3 dg = box_diag(g.box);
        const float dmax = srf_norm3f(dg.x, dg.y, dg.z);
        const V3 z = v3((pos.x - 0.5f) * 2.f, (pos.y - 0.5f) * 2.f, (pos.z - 0.5f) * 2.f);
        const float mag = srf_norm3f(z.x, z.y, z.z);
        x = v3(z.x * mag * dmax + 0.5f, z.y * mag * dmax + 0.5f, z.z * mag * dmax + 0.5f);
    } break;
    case SRF_WARP_SIGMOID: {                                         /* :489-493, logit(x) = -log(1/x - 1) [M] */
        x = v3(-srf_logf(1.f / pos.x - 1.f) + 0.5f, -srf_logf(1.f / pos.y - 1.f) + 0.5f,
               -srf_logf(1.f / pos.z - 1.f) + 0.5f);
    } break;
    case SRF_WARP_ERP:            /* :494-507 falls through as well */
    case SRF_WARP_SINUSOIDAL: {                                      /* :508-520 */
        const float phi = (float)((double)(pos.y - 0.5f) * kPi);     /* :510, fp64 */
        float sphi, cphi;
        srf_sincosf(phi, &sphi, &cphi);
        const float theta = (float)((double)((pos.x - 0.5f) * 2.f) * kPi / (double)cphi);   /* :511, fp64 */
        float p_mag = pos.z * 2.f;
        p_mag = (p_mag <= 1.f) ? p_mag : 1.f / (2.f - p_mag);
        float sth, cth;
        srf_sincosf(theta, &sth, &cth);
        x = v3(p_mag * cphi * cth + 0.5f, p_mag * cphi * sth + 0.5f, p_mag * sphi + 0.5f);
    } break;
    default: break;
    }
    return x;
}

/* ---- occupancy lookup: internal/sampler/occupancy_sampler.cu:349-469 ---------------------- */
uint32_t level_from_pos(const Cfg& g, const V3& pos, const V3& w) {   /* :349-398 */
    const uint32_t nc = g.c.num_cascades;
    float maxval = 0.f;
    switch (g.c.grid_distribution_type) {
    case SRF_GRID_WARPED_EXP: case SRF_GRID_WARPED_RECIPROCAL:
        maxval = fmaxf(fmaxf(fabsf(w.x - 0.5f), fabsf(w.y - 0.5f)), fabsf(w.z - 0.5f));
        break;
    default: {
        const V3 dg = box_diag(g.box);
        maxval = fmaxf(fmaxf(fabsf((pos.x - 0.5f) / dg.x), fabsf((pos.y - 0.5f) / dg.y)), fabsf((pos.z - 0.5f) / dg.z));
    } break;
    }
    maxval *= 2.f;
    uint32_t mip = 0;
    for (; mip + 1 < nc; ++mip) {
        bool got;
        if (g.c.grid_distribution_type == SRF_GRID_WARPED_EXP || g.c.grid_distribution_type == SRF_GRID_METRIC_EXP)
            got = maxval > scalbnf(1.f, -1 - (int)mip);
        else
            got = maxval > 1.f / (float)(mip + 2);
        if (got) break;
    }
    return nc - mip - 1;
}

uint32_t cascaded_grid_idx_at(const Cfg& g, const V3& pos, const V3& w, uint32_t level) {   /* :404-455 */
    const uint32_t nc = g.c.num_cascades, N = g.c.grid_size;
    V3 p = v3(0.f, 0.f, 0.f);
    float s;
    switch (g.c.grid_distribution_type) {
    case SRF_GRID_WARPED_EXP:
        s = scalbnf(1.0f, (int)(nc - level - 1));
        p = v3((w.x - 0.5f) * s + 0.5f, (w.y - 0.5f) * s + 0.5f, (w.z - 0.5f) * s + 0.5f);
        break;
    case SRF_GRID_WARPED_RECIPROCAL:
        s = (float)(nc - level);
        p = v3((w.x - 0.5f) * s + 0.5f, (w.y - 0.5f) * s + 0.5f, (w.z - 0.5f) * s + 0.5f);
        break;
    case SRF_GRID_METRIC_EXP: {
        const V3 dg = box_diag(g.box);
        s = scalbnf(1.0f, (int)(nc - level - 1));
        p = v3((pos.x - 0.5f) / dg.x * s + 0.5f, (pos.y - 0.5f) / dg.y * s + 0.5f, (pos.z - 0.5f) / dg.z * s + 0.5f);
    } break;
    case SRF_GRID_METRIC_RECIPROCAL: {
        const V3 dg = box_diag(g.box);
        s = (float)(nc - level);
        p = v3((pos.x - 0.5f) / dg.x * s + 0.5f, (pos.y - 0.5f) / dg.y * s + 0.5f, (pos.z - 0.5f) / dg.z * s + 0.5f);
    } break;
    default: break;
    }
    const float fn = (float)N;
    const int ix = srf_f2i_rz(p.x * fn), iy = srf_f2i_rz(p.y * fn), iz = srf_f2i_rz(p.z * fn);   /* :442 */
    const int hi = (int)N - 1;
    return morton3D((uint32_t)std::min(std::max(ix, 0), hi), (uint32_t)std::min(std::max(iy, 0), hi),
                    (uint32_t)std::min(std::max(iz, 0), hi));       /* :448-452 */
}

inline bool occupied_at(const Cfg& g, const uint8_t* bits, uint32_t idx, uint32_t level) {   /* :467-468 */
    return bits[idx / 8 + (g.cells * level) / 8] & (1u << (idx % 8));
}

/* ---- shard geometry ------------------------------------------------------------------------ */
uint64_t shard_rows_total(const srf_view_t& v) {
    const uint32_t sr = v.shard_rows ? v.shard_rows : 8, sc = v.shard_count ? v.shard_count : 1;
    const uint32_t n_blocks = (v.height + sr - 1) / sr;
    uint64_t rows = 0;
    for (uint32_t b = v.shard_rank; b < n_blocks; b += sc) rows += std::min(sr, v.height - b * sr);
    return rows;
}
inline uint32_t shard_ray_pixel(const srf_view_t& v, uint64_t i) {
    const uint32_t sr = v.shard_rows ? v.shard_rows : 8, sc = v.shard_count ? v.shard_count : 1;
    const uint64_t lr = i / v.width;
    const uint32_t x = (uint32_t)(i % v.width);
    const uint32_t b = v.shard_rank + (uint32_t)(lr / sr) * sc;
    const uint32_t y = b * sr + (uint32_t)(lr % sr);
    return x + v.width * y;
}

/* ---- one ray ----------------------------------------------------------------------------------- */
enum { END_EXIT = 0, END_DT0 = 1, END_STUCK = 2, END_LIMIT = 3, END_BORN_DEAD = 4, END_CAP = 5 };

struct Sample { V3 w; float dt; uint32_t ordinal, cell; float t; };

struct RayInit { bool alive; V3 o, d; float t; };

/* init_rays_with_payload_kernel_nerf (occupancy_sampler.cu:691-736) followed by the jitter of
   advance_pos_nerf (:766-768). */
RayInit init_ray(const Cfg& g, const srf_view_t& v, uint32_t pixel) {
    RayInit r;
    const uint32_t px = pixel % v.width, py = pixel / v.width;
    pixel_to_ray(v, g.c.snap_to_pixel_centers_in_rendering != 0, px, py, &r.o, &r.d);
    const float t = fmaxf(box_ray_tmin(g.box, r.o, r.d), 0.05f) + 1e-6f;   /* :721 */
    const V3 p = v3(fmaf(r.d.x, t, r.o.x), fmaf(r.d.y, t, r.o.y), fmaf(r.d.z, t, r.o.z));   /* :723 [E] */
    r.alive = box_contains(g.box, p);
    r.t = t;
    if (r.alive) {
        const float dt = calc_dt(g, t);                              /* :767 */
        r.t = fmaf(ld_random_val(v.spp_index, pixel * 786433u, 0), dt, t);   /* :768 */
    }
    return r;
}

/*
 * The march of one ray: the loop shared by advance_pos_nerf (:771-794) and
 * generate_coords_from_rays_regularly_kernel (:829-860), run to the end of the ray.
 * `emit` is called for every occupied step and returns false to stop the ray (early
 * termination by the compositor).  Returns the reason the ray ended; *steps counts loop
 * iterations.  The reference bounds nothing here (its host loop stops after MARCH_ITER
 * samples); `max_samples` restates that bound per ray and `hard_limit` guards the loop.
 */
template <class Emit>
int march_ray(const Cfg& g, const uint8_t* bits, const RayInit& r, uint32_t max_samples, uint64_t* steps, Emit emit) {
    float t = r.t;
    uint32_t ordinal = 0, n = 0;
    const uint32_t hard_limit = 1u << 24;
    for (;; ++ordinal) {
        if (ordinal >= hard_limit) { *steps += ordinal; return END_LIMIT; }
        const V3 pos = v3(fmaf(r.d.x, t, r.o.x), fmaf(r.d.y, t, r.o.y), fmaf(r.d.z, t, r.o.z));   /* :772,834 */
        if (!box_contains(g.box, pos)) { *steps += ordinal + 1; return END_EXIT; }
        const float dt = calc_dt(g, t);                              /* :785,847 */
        const V3 w = warp_position(g, pos);                          /* :786,848 */
        bool occ = true;
        uint32_t idx = 0;
        if (g.c.use_grid) {
            const uint32_t level = level_from_pos(g, pos, w);        /* :787,849 */
            idx = cascaded_grid_idx_at(g, pos, w, level);
            occ = occupied_at(g, bits, idx, level);                  /* :788,850 */
            idx += level * g.cells;
        }
        if (occ) {
            if (dt == 0.f) { *steps += ordinal + 1; return END_STUCK; }   /* zero-width samples forever: see header */
            if (n >= max_samples) { *steps += ordinal + 1; return END_CAP; }
            Sample s = { w, dt, ordinal, idx, t };
            ++n;
            if (!emit(s)) { *steps += ordinal + 1; return -1; }
            t += dt;                                                 /* :859 */
        } else {
            t += dt;                                                 /* :789,851 */
            if (dt == 0.f) { *steps += ordinal + 1; return END_DT0; }   /* :790-793,852-855 */
        }
    }
}

inline uint32_t sample_cap(const Cfg& g) {
    /* Testbed::render_frame stops after MARCH_ITER-1 samples of a ray (testbed.cu:520-523,582). */
    uint32_t cap = g.c.march_iter ? g.c.march_iter - 1 : 9999u;
    if (g.c.max_samples_per_ray && g.c.max_samples_per_ray < cap) cap = g.c.max_samples_per_ray;
    return cap;
}

/* ---- network [T] ------------------------------------------------------------------------------- */
struct GridLayout { std::vector<uint32_t> offsets, res; std::vector<float> scale; };

GridLayout grid_layout(const Cfg& g) {
    GridLayout L;
    const uint32_t nl = g.c.n_levels;
    L.offsets.resize(nl + 1); L.res.resize(nl); L.scale.resize(nl);
    uint32_t off = 0;
    const uint64_t T = 1ull << g.c.log2_hashmap_size;
    for (uint32_t l = 0; l < nl; ++l) {
        const double s = (double)g.c.base_resolution * std::pow((double)g.per_level_scale, (double)l) - 1.0;
        const float sf = (float)s;
        const uint32_t res = (uint32_t)std::ceil(sf) + 1u;
        uint64_t n = (uint64_t)res * res * res;
        n = (n + 7ull) / 8ull * 8ull;
        if (n > T) n = T;
        L.offsets[l] = off; L.res[l] = res; L.scale[l] = sf;
        off += (uint32_t)n;
    }
    L.offsets[nl] = off;
    return L;
}

inline uint32_t grid_index(uint32_t gx, uint32_t gy, uint32_t gz, uint32_t res, uint32_t size) {
    const uint64_t dense = (uint64_t)res * res * res;
    uint32_t idx;
    if (dense <= size) idx = gx + gy * res + gz * res * res;
    else idx = (gx * 1u) ^ (gy * 2654435761u) ^ (gz * 805459861u);
    return idx % size;
}

void hash_encode(const Cfg& g, const GridLayout& L, const uint16_t* table, const float* x3, uint16_t* out32) {
    const uint32_t F = g.c.n_features_per_level;
    for (uint32_t l = 0; l < g.c.n_levels; ++l) {
        const float sc = L.scale[l];
        const uint32_t res = L.res[l], size = L.offsets[l + 1] - L.offsets[l];
        float w[3]; uint32_t ig[3];
        for (int d = 0; d < 3; ++d) {
            const float p = fmaf(sc, x3[d], 0.5f);
            const float fl = floorf(p);
            w[d] = p - fl;
            ig[d] = (uint32_t)srf_f2i_rz(fl);
        }
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t c = 0; c < 8; ++c) {
            float wt = 1.f; uint32_t gp[3];
            for (int d = 0; d < 3; ++d) {
                if ((c >> d) & 1u) { wt *= w[d]; gp[d] = ig[d] + 1u; }
                else { wt *= 1.f - w[d]; gp[d] = ig[d]; }
            }
            const uint32_t idx = grid_index(gp[0], gp[1], gp[2], res, size);
            const uint16_t* e = table + (size_t)(L.offsets[l] + idx) * F;
            for (uint32_t f = 0; f < F; ++f) acc[f] = fmaf(wt, h2f(e[f]), acc[f]);
        }
        for (uint32_t f = 0; f < F; ++f) out32[l * F + f] = f2h(acc[f]);
    }
}

/* Real spherical harmonics up to degree 3 (16 values) of the direction 2*d - 1. */
void sh_encode(const float* dir3, uint16_t* out16) {
    const float x = fmaf(dir3[0], 2.f, -1.f), y = fmaf(dir3[1], 2.f, -1.f), z = fmaf(dir3[2], 2.f, -1.f);
    const float xy = x * y, xz = x * z, yz = y * z, x2 = x * x, y2 = y * y, z2 = z * z;
    float o[16];
    o[0] = 0.28209479177387814f;
    o[1] = -0.48860251190291987f * y;
    o[2] = 0.48860251190291987f * z;
    o[3] = -0.48860251190291987f * x;
    o[4] = 1.0925484305920792f * xy;
    o[5] = -1.0925484305920792f * yz;
    o[6] = fmaf(0.94617469575755997f, z2, -0.31539156525251999f);
    o[7] = -1.0925484305920792f * xz;
    o[8] = 0.54627421529603959f * x2 - 0.54627421529603959f * y2;
    o[9] = 0.59004358992664352f * y * (fmaf(-3.f, x2, y2));
    o[10] = 2.8906114426405538f * xy * z;
    o[11] = 0.45704579946446572f * y * (fmaf(-5.f, z2, 1.f));
    o[12] = 0.3731763325901154f * z * (fmaf(5.f, z2, -3.f));
    o[13] = 0.45704579946446572f * x * (fmaf(-5.f, z2, 1.f));
    o[14] = 1.4453057213202769f * z * (x2 - y2);
    o[15] = 0.59004358992664352f * x * (fmaf(3.f, y2, -x2));
    for (int i = 0; i < 16; ++i) out16[i] = f2h(o[i]);
}

/* out[o] = act(sum_k W[o][k] * in[k]), fp32 accumulation in k order, rounded to fp16. */
void dense_layer(const float* W, uint32_t n_out, uint32_t n_in, const uint16_t* in, uint16_t* out, bool relu) {
    float x[64];
    for (uint32_t k = 0; k < n_in; ++k) x[k] = h2f(in[k]);
    for (uint32_t o = 0; o < n_out; ++o) {
        float acc = 0.f;
        for (uint32_t k = 0; k < n_in; ++k) acc = fmaf(W[o * n_in + k], x[k], acc);
        if (relu && !(acc > 0.f)) acc = 0.f;
        out[o] = f2h(acc);
    }
}

/* The fp16 MLP weights converted to float once (exact), so that the inner loops stay simple. */
struct Weights {
    std::vector<float> d, c;
    explicit Weights(const srfo_model_t& m) {
        if (m.density_mlp) { d.resize(64 * 32 + 16 * 64); for (size_t i = 0; i < d.size(); ++i) d[i] = h2f(m.density_mlp[i]); }
        if (m.rgb_mlp) { c.resize(64 * 32 + 64 * 64 + 16 * 64); for (size_t i = 0; i < c.size(); ++i) c[i] = h2f(m.rgb_mlp[i]); }
    }
};

void density_net(const Cfg& g, const GridLayout& L, const srfo_model_t& m, const Weights& W, const float* x3, uint16_t* out16) {
    uint16_t enc[32], h[64];
    hash_encode(g, L, m.hash_table, x3, enc);
    dense_layer(W.d.data(), 64, 32, enc, h, true);
    dense_layer(W.d.data() + 64 * 32, 16, 64, h, out16, false);
}

/* Density output 0 and its gradient with respect to the (warped) position: what
   NGPNetwork::input_gradient(stream, 3, coords, coords) leaves in the position rows for the Normals render
   mode (testbed.cu:557-559).  [T] The reference's dependency runs this backward pass in fp16 with a loss
   scale; the canonical definition here is fp32 throughout:
     d enc[l,f] / d x_d = scale_l * sum over the 4 corner pairs along d of (w_a' * w_b') * (v_hi - v_lo),
       pairs ordered by the other two axes a < b, a's bit first;
     g_h[j] = W2[0][j] where the (fp16, ReLU) hidden unit j is positive, else 0;
     g_enc[k] = sum_j W1[j][k] * g_h[j] (j ascending, fused multiply-add);
     grad[d]  = sum_k g_enc[k] * d enc[k] / d x_d (k ascending, fused multiply-add). */
void density_with_gradient(const Cfg& g, const GridLayout& L, const srfo_model_t& m, const Weights& W, const float* x3,
                           uint16_t* sigma_out, float* grad3) {
    const uint32_t F = g.c.n_features_per_level;
    uint16_t enc[32], h[64], out16[16];
    float dydx[32][3];
    for (uint32_t l = 0; l < g.c.n_levels; ++l) {
        const float sc = L.scale[l];
        const uint32_t res = L.res[l], size = L.offsets[l + 1] - L.offsets[l];
        float w[3]; uint32_t ig[3];
        for (int d = 0; d < 3; ++d) {
            const float p = fmaf(sc, x3[d], 0.5f);
            const float fl = floorf(p);
            w[d] = p - fl;
            ig[d] = (uint32_t)srf_f2i_rz(fl);
        }
        float v[8][8];
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (uint32_t c = 0; c < 8; ++c) {
            float wt = 1.f; uint32_t gp[3];
            for (int d = 0; d < 3; ++d) {
                if ((c >> d) & 1u) { wt *= w[d]; gp[d] = ig[d] + 1u; }
                else { wt *= 1.f - w[d]; gp[d] = ig[d]; }
            }
            const uint16_t* e = m.hash_table + (size_t)(L.offsets[l] + grid_index(gp[0], gp[1], gp[2], res, size)) * F;
            for (uint32_t f = 0; f < F; ++f) { v[c][f] = h2f(e[f]); acc[f] = fmaf(wt, v[c][f], acc[f]); }
        }
        for (uint32_t f = 0; f < F; ++f) enc[l * F + f] = f2h(acc[f]);
        for (int d = 0; d < 3; ++d) {
            const int a = d == 0 ? 1 : 0, b = d == 2 ? 1 : 2;
            for (uint32_t f = 0; f < F; ++f) {
                float gs = 0.f;
                for (uint32_t c2 = 0; c2 < 4; ++c2) {
                    const uint32_t ba = c2 & 1u, bb = c2 >> 1;
                    const float wt = (ba ? w[a] : 1.f - w[a]) * (bb ? w[b] : 1.f - w[b]);
                    const uint32_t lo = (ba << a) | (bb << b), hi = lo | (1u << d);
                    gs = fmaf(wt, v[hi][f] - v[lo][f], gs);
                }
                dydx[l * F + f][d] = sc * gs;
            }
        }
    }
    dense_layer(W.d.data(), 64, 32, enc, h, true);
    dense_layer(W.d.data() + 64 * 32, 16, 64, h, out16, false);
    *sigma_out = out16[0];
    float g_enc[32];
    for (int k = 0; k < 32; ++k) {
        float acc = 0.f;
        for (int j = 0; j < 64; ++j) {
            const float gh = h2f(h[j]) > 0.f ? W.d[64 * 32 + j] : 0.f;
            acc = fmaf(W.d[j * 32 + k], gh, acc);
        }
        g_enc[k] = acc;
    }
    for (int d = 0; d < 3; ++d) {
        float acc = 0.f;
        for (int k = 0; k < 32; ++k) acc = fmaf(g_enc[k], dydx[k][d], acc);
        grad3[d] = acc;
    }
}

/* NGPNetwork::inference_mixed_precision (ngp_network.h:212-279): (r,g,b) from the colour MLP,
   sigma = density output 0. */
void network_eval(const Cfg& g, const GridLayout& L, const srfo_model_t& m, const Weights& W, const float* pos3, const float* dir3, uint16_t* rgbs4) {
    uint16_t in[32], h1[64], h2[64], o[16];
    density_net(g, L, m, W, pos3, in);                                  /* rows 0..15 (:256-262) */
    sh_encode(dir3, in + 16);                                        /* rows 16..31 (:245) */
    dense_layer(W.c.data(), 64, 32, in, h1, true);
    dense_layer(W.c.data() + 64 * 32, 64, 64, h1, h2, true);
    dense_layer(W.c.data() + 64 * 32 + 64 * 64, 16, 64, h2, o, false);
    rgbs4[0] = o[0]; rgbs4[1] = o[1]; rgbs4[2] = o[2]; rgbs4[3] = in[0];   /* :63-78 */
}

/* Stand-in analytic scene (no reference counterpart): fp32 (r,g,b logits, sigma). */
void blobs_eval(const Cfg& g, const srfo_model_t& m, const V3& w, float* rgbs4) {
    const V3 x = unwarp_position(g, w);
    float sigma = 0.f;
    for (uint32_t i = 0; i < m.n_blobs; ++i) {
        const float* b = m.blobs + 5 * i;
        const float dx = x.x - b[0], dy = x.y - b[1], dz = x.z - b[2];
        const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
        const float inv = -0.5f / (b[3] * b[3]);
        sigma = fmaf(b[4], srf_expf(d2 * inv), sigma);
    }
    const float px = x.x - 0.5f, py = x.y - 0.5f, pz = x.z - 0.5f;
    const float* M = m.color_map;
    rgbs4[0] = fmaf(M[2], pz, fmaf(M[1], py, M[0] * px));
    rgbs4[1] = fmaf(M[5], pz, fmaf(M[4], py, M[3] * px));
    rgbs4[2] = fmaf(M[8], pz, fmaf(M[7], py, M[6] * px));
    rgbs4[3] = sigma;
}

/* ---- activations: internal/utils/common_device.h:320-351 [M] ------------------------------------ */
inline float network_to_rgb(float v, int act) {
    switch (act) {
    case SRF_ACT_NONE: return v;
    case SRF_ACT_RELU: return v > 0.f ? v : 0.f;
    case SRF_ACT_LOGISTIC: return srf_logisticf(v);
    case SRF_ACT_EXPONENTIAL: return srf_expf(clampf(v, -10.f, 10.f));
    default: return 0.f;
    }
}
inline float network_to_density(float v, int act) {
    switch (act) {
    case SRF_ACT_NONE: return v;
    case SRF_ACT_RELU: return v > 0.f ? v : 0.f;
    case SRF_ACT_LOGISTIC: return srf_logisticf(v);
    case SRF_ACT_EXPONENTIAL: return srf_expf(v);
    default: return 0.f;
    }
}

/* ---- colour: internal/utils/common_device.h:70-88 [M] ------------------------------------------- */
#if defined(SRF_CANON_PLAIN)
inline float srf_powf(float x, float y) { return powf(x, y); }       /* the C library's, as a host compile of the reference uses */
#else
inline float srf_powf(float x, float y) { return x > 0.f ? srf_expf(y * srf_logf(x)) : 0.f; }
#endif
inline float srgb_to_linear(float s) { return s <= 0.04045f ? s / 12.92f : srf_powf((s + 0.055f) / 1.055f, 2.4f); }
inline float linear_to_srgb(float l) { return l < 0.0031308f ? 12.92f * l : 1.055f * srf_powf(l, 0.41666f) - 0.055f; }

/* tonemap(): internal/utils/render_buffer.cu:84-140 */
void tonemap3(float* x, int curve) {
    if (curve == SRF_TONEMAP_IDENTITY) return;
    for (int i = 0; i < 3; ++i) x[i] = fmaxf(x[i], 0.f);
    float k0, k1, k2, k3, k4, k5;
    if (curve == SRF_TONEMAP_ACES) {
        k0 = 0.6f * 0.6f * 2.51f; k1 = 0.6f * 0.03f; k2 = 0.0f; k3 = 0.6f * 0.6f * 2.43f; k4 = 0.6f * 0.59f; k5 = 0.14f;
    } else if (curve == SRF_TONEMAP_HABLE) {
        const float A = 0.15f, B = 0.50f, C = 0.10f, D = 0.20f, E = 0.02f, F = 0.30f;
        k0 = A * F - A * E; k1 = C * B * F - B * E; k2 = 0.0f; k3 = A * F; k4 = B * F; k5 = D * F * F;
        const float W = 11.2f;
        const float nom = k0 * (W * W) + k1 * W + k2;
        const float denom = k3 * (W * W) + k4 * W + k5;
        const float whiteScale = denom / nom;
        k0 = 4.0f * k0 * whiteScale; k1 = 2.0f * k1 * whiteScale; k2 = k2 * whiteScale; k3 = 4.0f * k3; k4 = 2.0f * k4;
    } else {
        const float Y = srf_dot3f(0.2126f, x[0], 0.7152f, x[1], 0.0722f, x[2]);
        const float s = 1.f / (Y + 1.0f);
        for (int i = 0; i < 3; ++i) x[i] = x[i] * s;
        return;
    }
    for (int i = 0; i < 3; ++i) {
        const float sq = x[i] * x[i];
        const float nom = fmaf(k1, x[i], sq * k0) + k2;
        const float denom = fmaf(k4, x[i], k3 * sq) + k5;
        x[i] = nom / denom;
    }
}

/* shade_kernel + accumulate_kernel + tonemap_kernel for one pixel
   (testbed.cu:448-477, render_buffer.cu:46-82,142-181). `hit` = the ray reached the hit buffer. */
void finish_pixel(const Cfg& g, const srf_view_t& v, const srf_post_t& post, bool hit, const float rgba_in[4],
                  uint32_t n_steps_total, float* accum4, float* out4) {
    float fb[4] = {0.f, 0.f, 0.f, 0.f};                              /* cleared frame buffer (testbed.cu:502) */
    if (hit) {
        float tmp[4] = {rgba_in[0], rgba_in[1], rgba_in[2], rgba_in[3]};
        if (v.render_mode == SRF_MODE_NORMALS) {                     /* :463-465 */
            const float nn = srf_norm3f(tmp[0], tmp[1], tmp[2]);
            for (int i = 0; i < 3; ++i) tmp[i] = (0.5f * (nn > 0.f ? tmp[i] / nn : tmp[i]) + 0.5f) * tmp[3];
        } else if (v.render_mode == SRF_MODE_COST) {                 /* :465-468 */
            const float col = (float)n_steps_total / 128;
            tmp[0] = tmp[1] = tmp[2] = col; tmp[3] = 1.0f;
        }
        if (!g.c.train_in_linear_color && v.render_mode == SRF_MODE_SHADE)   /* :470-473 */
            for (int i = 0; i < 3; ++i) tmp[i] = srgb_to_linear(tmp[i]);
        for (int i = 0; i < 4; ++i) fb[i] = tmp[i];                  /* :476: frame buffer was 0 */
    }
    /* accumulate */
    const float sc = (float)v.spp_index;
    float tmp[4] = {0.f, 0.f, 0.f, 0.f};
    if (v.spp_index != 0) for (int i = 0; i < 4; ++i) tmp[i] = accum4[i];   /* render_buffer.cu:204-206 */
    float color[4] = {fb[0], fb[1], fb[2], fb[3]};
    switch (post.color_space) {
    case SRF_COLOR_VISPOSNEG: {                                      /* :61-71 */
        const float val = color[0] - color[1];
        float tv = tmp[0] - tmp[1];
        tv = fmaf(tv, sc, val) / (sc + 1);
        tmp[0] = fmaxf(tv, 0.f); tmp[1] = fmaxf(-tv, 0.f);
    } break;
    case SRF_COLOR_SRGB:
        for (int i = 0; i < 3; ++i) color[i] = linear_to_srgb(color[i]);   /* :73 */
        /* fall through */
    default:
        for (int i = 0; i < 3; ++i) tmp[i] = fmaf(tmp[i], sc, color[i]) / (sc + 1);   /* :76 */
        break;
    }
    tmp[3] = fmaf(tmp[3], sc, color[3]) / (sc + 1);                  /* :79 */
    for (int i = 0; i < 4; ++i) accum4[i] = tmp[i];
    /* tonemap */
    float c[4] = {tmp[0], tmp[1], tmp[2], tmp[3]};
    const float scale = srf_powf(2.0f, post.exposure);               /* :155 */
    for (int i = 0; i < 3; ++i) c[i] *= scale;
    float bg[4] = {post.background_color[0], post.background_color[1], post.background_color[2], post.background_color[3]};
    if (post.color_space != SRF_COLOR_SRGB) for (int i = 0; i < 3; ++i) bg[i] = srgb_to_linear(bg[i]);   /* :160-162 */
    const float weight = (1 - c[3]) * bg[3];                         /* :164 */
    for (int i = 0; i < 3; ++i) c[i] = fmaf(bg[i], weight, c[i]);
    c[3] += weight;
    if (post.color_space == SRF_COLOR_SRGB) for (int i = 0; i < 3; ++i) c[i] = srgb_to_linear(c[i]);   /* :170-172 */
    tonemap3(c, post.tonemap_curve);
    if (post.to_srgb) for (int i = 0; i < 3; ++i) c[i] = linear_to_srgb(c[i]);   /* :177-179 */
    for (int i = 0; i < 4; ++i) out4[i] = c[i];
}

/* ---- PCG32 [T] --------------------------------------------------------------------------------- */
const uint64_t kPcgMult = 0x5851f42d4c957f2dULL;
inline uint32_t pcg_next_uint(srfo_rng_t& r) {
    const uint64_t old = r.state;
    r.state = old * kPcgMult + r.inc;
    const uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    const uint32_t rot = (uint32_t)(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31));
}
inline float pcg_next_float(srfo_rng_t& r) {
    return srf_u32_as_f32((pcg_next_uint(r) >> 9) | 0x3f800000u) - 1.0f;
}
inline void pcg_advance(srfo_rng_t& r, uint64_t delta) {
    uint64_t cur_mult = kPcgMult, cur_plus = r.inc, acc_mult = 1u, acc_plus = 0u;
    while (delta > 0) {
        if (delta & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
        cur_plus = (cur_mult + 1) * cur_plus;
        cur_mult *= cur_mult;
        delta >>= 1;
    }
    r.state = acc_mult * r.state + acc_plus;
}

/* The definition of the grid mean's summation order [T]: chunks of 1024 consecutive values
   (the last one zero-padded) are each summed by stride halving (v[i] += v[i+512], then 256,
   ... 1); the chunk sums are reduced the same way until one value is left. */
float tree_sum(std::vector<float> v) {
    while (true) {
        const size_t n_chunks = (v.size() + 1023) / 1024;
        v.resize(n_chunks * 1024, 0.f);
        std::vector<float> sums(n_chunks);
        for (size_t c = 0; c < n_chunks; ++c) {
            float* p = &v[c * 1024];
            for (size_t h = 512; h >= 1; h /= 2)
                for (size_t i = 0; i < h; ++i) p[i] = p[i] + p[i + h];
            sums[c] = p[0];
        }
        if (n_chunks == 1) return sums[0];
        v.swap(sums);
    }
}

}  // namespace

/* ================================================================================================== */
extern "C" {

int srfo_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Sets the OpenMP thread count (launchers such as torchrun export OMP_NUM_THREADS=1); n <= 0: one per available core. */
void srfo_set_num_threads(int n) {
#ifdef _OPENMP
    if (n <= 0) n = omp_get_num_procs();
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int srfo_hashgrid_layout(const srf_config_t* cfg, uint32_t* offsets, uint32_t* resolutions, float* scales) {
    const Cfg g = resolve(cfg);
    const GridLayout L = grid_layout(g);
    for (uint32_t l = 0; l < cfg->n_levels; ++l) {
        if (offsets) offsets[l] = L.offsets[l];
        if (resolutions) resolutions[l] = L.res[l];
        if (scales) scales[l] = L.scale[l];
    }
    if (offsets) offsets[cfg->n_levels] = L.offsets[cfg->n_levels];
    return 0;
}

int srfo_eval_math(int op, const float* a, const float* b, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        switch (op) {
        case 0: out[i] = srf_atan2f(a[i], b[i]); break;
        case 1: out[i] = srf_asinf(a[i]); break;
        case 2: out[i] = srf_cosf(a[i]); break;
        case 3: out[i] = srf_sinf(a[i]); break;
        case 4: out[i] = srf_expf(a[i]); break;
        case 5: out[i] = srf_logf(a[i]); break;
        default: return 1;
        }
    }
    return 0;
}

int srfo_warp_position(const srf_config_t* cfg, const float* pos, float* out, size_t n, int inverse) {
    const Cfg g = resolve(cfg);
    for (size_t i = 0; i < n; ++i) {
        const V3 p = v3(pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]);
        const V3 r = inverse ? unwarp_position(g, p) : warp_position(g, p);
        out[3 * i] = r.x; out[3 * i + 1] = r.y; out[3 * i + 2] = r.z;
    }
    return 0;
}

uint64_t srfo_shard_ray_count(const srf_view_t* view) { return shard_rows_total(*view) * view->width; }

/* taps for the known-answer tests: one reference function each, on arrays */
int srfo_calc_dt(const srf_config_t* cfg, const float* t, float* dt, size_t n) {
    const Cfg g = resolve(cfg);
    for (size_t i = 0; i < n; ++i) dt[i] = calc_dt(g, t[i]);
    return 0;
}
int srfo_grid_index(const srf_config_t* cfg, const float* pos, uint32_t* level_out, uint32_t* idx_out, size_t n) {
    const Cfg g = resolve(cfg);
    for (size_t i = 0; i < n; ++i) {
        const V3 p = v3(pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]);
        const V3 w = warp_position(g, p);
        const uint32_t level = level_from_pos(g, p, w);
        level_out[i] = level;
        idx_out[i] = cascaded_grid_idx_at(g, p, w, level);
    }
    return 0;
}
void srfo_pixel_offset(uint32_t spp, float* out2) { ld_random_pixel_offset(spp, &out2[0], &out2[1]); }

/* ---- training compositor: internal/render/ray_marcher.cu:9-202, internal/utils/loss.cu:18-101 ---- */
namespace {
inline float rgb_derivative(float v, int act) {                      /* common_device.h:331-340 */
    switch (act) {
    case SRF_ACT_NONE: return 1.0f;
    case SRF_ACT_RELU: return v > 0.f ? 1.0f : 0.0f;
    case SRF_ACT_LOGISTIC: { const float d = srf_logisticf(v); return d * (1.f - d); }
    case SRF_ACT_EXPONENTIAL: return srf_expf(clampf(v, -10.f, 10.f));
    default: return 0.f;
    }
}
inline float density_derivative(float v, int act) {                  /* common_device.h:353-362 */
    switch (act) {
    case SRF_ACT_NONE: return 1.0f;
    case SRF_ACT_RELU: return v > 0.f ? 1.0f : 0.0f;
    case SRF_ACT_LOGISTIC: { const float d = srf_logisticf(v); return d * (1.f - d); }
    case SRF_ACT_EXPONENTIAL: return srf_expf(clampf(v, -15.f, 15.f));
    default: return 0.f;
    }
}
inline void loss_channel(int type, float target, float pred, float* loss, float* grad) {
    const float d = pred - target;
    switch (type) {
    case SRF_LOSS_RELATIVE_L2: { const float f = 1.f / (pred * pred + 1e-2f); *loss = d * d * f; *grad = 2.0f * d * f; } break;   /* :26-33 */
    case SRF_LOSS_L1: *loss = fabsf(d); *grad = copysignf(1.0f, d); break;                                                        /* :35-41 */
    case SRF_LOSS_MAPE: { const float f = 1.f / (fabsf(pred) + 1e-2f); *loss = fabsf(d) * f; *grad = copysignf(f, d); } break;     /* :80-87 */
    case SRF_LOSS_SMAPE: { const float f = 1.f / (0.5f * (fabsf(pred) + fabsf(target)) + 1e-2f); *loss = fabsf(d) * f; *grad = copysignf(f, d); } break;   /* :71-78 */
    case SRF_LOSS_SMOOTH_L1: {                                                                                                    /* :43-59, alpha 0.1 (:95) */
        const float a = 0.1f, ad = fabsf(d);
        const float sq = 0.5f / a * d * d;
        *loss = ad > a ? (ad - 0.5f * a) : sq;
        *grad = ad > a ? (d > 0.f ? 1.0f : -1.0f) : (d / a);
    } break;
    case SRF_LOSS_LOG_L1: { const float dv = fabsf(d) + 1.0f; *loss = srf_logf(dv); *grad = copysignf(1.f / dv, d); } break;      /* :61-69 */
    default: *loss = d * d; *grad = 2.0f * d; break;                                                                             /* :18-24 */
    }
}
}  // namespace

int srfo_tonemap(const float* rgb, float* out, size_t n, int curve) {
    for (size_t i = 0; i < n; ++i) {
        float c[3] = {rgb[3 * i], rgb[3 * i + 1], rgb[3 * i + 2]};
        tonemap3(c, curve);
        out[3 * i] = c[0]; out[3 * i + 1] = c[1]; out[3 * i + 2] = c[2];
    }
    return 0;
}
int srfo_srgb(const float* in, float* out, size_t n, int to_linear) {
    for (size_t i = 0; i < n; ++i) out[i] = to_linear ? srgb_to_linear(in[i]) : linear_to_srgb(in[i]);
    return 0;
}
int srfo_loss(const float* target, const float* prediction, float* loss, float* gradient, size_t n, int loss_type) {
    for (size_t i = 0; i < 3 * n; ++i) loss_channel(loss_type, target[i], prediction[i], &loss[i], &gradient[i]);
    return 0;
}

/* All pointers are HOST pointers.  `mean_density` is the grid mean the sampler holds (update_grid_bitfield). */
int srfo_volume_rendering_loss(const srf_config_t* cfg, const srf_loss_params_t* p, uint32_t n_rays_kept,
                               uint32_t* ray_coord_indices, const float* rays_rgba, const float* coords,
                               const uint16_t* network_output, float mean_density, float* compacted_coords,
                               uint32_t* n_compacted_counter, uint16_t* dloss_doutput, float* loss_output,
                               float* reg_distortion) {
    float bg_in[3] = {p->background_color[0], p->background_color[1], p->background_color[2]};
    if (p->train_with_random_bg_color) {                             /* :83-85 */
        srfo_rng_t r = {p->rng_state, p->rng_inc};
        for (int c = 0; c < 3; ++c) bg_in[c] = pcg_next_float(r);
    }
    float bg_linear[3];
    for (int c = 0; c < 3; ++c) bg_linear[c] = srgb_to_linear(bg_in[c]);   /* :86 */
    const bool til = cfg->train_in_linear_color != 0;
    *n_compacted_counter = 0;
    for (uint32_t i = 0; i < n_rays_kept && i < p->n_rays; ++i) {
        const uint32_t numsteps = ray_coord_indices[i * 2], base = ray_coord_indices[i * 2 + 1];
        const float* co = coords + (size_t)base * 7;
        const uint16_t* no = network_output + (size_t)base * 4;
        float T = 1.f, rgb_ray[3] = {0.f, 0.f, 0.f};
        uint32_t n = 0;
        for (; n < numsteps; ++n) {                                  /* :62-80 */
            if (T < cfg->transmittance_threshold) break;
            const float density = network_to_density(h2f(no[4 * n + 3]), cfg->density_activation);
            const float dt = co[7 * n + 3];
            const float alpha = 1.f - srf_expf(-density * dt);
            const float weight = alpha * T;
            for (int c = 0; c < 3; ++c) rgb_ray[c] += weight * network_to_rgb(h2f(no[4 * n + c]), cfg->rgb_activation);
            T *= (1.f - alpha);
        }
        float bg[3] = {bg_linear[0], bg_linear[1], bg_linear[2]};
        const float* tex = rays_rgba + (size_t)i * 4;
        float target[3] = {0.f, 0.f, 0.f};
        if (til || p->color_space == SRF_COLOR_LINEAR) {             /* :91-98 */
            for (int c = 0; c < 3; ++c) target[c] = tex[c] + (1.f - tex[3]) * bg[c];
            if (!til) for (int c = 0; c < 3; ++c) { target[c] = linear_to_srgb(target[c]); bg[c] = linear_to_srgb(bg[c]); }
        } else if (p->color_space == SRF_COLOR_SRGB) {               /* :99-106 */
            for (int c = 0; c < 3; ++c) bg[c] = linear_to_srgb(bg[c]);
            for (int c = 0; c < 3; ++c)
                target[c] = tex[3] > 0.f ? linear_to_srgb(tex[c] / tex[3]) * tex[3] + (1.f - tex[3]) * bg[c] : bg[c];
        }
        if (n == numsteps) for (int c = 0; c < 3; ++c) rgb_ray[c] += T * bg[c];   /* :108-111 */
        const uint32_t compacted_base = *n_compacted_counter;        /* :118 atomicAdd */
        *n_compacted_counter += n;
        const uint32_t n_max = p->n_max_compacted_coords;
        n = std::min(n_max - std::min(n_max, compacted_base), n);    /* :119 */
        ray_coord_indices[i * 2] = n;
        ray_coord_indices[i * 2 + 1] = compacted_base;
        if (n == 0) continue;
        float loss[3], grad[3];
        for (int c = 0; c < 3; ++c) loss_channel(p->loss_type, target[c], rgb_ray[c], &loss[c], &grad[c]);   /* :129 */
        const float n_rays_f = (float)p->n_rays;
        if (loss_output) loss_output[i] = (loss[0] + (loss[1] + loss[2])) / 3.0f / n_rays_f;   /* :131-132; [E] mean() reduces as t0 + (t1 + t2) */
        const float loss_scale = p->loss_scale / n_rays_f;           /* :134 */
        const float output_l2_reg = cfg->rgb_activation == SRF_ACT_EXPONENTIAL ? 1e-4f : 0.0f;
        const float output_l1_reg_density = (cfg->use_grid && (mean_density < cfg->min_optical_thickness)) ? 1e-4f : 0.0f;
        if (p->regularization_type == SRF_REG_DISTORTION && reg_distortion) {   /* :143-167: T stays 1 in this loop */
            float sum_w = 0.f, sum_wp = 0.f;
            float* rd = reg_distortion + (size_t)compacted_base * 2;
            for (uint32_t j = 0; j < n; ++j) {
                const float alpha = 1.f - srf_expf(-network_to_density(h2f(no[4 * j + 3]), cfg->density_activation) * co[7 * j + 3]);
                const float weight = alpha * 1.f;
                sum_w += weight;
                sum_wp += weight * (float)(j + 1) / (float)n;
                rd[2 * j] = sum_w;
                rd[2 * j + 1] = sum_wp;
            }
        }
        T = 1.f;
        float r2[3] = {0.f, 0.f, 0.f};
        float* cc = compacted_coords + (size_t)compacted_base * 7;
        uint16_t* dl = dloss_doutput + (size_t)compacted_base * p->padded_output_width;
        for (uint32_t j = 0; j < n; ++j) {                           /* :170-201 */
            for (int k = 0; k < 7; ++k) cc[(size_t)j * 7 + k] = co[7 * j + k];
            const float dt = co[7 * j + 3];
            float raw[4], rgb[3];
            for (int k = 0; k < 4; ++k) raw[k] = h2f(no[4 * j + k]);
            for (int k = 0; k < 3; ++k) rgb[k] = network_to_rgb(raw[k], cfg->rgb_activation);
            const float density = network_to_density(raw[3], cfg->density_activation);
            const float alpha = 1.f - srf_expf(-density * dt);
            const float weight = alpha * T;
            for (int k = 0; k < 3; ++k) r2[k] += weight * rgb[k];
            T *= (1.f - alpha);
            float out[4], v[3];
            for (int k = 0; k < 3; ++k) {
                const float dloss_by_drgb = weight * grad[k];
                out[k] = loss_scale * (dloss_by_drgb * rgb_derivative(raw[k], cfg->rgb_activation) + fmaxf(0.0f, output_l2_reg * raw[k]));
                v[k] = T * rgb[k] - (rgb_ray[k] - r2[k]);
            }
            const float dot = srf_dot3f(grad[0], v[0], grad[1], v[1], grad[2], v[2]);   /* [E] dot */
            const float dloss_by_dmlp = density_derivative(raw[3], cfg->density_activation) * (dt * dot);
            out[3] = loss_scale * dloss_by_dmlp + (raw[3] < 0.f ? -output_l1_reg_density : 0.0f);
            for (int k = 0; k < 4; ++k) dl[(size_t)j * p->padded_output_width + k] = f2h(out[k]);
        }
    }
    return 0;
}

/* mark_untrained_density_grid (occupancy_sampler.cu:12-102).  views holds HOST pointers here.
   grid_out: cells * cascades floats: 0 where some training view sees the cell, -1 elsewhere. */
int srfo_mark_untrained(const srf_config_t* cfg, const srf_train_views_t* tv, float* grid_out) {
    const Cfg g = resolve(cfg);
    const uint32_t N = cfg->grid_size, nc = cfg->num_cascades;
    const int64_t n = (int64_t)g.cells * nc;
    const float fn = (float)N, fa = (float)cfg->aabb_scale;
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t level = (uint32_t)(i / g.cells), pos_idx = (uint32_t)(i % g.cells);   /* :29-30 */
        const uint32_t x = morton3D_invert(pos_idx >> 0), y = morton3D_invert(pos_idx >> 1), z = morton3D_invert(pos_idx >> 2);
        V3 pos = v3(((float)x + 0.5f) / fn - 0.5f, ((float)y + 0.5f) / fn - 0.5f, ((float)z + 0.5f) / fn - 0.5f);   /* :37 */
        const int down = -(int)(nc - level - 1);
        const float fl = (float)(nc - level);
        float s;
        switch (cfg->grid_distribution_type) {
        case SRF_GRID_WARPED_EXP:                                    /* :40-45 */
            s = scalbnf(1.0f, down);
            pos = v3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
            pos = unwarp_position(g, pos);
            break;
        case SRF_GRID_WARPED_RECIPROCAL:                             /* :46-51 */
            pos = v3(pos.x / fl + 0.5f, pos.y / fl + 0.5f, pos.z / fl + 0.5f);
            pos = unwarp_position(g, pos);
            break;
        case SRF_GRID_METRIC_EXP:                                    /* :52-54, falls through (no break) */
            s = scalbnf(fa, down);
            pos = v3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
            /* fallthrough */
        case SRF_GRID_METRIC_RECIPROCAL:                             /* :55-57 */
            s = fa / fl;
            pos = v3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
            break;
        default: break;
        }
        const float half_resx = (float)tv->width * 0.5f, half_resy = (float)tv->height * 0.5f;   /* :61-62 */
        float voxel_radius = 0.5f * 1.73205080757f * fa / fn;        /* :63 */
        if (cfg->grid_distribution_type == SRF_GRID_WARPED_EXP || cfg->grid_distribution_type == SRF_GRID_METRIC_EXP)
            voxel_radius *= scalbnf(1.0f, down);                     /* :66-69,74-76 */
        else
            voxel_radius /= fl;                                      /* :70-73,77-79 */
        bool seen = false;
        for (uint32_t j = 0; j < tv->n_images && !seen; ++j) {       /* :84-99 */
            const float* m = tv->d_xforms + (size_t)j * 12;          /* column-major 3x4 */
            const V3 ploc = v3(pos.x - m[9], pos.y - m[10], pos.z - m[11]);
            const float cx = srf_dot3f(ploc.x, m[0], ploc.y, m[1], ploc.z, m[2]);     /* [E] dot */
            const float cy = srf_dot3f(ploc.x, m[3], ploc.y, m[4], ploc.z, m[5]);
            const float cz = srf_dot3f(ploc.x, m[6], ploc.y, m[7], ploc.z, m[8]);
            if (cz > 0.f)
                seen = fabsf(cx) - voxel_radius < cz / tv->focal_length[0] * half_resx &&
                       fabsf(cy) - voxel_radius < cz / tv->focal_length[1] * half_resy;
        }
        grid_out[i] = seen ? 0.f : -1.f;                             /* :101 */
    }
    return 0;
}

/* generate_training_samples_nerf (occupancy_sampler.cu:513-689) executed serially, ray 0 first: the atomic
   counters of the reference then hand out bases and ray slots in ray order.  views holds HOST pointers.
   Output capacities: rays n_rays*6, rgba n_rays*4, numsteps n_rays*2, coords n_coords*7. */
int srfo_sample_training_rays(const srf_config_t* cfg, const srf_train_views_t* tv, const uint8_t* bitfield,
                              uint32_t n_rays, uint32_t n_rays_shift, uint32_t n_coords, const srfo_rng_t* rng0,
                              int snap, uint32_t* ray_counter, uint32_t* numsteps_counter, float* rays_out,
                              float* rays_rgba, uint32_t* numsteps_out, float* coords_out) {
    const Cfg g = resolve(cfg);
    const uint32_t n_max_steps = cfg->maximum_marching_steps;
    *ray_counter = 0;
    *numsteps_counter = 0;
    const float rw = (float)tv->width, rh = (float)tv->height;
    for (uint32_t i = 0; i < n_rays; ++i) {
        const uint32_t img = (((n_rays_shift + i) * tv->n_images) / n_rays) % tv->n_images;   /* :544 */
        srfo_rng_t rng = *rng0;
        pcg_advance(rng, (uint64_t)(uint32_t)(i * 8u));              /* :551 */
        float xx = pcg_next_float(rng);                              /* :552, random_val.cuh:21-23 */
        float yy = pcg_next_float(rng);
        if (snap) {                                                  /* :553-555 */
            xx = ((float)std::min(std::max(srf_f2i_rz(xx * rw), 0), tv->width - 1) + 0.5f) / rw;
            yy = ((float)std::min(std::max(srf_f2i_rz(yy * rh), 0), tv->height - 1) + 0.5f) / rh;
        }
        const int px = std::max(std::min(srf_f2i_rz(xx * rw), tv->width - 1), 0);   /* common_device.h:191-197 */
        const int py = std::max(std::min(srf_f2i_rz(yy * rh), tv->height - 1), 0);
        const uint64_t pixel = (uint64_t)(int64_t)(px + py * tv->width) + (uint64_t)img * (uint64_t)tv->width * (uint64_t)tv->height;
        if (tv->d_sampling_probability && h2f(tv->d_sampling_probability[pixel]) <= 0.f) continue;   /* :570-571 */
        const float* m = tv->d_xforms + (size_t)img * 12;
        const V3 o = v3(m[9], m[10], m[11]);                         /* :576 */
        const float dx = (xx - tv->principal_point[0]) * rw / tv->focal_length[0];   /* :577-581 */
        const float dy = (yy - tv->principal_point[1]) * rh / tv->focal_length[1];
        const float rx = srf_dot3f(m[0], dx, m[3], dy, m[6], 1.0f);                  /* :582 [E] */
        const float ry = srf_dot3f(m[1], dx, m[4], dy, m[7], 1.0f);
        const float rz = srf_dot3f(m[2], dx, m[5], dy, m[8], 1.0f);
        const float nrm = srf_norm3f(rx, ry, rz);
        const V3 d = v3(rx / nrm, ry / nrm, rz / nrm);
        const float t0 = fmaxf(box_ray_tmin(g.box, o, d), cfg->near_distance);       /* :585-587 */
        const float startt = fmaf(pcg_next_float(rng), calc_dt(g, t0), t0);          /* :596-597 */
        /* the march of :602-628 (count) and :652-688 (emit): `emit` false = count only */
        auto march = [&](uint32_t limit, float* coords) {
            uint32_t j = 0;
            float t = startt;
            const V3 wd = v3((d.x + 1.f) * 0.5f, (d.y + 1.f) * 0.5f, (d.z + 1.f) * 0.5f);   /* warp_direction */
            for (uint32_t it = 0; it < (1u << 24) && j < limit; ++it) {
                const V3 pos = v3(fmaf(d.x, t, o.x), fmaf(d.y, t, o.y), fmaf(d.z, t, o.z));
                if (!box_contains(g.box, pos)) break;
                const float dt = calc_dt(g, t);
                const V3 w = warp_position(g, pos);
                bool occ = true;
                if (cfg->use_grid) {
                    const uint32_t level = level_from_pos(g, pos, w);
                    occ = occupied_at(g, bitfield, cascaded_grid_idx_at(g, pos, w, level), level);
                }
                if (occ) {
                    if (coords) {
                        float* c = coords + (size_t)j * 7;
                        c[0] = w.x; c[1] = w.y; c[2] = w.z; c[3] = dt; c[4] = wd.x; c[5] = wd.y; c[6] = wd.z;
                    }
                    ++j;
                }
                t += dt;
                if (dt == 0.f) break;
            }
            return j;
        };
        const uint32_t numsteps = march(n_max_steps, nullptr);
        if (numsteps == 0) continue;                                 /* :630-632 */
        const uint32_t base = *numsteps_counter;                     /* :634 atomicAdd */
        *numsteps_counter += numsteps;
        if ((uint64_t)base + numsteps > n_coords) continue;          /* :635-637 */
        const uint32_t ray_idx = (*ray_counter)++;                   /* :642 */
        float* ro = rays_out + (size_t)ray_idx * 6;
        ro[0] = o.x; ro[1] = o.y; ro[2] = o.z; ro[3] = d.x; ro[4] = d.y; ro[5] = d.z;
        for (int k = 0; k < 4; ++k) rays_rgba[(size_t)ray_idx * 4 + k] = h2f(tv->d_images[pixel * 4 + k]);   /* :645 */
        numsteps_out[ray_idx * 2 + 0] = numsteps;
        numsteps_out[ray_idx * 2 + 1] = base;
        march(numsteps, coords_out + (size_t)base * 7);
    }
    return 0;
}

/* OccupancySampler::generate_rays_from_camera_matrix (occupancy_sampler.cu:1145-1188). */
int srfo_generate_rays(const srf_config_t* cfg, const srf_view_t* view, const uint8_t* bitfield,
                       float* dir, float* t_out, uint8_t* alive, uint32_t* pixel) {
    const Cfg g = resolve(cfg);
    const int64_t n = (int64_t)srfo_shard_ray_count(view);
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t i = 0; i < n; ++i) {
        const uint32_t pix = shard_ray_pixel(*view, (uint64_t)i);
        RayInit r = init_ray(g, *view, pix);
        bool al = r.alive;
        float t = r.t;
        if (al) {
            /* advance_pos_nerf :771-794: stop at the first occupied step, or the ray dies */
            uint64_t steps = 0;
            bool found = false;
            march_ray(g, bitfield, r, 1u, &steps, [&](const Sample& s) { found = true; t = s.t; return false; });
            al = found;
        }
        if (dir) { dir[3 * i] = r.d.x; dir[3 * i + 1] = r.d.y; dir[3 * i + 2] = r.d.z; }
        if (t_out) t_out[i] = al ? t : 0.f;
        if (alive) alive[i] = al ? 1 : 0;
        if (pixel) pixel[i] = pix;
    }
    return 0;
}

int srfo_march(const srf_config_t* cfg, const srf_view_t* view, const uint8_t* bitfield,
               uint64_t ray_first, uint64_t ray_count, uint64_t capacity, uint32_t* counts,
               float* pos_dt, uint32_t* ordinal, uint32_t* cell, uint64_t* n_total, uint64_t* n_march_steps) {
    const Cfg g = resolve(cfg);
    const uint32_t cap = sample_cap(g);
    uint64_t total = 0, steps = 0;
    for (uint64_t k = 0; k < ray_count; ++k) {
        const uint32_t pix = shard_ray_pixel(*view, ray_first + k);
        const RayInit r = init_ray(g, *view, pix);
        uint32_t n = 0;
        if (r.alive) {
            march_ray(g, bitfield, r, cap, &steps, [&](const Sample& s) {
                if (total + n < capacity) {
                    const uint64_t j = total + n;
                    if (pos_dt) { pos_dt[4 * j] = s.w.x; pos_dt[4 * j + 1] = s.w.y; pos_dt[4 * j + 2] = s.w.z; pos_dt[4 * j + 3] = s.dt; }
                    if (ordinal) ordinal[j] = s.ordinal;
                    if (cell) cell[j] = s.cell;
                }
                ++n;
                return true;
            });
        }
        counts[k] = n;
        total += n;
    }
    if (n_total) *n_total = total;
    if (n_march_steps) *n_march_steps = steps;
    return total > capacity ? 3 : 0;
}

int srfo_network_inference(const srf_config_t* cfg, const srfo_model_t* model, const float* coords,
                           uint64_t n, uint16_t* rgbsigma) {
    const Cfg g = resolve(cfg);
    const GridLayout L = grid_layout(g);
    const Weights W(*model);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i)
        network_eval(g, L, *model, W, coords + 7 * i, coords + 7 * i + 4, rgbsigma + 4 * i);
    return 0;
}

int srfo_network_density(const srf_config_t* cfg, const srfo_model_t* model, const float* positions,
                         uint64_t n, uint16_t* out16) {
    const Cfg g = resolve(cfg);
    const GridLayout L = grid_layout(g);
    const Weights W(*model);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n; ++i) density_net(g, L, *model, W, positions + 3 * i, out16 + 16 * i);
    return 0;
}

/* Testbed::render_frame (testbed.cu:479-606) per ray: the per-ray semantics of its host loop are
   described at march_ray and finish_pixel above. */
int srfo_render_frame(const srf_config_t* cfg, const srf_view_t* view, const srf_post_t* post,
                      const uint8_t* bitfield, const srfo_model_t* model, uint64_t ray_first,
                      uint64_t ray_count, float* out, float* accum, float* rgba_raw,
                      uint32_t* n_samples, uint32_t* n_composited, srf_frame_stats_t* stats) {
    const Cfg g = resolve(cfg);
    const GridLayout L = grid_layout(g);
    const Weights W(*model);
    if (view->render_mode == SRF_MODE_NORMALS && g.c.field_type != SRF_FIELD_NETWORK) return 1;
    const uint64_t n_all = srfo_shard_ray_count(view);
    if (ray_count == 0) ray_count = n_all - ray_first;
    const uint32_t cap = sample_cap(g);
    const float thr = 1.0f - g.c.transmittance_threshold;
    uint64_t s_alive = 0, s_steps = 0, s_samples = 0, s_comp = 0, s_hit = 0;
    const float* M = view->camera;
    const V3 cam_fwd = v3(M[2], M[6], M[10]);                        /* camera_matrix.col(2), ray_marcher.cu:233 */

#pragma omp parallel for schedule(dynamic, 64) reduction(+ : s_alive, s_steps, s_samples, s_comp, s_hit)
    for (int64_t k = 0; k < (int64_t)ray_count; ++k) {
        const uint64_t i = ray_first + (uint64_t)k;
        const uint32_t pix = shard_ray_pixel(*view, i);
        const RayInit r = init_ray(g, *view, pix);
        float rgba[4] = {0.f, 0.f, 0.f, 0.f};
        uint32_t ncomp = 0, nsamp = 0;
        bool terminated = false;
        int end = END_BORN_DEAD;
        uint64_t steps = 0;
        if (r.alive) {
            ++s_alive;
            float dir3[3] = {(r.d.x + 1.f) * 0.5f, (r.d.y + 1.f) * 0.5f, (r.d.z + 1.f) * 0.5f};   /* warp_direction, common_device.h:528-530 */
            end = march_ray(g, bitfield, r, cap, &steps, [&](const Sample& s) {
                ++nsamp;
                float raw[4];
                float normal[3] = {0.f, 0.f, 0.f};
                if (g.c.field_type == SRF_FIELD_BLOBS) {
                    blobs_eval(g, *model, s.w, raw);
                } else if (view->render_mode == SRF_MODE_NORMALS) {
                    /* testbed.cu:557-559 + ray_marcher.cu:250-255: the position rows hold d sigma_raw / d pos */
                    const float p3[3] = {s.w.x, s.w.y, s.w.z};
                    uint16_t sg; float grad[3];
                    density_with_gradient(g, L, *model, W, p3, &sg, grad);
                    raw[0] = raw[1] = raw[2] = 0.f; raw[3] = h2f(sg);
                    const float dd = -density_derivative(raw[3], g.c.density_activation);
                    for (int c = 0; c < 3; ++c) normal[c] = dd * grad[c];
                    const float nn = srf_norm3f(normal[0], normal[1], normal[2]);
                    if (nn > 0.f) for (int c = 0; c < 3; ++c) normal[c] /= nn;   /* [E] normalized() */
                } else {
                    uint16_t o[4];
                    const float p3[3] = {s.w.x, s.w.y, s.w.z};
                    network_eval(g, L, *model, W, p3, dir3, o);
                    for (int c = 0; c < 4; ++c) raw[c] = h2f(o[c]);
                }
                /* volume_rendering_kernel, ray_marcher.cu:236-274 */
                const float T = 1.f - rgba[3];
                const float alpha = 1.f - srf_expf(-network_to_density(raw[3], g.c.density_activation) * s.dt);   /* :246 [M] */
                const float weight = alpha * T;
                float rgb[3] = {network_to_rgb(raw[0], g.c.rgb_activation), network_to_rgb(raw[1], g.c.rgb_activation),
                                network_to_rgb(raw[2], g.c.rgb_activation)};
                if (view->render_mode == SRF_MODE_DEPTH || view->render_mode == SRF_MODE_DISTANCE) {
                    const V3 p = unwarp_position(g, s.w);
                    const float dx = p.x - r.o.x, dy = p.y - r.o.y, dz = p.z - r.o.z;
                    float zz;
                    if (view->render_mode == SRF_MODE_DEPTH) zz = srf_dot3f(cam_fwd.x, dx, cam_fwd.y, dy, cam_fwd.z, dz) * view->depth_scale;   /* :258 */
                    else zz = srf_norm3f(dx, dy, dz) * view->depth_scale;   /* :261 */
                    rgb[0] = rgb[1] = rgb[2] = zz;
                } else if (view->render_mode == SRF_MODE_AO) {
                    rgb[0] = rgb[1] = rgb[2] = alpha;                /* :264 */
                } else if (view->render_mode == SRF_MODE_NORMALS) {
                    rgb[0] = normal[0]; rgb[1] = normal[1]; rgb[2] = normal[2];   /* :255 */
                }
                rgba[0] = fmaf(rgb[0], weight, rgba[0]);             /* :268 */
                rgba[1] = fmaf(rgb[1], weight, rgba[1]);
                rgba[2] = fmaf(rgb[2], weight, rgba[2]);
                rgba[3] += weight;                                   /* :269 */
                ++ncomp;
                if (rgba[3] > thr) { terminated = true; return false; }   /* :271-273; the store at :272 is dead (:281) */
                return true;
            });
        }
        /* testbed.cu:438-445: a ray reaches the hit buffer when it is no longer alive and visible;
           rays that never stop being alive (stuck on dt == 0, cut by MARCH_ITER) leave the pixel 0. */
        const bool finished = terminated || end == END_EXIT || end == END_DT0;
        const bool hit = finished && rgba[3] > 0.001f;
        const uint32_t n_steps_total = terminated ? ncomp : 1u + ncomp;   /* ray_marcher.cu:276-279, testbed.cu:520,582 */
        s_steps += steps; s_samples += nsamp; s_comp += ncomp; s_hit += hit ? 1 : 0;
        if (rgba_raw) for (int c = 0; c < 4; ++c) rgba_raw[4 * i + c] = rgba[c];
        if (n_samples) n_samples[i] = nsamp;
        if (n_composited) n_composited[i] = ncomp;
        if (out) finish_pixel(g, *view, *post, hit, rgba, n_steps_total, accum + 4 * i, out + 4 * i);
    }
    if (stats) {
        memset(stats, 0, sizeof(*stats));
        stats->n_rays = ray_count; stats->n_rays_alive = s_alive; stats->n_march_steps = s_steps;
        stats->n_samples = s_samples; stats->n_samples_composited = s_comp; stats->n_rays_hit = s_hit;
        stats->n_batches = 1;
        stats->n_waves = 1;
    }
    return 0;
}

/* OccupancySampler::update_grid_bitfield (occupancy_sampler.cu:1063-1088) */
int srfo_update_grid_bitfield(const srf_config_t* cfg, const float* grid, uint8_t* bitfield, float* mean_out) {
    const Cfg g = resolve(cfg);
    const uint32_t n = g.cells;
    std::vector<float> v(n);
    for (uint32_t i = 0; i < n; ++i) v[i] = fmaxf(grid[i], 0.f) / (float)n;   /* :1069: divide, then add */
    const float mean = tree_sum(v);
    if (mean_out) *mean_out = mean;
    const float thresh = std::min(g.c.min_optical_thickness, mean);   /* :252 */
    const uint32_t total = n * g.c.num_cascades;
    for (uint32_t i = 0; i < total / 8; ++i) {                       /* grid_to_bitfield :240-260 */
        uint8_t bits = 0;
        for (uint32_t j = 0; j < 8; ++j) bits |= grid[i * 8 + j] > thresh ? (uint8_t)(1u << j) : 0;
        bitfield[i] = bits;
    }
    if (g.c.grid_distribution_type == SRF_GRID_WARPED_EXP || g.c.grid_distribution_type == SRF_GRID_METRIC_EXP) {
        const uint32_t N = g.c.grid_size;
        for (uint32_t level = 1; level < g.c.num_cascades; ++level) {   /* bitfield_max_pool :262-285 */
            const uint8_t* prev = bitfield + (size_t)n * (level - 1) / 8;
            uint8_t* next = bitfield + (size_t)n * level / 8;
            for (uint32_t i = 0; i < n / 64; ++i) {
                uint8_t bits = 0;
                for (uint32_t j = 0; j < 8; ++j) bits |= prev[i * 8 + j] > 0 ? (uint8_t)(1u << j) : 0;
                const uint32_t x = morton3D_invert(i >> 0) + N / 8;
                const uint32_t y = morton3D_invert(i >> 1) + N / 8;
                const uint32_t z = morton3D_invert(i >> 2) + N / 8;
                next[morton3D(x, y, z)] |= bits;
            }
        }
    }
    return 0;
}

void srfo_rng_seed_seq(srfo_rng_t* rng, uint64_t seed, uint64_t seq) {
    rng->state = 0u;
    rng->inc = (seq << 1u) | 1u;
    pcg_next_uint(*rng);
    rng->state += seed;
    pcg_next_uint(*rng);
}
void srfo_rng_seed(srfo_rng_t* rng, uint64_t seed) { srfo_rng_seed_seq(rng, seed, 1u); }
uint32_t srfo_rng_next_uint(srfo_rng_t* rng) { return pcg_next_uint(*rng); }
float srfo_rng_next_float(srfo_rng_t* rng) { return pcg_next_float(*rng); }
void srfo_rng_advance(srfo_rng_t* rng, uint64_t delta) { pcg_advance(*rng, delta); }
float srfo_ld_random_val(uint32_t index, uint32_t seed, uint32_t dim) { return ld_random_val(index, seed, dim); }
uint32_t srfo_morton3d(uint32_t x, uint32_t y, uint32_t z) { return morton3D(x, y, z); }
uint32_t srfo_sobol(uint32_t index, uint32_t dim) { return sobol(index, dim); }

/* Testbed::train_prep_nerf (testbed.cu:203-239). */
int srfo_refresh_grid(const srf_config_t* cfg, const srfo_model_t* model, float* grid, uint8_t* bitfield,
                      float* mean, uint32_t* refresh_step, uint32_t training_step, srfo_rng_t* rng) {
    const Cfg g = resolve(cfg);
    const GridLayout L = grid_layout(g);
    const Weights W(*model);
    const uint32_t nc = g.c.num_cascades, N = g.c.grid_size;
    const uint32_t total = g.cells * nc;
    const uint32_t n_uniform = training_step >= 256 ? total / 4 : total;      /* :206 */
    const uint32_t n_nonuniform = training_step >= 256 ? total / 4 : 0;       /* :207 */
    const uint32_t n_pos = n_uniform + n_nonuniform;
    std::vector<float> positions((size_t)n_pos * 3);
    std::vector<uint32_t> indices(n_pos);
    const uint32_t step = *refresh_step;

    /* sample_positions_from_grid (occupancy_sampler.cu:980-1029): two launches of
       generate_grid_samples_nerf_nonuniform (:104-185) */
    for (int pass = 0; pass < 2; ++pass) {
        const uint32_t n_el = pass == 0 ? n_uniform : n_nonuniform;
        const uint32_t base = pass == 0 ? 0 : n_uniform;
        const float thresh = pass == 0 ? (float)-0.01 : g.c.min_optical_thickness;   /* :1007,1026 */
        const srfo_rng_t rng0 = *rng;
#pragma omp parallel for schedule(static)
        for (int64_t ii = 0; ii < (int64_t)n_el; ++ii) {
            const uint32_t i = (uint32_t)ii;
            srfo_rng_t r = rng0;
            pcg_advance(r, (uint64_t)i * 4u);                        /* :125 */
            const uint32_t level = (uint32_t)(pcg_next_float(r) * (float)nc) % nc;   /* :126 */
            uint32_t idx = 0;
            for (uint32_t j = 0; j < 10; ++j) {                      /* :130-136 */
                idx = ((i + step * n_el) * 56924617u + j * 19349663u + 96925573u) % g.cells;
                idx += level * g.cells;
                if (grid[idx] > thresh) break;
            }
            const uint32_t pos_idx = idx % g.cells;
            const uint32_t x = morton3D_invert(pos_idx >> 0), y = morton3D_invert(pos_idx >> 1), z = morton3D_invert(pos_idx >> 2);
            const float u0 = pcg_next_float(r), u1 = pcg_next_float(r), u2 = pcg_next_float(r);   /* :146 */
            float p[3] = {((float)x + u0) / (float)N - 0.5f, ((float)y + u1) / (float)N - 0.5f, ((float)z + u2) / (float)N - 0.5f};
            V3 pos = v3(0.f, 0.f, 0.f);
            switch (g.c.grid_distribution_type) {
            case SRF_GRID_WARPED_EXP: {                              /* :149-155 */
                const float s = scalbnf(1.0f, -(int)(nc - level - 1));
                pos = v3(p[0] * s + 0.5f, p[1] * s + 0.5f, p[2] * s + 0.5f);
            } break;
            case SRF_GRID_WARPED_RECIPROCAL: {                       /* :156-162 */
                const float s = 1.f / (float)(nc - level);
                pos = v3(p[0] * s + 0.5f, p[1] * s + 0.5f, p[2] * s + 0.5f);
            } break;
            case SRF_GRID_METRIC_EXP: {                              /* :163-170 */
                const float s = scalbnf((float)g.c.aabb_scale, -(int)(nc - level - 1));
                pos = warp_position(g, v3(p[0] * s + 0.5f, p[1] * s + 0.5f, p[2] * s + 0.5f));
            } break;
            default: {                                               /* :171-178 */
                const float s = (float)g.c.aabb_scale / (float)(nc - level);
                pos = warp_position(g, v3(p[0] * s + 0.5f, p[1] * s + 0.5f, p[2] * s + 0.5f));
            } break;
            }
            positions[(size_t)(base + i) * 3] = pos.x; positions[(size_t)(base + i) * 3 + 1] = pos.y; positions[(size_t)(base + i) * 3 + 2] = pos.z;
            indices[base + i] = idx;
        }
        pcg_advance(*rng, 1ull << 32);                               /* :1009,1028: rng.advance() */
    }

    /* NGPNetwork::density (testbed.cu:220-227) + update_grid (occupancy_sampler.cu:1031-1061) */
    std::vector<float> current(total, 0.f);                          /* :1039 */
    std::vector<float> thick(n_pos);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < (int64_t)n_pos; ++i) {
        uint16_t o[16];
        density_net(g, L, *model, W, &positions[(size_t)i * 3], o);
        const float mlp = network_to_density(h2f(o[0]), g.c.density_activation);   /* :206 */
        thick[i] = mlp * g.min_step;                                 /* :207: scalbnf(min_cone_stepsize, 0) */
    }
    for (uint32_t i = 0; i < n_pos; ++i) {                           /* :211 atomicMax on the bit pattern */
        uint32_t a, b;
        memcpy(&a, &current[indices[i]], 4); memcpy(&b, &thick[i], 4);
        if (b > a) current[indices[i]] = thick[i];
    }
    for (uint32_t i = 0; i < total; ++i) {                           /* ema_grid_samples_nerf :214-238 */
        const float prev = grid[i];
        grid[i] = (prev < 0.f) ? prev : fmaxf(prev * g.c.ema_decay, current[i]);
    }
    *refresh_step = step + 1;                                        /* :1060 */
    return srfo_update_grid_bitfield(cfg, grid, bitfield, mean);     /* testbed.cu:238 */
}

}  // extern "C"
