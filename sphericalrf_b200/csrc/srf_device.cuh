// srf_device.cuh -- device-side building blocks of the sampler: ray generation, step size,
// space warps, occupancy lookup and the march loop.
//
// Arithmetic contract: every float operation here is an IEEE-754 correctly rounded primitive
// and fused multiply-adds appear only where fmaf()/fma() is written (the library is compiled
// with -fmad=false).  Evaluation order follows the reference's statements; file:line
// citations point into the reference project.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/srf_abi.h"
#include "../../include/srf_canon_math.h"

namespace srf {

// Resolved configuration handed to kernels by value.
struct DevCfg {
    int warping_type, grid_dist, sampling_type, use_grid;
    uint32_t grid_size, n_cascades, cells;
    float box_min, box_max, box_diag;        // the box is a cube: one value per bound
    float min_step, max_step, cone_angle;
    float near_distance, far_distance;
    float ds;                                // 1 / maximum_marching_steps
    float g_far, g_near, g_diff;             // Disparity: 1/far, 1/near, their difference; Log: logs
    uint32_t sample_cap;                     // samples a ray may emit before it is cut
    uint32_t step_limit;                     // hard bound of the march loop
    int snap;
    // compositing
    float transmittance_keep;                // 1 - transmittance_threshold
    int density_activation, rgb_activation, train_in_linear_color, field_type;
    // exact empty-space tests in front of the full lookup (sinusoidal warp, one cascade): see march_ray
    const uint32_t* skip_shell;              // bit z: some occupied cell has radial index z
    const uint32_t* skip_yz;                 // bit z*N + y: some occupied cell has radial index z and latitude index y
};

// Per-call view constants.
struct DevView {
    float cam[12];                           // row-major 3x4
    uint32_t width, height;
    float rw, rh;                            // (float) resolution
    float fx, fy;                            // focal length in pixels
    float ppx, ppy;
    float off_x, off_y;                      // sub-pixel offset of this spp pass (same for all pixels)
    uint32_t spp_index;
    int render_mode;
    float depth_scale;
    uint32_t shard_rows, shard_count, shard_rank;
    uint64_t n_rays;
    int out_by_pixel;                        // output stage writes out[pixel] (whole-image buffer) instead of out[shard ray]
};

struct V3 { float x, y, z; };
__device__ __forceinline__ V3 mk3(float x, float y, float z) { V3 r; r.x = x; r.y = y; r.z = z; return r; }

// ---- Morton code (x -> bit 0, y -> bit 1, z -> bit 2) -----------------------------------------
__host__ __device__ __forceinline__ uint32_t expand_bits(uint32_t v) {
    v = (v * 0x00010001u) & 0xFF0000FFu;
    v = (v * 0x00000101u) & 0x0F00F00Fu;
    v = (v * 0x00000011u) & 0xC30C30C3u;
    v = (v * 0x00000005u) & 0x49249249u;
    return v;
}
__host__ __device__ __forceinline__ uint32_t morton3D(uint32_t x, uint32_t y, uint32_t z) {
    return expand_bits(x) | (expand_bits(y) << 1) | (expand_bits(z) << 2);
}
__host__ __device__ __forceinline__ uint32_t morton3D_invert(uint32_t x) {
    x = x & 0x49249249u;
    x = (x | (x >> 2)) & 0xc30c30c3u;
    x = (x | (x >> 4)) & 0x0f00f00fu;
    x = (x | (x >> 8)) & 0xff0000ffu;
    x = (x | (x >> 16)) & 0x0000ffffu;
    return x;
}

// ---- low-discrepancy jitter: internal/utils/random_val.cuh:137-273 ----------------------------
// Sobol dimension 0 is the bit reversal, dimension 1 has direction numbers v[k] = v[k-1]^(v[k-1]>>1).
__host__ __device__ __forceinline__ uint32_t reverse_bits32(uint32_t x) {
#if defined(__CUDA_ARCH__)
    return __brev(x);
#else
    x = (((x & 0xaaaaaaaau) >> 1) | ((x & 0x55555555u) << 1));
    x = (((x & 0xccccccccu) >> 2) | ((x & 0x33333333u) << 2));
    x = (((x & 0xf0f0f0f0u) >> 4) | ((x & 0x0f0f0f0fu) << 4));
    x = (((x & 0xff00ff00u) >> 8) | ((x & 0x00ff00ffu) << 8));
    return ((x >> 16) | (x << 16));
#endif
}
__host__ __device__ __forceinline__ uint32_t sobol_dim(uint32_t index, uint32_t dim) {
    if (dim == 0) return reverse_bits32(index);
    uint32_t X = 0, v = 0x80000000u;
    for (uint32_t bit = 0; bit < 32; ++bit) {
        if ((index >> bit) & 1u) X ^= v;
        v ^= v >> 1;
    }
    return X;
}
__host__ __device__ __forceinline__ uint32_t hash_combine(uint32_t seed, uint32_t v) {
    return seed ^ (v + (seed << 6) + (seed >> 2));
}
__host__ __device__ __forceinline__ uint32_t laine_karras(uint32_t x, uint32_t seed) {
    x += seed;
    x ^= x * 0x6c50b47cu;
    x ^= x * 0xb82f1e52u;
    x ^= x * 0xc7afe638u;
    x ^= x * 0x8d22f6e6u;
    return x;
}
__host__ __device__ __forceinline__ uint32_t owen_scramble(uint32_t x, uint32_t seed) {
    return reverse_bits32(laine_karras(reverse_bits32(x), seed));
}
__host__ __device__ __forceinline__ float ld_random_val(uint32_t index, uint32_t seed, uint32_t dim) {
    index = owen_scramble(index, seed);
    return (float)owen_scramble(sobol_dim(index, dim), hash_combine(seed, dim)) * 2.3283064365386963e-10f;
}
// ld_random_pixel_offset (:268-273); identical for every pixel, so the host evaluates it once.
inline void ld_random_pixel_offset_host(uint32_t spp, float* ox, float* oy) {
    const float a0 = ld_random_val(0, 0xdeadbeefu, 0), b0 = ld_random_val(0, 0xdeadbeefu, 1);
    const float a1 = ld_random_val(spp, 0xdeadbeefu, 0), b1 = ld_random_val(spp, 0xdeadbeefu, 1);
    const float x = (0.5f - a0) + a1, y = (0.5f - b0) + b1;
    *ox = x - floorf(x);
    *oy = y - floorf(y);
}

// ---- shard geometry ----------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t shard_ray_pixel(const DevView& v, uint64_t i) {
    const uint64_t lr = i / v.width;
    const uint32_t x = (uint32_t)(i - lr * v.width);
    const uint32_t b = v.shard_rank + (uint32_t)(lr / v.shard_rows) * v.shard_count;
    const uint32_t y = b * v.shard_rows + (uint32_t)(lr % v.shard_rows);
    return x + v.width * y;
}

// ---- bounding box: internal/sampler/bounding_box.h:145-191 -------------------------------------
__device__ __forceinline__ bool box_contains(const DevCfg& g, const V3& p) {
    return p.x >= g.box_min && p.x <= g.box_max && p.y >= g.box_min && p.y <= g.box_max &&
           p.z >= g.box_min && p.z <= g.box_max;
}
__device__ __forceinline__ void swapf(float& a, float& b) { const float t = a; a = b; b = t; }
__device__ __forceinline__ float box_ray_tmin(const DevCfg& g, const V3& pos, const V3& dir) {
    float tmin = (g.box_min - pos.x) / dir.x;
    float tmax = (g.box_max - pos.x) / dir.x;
    if (tmin > tmax) swapf(tmin, tmax);
    float tymin = (g.box_min - pos.y) / dir.y;
    float tymax = (g.box_max - pos.y) / dir.y;
    if (tymin > tymax) swapf(tymin, tymax);
    if ((tmin > tymax) || (tymin > tmax)) return 100000.0f;
    if (tymin > tmin) tmin = tymin;
    if (tymax < tmax) tmax = tymax;
    float tzmin = (g.box_min - pos.z) / dir.z;
    float tzmax = (g.box_max - pos.z) / dir.z;
    if (tzmin > tzmax) swapf(tzmin, tzmax);
    if ((tmin > tzmax) || (tzmin > tmax)) return 100000.0f;
    if (tzmin > tmin) tmin = tzmin;
    return tmin;
}

// ---- camera: internal/utils/common_device.h:143-165 ---------------------------------------------
__device__ __forceinline__ void pixel_to_ray(const DevView& v, uint32_t px, uint32_t py, V3* o, V3* d) {
    const float xx = ((float)px + v.off_x) / v.rw;
    const float yy = ((float)py + v.off_y) / v.rh;
    const float dx = (xx - v.ppx) * v.rw / v.fx;
    const float dy = (yy - v.ppy) * v.rh / v.fy;
    const float* m = v.cam;
    *o = mk3(m[3], m[7], m[11]);
    const float rx = srf_dot3f(m[0], dx, m[1], dy, m[2], 1.0f);
    const float ry = srf_dot3f(m[4], dx, m[5], dy, m[6], 1.0f);
    const float rz = srf_dot3f(m[8], dx, m[9], dy, m[10], 1.0f);
    const float n = srf_norm3f(rx, ry, rz);
    *d = mk3(rx / n, ry / n, rz / n);
}

// ---- step size: internal/sampler/occupancy_sampler.cu:287-331 ----------------------------------
__device__ __forceinline__ float calc_dt(const DevCfg& g, float t) {
    float dt = 0.f;
    switch (g.sampling_type) {
    case SRF_SAMPLING_ORIGINAL:
        dt = fminf(fmaxf(t * g.cone_angle, g.min_step), g.max_step);
        break;
    case SRF_SAMPLING_DISPARITY: {
        const float g_t0 = 1.f / t;
        const float g_t1 = fmaf(g.ds, g.g_diff, g_t0);
        const float t1 = 1.f / g_t1;
        dt = t1 - t;
        if (dt < 0.f) dt = t >= g.far_distance ? 0.f : g.far_distance - t;
    } break;
    case SRF_SAMPLING_LOG: {
        const float g_t0 = srf_logf(t);
        const float g_t1 = fmaf(g.ds, g.g_diff, g_t0);
        float t1 = srf_expf(g_t1);
        t1 = t1 < g.far_distance ? t1 : g.far_distance;
        dt = t1 - t;
    } break;
    default: break;
    }
    return dt;
}

// ---- warps: internal/utils/common_device.h:375-526 ---------------------------------------------
#define SRF_INV_PI 0.318309886183790671537767526745028724
#define SRF_PI 3.14159265358979323846

__device__ __forceinline__ V3 warp_sinusoidal(const V3& pos) {
    const V3 p = mk3(pos.x - 0.5f, pos.y - 0.5f, pos.z - 0.5f);
    float p_mag = srf_norm3f(p.x, p.y, p.z);
    const float p_mag_inv = 1.f / p_mag;
    const float theta = srf_atan2f(p.y, p.x);
    const float phi = srf_asinf(p.z * p_mag_inv);
    p_mag = (p_mag <= 1.f) ? p_mag : (2.f - p_mag_inv);
    p_mag *= 0.5f;
    V3 z;
    // M_1_PI is a double in the reference: both expressions are evaluated in fp64 (:443-444)
    const double tx = (double)(theta * srf_cosf(phi)) * SRF_INV_PI;
    z.x = (float)fma(tx, 0.5, 0.5);
    z.y = (float)fma((double)phi, SRF_INV_PI, 0.5);
    z.z = p_mag;
    return z;
}

__device__ __forceinline__ V3 warp_position(const DevCfg& g, const V3& pos) {
    V3 z = mk3(0.f, 0.f, 0.f);
    switch (g.warping_type) {
    case SRF_WARP_NGP:
        z = mk3((pos.x - g.box_min) / g.box_diag, (pos.y - g.box_min) / g.box_diag, (pos.z - g.box_min) / g.box_diag);
        break;
    case SRF_WARP_MIPNERF360: {
        const V3 x = mk3((pos.x - 0.5f) * 2.f, (pos.y - 0.5f) * 2.f, (pos.z - 0.5f) * 2.f);
        const float mag = srf_norm3f(x.x, x.y, x.z);
        const float inv = 1.f / mag;
        if (mag <= 1.f) z = x;
        else { const float s = (2.f - inv) * inv; z = mk3(s * x.x, s * x.y, s * x.z); }
        z = mk3(fmaf(z.x, 0.25f, 0.5f), fmaf(z.y, 0.25f, 0.5f), fmaf(z.z, 0.25f, 0.5f));
    } break;
    case SRF_WARP_DONERF: {
        const float dmax = srf_norm3f(g.box_diag, g.box_diag, g.box_diag);
        const V3 x = mk3(pos.x - 0.5f, pos.y - 0.5f, pos.z - 0.5f);
        const float mag = srf_norm3f(x.x, x.y, x.z);
        if (mag == 0.f) z = x;
        else { const float q = sqrtf(mag * dmax); z = mk3(x.x / q, x.y / q, x.z / q); }
        z = mk3(fmaf(z.x, 0.5f, 0.5f), fmaf(z.y, 0.5f, 0.5f), fmaf(z.z, 0.5f, 0.5f));
    } break;
    case SRF_WARP_SIGMOID:
        z = mk3(srf_logisticf(pos.x - 0.5f), srf_logisticf(pos.y - 0.5f), srf_logisticf(pos.z - 0.5f));
        break;
    case SRF_WARP_ERP:           // the reference's ERP case has no break and is overwritten by the next one
    case SRF_WARP_SINUSOIDAL:
        z = warp_sinusoidal(pos);
        break;
    default: break;
    }
    return z;
}

__device__ __forceinline__ V3 unwarp_position(const DevCfg& g, const V3& pos) {
    V3 x = mk3(0.f, 0.f, 0.f);
    switch (g.warping_type) {
    case SRF_WARP_NGP:
        x = mk3(fmaf(pos.x, g.box_diag, g.box_min), fmaf(pos.y, g.box_diag, g.box_min), fmaf(pos.z, g.box_diag, g.box_min));
        break;
    case SRF_WARP_MIPNERF360: {
        const V3 z = mk3((pos.x - 0.5f) * 4.f, (pos.y - 0.5f) * 4.f, (pos.z - 0.5f) * 4.f);
        const float mag = srf_norm3f(z.x, z.y, z.z);
        const float inv = 1.f / mag;
        if (mag <= 1.f) x = z;
        else { const float s = 1.f / (2.f - mag) * inv; x = mk3(s * z.x, s * z.y, s * z.z); }
        x = mk3(fmaf(x.x, 0.5f, 0.5f), fmaf(x.y, 0.5f, 0.5f), fmaf(x.z, 0.5f, 0.5f));
    } break;
    case SRF_WARP_DONERF: {
        const float dmax = srf_norm3f(g.box_diag, g.box_diag, g.box_diag);
        const V3 z = mk3((pos.x - 0.5f) * 2.f, (pos.y - 0.5f) * 2.f, (pos.z - 0.5f) * 2.f);
        const float mag = srf_norm3f(z.x, z.y, z.z);
        x = mk3(z.x * mag * dmax + 0.5f, z.y * mag * dmax + 0.5f, z.z * mag * dmax + 0.5f);
    } break;
    case SRF_WARP_SIGMOID:
        x = mk3(-srf_logf(1.f / pos.x - 1.f) + 0.5f, -srf_logf(1.f / pos.y - 1.f) + 0.5f, -srf_logf(1.f / pos.z - 1.f) + 0.5f);
        break;
    case SRF_WARP_ERP:
    case SRF_WARP_SINUSOIDAL: {
        const float phi = (float)((double)(pos.y - 0.5f) * SRF_PI);
        float sphi, cphi;
        srf_sincosf(phi, &sphi, &cphi);
        const float theta = (float)((double)((pos.x - 0.5f) * 2.f) * SRF_PI / (double)cphi);
        float p_mag = pos.z * 2.f;
        p_mag = (p_mag <= 1.f) ? p_mag : 1.f / (2.f - p_mag);
        float sth, cth;
        srf_sincosf(theta, &sth, &cth);
        x = mk3(p_mag * cphi * cth + 0.5f, p_mag * cphi * sth + 0.5f, p_mag * sphi + 0.5f);
    } break;
    default: break;
    }
    return x;
}

// ---- occupancy lookup: internal/sampler/occupancy_sampler.cu:349-469 ---------------------------
__device__ __forceinline__ uint32_t level_from_pos(const DevCfg& g, const V3& pos, const V3& w) {
    const uint32_t nc = g.n_cascades;
    if (nc == 1) return 0;
    float maxval;
    if (g.grid_dist == SRF_GRID_WARPED_EXP || g.grid_dist == SRF_GRID_WARPED_RECIPROCAL)
        maxval = fmaxf(fmaxf(fabsf(w.x - 0.5f), fabsf(w.y - 0.5f)), fabsf(w.z - 0.5f));
    else
        maxval = fmaxf(fmaxf(fabsf((pos.x - 0.5f) / g.box_diag), fabsf((pos.y - 0.5f) / g.box_diag)),
                       fabsf((pos.z - 0.5f) / g.box_diag));
    maxval *= 2.f;
    uint32_t mip = 0;
    for (; mip + 1 < nc; ++mip) {
        bool got;
        if (g.grid_dist == SRF_GRID_WARPED_EXP || g.grid_dist == SRF_GRID_METRIC_EXP)
            got = maxval > scalbnf(1.f, -1 - (int)mip);
        else
            got = maxval > 1.f / (float)(mip + 2);
        if (got) break;
    }
    return nc - mip - 1;
}

__device__ __forceinline__ uint32_t cascaded_grid_idx_at(const DevCfg& g, const V3& pos, const V3& w, uint32_t level) {
    const uint32_t nc = g.n_cascades, N = g.grid_size;
    V3 p;
    float s;
    switch (g.grid_dist) {
    case SRF_GRID_WARPED_EXP:
        s = scalbnf(1.0f, (int)(nc - level - 1));
        p = mk3((w.x - 0.5f) * s + 0.5f, (w.y - 0.5f) * s + 0.5f, (w.z - 0.5f) * s + 0.5f);
        break;
    case SRF_GRID_WARPED_RECIPROCAL:
        s = (float)(nc - level);
        p = mk3((w.x - 0.5f) * s + 0.5f, (w.y - 0.5f) * s + 0.5f, (w.z - 0.5f) * s + 0.5f);
        break;
    case SRF_GRID_METRIC_EXP:
        s = scalbnf(1.0f, (int)(nc - level - 1));
        p = mk3((pos.x - 0.5f) / g.box_diag * s + 0.5f, (pos.y - 0.5f) / g.box_diag * s + 0.5f,
                (pos.z - 0.5f) / g.box_diag * s + 0.5f);
        break;
    default:
        s = (float)(nc - level);
        p = mk3((pos.x - 0.5f) / g.box_diag * s + 0.5f, (pos.y - 0.5f) / g.box_diag * s + 0.5f,
                (pos.z - 0.5f) / g.box_diag * s + 0.5f);
        break;
    }
    const float fn = (float)N;
    const int hi = (int)N - 1;
    const int ix = min(max(srf_f2i_rz(p.x * fn), 0), hi);
    const int iy = min(max(srf_f2i_rz(p.y * fn), 0), hi);
    const int iz = min(max(srf_f2i_rz(p.z * fn), 0), hi);
    return morton3D((uint32_t)ix, (uint32_t)iy, (uint32_t)iz);
}

// ---- PCG32 (the generator behind the reference's default_rng_t) ------------------------------------
struct Pcg { uint64_t state, inc; };
constexpr uint64_t kPcgMult = 0x5851f42d4c957f2dULL;
__device__ __forceinline__ uint32_t pcg_next_uint(Pcg& r) {
    const uint64_t old = r.state;
    r.state = old * kPcgMult + r.inc;
    const uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    const uint32_t rot = (uint32_t)(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31));
}
__device__ __forceinline__ float pcg_next_float(Pcg& r) {
    return __uint_as_float((pcg_next_uint(r) >> 9) | 0x3f800000u) - 1.0f;
}
__device__ __forceinline__ void pcg_advance(Pcg& r, uint64_t delta) {
    uint64_t cur_mult = kPcgMult, cur_plus = r.inc, acc_mult = 1u, acc_plus = 0u;
    while (delta > 0) {
        if (delta & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
        cur_plus = (cur_mult + 1) * cur_plus;
        cur_mult *= cur_mult;
        delta >>= 1;
    }
    r.state = acc_mult * r.state + acc_plus;
}

// pcg_advance for 32-bit distances without the 32-iteration square-and-multiply loop: the jump by
// delta = sum_k b_k * 256^k is the composition of four table jumps.  A jump by d maps state to
// m^d * state + inc * (1 + m + ... + m^(d-1)); the table holds both factors for every d = b * 256^k
// (they depend only on the generator's multiplier), 16 KB of constants computed at compile time.
struct PcgJumpTable { uint64_t mult[4][256]; uint64_t geo[4][256]; };
constexpr PcgJumpTable make_pcg_jump_table() {
    PcgJumpTable t{};
    for (int k = 0; k < 4; ++k)
        for (int b = 0; b < 256; ++b) {
            uint64_t delta = (uint64_t)b << (8 * k);
            uint64_t cur_mult = kPcgMult, cur_plus = 1u, acc_mult = 1u, acc_plus = 0u;
            while (delta > 0) {
                if (delta & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
                cur_plus = (cur_mult + 1) * cur_plus;
                cur_mult *= cur_mult;
                delta >>= 1;
            }
            t.mult[k][b] = acc_mult;
            t.geo[k][b] = acc_plus;
        }
    return t;
}
static __device__ const PcgJumpTable kPcgJump = make_pcg_jump_table();
__device__ __forceinline__ void pcg_jump(Pcg& r, uint32_t delta) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t b = (delta >> (8 * k)) & 255u;
        if (b) r.state = kPcgJump.mult[k][b] * r.state + kPcgJump.geo[k][b] * r.inc;
    }
}

// ---- one ray ---------------------------------------------------------------------------------------
enum RayEnd : uint32_t {
    RAY_END_EXIT = 0,       // left the box
    RAY_END_DT0 = 1,        // step size reached 0 in an empty cell
    RAY_END_STUCK = 2,      // step size reached 0 in an occupied cell: alive until the reference's loop bound
    RAY_END_LIMIT = 3,      // the march loop's hard bound (an error)
    RAY_END_BORN_DEAD = 4,  // entry point outside the box
    RAY_END_CAP = 5,        // sample cap reached
    RAY_END_TERMINATED = 6, // stopped by the consumer (early termination)
    RAY_END_PAUSED = 7,     // the wave's step budget is used up: the march resumes later from the saved MarchState
    RAY_END_DONE = 8        // frame path: the ray's pixel has been written by an earlier wave
};

// Where a march stands: ray parameter, loop iterations so far, samples emitted so far.
struct MarchState { float t; uint32_t ordinal, n; };

struct RayInit { bool alive; V3 o, d; float t; };

// init_rays_with_payload_kernel_nerf (:691-736) + the jitter of advance_pos_nerf (:766-768)
__device__ __forceinline__ RayInit init_ray(const DevCfg& g, const DevView& v, uint32_t pixel) {
    RayInit r;
    const uint32_t py = pixel / v.width, px = pixel - py * v.width;
    pixel_to_ray(v, px, py, &r.o, &r.d);
    const float t = fmaxf(box_ray_tmin(g, r.o, r.d), 0.05f) + 1e-6f;
    const V3 p = mk3(fmaf(r.d.x, t, r.o.x), fmaf(r.d.y, t, r.o.y), fmaf(r.d.z, t, r.o.z));
    r.alive = box_contains(g, p);
    r.t = t;
    if (r.alive) {
        const float dt = calc_dt(g, t);
        r.t = fmaf(ld_random_val(v.spp_index, pixel * 786433u, 0), dt, t);
    }
    return r;
}

// One march step's occupancy lookup: warped position *w, Morton cell index *idx (+ level * cells), and
// whether the cell's bit is set (warp_position + level_from_pos + density_grid_occupied_at,
// occupancy_sampler.cu:786-788).  Without a grid every step counts as occupied.  When the lookup says
// "empty", *w and *idx may be partly unset: callers use them only for occupied steps.
__device__ __forceinline__ bool grid_lookup(const DevCfg& g, const uint8_t* __restrict__ bits, const V3& pos, V3* w_out,
                                            uint32_t* idx_out) {
    V3 w;
    bool occ = true;
    uint32_t idx = 0;
    if (g.skip_shell) {
        // Staged evaluation of warp_sinusoidal + cascaded_grid_idx_at for one cascade: the radial cell
        // index needs only |p|, the latitude index only asin; a 1-D and a 2-D summary of the bitfield
        // tell whether any occupied cell has these indices.  Every expression is the one the full path
        // evaluates, so the decision (and the sample, when there is one) is bit-identical to it; the
        // atan2 / cos / fp64 part -- most of a step's cost -- runs only where it can matter.
        const uint32_t N = g.grid_size;
        const float fn = (float)N, s1 = 1.0f;
        const int hi = (int)N - 1;
        const V3 p = mk3(pos.x - 0.5f, pos.y - 0.5f, pos.z - 0.5f);
        float p_mag = srf_norm3f(p.x, p.y, p.z);
        const float p_mag_inv = 1.f / p_mag;
        p_mag = (p_mag <= 1.f) ? p_mag : (2.f - p_mag_inv);
        w.z = p_mag * 0.5f;
        w.x = w.y = 0.f;
        const uint32_t iz = (uint32_t)min(max(srf_f2i_rz(((w.z - 0.5f) * s1 + 0.5f) * fn), 0), hi);
        occ = (__ldg(g.skip_shell + (iz >> 5)) >> (iz & 31u)) & 1u;
        if (occ) {
            const float phi = srf_asinf(p.z * p_mag_inv);
            w.y = (float)fma((double)phi, SRF_INV_PI, 0.5);
            const uint32_t iy = (uint32_t)min(max(srf_f2i_rz(((w.y - 0.5f) * s1 + 0.5f) * fn), 0), hi);
            const uint32_t yz = iz * N + iy;
            occ = (__ldg(g.skip_yz + (yz >> 5)) >> (yz & 31u)) & 1u;
            if (occ) {
                const float theta = srf_atan2f(p.y, p.x);
                const double tx = (double)(theta * srf_cosf(phi)) * SRF_INV_PI;
                w.x = (float)fma(tx, 0.5, 0.5);
                const uint32_t ix = (uint32_t)min(max(srf_f2i_rz(((w.x - 0.5f) * s1 + 0.5f) * fn), 0), hi);
                idx = morton3D(ix, iy, iz);
                occ = (__ldg(bits + (idx >> 3)) >> (idx & 7u)) & 1u;
            }
        }
    } else {
        w = warp_position(g, pos);
        if (g.use_grid) {
            const uint32_t level = level_from_pos(g, pos, w);
            idx = cascaded_grid_idx_at(g, pos, w, level) + level * g.cells;
            occ = (__ldg(bits + (idx >> 3)) >> (idx & 7u)) & 1u;
        }
    }
    *w_out = w;
    *idx_out = idx;
    return occ;
}

// grid_lookup for two positions at once (staged path only: g.skip_shell set).  Each stage is evaluated for both
// positions when either needs it, so that the two dependent chains overlap; every expression is the one
// grid_lookup evaluates, and a stage computed for a position that did not need it is simply not used.
__device__ __forceinline__ void grid_lookup_pair(const DevCfg& g, const uint8_t* __restrict__ bits, const V3& pos0, const V3& pos1,
                                                 V3* w0_out, uint32_t* idx0_out, bool* occ0_out, V3* w1_out, uint32_t* idx1_out,
                                                 bool* occ1_out) {
    const uint32_t N = g.grid_size;
    const float fn = (float)N, s1 = 1.0f;
    const int hi = (int)N - 1;
    const V3 p0 = mk3(pos0.x - 0.5f, pos0.y - 0.5f, pos0.z - 0.5f), p1 = mk3(pos1.x - 0.5f, pos1.y - 0.5f, pos1.z - 0.5f);
    float m0 = srf_norm3f(p0.x, p0.y, p0.z), m1 = srf_norm3f(p1.x, p1.y, p1.z);
    const float inv0 = 1.f / m0, inv1 = 1.f / m1;
    m0 = (m0 <= 1.f) ? m0 : (2.f - inv0);
    m1 = (m1 <= 1.f) ? m1 : (2.f - inv1);
    V3 w0 = mk3(0.f, 0.f, m0 * 0.5f), w1 = mk3(0.f, 0.f, m1 * 0.5f);
    const uint32_t iz0 = (uint32_t)min(max(srf_f2i_rz(((w0.z - 0.5f) * s1 + 0.5f) * fn), 0), hi);
    const uint32_t iz1 = (uint32_t)min(max(srf_f2i_rz(((w1.z - 0.5f) * s1 + 0.5f) * fn), 0), hi);
    bool occ0 = (__ldg(g.skip_shell + (iz0 >> 5)) >> (iz0 & 31u)) & 1u;
    bool occ1 = (__ldg(g.skip_shell + (iz1 >> 5)) >> (iz1 & 31u)) & 1u;
    uint32_t idx0 = 0, idx1 = 0;
    if (occ0 | occ1) {
        const float phi0 = srf_asinf(p0.z * inv0), phi1 = srf_asinf(p1.z * inv1);
        w0.y = (float)fma((double)phi0, SRF_INV_PI, 0.5);
        w1.y = (float)fma((double)phi1, SRF_INV_PI, 0.5);
        const uint32_t iy0 = (uint32_t)min(max(srf_f2i_rz(((w0.y - 0.5f) * s1 + 0.5f) * fn), 0), hi);
        const uint32_t iy1 = (uint32_t)min(max(srf_f2i_rz(((w1.y - 0.5f) * s1 + 0.5f) * fn), 0), hi);
        const uint32_t yz0 = iz0 * N + iy0, yz1 = iz1 * N + iy1;
        occ0 = occ0 && ((__ldg(g.skip_yz + (yz0 >> 5)) >> (yz0 & 31u)) & 1u);
        occ1 = occ1 && ((__ldg(g.skip_yz + (yz1 >> 5)) >> (yz1 & 31u)) & 1u);
        if (occ0 | occ1) {
            const float th0 = srf_atan2f(p0.y, p0.x), th1 = srf_atan2f(p1.y, p1.x);
            const double tx0 = (double)(th0 * srf_cosf(phi0)) * SRF_INV_PI, tx1 = (double)(th1 * srf_cosf(phi1)) * SRF_INV_PI;
            w0.x = (float)fma(tx0, 0.5, 0.5);
            w1.x = (float)fma(tx1, 0.5, 0.5);
            const uint32_t ix0 = (uint32_t)min(max(srf_f2i_rz(((w0.x - 0.5f) * s1 + 0.5f) * fn), 0), hi);
            const uint32_t ix1 = (uint32_t)min(max(srf_f2i_rz(((w1.x - 0.5f) * s1 + 0.5f) * fn), 0), hi);
            idx0 = morton3D(ix0, iy0, iz0);
            idx1 = morton3D(ix1, iy1, iz1);
            occ0 = occ0 && ((__ldg(bits + (idx0 >> 3)) >> (idx0 & 7u)) & 1u);
            occ1 = occ1 && ((__ldg(bits + (idx1 >> 3)) >> (idx1 & 7u)) & 1u);
        }
    }
    *w0_out = w0; *idx0_out = idx0; *occ0_out = occ0;
    *w1_out = w1; *idx1_out = idx1; *occ1_out = occ1;
}

// The loop shared by advance_pos_nerf (:771-794) and generate_coords_from_rays_regularly_kernel
// (:829-860), run from `st` until the ray ends, the consumer stops it, or the loop has made `pause_at`
// iterations in all (RAY_END_PAUSED: `st` then holds the state to resume from).  emit(w, dt, ordinal, cell, t)
// is called for every occupied step and returns false to stop.  Returns the RayEnd; st.ordinal counts the
// loop iterations of the whole ray.  Pausing on the iteration count (not on the number of samples) keeps the
// lanes of a warp in step: they all pause after the same number of iterations.
template <class Emit>
__device__ __forceinline__ uint32_t march_ray_from(const DevCfg& g, const uint8_t* __restrict__ bits, const V3& o,
                                                   const V3& d, MarchState& st, uint32_t pause_at, Emit emit) {
    float t = st.t;
    uint32_t ordinal = st.ordinal, n = st.n;
    const uint32_t stop = pause_at < g.step_limit ? pause_at : g.step_limit;
    uint32_t end = pause_at < g.step_limit ? RAY_END_PAUSED : RAY_END_LIMIT;
    // Two steps per iteration where the staged lookup applies: t advances by calc_dt(t) whether or not a step is
    // occupied, so step k+1's position does not wait for step k's lookup and the two lookups overlap (one dependent
    // chain per thread left half of the issue slots empty: 28.2 -> 21.4 ms per benchmark frame; three and four steps
    // in flight were no faster).  The steps are then consumed in order exactly as the loop below consumes them; what
    // was computed for a step behind a stop is dropped.
    bool stopped = false;
#if !defined(SRF_MARCH_SINGLE_STEP)
    if (g.skip_shell) {
        while (ordinal + 1 < stop) {
            const float t0 = t;
            const V3 pos0 = mk3(fmaf(d.x, t0, o.x), fmaf(d.y, t0, o.y), fmaf(d.z, t0, o.z));
            const float dt0 = calc_dt(g, t0);
            const float t1 = t0 + dt0;
            const V3 pos1 = mk3(fmaf(d.x, t1, o.x), fmaf(d.y, t1, o.y), fmaf(d.z, t1, o.z));
            const float dt1 = calc_dt(g, t1);
            if (!box_contains(g, pos0)) { end = RAY_END_EXIT; ++ordinal; stopped = true; break; }
            V3 w0, w1;
            uint32_t idx0, idx1;
            bool occ0, occ1;
            grid_lookup_pair(g, bits, pos0, pos1, &w0, &idx0, &occ0, &w1, &idx1, &occ1);
            if (occ0) {
                if (dt0 == 0.f) { end = RAY_END_STUCK; ++ordinal; stopped = true; break; }
                if (n >= g.sample_cap) { end = RAY_END_CAP; ++ordinal; stopped = true; break; }
                ++n;
                if (!emit(w0, dt0, ordinal, idx0, t0)) { end = RAY_END_TERMINATED; ++ordinal; stopped = true; break; }
                t = t1;
            } else {
                t = t1;
                if (dt0 == 0.f) { end = RAY_END_DT0; ++ordinal; stopped = true; break; }
            }
            ++ordinal;
            if (!box_contains(g, pos1)) { end = RAY_END_EXIT; ++ordinal; stopped = true; break; }
            if (occ1) {
                if (dt1 == 0.f) { end = RAY_END_STUCK; ++ordinal; stopped = true; break; }
                if (n >= g.sample_cap) { end = RAY_END_CAP; ++ordinal; stopped = true; break; }
                ++n;
                if (!emit(w1, dt1, ordinal, idx1, t1)) { end = RAY_END_TERMINATED; ++ordinal; stopped = true; break; }
                t = t1 + dt1;
            } else {
                t = t1 + dt1;
                if (dt1 == 0.f) { end = RAY_END_DT0; ++ordinal; stopped = true; break; }
            }
            ++ordinal;
        }
    }
#endif
    if (!stopped)
    for (; ordinal < stop; ++ordinal) {
        const V3 pos = mk3(fmaf(d.x, t, o.x), fmaf(d.y, t, o.y), fmaf(d.z, t, o.z));
        if (!box_contains(g, pos)) { end = RAY_END_EXIT; ++ordinal; break; }
        const float dt = calc_dt(g, t);
        V3 w;
        uint32_t idx;
        const bool occ = grid_lookup(g, bits, pos, &w, &idx);
        if (occ) {
            if (dt == 0.f) { end = RAY_END_STUCK; ++ordinal; break; }
            if (n >= g.sample_cap) { end = RAY_END_CAP; ++ordinal; break; }
            ++n;
            if (!emit(w, dt, ordinal, idx, t)) { end = RAY_END_TERMINATED; ++ordinal; break; }
            t += dt;
        } else {
            t += dt;
            if (dt == 0.f) { end = RAY_END_DT0; ++ordinal; break; }
        }
    }
    st.t = t; st.ordinal = ordinal; st.n = n;
    return end;
}

// The whole march in one go.  *n_steps receives the loop iterations.
template <class Emit>
__device__ __forceinline__ uint32_t march_ray(const DevCfg& g, const uint8_t* __restrict__ bits, const V3& o,
                                              const V3& d, float t, uint32_t* n_steps, Emit emit) {
    MarchState st = {t, 0u, 0u};
    const uint32_t end = march_ray_from(g, bits, o, d, st, 0xffffffffu, emit);
    *n_steps = st.ordinal;
    return end;
}

// ---- activations and colour (internal/utils/common_device.h:70-88,320-351) -----------------------
__device__ __forceinline__ float network_to_rgb(float v, int act) {
    switch (act) {
    case SRF_ACT_NONE: return v;
    case SRF_ACT_RELU: return v > 0.f ? v : 0.f;
    case SRF_ACT_LOGISTIC: return srf_logisticf(v);
    case SRF_ACT_EXPONENTIAL: return srf_expf(fminf(fmaxf(v, -10.f), 10.f));
    default: return 0.f;
    }
}
__device__ __forceinline__ float network_to_density(float v, int act) {
    switch (act) {
    case SRF_ACT_NONE: return v;
    case SRF_ACT_RELU: return v > 0.f ? v : 0.f;
    case SRF_ACT_LOGISTIC: return srf_logisticf(v);
    case SRF_ACT_EXPONENTIAL: return srf_expf(v);
    default: return 0.f;
    }
}
__device__ __forceinline__ float network_to_rgb_derivative(float v, int act) {          // common_device.h:331-340
    switch (act) {
    case SRF_ACT_NONE: return 1.0f;
    case SRF_ACT_RELU: return v > 0.f ? 1.0f : 0.0f;
    case SRF_ACT_LOGISTIC: { const float d = srf_logisticf(v); return d * (1.f - d); }
    case SRF_ACT_EXPONENTIAL: return srf_expf(fminf(fmaxf(v, -10.f), 10.f));
    default: return 0.f;
    }
}
__device__ __forceinline__ float network_to_density_derivative(float v, int act) {      // common_device.h:353-362
    switch (act) {
    case SRF_ACT_NONE: return 1.0f;
    case SRF_ACT_RELU: return v > 0.f ? 1.0f : 0.0f;
    case SRF_ACT_LOGISTIC: { const float d = srf_logisticf(v); return d * (1.f - d); }
    case SRF_ACT_EXPONENTIAL: return srf_expf(fminf(fmaxf(v, -15.f), 15.f));
    default: return 0.f;
    }
}

#if defined(SRF_CANON_CUDA_MATH)
__device__ __forceinline__ float srf_powf(float x, float y) { return powf(x, y); }      // test-only build: see srf_canon_math.h
#else
__device__ __forceinline__ float srf_powf(float x, float y) { return x > 0.f ? srf_expf(y * srf_logf(x)) : 0.f; }
#endif
__device__ __forceinline__ float srgb_to_linear(float s) {
    return s <= 0.04045f ? s / 12.92f : srf_powf((s + 0.055f) / 1.055f, 2.4f);
}
__device__ __forceinline__ float linear_to_srgb(float l) {
    return l < 0.0031308f ? 12.92f * l : 1.055f * srf_powf(l, 0.41666f) - 0.055f;
}

// What the compositor needs from one sample: the activated colour and the opacity of the step
// (volume_rendering_kernel, internal/render/ray_marcher.cu:236-265).  raw = (r, g, b, sigma) as the
// field returned them; w = warped position (for the depth modes).
__device__ __forceinline__ float4 shade_finish(const DevCfg& g, const DevView& v, float sigma, float cr, float cg, float cb,
                                               float dt, const V3& w) {
    const float alpha = 1.f - srf_expf(-sigma * dt);
    if (v.render_mode == SRF_MODE_DEPTH || v.render_mode == SRF_MODE_DISTANCE) {
        const V3 p = unwarp_position(g, w);
        const float dx = p.x - v.cam[3], dy = p.y - v.cam[7], dz = p.z - v.cam[11];
        float zz;
        if (v.render_mode == SRF_MODE_DEPTH) zz = srf_dot3f(v.cam[2], dx, v.cam[6], dy, v.cam[10], dz) * v.depth_scale;
        else zz = srf_norm3f(dx, dy, dz) * v.depth_scale;
        cr = cg = cb = zz;
    } else if (v.render_mode == SRF_MODE_AO) {
        cr = cg = cb = alpha;
    }
    return make_float4(cr, cg, cb, alpha);
}
__device__ __forceinline__ float4 shade_sample(const DevCfg& g, const DevView& v, const float (&raw)[4], float dt, const V3& w) {
    return shade_finish(g, v, network_to_density(raw[3], g.density_activation), network_to_rgb(raw[0], g.rgb_activation),
                        network_to_rgb(raw[1], g.rgb_activation), network_to_rgb(raw[2], g.rgb_activation), dt, w);
}
// The same with the activations read from a table.  The network's outputs are fp16 numbers, so an activation has
// 65 536 possible arguments: lut[h] = network_to_rgb(value of the half with bits h), lut[65536 + h] =
// network_to_density(...), filled by the functions above (the table holds exactly what they return).
__device__ __forceinline__ float4 shade_sample_lut(const DevCfg& g, const DevView& v, const float* __restrict__ lut,
                                                   uint32_t hr, uint32_t hg, uint32_t hb, uint32_t hs, float dt, const V3& w) {
    return shade_finish(g, v, __ldg(lut + 65536 + hs), __ldg(lut + hr), __ldg(lut + hg), __ldg(lut + hb), dt, w);
}

}  // namespace srf
