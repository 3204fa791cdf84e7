// srf_training.cu -- the sampler's training-side entry points.
//
//   k_mark_untrained      mark_untrained_density_grid (internal/sampler/occupancy_sampler.cu:12-102)
//   k_train_count / emit  generate_training_samples_nerf (:513-689)
//
// The reference's training sampler reserves each ray's slots with atomicAdd on two global counters, so the
// order of rays and samples in its output changes from run to run.  Here the same per-ray work is split into
// a counting march (a warp per ray: see train_march_warp), two exclusive scans (samples per ray -> base; "has samples" -> compacted ray index) and
// an emitting march: the output is the one a serial execution of the reference kernel (ray 0, 1, 2, ...)
// would produce, every time, and sample writes of neighbouring rays land next to each other.
#include "srf_kernels.cuh"

namespace srf {

namespace {


__device__ __forceinline__ float dot3(const V3& a, const float* b) {
    return srf_dot3f(a.x, b[0], a.y, b[1], a.z, b[2]);
}

__global__ void __launch_bounds__(256)
k_mark_untrained(const DevCfg g, uint32_t n_elements, uint32_t aabb_scale, uint32_t n_images, int width, int height,
                 float focal_x, float focal_y, const float* __restrict__ xforms, float* __restrict__ grid_out) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elements) return;
    const uint32_t N = g.grid_size, nc = g.n_cascades;
    const uint32_t level = i / g.cells, pos_idx = i % g.cells;
    const uint32_t x = morton3D_invert(pos_idx >> 0), y = morton3D_invert(pos_idx >> 1), z = morton3D_invert(pos_idx >> 2);
    const float fn = (float)N;
    V3 pos = mk3(((float)x + 0.5f) / fn - 0.5f, ((float)y + 0.5f) / fn - 0.5f, ((float)z + 0.5f) / fn - 0.5f);
    const int down = -(int)(nc - level - 1);
    const float fa = (float)aabb_scale, fl = (float)(nc - level);
    float s;
    switch (g.grid_dist) {
    case SRF_GRID_WARPED_EXP:
        s = scalbnf(1.0f, down);
        pos = mk3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
        pos = unwarp_position(g, pos);
        break;
    case SRF_GRID_WARPED_RECIPROCAL:
        pos = mk3(pos.x / fl + 0.5f, pos.y / fl + 0.5f, pos.z / fl + 0.5f);
        pos = unwarp_position(g, pos);
        break;
    case SRF_GRID_METRIC_EXP:
        s = scalbnf(fa, down);
        pos = mk3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
        // the reference has no `break` here (:52-57): the reciprocal scaling is applied on top
    case SRF_GRID_METRIC_RECIPROCAL:
        s = fa / fl;
        pos = mk3(pos.x * s + 0.5f, pos.y * s + 0.5f, pos.z * s + 0.5f);
        break;
    default: break;
    }
    const float half_resx = (float)width * 0.5f, half_resy = (float)height * 0.5f;
    float voxel_radius = 0.5f * 1.73205080757f * fa / fn;
    if (g.grid_dist == SRF_GRID_WARPED_EXP || g.grid_dist == SRF_GRID_METRIC_EXP) voxel_radius *= scalbnf(1.0f, down);
    else voxel_radius /= fl;
    bool seen = false;
    for (uint32_t j = 0; j < n_images && !seen; ++j) {
        const float* m = xforms + (size_t)j * 12;            // 3x4, column-major
        const V3 ploc = mk3(pos.x - m[9], pos.y - m[10], pos.z - m[11]);
        const float cx = dot3(ploc, m + 0), cy = dot3(ploc, m + 3), cz = dot3(ploc, m + 6);
        if (cz > 0.f)
            seen = fabsf(cx) - voxel_radius < cz / focal_x * half_resx && fabsf(cy) - voxel_radius < cz / focal_y * half_resy;
    }
    grid_out[i] = seen ? 0.f : -1.f;
}

struct TrainRay {
    bool valid;
    V3 o, d;
    float t;              // start of the march (after the jitter)
    uint64_t pixel;       // pixel_idx: x + y*W + img*W*H
};

// Lines :544-594 of the reference kernel: image, pixel, probability test, ray, box entry, jitter.
__device__ __forceinline__ TrainRay train_ray_setup(const DevCfg& g, const TrainViews& tv, uint32_t i, uint32_t n_rays,
                                                    uint32_t n_rays_shift, Pcg rng, int snap) {
    TrainRay r;
    r.valid = false;
    const uint32_t img = (((n_rays_shift + i) * tv.n_images) / n_rays) % tv.n_images;      // u32 arithmetic (:544)
    pcg_jump(rng, i * 8u);                                  // rng.advance(i * 8) with the reference's u32 product (:551)
    float xx = pcg_next_float(rng);
    float yy = pcg_next_float(rng);
    const float rw = (float)tv.width, rh = (float)tv.height;
    if (snap) {
        xx = ((float)min(max(srf_f2i_rz(xx * rw), 0), tv.width - 1) + 0.5f) / rw;
        yy = ((float)min(max(srf_f2i_rz(yy * rh), 0), tv.height - 1) + 0.5f) / rh;
    }
    const int px = max(min(srf_f2i_rz(xx * rw), tv.width - 1), 0), py = max(min(srf_f2i_rz(yy * rh), tv.height - 1), 0);
    r.pixel = (uint64_t)(int64_t)(px + py * tv.width) + (uint64_t)img * (uint64_t)tv.width * (uint64_t)tv.height;
    if (tv.sampling_probability && __half2float(tv.sampling_probability[r.pixel]) <= 0.f) return r;     // :570-571
    const float* m = tv.xforms + (size_t)img * 12;            // 3x4, column-major
    r.o = mk3(m[9], m[10], m[11]);
    const float dx = (xx - tv.pp_x) * rw / tv.focal_x;
    const float dy = (yy - tv.pp_y) * rh / tv.focal_y;
    const float rx = srf_dot3f(m[0], dx, m[3], dy, m[6], 1.0f);
    const float ry = srf_dot3f(m[1], dx, m[4], dy, m[7], 1.0f);
    const float rz = srf_dot3f(m[2], dx, m[5], dy, m[8], 1.0f);
    const float n = srf_norm3f(rx, ry, rz);
    r.d = mk3(rx / n, ry / n, rz / n);
    const float t0 = fmaxf(box_ray_tmin(g, r.o, r.d), g.near_distance);
    r.t = fmaf(pcg_next_float(rng), calc_dt(g, t0), t0);
    r.valid = true;
    return r;
}

// The two marches of the reference kernel (:596-628 and :650-688), run by a whole warp for one ray.  The
// recurrence t += calc_dt(t) is cheap and inherently serial: every lane replays 32 steps of it and keeps the t
// of "its" step; the expensive part of a step (box test, warp, level, bit lookup) then runs on the 32 steps in
// parallel, and ballots give each occupied step its index within the ray.  The values of t, dt and the
// positions are exactly those of the serial loop; emit(j, w, dt) is called by the lane that owns occupied step
// j, for j < limit.  Returns the number of occupied steps (the same in all lanes), at most `limit`.
template <class Emit>
__device__ __forceinline__ uint32_t train_march_warp(const DevCfg& g, const uint8_t* __restrict__ bits, const TrainRay& r,
                                                     uint32_t limit, Emit emit) {
    const int lane = threadIdx.x & 31;
    uint32_t j = 0;
    float t = r.t;
    for (uint32_t block = 0; block < (g.step_limit >> 5) && j < limit; ++block) {
        float my_t = 0.f, my_dt = 0.f;
#pragma unroll 4
        for (int k = 0; k < 32; ++k) {
            const float dt = calc_dt(g, t);
            if (k == lane) { my_t = t; my_dt = dt; }
            t += dt;
        }
        const V3 pos = mk3(fmaf(r.d.x, my_t, r.o.x), fmaf(r.d.y, my_t, r.o.y), fmaf(r.d.z, my_t, r.o.z));
        const bool inside = box_contains(g, pos);
        const unsigned out_mask = __ballot_sync(0xffffffffu, !inside);          // the loop ends before the first such step
        const unsigned zero_mask = __ballot_sync(0xffffffffu, my_dt == 0.f);    // and after the first step with dt == 0
        unsigned valid = out_mask ? ((1u << (__ffs(out_mask) - 1)) - 1u) : 0xffffffffu;
        if (zero_mask) {
            const int z = __ffs(zero_mask) - 1;
            valid &= (z == 31) ? 0xffffffffu : ((2u << z) - 1u);
        }
        const bool mine = (valid >> lane) & 1u;
        V3 w = mk3(0.f, 0.f, 0.f);
        uint32_t idx;
        bool occ = false;
        if (mine) occ = grid_lookup(g, bits, pos, &w, &idx);
        const unsigned occ_mask = __ballot_sync(0xffffffffu, occ);
        const uint32_t my_j = j + __popc(occ_mask & ((1u << lane) - 1u));
        if (occ && my_j < limit) emit(my_j, w, my_dt);
        j += __popc(occ_mask);
        if (valid != 0xffffffffu) break;
    }
    return j < limit ? j : limit;
}

constexpr int kTrainWarpBlock = 128;      // 4 rays per block

__global__ void __launch_bounds__(kTrainWarpBlock)
k_train_count(const DevCfg g, const TrainViews tv, const uint8_t* __restrict__ bits, uint32_t n_rays, uint32_t n_rays_shift,
              uint32_t n_max_steps, Pcg rng, int snap, uint32_t* __restrict__ counts, uint32_t* __restrict__ flags) {
    const uint32_t i = (blockIdx.x * kTrainWarpBlock + threadIdx.x) >> 5;
    if (i >= n_rays) return;
    const TrainRay r = train_ray_setup(g, tv, i, n_rays, n_rays_shift, rng, snap);
    uint32_t n = 0;
    if (r.valid) n = train_march_warp(g, bits, r, n_max_steps, [](uint32_t, const V3&, float) {});
    if ((threadIdx.x & 31) == 0) {
        counts[i] = n;
        flags[i] = n ? 1u : 0u;
    }
}

__global__ void __launch_bounds__(kTrainWarpBlock)
k_train_emit(const DevCfg g, const TrainViews tv, const uint8_t* __restrict__ bits, uint32_t n_rays, uint32_t n_rays_shift,
             uint32_t n_coords, Pcg rng, int snap, const uint32_t* __restrict__ counts, const uint64_t* __restrict__ offsets,
             const uint64_t* __restrict__ ray_rank, uint32_t* __restrict__ ray_counter, uint32_t* __restrict__ numsteps_counter,
             float* __restrict__ rays_out, float* __restrict__ rays_rgba, uint32_t* __restrict__ numsteps_out,
             float* __restrict__ coords_out) {
    const uint32_t i = (blockIdx.x * kTrainWarpBlock + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i == 0 && lane == 0) *numsteps_counter = (uint32_t)offsets[n_rays];   // includes the rays that found no room, as :633 does
    if (i >= n_rays) return;
    const uint32_t numsteps = counts[i];
    if (numsteps == 0) return;
    const uint64_t base = offsets[i];
    if (base + numsteps > (uint64_t)n_coords) return;                  // :634-636
    const uint32_t ray_idx = (uint32_t)ray_rank[i];
    const TrainRay r = train_ray_setup(g, tv, i, n_rays, n_rays_shift, rng, snap);
    if (lane == 0) {
        atomicAdd(ray_counter, 1u);                                    // a count only: the index comes from the scan
        float* ro = rays_out + (size_t)ray_idx * 6;
        ro[0] = r.o.x; ro[1] = r.o.y; ro[2] = r.o.z; ro[3] = r.d.x; ro[4] = r.d.y; ro[5] = r.d.z;
        const uint2 texel = reinterpret_cast<const uint2*>(tv.images)[r.pixel];     // 4 halves (read_rgba, common_device.h:203-213)
        const __half2 rg = *reinterpret_cast<const __half2*>(&texel.x), ba = *reinterpret_cast<const __half2*>(&texel.y);
        reinterpret_cast<float4*>(rays_rgba)[ray_idx] = make_float4(__low2float(rg), __high2float(rg), __low2float(ba), __high2float(ba));
        numsteps_out[ray_idx * 2 + 0] = numsteps;
        numsteps_out[ray_idx * 2 + 1] = (uint32_t)base;
    }
    const V3 wd = mk3((r.d.x + 1.f) * 0.5f, (r.d.y + 1.f) * 0.5f, (r.d.z + 1.f) * 0.5f);   // warp_direction
    float* c0 = coords_out + base * 7;
    train_march_warp(g, bits, r, numsteps, [&](uint32_t j, const V3& w, float dt) {
        float* c = c0 + (size_t)j * 7;
        c[0] = w.x; c[1] = w.y; c[2] = w.z; c[3] = dt; c[4] = wd.x; c[5] = wd.y; c[6] = wd.z;
    });
}

}  // namespace

void launch_mark_untrained(const DevCfg& g, uint32_t aabb_scale, const TrainViews& tv, float* grid_out, cudaStream_t stream) {
    const uint32_t n = g.cells * g.n_cascades;
    k_mark_untrained<<<(n + 255) / 256, 256, 0, stream>>>(g, n, aabb_scale, tv.n_images, tv.width, tv.height, tv.focal_x,
                                                          tv.focal_y, tv.xforms, grid_out);
}

void launch_train_count(const DevCfg& g, const TrainViews& tv, const uint8_t* bits, uint32_t n_rays, uint32_t n_rays_shift,
                        uint32_t n_max_steps, RefreshRng rng, int snap, uint32_t* counts, uint32_t* flags, cudaStream_t stream) {
    if (n_rays == 0) return;
    const Pcg r = {rng.state, rng.inc};
    k_train_count<<<(unsigned int)(((uint64_t)n_rays * 32 + kTrainWarpBlock - 1) / kTrainWarpBlock), kTrainWarpBlock, 0, stream>>>(g, tv, bits, n_rays, n_rays_shift,
                                                                                       n_max_steps, r, snap, counts, flags);
}

void launch_train_emit(const DevCfg& g, const TrainViews& tv, const uint8_t* bits, uint32_t n_rays, uint32_t n_rays_shift,
                       uint32_t n_coords, RefreshRng rng, int snap, const uint32_t* counts, const uint64_t* offsets,
                       const uint64_t* ray_rank, uint32_t* ray_counter, uint32_t* numsteps_counter, float* rays_out,
                       float* rays_rgba, uint32_t* numsteps_out, float* coords_out, cudaStream_t stream) {
    if (n_rays == 0) return;
    const Pcg r = {rng.state, rng.inc};
    k_train_emit<<<(unsigned int)(((uint64_t)n_rays * 32 + kTrainWarpBlock - 1) / kTrainWarpBlock), kTrainWarpBlock, 0, stream>>>(
        g, tv, bits, n_rays, n_rays_shift, n_coords, r, snap, counts, offsets, ray_rank, ray_counter, numsteps_counter, rays_out,
        rays_rgba, numsteps_out, coords_out);
}

}  // namespace srf
