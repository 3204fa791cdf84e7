// ref_harness.cpp -- runs the REFERENCE's own kernels on the host.  TEST INFRASTRUCTURE ONLY.
//
// oracle/build_ref.py cuts the kernel and device-function line ranges out of the reference's .cu files where
// they lie (a read-only mount of the reference project; nothing is copied into this repository), writes them
// to a temporary directory as *.inc files and compiles this file with them into oracle/_ref/libsrf_ref.so.
// The reference's headers internal/utils/{common,common_device,loss}.h, random_val.cuh and
// internal/sampler/bounding_box.h are included whole.  What the reference takes from libraries that are not
// available (Eigen, tiny-cuda-nn, the CUDA runtime's device built-ins) comes from the stand-ins under
// oracle/ref_stub/: a kernel is an ordinary function, this file sets threadIdx/blockIdx and calls it once per
// "thread", in index order.
//
// What this pins: the reference's control flow, statement order, integer arithmetic (Sobol/Owen jitter, Morton
// indices, cell pick of the refresh), the float expressions as its source writes them (evaluated without fused
// multiply-adds, with the C library's elementary functions and Eigen's reduction order), its compaction and
// termination rules, its output stage.  What it cannot pin: the bits of the CUDA math library's
// atan2f/asinf/cosf/__expf/__logf, which multiply-adds nvcc fuses, and the network (tiny-cuda-nn): the field is
// supplied by the caller through a function pointer.
//
// Only the host loops below (the launch sequences of Testbed::render_frame, OccupancySampler::update_grid...,
// written here from the reference's host code, cited per function) are this repository's code.
#include "srf_cuda_on_host.h"
#ifdef _OPENMP
#include <omp.h>
#endif

thread_local SrfThreadIndex threadIdx, blockIdx, blockDim, gridDim;

#include "internal/utils/common_device.h"
#include "internal/utils/loss.h"

#include "loss.inc"                    // internal/utils/loss.cu: the seven losses
#include "sampler_kernels.inc"         // internal/sampler/occupancy_sampler.cu: every kernel and device function
#include "marcher_kernels.inc"         // internal/render/ray_marcher.cu: both compositing kernels
#include "testbed_kernels.inc"         // internal/testbed.cu: compact_rays_kernel, shade_kernel
#include "render_buffer_kernels.inc"   // internal/utils/render_buffer.cu: accumulate, tonemap

#include "../include/srf_abi.h"        // configuration / view / post structs only

namespace {

// linear_kernel(...) of tiny-cuda-nn: one thread per element, 128 threads per block.  "Threads" run in index order
// on one host thread: kernels that take slots from atomic counters then behave like a serial execution.
template <typename K, typename... Args>
void run_linear(K kernel, uint32_t n_elements, Args... args) {
    blockDim.x = 128; blockDim.y = blockDim.z = 1;
    for (uint32_t i = 0; i < n_elements; ++i) {
        blockIdx.x = i / 128; blockIdx.y = blockIdx.z = 0;
        threadIdx.x = i % 128; threadIdx.y = threadIdx.z = 0;
        kernel(n_elements, args...);
    }
}

// The same for kernels whose threads touch disjoint data (no counters): spread over the host cores with OpenMP.
// threadIdx / blockIdx are thread_local, so every host thread has its own.
template <typename K, typename... Args>
void run_linear_parallel(K kernel, uint32_t n_elements, Args... args) {
#pragma omp parallel for schedule(dynamic, 64)
    for (int64_t i = 0; i < (int64_t)n_elements; ++i) {
        blockDim.x = 128; blockDim.y = blockDim.z = 1;
        blockIdx.x = (uint32_t)i / 128; blockIdx.y = blockIdx.z = 0;
        threadIdx.x = (uint32_t)i % 128; threadIdx.y = threadIdx.z = 0;
        kernel(n_elements, args...);
    }
}

// A 16 x 8 launch over an image, as the reference's 2-D kernels use.
template <typename K, typename... Args>
void run_image(K kernel, int width, int height, Args... args) {
    blockDim.x = 16; blockDim.y = 8; blockDim.z = 1;
    for (int y = 0; y < height; ++y)
        for (int x = 0; x < width; ++x) {
            blockIdx.x = x / 16; blockIdx.y = y / 8; blockIdx.z = 0;
            threadIdx.x = x % 16; threadIdx.y = y % 8; threadIdx.z = 0;
            kernel(args...);
        }
}

// The sampler's members as OccupancySampler::OccupancySampler derives them (occupancy_sampler.cu:909-944).
struct Sampler {
    EWarpingType warping_type;
    uint32_t aabb_scale;
    BoundingBox aabb;
    bool use_grid;
    uint32_t n_grid_size, n_grid_elements, n_cascades, n_total_elements;
    float ema_decay;
    EGridDistType griddist_type;
    uint32_t n_max_steps;
    float cone_angle_constant, min_cone_stepsize, max_cone_stepsize, near_distance, far_distance;
    ESamplingType sampling_type;
    bool snap_rendering;
    float min_optical_thickness;
};

Sampler make_sampler(const srf_config_t& c) {
    Sampler s;
    s.warping_type = (EWarpingType)c.warping_type;
    s.aabb_scale = c.aabb_scale;
    s.aabb = BoundingBox{Eigen::Vector3f::Constant(0.5f), Eigen::Vector3f::Constant(0.5f)};
    s.aabb.inflate(0.5f * s.aabb_scale);
    s.use_grid = c.use_grid != 0;
    s.n_grid_size = c.grid_size;
    s.n_grid_elements = s.n_grid_size * s.n_grid_size * s.n_grid_size;
    s.n_cascades = c.num_cascades;
    s.n_total_elements = s.n_grid_elements * s.n_cascades;
    s.ema_decay = c.ema_decay;
    s.griddist_type = (EGridDistType)c.grid_distribution_type;
    s.n_max_steps = c.maximum_marching_steps;
    s.cone_angle_constant = c.cone_angle_constant;
    s.min_cone_stepsize = c.min_cone_stepsize > 0.f ? c.min_cone_stepsize : SQRT3() / s.n_max_steps;
    s.max_cone_stepsize = c.max_cone_stepsize > 0.f ? c.max_cone_stepsize
                        : (s.use_grid ? (SQRT3() * (1 << (s.n_cascades - 1)) / s.n_grid_size) : s.min_cone_stepsize);
    s.near_distance = c.near_distance;
    s.far_distance = c.far_distance;
    s.sampling_type = (ESamplingType)c.sampling_type;
    s.snap_rendering = c.snap_to_pixel_centers_in_rendering != 0;
    s.min_optical_thickness = c.min_optical_thickness;
    return s;
}

Eigen::Matrix<float, 3, 4> camera_of(const float* row_major12) {
    Eigen::Matrix<float, 3, 4> m;
    for (int r = 0; r < 3; ++r) for (int c = 0; c < 4; ++c) m(r, c) = row_major12[r * 4 + c];
    return m;
}

}  // namespace

extern "C" {

// OpenMP threads of the per-ray kernels (n <= 0: one per available core); returns the count in force.
int refh_set_num_threads(int n) {
#ifdef _OPENMP
    if (n <= 0) n = omp_get_num_procs();
    omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}

// The field a frame queries: Coordinate records (n x 7 floats) -> n x 4 halves (r, g, b, sigma raw).  Same
// signature as the oracle's srfo_network_inference, so that function can be passed directly.
typedef int (*refh_field_fn)(const void* cfg, const void* model, const float* coords, uint64_t n, uint16_t* rgbsigma);
// Positions (n x 3 floats) -> n x 16 halves (the density network's padded output); srfo_network_density's signature.
typedef int (*refh_density_fn)(const void* cfg, const void* model, const float* positions, uint64_t n, uint16_t* out16);

// ---- small taps (known-answer material for the oracle) --------------------------------------------------------
float refh_ld_random_val(uint32_t index, uint32_t seed, uint32_t dim) { return ld_random_val(index, seed, dim); }
uint32_t refh_sobol(uint32_t index, uint32_t dim) { return sobol(index, dim); }
void refh_ld_random_pixel_offset(uint32_t spp, uint32_t x, uint32_t y, float* out2) {
    const Eigen::Vector2f o = ld_random_pixel_offset(spp, x, y);
    out2[0] = o.x(); out2[1] = o.y();
}

// warp_position / unwarp_position of n positions (internal/utils/common_device.h:375-526)
void refh_warp_position(const srf_config_t* cfg, const float* pos, float* out, size_t n, int inverse) {
    const Sampler s = make_sampler(*cfg);
    for (size_t i = 0; i < n; ++i) {
        const Eigen::Vector3f p(pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]);
        const Eigen::Vector3f w = inverse ? unwarp_position(p, s.aabb, s.warping_type) : warp_position(p, s.aabb, s.warping_type);
        out[3 * i] = w.x(); out[3 * i + 1] = w.y(); out[3 * i + 2] = w.z();
    }
}

// calc_dt (internal/sampler/occupancy_sampler.cu:287-331) for n values of t
void refh_calc_dt(const srf_config_t* cfg, const float* t, float* dt, size_t n) {
    const Sampler s = make_sampler(*cfg);
    for (size_t i = 0; i < n; ++i)
        dt[i] = calc_dt(t[i], s.n_max_steps, s.cone_angle_constant, s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance,
                        s.far_distance, s.sampling_type);
}

// level_from_pos + cascaded_grid_idx_at (occupancy_sampler.cu:349-456) for n metric positions: level and Morton index
void refh_grid_index(const srf_config_t* cfg, const float* pos, uint32_t* level_out, uint32_t* idx_out, size_t n) {
    const Sampler s = make_sampler(*cfg);
    for (size_t i = 0; i < n; ++i) {
        const Eigen::Vector3f p(pos[3 * i], pos[3 * i + 1], pos[3 * i + 2]);
        const Eigen::Vector3f w = warp_position(p, s.aabb, s.warping_type);
        const uint32_t level = level_from_pos(p, w, s.aabb, s.n_cascades, s.griddist_type);
        level_out[i] = level;
        idx_out[i] = cascaded_grid_idx_at(p, w, s.aabb, level, s.n_grid_size, s.n_cascades, s.griddist_type);
    }
}

// tonemap() (internal/utils/render_buffer.cu:84-140) and the sRGB pair (common_device.h:70-88) on n colours
void refh_tonemap(const float* rgb, float* out, size_t n, int curve) {
    for (size_t i = 0; i < n; ++i) {
        const Eigen::Array3f c = tonemap(Eigen::Array3f(rgb[3 * i], rgb[3 * i + 1], rgb[3 * i + 2]), (ETonemapCurve)curve);
        out[3 * i] = c.x(); out[3 * i + 1] = c.y(); out[3 * i + 2] = c.z();
    }
}
void refh_srgb(const float* in, float* out, size_t n, int to_linear) {
    for (size_t i = 0; i < n; ++i) out[i] = to_linear ? srgb_to_linear(in[i]) : linear_to_srgb(in[i]);
}

// loss_and_gradient (internal/utils/loss.cu:88-99): loss[3] and gradient[3] per (target, prediction) pair
void refh_loss(const float* target, const float* prediction, float* loss, float* gradient, size_t n, int loss_type) {
    for (size_t i = 0; i < n; ++i) {
        const LossAndGradient lg = loss_and_gradient(Eigen::Vector3f(target[3 * i], target[3 * i + 1], target[3 * i + 2]),
                                                     Eigen::Vector3f(prediction[3 * i], prediction[3 * i + 1], prediction[3 * i + 2]),
                                                     (ELossType)loss_type);
        for (int k = 0; k < 3; ++k) { loss[3 * i + k] = lg.loss[k]; gradient[3 * i + k] = lg.gradient[k]; }
    }
}

// ---- rays only: OccupancySampler::generate_rays_from_camera_matrix (occupancy_sampler.cu:1145-1188) ----------------
// Per pixel: direction, t after advance_pos_nerf, alive.
int refh_generate_rays(const srf_config_t* cfg, const srf_view_t* view, const uint8_t* bitfield, float* dir, float* t,
                       uint8_t* alive) {
    const Sampler s = make_sampler(*cfg);
    const Eigen::Vector2i resolution((int)view->width, (int)view->height);
    const Eigen::Vector2f focal(resolution.x() * view->relative_focal_length[0], resolution.y() * view->relative_focal_length[1]);
    const Eigen::Vector2f pp(view->principal_point[0], view->principal_point[1]);
    const Eigen::Matrix<float, 3, 4> cam = camera_of(view->camera);
    const uint32_t n_pixels = view->width * view->height;
    std::vector<RayPayload> payloads(n_pixels);
    memset((void*)payloads.data(), 0, sizeof(RayPayload) * n_pixels);
    run_image(init_rays_with_payload_kernel_nerf, (int)view->width, (int)view->height, resolution, focal, pp, cam, view->spp_index,
              s.snap_rendering, s.aabb, payloads.data());
    run_linear(advance_pos_nerf, n_pixels, view->spp_index, payloads.data(), s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
               s.griddist_type, s.use_grid ? bitfield : (const uint8_t*)nullptr, s.n_max_steps, s.cone_angle_constant,
               s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type);
    for (uint32_t i = 0; i < n_pixels; ++i) {
        // a ray that was never alive keeps d unset in the reference; report zeros for it
        const bool born = payloads[i].alive || payloads[i].t != 0.f;
        if (dir) for (int k = 0; k < 3; ++k) dir[3 * i + k] = born ? payloads[i].d[k] : 0.f;
        if (t) t[i] = payloads[i].t;
        if (alive) alive[i] = payloads[i].alive ? 1 : 0;
    }
    return 0;
}

// ---- a frame: Testbed::render_frame (internal/testbed.cu:479-606) ----------------------------------------------------
// One sample-per-pixel pass (view->spp_index) over the whole image.  Outputs, all indexed by pixel (any may be NULL):
//   out        H*W*4  the tonemapped image (what tonemap_kernel writes to the surface)
//   accum      H*W*4  accumulate buffer, kept by the caller between passes (cleared here when spp_index == 0)
//   rgba_raw   H*W*4  premultiplied colour/opacity of the ray when it stopped being alive (0 for rays still alive at
//                     the loop bound and for rays that never entered the box)
//   n_samples  H*W    samples the sampler emitted for the ray (sum of payload.n_steps over all rounds)
//   hit        H*W    1 when the ray reached the hit buffer
// Sample capture (parity tap): the samples of pixels [cap_first, cap_first + cap_count) in emission order, pixel after
// pixel: cap_counts[cap_count], cap_pos_dt[* x 4] (at most cap_capacity samples; *cap_total receives the number).
int refh_render_frame(const srf_config_t* cfg, const srf_view_t* view, const srf_post_t* post, const uint8_t* bitfield,
                      refh_field_fn field, const void* field_cfg, const void* field_model, float* out, float* accum,
                      float* rgba_raw, uint32_t* n_samples, uint8_t* hit, uint32_t cap_first, uint32_t cap_count,
                      uint64_t cap_capacity, uint32_t* cap_counts, float* cap_pos_dt, uint64_t* cap_total,
                      uint64_t* n_rounds_out) {
    const Sampler s = make_sampler(*cfg);
    const Eigen::Vector2i resolution((int)view->width, (int)view->height);
    const Eigen::Vector2f focal(resolution.x() * view->relative_focal_length[0], resolution.y() * view->relative_focal_length[1]);
    const Eigen::Vector2f pp(view->principal_point[0], view->principal_point[1]);
    const Eigen::Matrix<float, 3, 4> cam = camera_of(view->camera);
    const uint32_t n_pixels = view->width * view->height;
    const ERenderMode render_mode = (ERenderMode)view->render_mode;
    const uint32_t kMinSteps = 1, kMaxSteps = 8;                      // testbed.h: MIN/MAX_STEPS_INBETWEEN_COMPACTION
    const uint32_t padded_output_width = 4;
    const uint32_t n_elements = tcnn::next_multiple(n_pixels, BATCH_SIZE_MULTIPLE);

    std::vector<RayPayload> pay[2] = {std::vector<RayPayload>(n_elements), std::vector<RayPayload>(n_elements)};
    std::vector<Eigen::Array4f> rgba[2] = {std::vector<Eigen::Array4f>(n_elements), std::vector<Eigen::Array4f>(n_elements)};
    std::vector<RayPayload> pay_hit(n_elements);
    std::vector<Eigen::Array4f> rgba_hit(n_elements);
    for (int k = 0; k < 2; ++k) memset((void*)pay[k].data(), 0, sizeof(RayPayload) * n_elements);
    memset((void*)pay_hit.data(), 0, sizeof(RayPayload) * n_elements);
    std::vector<float> coords((size_t)n_elements * kMaxSteps * 7, 0.f);
    std::vector<uint16_t> rgbsigma((size_t)n_elements * kMaxSteps * padded_output_width, 0);
    std::vector<Eigen::Array4f> frame(n_pixels);                    // clear_frame_buffer
    std::vector<std::vector<float>> captured(cap_count);
    if (n_samples) memset(n_samples, 0, sizeof(uint32_t) * n_pixels);
    if (rgba_raw) memset(rgba_raw, 0, sizeof(float) * 4 * n_pixels);
    if (hit) memset(hit, 0, n_pixels);

    // generate_rays_from_camera_matrix
    run_image(init_rays_with_payload_kernel_nerf, (int)view->width, (int)view->height, resolution, focal, pp, cam, view->spp_index,
              s.snap_rendering, s.aabb, pay[0].data());
    run_linear_parallel(advance_pos_nerf, n_pixels, view->spp_index, pay[0].data(), s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
               s.griddist_type, s.use_grid ? bitfield : (const uint8_t*)nullptr, s.n_max_steps, s.cone_angle_constant,
               s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type);
    // rays that never entered the box carry no pixel index; give them one so the per-pixel taps stay aligned
    // (nothing below reads it for a dead ray with zero opacity)
    uint32_t n_hit = 0, n_alive = n_pixels, i_steps_offset = 1, double_buffer_index = 0;
    uint64_t n_rounds = 0;
    while (i_steps_offset < MARCH_ITER) {
        std::vector<RayPayload>& prev_p = pay[double_buffer_index % 2];
        std::vector<Eigen::Array4f>& prev_c = rgba[double_buffer_index % 2];
        std::vector<RayPayload>& cur_p = pay[(double_buffer_index + 1) % 2];
        std::vector<Eigen::Array4f>& cur_c = rgba[(double_buffer_index + 1) % 2];
        ++double_buffer_index;
        uint32_t alive_counter = 0;
        // record what rays that just stopped being alive carry (before compaction drops the transparent ones)
        for (uint32_t i = 0; i < n_alive; ++i)
            if (!prev_p[i].alive && n_rounds > 0 && rgba_raw) {
                const uint32_t px = prev_p[i].idx;
                for (int k = 0; k < 4; ++k) rgba_raw[4 * px + k] = prev_c[i][k];
            }
        run_linear(compact_rays_kernel, n_alive, prev_p.data(), prev_c.data(), cur_p.data(), cur_c.data(), pay_hit.data(),
                   rgba_hit.data(), &alive_counter, &n_hit);
        n_alive = alive_counter;
        if (n_alive == 0) break;
        const uint32_t n_steps = tcnn::clamp(n_pixels / n_alive, kMinSteps, kMaxSteps);
        run_linear_parallel(generate_coords_from_rays_regularly_kernel, n_alive, n_steps, s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
                   s.griddist_type, s.use_grid ? bitfield : (const uint8_t*)nullptr, s.n_max_steps, s.cone_angle_constant,
                   s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type, cur_p.data(),
                   (Coordinate*)coords.data());
        for (uint32_t i = 0; i < n_alive; ++i) {
            const uint32_t px = cur_p[i].idx, m = cur_p[i].n_steps;
            if (n_samples) n_samples[px] += m;
            if (px >= cap_first && px < cap_first + cap_count)
                for (uint32_t j = 0; j < m; ++j) {
                    const float* c = coords.data() + ((size_t)i * n_steps + j) * 7;
                    std::vector<float>& v = captured[px - cap_first];
                    v.push_back(c[0]); v.push_back(c[1]); v.push_back(c[2]); v.push_back(c[3]);
                }
        }
        const uint32_t n_net = tcnn::next_multiple(n_alive * n_steps, BATCH_SIZE_MULTIPLE);
        if (field(field_cfg, field_model, coords.data(), n_net, rgbsigma.data()) != 0) return 2;
        run_linear_parallel(volume_rendering_kernel, n_alive, n_steps, i_steps_offset, cur_p.data(), cur_c.data(), (const Coordinate*)coords.data(),
                   (const precision_t*)rgbsigma.data(), padded_output_width, (EActivation)cfg->density_activation,
                   (EActivation)cfg->rgb_activation, render_mode, s.warping_type, s.aabb, s.n_cascades, s.min_cone_stepsize, cam,
                   view->depth_scale, cfg->transmittance_threshold);
        i_steps_offset += n_steps;
        ++n_rounds;
    }
    if (n_rounds_out) *n_rounds_out = n_rounds;
    run_linear(shade_kernel, n_hit, (const Eigen::Array4f*)rgba_hit.data(), (const RayPayload*)pay_hit.data(), frame.data(), render_mode,
               cfg->train_in_linear_color != 0);
    if (hit) for (uint32_t i = 0; i < n_hit; ++i) hit[pay_hit[i].idx] = 1;

    // render_buffer.accumulate + tonemap (internal/utils/render_buffer.cu:204-236)
    std::vector<Eigen::Array4f> acc(n_pixels);
    if (view->spp_index != 0 && accum) memcpy((void*)acc.data(), accum, sizeof(float) * 4 * n_pixels);
    run_image(accumulate_kernel, (int)view->width, (int)view->height, resolution, frame.data(), acc.data(), (float)view->spp_index,
              (EColorSpace)post->color_space);
    if (accum) memcpy(accum, (const void*)acc.data(), sizeof(float) * 4 * n_pixels);
    if (out) {
        SrfHostSurface surf = {reinterpret_cast<float4*>(out), (int)view->width};
        const Eigen::Array4f bg(post->background_color[0], post->background_color[1], post->background_color[2], post->background_color[3]);
        run_image(tonemap_kernel, (int)view->width, (int)view->height, resolution, post->exposure, bg, acc.data(),
                  (EColorSpace)post->color_space, post->to_srgb ? EColorSpace::SRGB : EColorSpace::Linear,
                  (ETonemapCurve)post->tonemap_curve, &surf);
    }
    uint64_t total = 0;
    for (uint32_t k = 0; k < cap_count; ++k) {
        const uint64_t m = captured[k].size() / 4;
        if (cap_counts) cap_counts[k] = (uint32_t)m;
        if (cap_pos_dt && total + m <= cap_capacity) memcpy(cap_pos_dt + total * 4, captured[k].data(), m * 4 * sizeof(float));
        total += m;
    }
    if (cap_total) *cap_total = total;
    return total > cap_capacity && cap_pos_dt ? 3 : 0;
}

// ---- grid refresh: Testbed::train_prep_nerf (internal/testbed.cu:203-239) ----------------------------------------------
// = sample_positions_from_grid + NGPNetwork::density + update_grid (occupancy_sampler.cu:980-1061).  The grid mean and
// the bitfield are a separate step (refh_grid_to_bitfield) because the mean's summation order belongs to tiny-cuda-nn.
// rng_state/rng_inc: the sampler's generator, advanced as the reference advances it; *i_step its refresh counter.
// positions_out (n_total x 3) and indices_out (n_total), optional, receive what the two sampling launches produced.
int refh_update_grid(const srf_config_t* cfg, float* grid, uint32_t n_uniform, uint32_t n_nonuniform, uint64_t* rng_state,
                     uint64_t* rng_inc, uint32_t* i_step, refh_density_fn density, const void* field_cfg, const void* field_model,
                     float* positions_out, uint32_t* indices_out) {
    const Sampler s = make_sampler(*cfg);
    const uint32_t n_total = n_uniform + n_nonuniform;
    tcnn::default_rng_t rng;
    rng.state = *rng_state; rng.inc = *rng_inc;
    std::vector<Position> positions(n_total, Position(Eigen::Vector3f::Zero(), 0.f));
    std::vector<uint32_t> indices(n_total, 0u);
    run_linear(generate_grid_samples_nerf_nonuniform, n_uniform, rng, *i_step, s.warping_type, s.aabb_scale, s.aabb, s.griddist_type,
               (const float*)grid, positions.data(), indices.data(), s.n_grid_size, s.n_grid_elements, s.n_cascades,
               s.min_cone_stepsize, (float)-0.01);
    rng.advance();
    run_linear(generate_grid_samples_nerf_nonuniform, n_nonuniform, rng, *i_step, s.warping_type, s.aabb_scale, s.aabb, s.griddist_type,
               (const float*)grid, positions.data() + n_uniform, indices.data() + n_uniform, s.n_grid_size, s.n_grid_elements,
               s.n_cascades, s.min_cone_stepsize, s.min_optical_thickness);
    rng.advance();
    static_assert(sizeof(Position) == 3 * sizeof(float), "Position is three floats");
    if (positions_out) memcpy(positions_out, (const void*)positions.data(), sizeof(float) * 3 * n_total);
    if (indices_out) memcpy(indices_out, indices.data(), sizeof(uint32_t) * n_total);
    const uint32_t padded = 16;
    std::vector<uint16_t> dens((size_t)n_total * padded, 0);
    if (n_total && density(field_cfg, field_model, (const float*)positions.data(), n_total, dens.data()) != 0) return 2;
    std::vector<float> current(s.n_total_elements, 0.f);               // density_grid_current, cleared (:1039)
    run_linear(splat_grid_samples_nerf_max_nearest_neighbor, n_total, (const uint32_t*)indices.data(), (int)padded,
               (const tcnn::network_precision_t*)dens.data(), (EActivation)cfg->density_activation, s.n_grid_size, s.min_cone_stepsize,
               current.data());
    run_linear(ema_grid_samples_nerf, s.n_total_elements, (const float*)current.data(), s.ema_decay, *i_step, grid);
    ++*i_step;
    *rng_state = rng.state; *rng_inc = rng.inc;
    return 0;
}

// grid_to_bitfield + bitfield_max_pool (occupancy_sampler.cu:1072-1088) for a given mean.
int refh_grid_to_bitfield(const srf_config_t* cfg, const float* grid, float mean, uint8_t* bitfield) {
    const Sampler s = make_sampler(*cfg);
    run_linear(grid_to_bitfield, s.n_total_elements / 8, grid, bitfield, (const float*)&mean, s.min_optical_thickness);
    if (s.griddist_type == EGridDistType::WarpedSpace_Exp || s.griddist_type == EGridDistType::MetricSpace_Exp)
        for (uint32_t level = 1; level < s.n_cascades; ++level)
            run_linear(bitfield_max_pool, s.n_grid_elements / 64, s.n_grid_size,
                       (const uint8_t*)(bitfield + s.n_grid_elements * (level - 1) / 8), bitfield + s.n_grid_elements * level / 8);
    return 0;
}

// mark_untrained_density_grid (occupancy_sampler.cu:12-102); xforms: n_images x 12 floats, column-major 3x4.
int refh_mark_untrained(const srf_config_t* cfg, uint32_t n_images, int width, int height, const float* focal2,
                        const float* xforms, float* grid_out) {
    const Sampler s = make_sampler(*cfg);
    static_assert(sizeof(Eigen::Matrix<float, 3, 4>) == 12 * sizeof(float), "3x4 matrix is twelve floats");
    run_linear(mark_untrained_density_grid, s.n_total_elements, s.n_grid_size, s.n_cascades, n_images, Eigen::Vector2i(width, height),
               Eigen::Vector2f(focal2[0], focal2[1]), (const Eigen::Matrix<float, 3, 4>*)xforms, s.aabb_scale, s.aabb, s.warping_type,
               s.griddist_type, grid_out);
    return 0;
}

// ---- training rays: generate_training_samples_nerf (occupancy_sampler.cu:513-689) ---------------------------------------
// Threads run in index order, so the two atomic counters hand out bases and ray slots in ray order.
int refh_sample_training_rays(const srf_config_t* cfg, const uint8_t* bitfield, uint32_t n_rays, uint32_t n_rays_shift,
                              uint32_t n_coords, uint32_t n_images, int width, int height, const float* focal2, const float* pp2,
                              const float* xforms, const uint16_t* images, const uint16_t* sampling_probability,
                              uint64_t rng_state, uint64_t rng_inc, int snap, uint32_t* ray_counter, uint32_t* numsteps_counter,
                              float* rays_out, float* rays_rgba, uint32_t* numsteps_out, float* coords_out) {
    const Sampler s = make_sampler(*cfg);
    tcnn::default_rng_t rng;
    rng.state = rng_state; rng.inc = rng_inc;
    *ray_counter = 0; *numsteps_counter = 0;
    static_assert(sizeof(Ray) == 6 * sizeof(float) && sizeof(Coordinate) == 7 * sizeof(float), "record sizes");
    run_linear(generate_training_samples_nerf, n_rays, n_rays_shift, n_coords, n_images, Eigen::Vector2i(width, height),
               Eigen::Vector2f(focal2[0], focal2[1]), Eigen::Vector2f(pp2[0], pp2[1]), (const Eigen::Matrix<float, 3, 4>*)xforms,
               (const __half*)images, (const __half*)sampling_probability, s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
               s.griddist_type, bitfield, s.use_grid, snap != 0, s.n_max_steps, s.cone_angle_constant, s.min_cone_stepsize,
               s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type, ray_counter, numsteps_counter, (Ray*)rays_out,
               (Eigen::Array4f*)rays_rgba, numsteps_out, (Coordinate*)coords_out, rng);
    return 0;
}

// ---- training compositor: volume_rendering_with_loss_and_gradient_kernal (internal/render/ray_marcher.cu:9-202) ----------
int refh_volume_rendering_loss(const srf_config_t* cfg, const srf_loss_params_t* p, uint32_t n_rays_kept, uint32_t* ray_coord_indices,
                               const float* rays_rgba, const float* coords, const uint16_t* network_output, float mean_density,
                               float* compacted_coords, uint32_t* n_compacted_counter, uint16_t* dloss_doutput, float* loss_output,
                               float* reg_distortion) {
    const Sampler s = make_sampler(*cfg);
    tcnn::default_rng_t rng;
    rng.state = p->rng_state; rng.inc = p->rng_inc;
    *n_compacted_counter = 0;
    const uint32_t counter = n_rays_kept;
    run_linear(volume_rendering_with_loss_and_gradient_kernal, p->n_rays, p->n_max_compacted_coords, (const Ray*)nullptr,
               (const Eigen::Array4f*)rays_rgba, (const uint32_t*)&counter, ray_coord_indices, (const Coordinate*)coords,
               (Coordinate*)compacted_coords, n_compacted_counter, (const precision_t*)network_output, (precision_t*)dloss_doutput,
               (int)p->padded_output_width, (EActivation)cfg->rgb_activation, (EActivation)cfg->density_activation, loss_output,
               reg_distortion, (ELossType)p->loss_type, p->loss_scale, (ERegularizationType)p->regularization_type, s.aabb, s.n_cascades,
               s.min_cone_stepsize, (const float*)&mean_density, s.min_optical_thickness, s.use_grid,
               Eigen::Array3f(p->background_color[0], p->background_color[1], p->background_color[2]), (EColorSpace)p->color_space,
               p->train_with_random_bg_color != 0, cfg->train_in_linear_color != 0, cfg->transmittance_threshold, rng);
    return 0;
}

}  // extern "C"
