// srf_shim.hpp -- header-only C++ classes with the reference's names and method order that
// forward to the C-ABI of libsrf_b200.so (srf_abi.h) and turn status codes into
// std::runtime_error, the reference's error convention (CUDA_CHECK_THROW everywhere).
//
// A reference maintainer swaps the bodies of OccupancySampler / NGPNetwork / RayMarcher /
// Testbed::render_frame for these forwards; device buffers stay owned by the caller, as
// tcnn::GPUMemory buffers are in the reference, and are passed as raw device pointers.
// Streams are cudaStream_t passed as void*.
#pragma once

#include <cstdint>
#include <stdexcept>
#include <string>

#include "srf_abi.h"

namespace srf_shim {

inline void check(srf_status st, const srf_ctx* ctx) {
    if (st != SRF_OK) throw std::runtime_error(std::string("srf: ") + srf_last_error(ctx));
}

// Owns one library context: the role of Testbed's model members (internal/testbed.h:100-117).
class Context {
public:
    Context(const srf_config_t& cfg, int device = 0) {
        srf_status st = srf_create(&cfg, device, &m_ctx);
        if (st != SRF_OK) throw std::runtime_error(std::string("srf: ") + srf_last_error(nullptr));
    }
    ~Context() { srf_destroy(m_ctx); }
    Context(const Context&) = delete;
    Context& operator=(const Context&) = delete;
    srf_ctx* get() const { return m_ctx; }
private:
    srf_ctx* m_ctx = nullptr;
};

// internal/sampler/occupancy_sampler.h:13-135
class OccupancySampler {
public:
    explicit OccupancySampler(Context& c) : m(c) {}
    // OccupancySampler::update_grid_bitfield(cudaStream_t)
    void update_grid_bitfield(void* stream) { check(srf_update_grid_bitfield(m.get(), stream), m.get()); }
    // OccupancySampler::generate_rays_from_camera_matrix(resolution, focal, pp, camera, payload, buffer, stream)
    void generate_rays_from_camera_matrix(const srf_view_t& view, float* d_dir, float* d_t, uint8_t* d_alive,
                                          uint32_t* d_pixel, void* stream) {
        check(srf_generate_rays(m.get(), &view, d_dir, d_t, d_alive, d_pixel, stream), m.get());
    }
    // OccupancySampler::generate_coords_from_rays(n_rays, n_steps, payloads, coords, stream): count, place, emit
    void count_samples(const srf_view_t& view, uint32_t* d_counts, void* stream) {
        check(srf_sample_count(m.get(), &view, d_counts, stream), m.get());
    }
    void sample_offsets(const uint32_t* d_counts, uint64_t n_rays, uint64_t* d_offsets, void* stream) {
        check(srf_sample_offsets(m.get(), d_counts, n_rays, d_offsets, stream), m.get());
    }
    void generate_coords_from_rays(const srf_view_t& view, const uint64_t* d_offsets, uint64_t capacity,
                                   float* d_coords, void* stream) {
        check(srf_sample_emit(m.get(), &view, d_offsets, capacity, d_coords, nullptr, nullptr, stream), m.get());
    }
    // OccupancySampler::init(n_images, resolution, focal, pp, camera_matrices, images, rng, stream)
    void init(const srf_train_views_t& views, bool init_grid_with_mask, uint64_t rng_seed, void* stream) {
        check(srf_sampler_init(m.get(), &views, init_grid_with_mask ? 1 : 0, rng_seed, stream), m.get());
    }
    // OccupancySampler::sample_coords_from_dataset(n_rays, n_rays_shift, n_coords, dataset, rays, rays_rgba,
    //     n_rays_counter, ray_coord_indices, coords, n_coords_counter, rng, stream)
    void sample_coords_from_dataset(uint32_t n_rays, uint32_t n_rays_shift, uint32_t n_coords, const srf_train_views_t& dataset,
                                    float* d_rays, float* d_rays_rgba, uint32_t* d_n_rays_counter, uint32_t* d_ray_coord_indices,
                                    float* d_coords, uint32_t* d_n_coords_counter, uint64_t rng_state, uint64_t rng_inc,
                                    bool snap_to_pixel_centers_in_training, void* stream) {
        check(srf_sample_training_rays(m.get(), &dataset, n_rays, n_rays_shift, n_coords, rng_state, rng_inc,
                                       snap_to_pixel_centers_in_training ? 1 : 0, d_n_rays_counter, d_n_coords_counter, d_rays,
                                       d_rays_rgba, d_ray_coord_indices, d_coords, stream), m.get());
    }
private:
    Context& m;
};

// internal/network/ngp_network.h:143-777
class NGPNetwork {
public:
    explicit NGPNetwork(Context& c) : m(c) {}
    uint32_t padded_output_width() const { return 4; }            // :542-544
    uint32_t padded_density_output_width() const { return 16; }   // :312-314
    // inference_mixed_precision(stream, input 7xB float, output 4xB half column-major)
    void inference_mixed_precision(void* stream, const float* d_coords, uint64_t batch, uint16_t* d_rgbsigma) {
        check(srf_network_inference(m.get(), d_coords, batch, d_rgbsigma, stream), m.get());
    }
    // density(stream, positions, output 16xB half)
    void density(void* stream, const float* d_positions, uint64_t batch, uint16_t* d_out) {
        check(srf_network_density(m.get(), d_positions, batch, d_out, stream), m.get());
    }
private:
    Context& m;
};

// internal/render/ray_marcher.h:13-81
class RayMarcher {
public:
    explicit RayMarcher(Context& c) : m(c) {}
    void volume_rendering(const srf_view_t& view, const uint64_t* d_offsets, uint64_t n_rays, const float* d_coords,
                          const uint16_t* d_rgbsigma, float* d_rgba, uint32_t* d_n_composited, void* stream) {
        check(srf_volume_rendering(m.get(), &view, d_offsets, n_rays, d_coords, d_rgbsigma, d_rgba, d_n_composited, stream), m.get());
    }
    // RayMarcher::volume_rendering_with_loss_and_gradient(n_rays, n_max_compacted_coords, rays, rays_rgba, n_rays_counter,
    //     ray_coord_indices, coords, compacted_coords, n_compacted_coords_counter, network_output, dloss_doutput, ...)
    void volume_rendering_with_loss_and_gradient(const srf_loss_params_t& params, const float* d_rays_rgba,
                                                 const uint32_t* d_n_rays_counter, uint32_t* d_ray_coord_indices,
                                                 const float* d_coords, float* d_compacted_coords,
                                                 uint32_t* d_n_compacted_coords_counter, const uint16_t* d_network_output,
                                                 uint16_t* d_dloss_doutput, float* d_loss_output, float* d_reg_distortion,
                                                 void* stream) {
        check(srf_volume_rendering_loss(m.get(), &params, d_n_rays_counter, d_ray_coord_indices, d_rays_rgba, d_coords,
                                        d_network_output, d_compacted_coords, d_n_compacted_coords_counter, d_dloss_doutput,
                                        d_loss_output, d_reg_distortion, stream), m.get());
    }
private:
    Context& m;
};

// internal/testbed.h: render_frame, train_prep_nerf, render
class Testbed {
public:
    explicit Testbed(const srf_config_t& cfg, int device = 0)
        : m_ctx(cfg, device), m_sampler(m_ctx), m_network(m_ctx), m_render(m_ctx) {}
    Context& context() { return m_ctx; }
    OccupancySampler& sampler() { return m_sampler; }
    NGPNetwork& network() { return m_network; }
    RayMarcher& render_stage() { return m_render; }
    void render_frame(const srf_view_t& view, const srf_post_t& post, float* d_out, float* d_accum, void* stream,
                      srf_frame_stats_t* stats = nullptr) {
        check(srf_render_frame(m_ctx.get(), &view, &post, d_out, d_accum, nullptr, nullptr, stats, stream), m_ctx.get());
    }
    void render(const srf_view_t& view, const srf_post_t& post, uint32_t spp, float* h_image) {
        check(srf_render(m_ctx.get(), &view, &post, spp, h_image, nullptr), m_ctx.get());
    }
    // RenderingBuffer::MIN/MAX_STEPS_INBETWEEN_COMPACTION have no meaning here; the counterpart is the wave schedule
    void set_wave_schedule(const uint32_t* steps, uint32_t n) { check(srf_set_wave_schedule(m_ctx.get(), steps, n), m_ctx.get()); }
    void train_prep_nerf(uint32_t training_step, void* stream) {
        check(srf_refresh_grid(m_ctx.get(), training_step, stream), m_ctx.get());
    }
private:
    Context m_ctx;
    OccupancySampler m_sampler;
    NGPNetwork m_network;
    RayMarcher m_render;
};

}  // namespace srf_shim
