/*
 * srf_oracle.h -- C interface of the CPU oracle (TEST INFRASTRUCTURE, not product code).
 *
 * The oracle restates, on the host, the algorithms of SphericalRF's render hot path and
 * density-grid refresh so that the CUDA library can be checked against it.  Only tests,
 * the smoke check and the benchmark's CPU-baseline leg may load it; the library never does.
 *
 * PARITY UNPINNED: the reference ships no tests, golden vectors or fixtures, cannot be
 * built here (no build files; tiny-cuda-nn, Eigen and others are absent) and is GPU-only,
 * so nothing pins this restatement to the reference's bits.  It follows the reference's
 * source line by line where the source exists and fixes documented canonical definitions
 * where the arithmetic lives in absent third-party code (see srf_oracle.cpp).
 */
#ifndef SRF_ORACLE_H_
#define SRF_ORACLE_H_

#include "../include/srf_abi.h"   /* configuration / view / post structs and enumerators only */

#ifdef __cplusplus
extern "C" {
#endif

typedef struct srfo_model_t {
    const uint16_t* hash_table;   /* fp16, layout of srf_hashgrid_layout */
    const uint16_t* density_mlp;  /* fp16 64x32, 16x64 */
    const uint16_t* rgb_mlp;      /* fp16 64x32, 64x64, 16x64 */
    const float*    blobs;        /* n_blobs x (cx,cy,cz,sigma,peak) */
    uint32_t        n_blobs;
    const float*    color_map;    /* 3x3 row-major */
} srfo_model_t;

typedef struct srfo_rng_t { uint64_t state, inc; } srfo_rng_t;

int srfo_num_threads(void);
void srfo_set_num_threads(int n);   /* n <= 0: one per available core */
int srfo_hashgrid_layout(const srf_config_t* cfg, uint32_t* offsets, uint32_t* resolutions, float* scales);
int srfo_eval_math(int op, const float* a, const float* b, float* out, size_t n);
int srfo_warp_position(const srf_config_t* cfg, const float* pos, float* out, size_t n, int inverse);
uint64_t srfo_shard_ray_count(const srf_view_t* view);
/* one reference function each, on arrays (known-answer taps) */
int srfo_calc_dt(const srf_config_t* cfg, const float* t, float* dt, size_t n);
int srfo_grid_index(const srf_config_t* cfg, const float* pos, uint32_t* level_out, uint32_t* idx_out, size_t n);
void srfo_pixel_offset(uint32_t spp, float* out2);
int srfo_tonemap(const float* rgb, float* out, size_t n, int curve);
int srfo_srgb(const float* in, float* out, size_t n, int to_linear);
int srfo_loss(const float* target, const float* prediction, float* loss, float* gradient, size_t n, int loss_type);

int srfo_generate_rays(const srf_config_t* cfg, const srf_view_t* view, const uint8_t* bitfield,
                       float* dir, float* t, uint8_t* alive, uint32_t* pixel);

/* Full march of rays [ray_first, ray_first+ray_count) without early termination. */
int srfo_march(const srf_config_t* cfg, const srf_view_t* view, const uint8_t* bitfield,
               uint64_t ray_first, uint64_t ray_count, uint64_t capacity, uint32_t* counts,
               float* pos_dt, uint32_t* ordinal, uint32_t* cell, uint64_t* n_total,
               uint64_t* n_march_steps);

/* Training-side sampler; `views` carries HOST pointers in the oracle. */
int srfo_mark_untrained(const srf_config_t* cfg, const srf_train_views_t* views, float* grid_out);
int srfo_sample_training_rays(const srf_config_t* cfg, const srf_train_views_t* views, const uint8_t* bitfield,
                              uint32_t n_rays, uint32_t n_rays_shift, uint32_t n_coords, const srfo_rng_t* rng,
                              int snap_to_pixel_centers, uint32_t* ray_counter, uint32_t* numsteps_counter,
                              float* rays_out, float* rays_rgba, uint32_t* numsteps_out, float* coords_out);

/* Training compositor (host pointers); n_rays_kept is the training sampler's ray counter. */
int srfo_volume_rendering_loss(const srf_config_t* cfg, const srf_loss_params_t* params, uint32_t n_rays_kept,
                               uint32_t* ray_coord_indices, const float* rays_rgba, const float* coords,
                               const uint16_t* network_output, float mean_density, float* compacted_coords,
                               uint32_t* n_compacted_counter, uint16_t* dloss_doutput, float* loss_output,
                               float* reg_distortion);

int srfo_network_inference(const srf_config_t* cfg, const srfo_model_t* model, const float* coords,
                           uint64_t n, uint16_t* rgbsigma);
int srfo_network_density(const srf_config_t* cfg, const srfo_model_t* model, const float* positions,
                         uint64_t n, uint16_t* out16);

/* One sample-per-pixel pass over rays [ray_first, ray_first+ray_count) of the view's shard
   (ray_count = 0: all).  Output arrays are indexed by shard ray. */
int srfo_render_frame(const srf_config_t* cfg, const srf_view_t* view, const srf_post_t* post,
                      const uint8_t* bitfield, const srfo_model_t* model, uint64_t ray_first,
                      uint64_t ray_count, float* out, float* accum, float* rgba_raw,
                      uint32_t* n_samples, uint32_t* n_composited, srf_frame_stats_t* stats);

int srfo_update_grid_bitfield(const srf_config_t* cfg, const float* grid, uint8_t* bitfield, float* mean);
void srfo_rng_seed(srfo_rng_t* rng, uint64_t seed);
/* small taps for known-answer tests */
void srfo_rng_seed_seq(srfo_rng_t* rng, uint64_t seed, uint64_t seq);
uint32_t srfo_rng_next_uint(srfo_rng_t* rng);
float srfo_rng_next_float(srfo_rng_t* rng);
void srfo_rng_advance(srfo_rng_t* rng, uint64_t delta);
float srfo_ld_random_val(uint32_t index, uint32_t seed, uint32_t dim);
uint32_t srfo_morton3d(uint32_t x, uint32_t y, uint32_t z);
uint32_t srfo_sobol(uint32_t index, uint32_t dim);
int srfo_refresh_grid(const srf_config_t* cfg, const srfo_model_t* model, float* grid, uint8_t* bitfield,
                      float* mean, uint32_t* refresh_step, uint32_t training_step, srfo_rng_t* rng);

#ifdef __cplusplus
}
#endif
#endif
