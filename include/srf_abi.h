/*
 * srf_abi.h -- C-ABI of libsrf_b200.so: the sm_100a replacement for the render hot path
 * and the density-grid refresh of SphericalRF.
 *
 * Every entry point states the reference interface it replaces (paths are relative to
 * the reference project root).  Conventions:
 *   - all functions return an srf_status; srf_last_error() gives text for the last failure;
 *   - no C++ exception crosses this boundary, nothing falls back to the CPU;
 *   - pointers named d_* are device pointers, h_* host pointers;
 *   - `stream` is a cudaStream_t passed as void* (0 = the legacy default stream); work is
 *     enqueued on it and, unless a function says otherwise, not synchronised;
 *   - one context per GPU; a context is not re-entrant (the reference's Testbed is not
 *     either: internal/network/ngp_network.h:223-226 caches scratch per batch size).
 */
#ifndef SRF_ABI_H_
#define SRF_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SRF_ABI_VERSION 1u

typedef enum srf_status {
    SRF_OK = 0,
    SRF_ERR_ARG = 1,        /* bad argument or unsupported configuration value */
    SRF_ERR_CUDA = 2,       /* a CUDA runtime call failed */
    SRF_ERR_CAPACITY = 3,   /* a caller-provided buffer or a stated maximum is too small */
    SRF_ERR_TIMEOUT = 4,    /* a bounded device-side loop or wait hit its limit */
    SRF_ERR_STATE = 5       /* call order: e.g. rendering before weights were uploaded */
} srf_status;

/* Enumerators keep the reference's order (internal/utils/common.h:61-115). */
enum { SRF_ACT_NONE = 0, SRF_ACT_RELU = 1, SRF_ACT_LOGISTIC = 2, SRF_ACT_EXPONENTIAL = 3 };
enum { SRF_MODE_AO = 0, SRF_MODE_SHADE = 1, SRF_MODE_NORMALS = 2, SRF_MODE_DEPTH = 3,
       SRF_MODE_DISTANCE = 4, SRF_MODE_COST = 5 };
enum { SRF_COLOR_LINEAR = 0, SRF_COLOR_SRGB = 1, SRF_COLOR_VISPOSNEG = 2 };
/* ELossType (internal/utils/loss.h:10-18) and ERegularizationType (internal/render/ray_marcher.h) */
enum { SRF_LOSS_L2 = 0, SRF_LOSS_L1 = 1, SRF_LOSS_MAPE = 2, SRF_LOSS_SMAPE = 3, SRF_LOSS_SMOOTH_L1 = 4, SRF_LOSS_LOG_L1 = 5, SRF_LOSS_RELATIVE_L2 = 6 };
enum { SRF_REG_NONE = 0, SRF_REG_DISTORTION = 1 };
enum { SRF_TONEMAP_IDENTITY = 0, SRF_TONEMAP_ACES = 1, SRF_TONEMAP_HABLE = 2, SRF_TONEMAP_REINHARD = 3 };
enum { SRF_WARP_NGP = 0, SRF_WARP_MIPNERF360 = 1, SRF_WARP_DONERF = 2, SRF_WARP_SIGMOID = 3,
       SRF_WARP_ERP = 4, SRF_WARP_SINUSOIDAL = 5 };
enum { SRF_SAMPLING_ORIGINAL = 0, SRF_SAMPLING_DISPARITY = 1, SRF_SAMPLING_LOG = 2 };
enum { SRF_GRID_WARPED_EXP = 0, SRF_GRID_WARPED_RECIPROCAL = 1, SRF_GRID_METRIC_EXP = 2,
       SRF_GRID_METRIC_RECIPROCAL = 3 };

/* Which field answers (r,g,b,sigma) for a sample. */
enum { SRF_FIELD_NETWORK = 0,     /* hash grid + SH + two MLPs (internal/network/ngp_network.h) */
       SRF_FIELD_BLOBS = 1 };     /* closed-form Gaussian blobs, fp32: a seed-generated stand-in scene */

/*
 * Model configuration: the fields the reference reads from its JSON config
 * (sampler section "samlper": internal/sampler/occupancy_sampler.cu:909-944; "render":
 * internal/render/ray_marcher.cu:294-301; "network": internal/network/ngp_network.h:148-194,
 * 597-637) plus the Testbed members that steer rendering (internal/testbed.h:114-117).
 * Fill it with srf_config_default() first, then override.
 */
typedef struct srf_config_t {
    uint32_t struct_size;            /* sizeof(srf_config_t), checked */
    uint32_t version;                /* SRF_ABI_VERSION */
    /* sampler */
    int32_t  warping_type;           /* SRF_WARP_*  ("ERP" behaves as SINUSOIDAL: missing break) */
    uint32_t aabb_scale;
    int32_t  use_grid;
    uint32_t grid_size;
    uint32_t num_cascades;
    float    ema_decay;
    int32_t  grid_distribution_type; /* SRF_GRID_* */
    uint32_t maximum_marching_steps;
    float    cone_angle_constant;
    float    min_cone_stepsize;      /* <= 0: sqrt(3)/maximum_marching_steps */
    float    max_cone_stepsize;      /* <= 0: the reference's default */
    float    near_distance;
    float    far_distance;
    int32_t  sampling_type;          /* SRF_SAMPLING_* */
    int32_t  snap_to_pixel_centers_in_rendering;
    float    min_optical_thickness;
    /* render */
    float    transmittance_threshold;
    int32_t  train_in_linear_color;
    /* network */
    uint32_t n_levels;
    uint32_t n_features_per_level;
    uint32_t log2_hashmap_size;
    uint32_t base_resolution;
    float    per_level_scale;        /* <= 0: exp(log(desired_resolution/base)/(n_levels-1)) */
    float    desired_resolution;
    /* testbed members */
    int32_t  density_activation;     /* SRF_ACT_* */
    int32_t  rgb_activation;
    int32_t  field_type;             /* SRF_FIELD_* */
    /* limits */
    uint32_t march_iter;             /* the reference's MARCH_ITER (internal/utils/common.h:52) */
    uint32_t max_samples_per_ray;    /* 0 = no cap (the reference has none when rendering) */
    uint32_t reserved[8];
} srf_config_t;

/* Per-call camera and image description (internal/testbed.cu:479-487). */
typedef struct srf_view_t {
    float    camera[12];               /* row-major 3x4 camera-to-world, already in the reference's
                                          internal convention (after spec_opengl_to_opencv) */
    uint32_t width, height;
    float    relative_focal_length[2]; /* focal length / resolution per axis */
    float    principal_point[2];
    uint32_t spp_index;                /* CudaRenderBuffer::spp(): index of this sample-per-pixel pass */
    int32_t  render_mode;              /* SRF_MODE_* */
    float    depth_scale;              /* 1 / scene scale */
    /* Ray subset of this call: image rows are cut into blocks of `shard_rows` rows and block b
       belongs to shard b % shard_count.  shard_count = 1 renders everything. */
    uint32_t shard_rows, shard_count, shard_rank;
} srf_view_t;

/* Output stage parameters (internal/utils/render_buffer.cu:46-236, internal/testbed.cu:600-604). */
typedef struct srf_post_t {
    float   exposure;
    float   background_color[4];
    int32_t color_space;       /* SRF_COLOR_* (Testbed::m_color_space) */
    int32_t tonemap_curve;     /* SRF_TONEMAP_* */
    int32_t to_srgb;           /* output colour space */
} srf_post_t;

/* Counters of one rendered frame (all rays of the call's shard). */
typedef struct srf_frame_stats_t {
    uint64_t n_rays;           /* rays in the shard */
    uint64_t n_rays_alive;     /* rays that enter the box */
    uint64_t n_march_steps;    /* march-loop iterations over all rays */
    uint64_t n_samples;        /* live (occupied-cell) samples found by the sampler */
    uint64_t n_samples_composited; /* samples consumed before early termination */
    uint64_t n_rays_hit;       /* rays with final opacity > 0.001 */
    uint32_t n_batches;        /* sample-buffer batches the frame was cut into */
    uint32_t error_flags;      /* bit 0: a bounded device loop hit its limit */
    float    ms_sampler, ms_field, ms_composite, ms_post; /* CUDA-event times, when timing is on */
    uint32_t n_waves;          /* sampler / field / compositor launches per batch (see srf_set_wave_schedule) */
} srf_frame_stats_t;

typedef struct srf_ctx srf_ctx;

/* ---- context --------------------------------------------------------------------------- */

/* The reference's defaults for every field (occupancy_sampler.cu:909-944 and the shipped
   configs' common values for the network). */
void srf_config_default(srf_config_t* cfg);

/* Testbed::Testbed + Testbed::load_model_config (internal/testbed.cu:15-80): validates the
   configuration, binds the context to `device`, allocates grids and parameter storage. */
srf_status srf_create(const srf_config_t* cfg, int device, srf_ctx** out);
void srf_destroy(srf_ctx* ctx);
const char* srf_last_error(const srf_ctx* ctx);   /* ctx may be NULL: creation errors */
/* Turn per-stage CUDA-event timing in srf_frame_stats_t on or off (default off). */
srf_status srf_set_timing(srf_ctx* ctx, int enabled);

/* ---- parameters (Trainer::deserialize, internal/testbed.cu:151-171) -------------------- */

/* Layout of the multiresolution hash table the context expects: entry offsets per level
   (n_levels + 1 values; an entry is n_features_per_level halves), grid resolution and the
   position scale per level. Any output pointer may be NULL. */
srf_status srf_hashgrid_layout(const srf_config_t* cfg, uint32_t* offsets, uint32_t* resolutions,
                               float* scales);
/* Host fp16 arrays: the hash table (offsets[n_levels] * n_features_per_level halves), the
   density MLP (64x32 then 16x64, row-major [out][in]) and the colour MLP (64x32, 64x64,
   16x64 with rows 3..15 ignored). Parameter order follows NGPNetwork::initialize_params
   (internal/network/ngp_network.h:491-536): density MLP, colour MLP, hash grid. */
srf_status srf_upload_network(srf_ctx* ctx, const uint16_t* h_hash_table, size_t n_table_halves,
                              const uint16_t* h_density_mlp, size_t n_density_halves,
                              const uint16_t* h_rgb_mlp, size_t n_rgb_halves);
/* Stand-in scene for SRF_FIELD_BLOBS: n blobs of (cx,cy,cz,sigma,peak) and a row-major 3x3
   colour map; sigma = sum peak*exp(-|x-c|^2/(2 sigma^2)), rgb logits = M (x - 0.5). No
   counterpart in the reference. */
srf_status srf_upload_blobs(srf_ctx* ctx, const float* h_blobs, uint32_t n_blobs, const float* h_color_map);

/* ---- occupancy grid (OccupancySampler members, internal/sampler/occupancy_sampler.h:120-131) */

/* density_grid = snapshot["density_grid"] (internal/testbed.cu:167): n = cells * cascades floats
   in Morton order.  Does not rebuild the bitfield. */
srf_status srf_upload_density_grid(srf_ctx* ctx, const float* h_grid, size_t n, void* stream);
srf_status srf_download_density_grid(srf_ctx* ctx, float* h_grid, size_t n, void* stream);
srf_status srf_upload_bitfield(srf_ctx* ctx, const uint8_t* h_bits, size_t n_bytes, void* stream);
srf_status srf_download_bitfield(srf_ctx* ctx, uint8_t* h_bits, size_t n_bytes, void* stream);
/* The grid mean computed by the last bitfield rebuild (density_grid_mean). Synchronises. */
srf_status srf_download_grid_mean(srf_ctx* ctx, float* h_mean, void* stream);
/* OccupancySampler::update_grid_bitfield (internal/sampler/occupancy_sampler.cu:1063-1088):
   mean, threshold min(min_optical_thickness, mean), 8 cells -> 1 byte, max-pool for cascades. */
srf_status srf_update_grid_bitfield(srf_ctx* ctx, void* stream);
/* Testbed::train_prep_nerf (internal/testbed.cu:203-239) = sample_positions_from_grid +
   NGPNetwork::density + update_grid + update_grid_bitfield as one fused pass.
   `training_step` is Testbed's optimiser-step counter (selects all-cells vs quarter sampling);
   the sampler's own refresh counter and RNG stream live in the context and advance here.
   srf_refresh_reset() restarts them (OccupancySampler::init, occupancy_sampler.cu:956-957). */
srf_status srf_refresh_reset(srf_ctx* ctx, uint64_t rng_seed);
srf_status srf_refresh_grid(srf_ctx* ctx, uint32_t training_step, void* stream);

/* ---- stage entry points (the reference's class methods) -------------------------------- */

/* Number of rays of a view's shard, and the pixel index of each of them. */
srf_status srf_shard_ray_count(const srf_view_t* view, uint64_t* n_rays);

/* OccupancySampler::generate_rays_from_camera_matrix (occupancy_sampler.cu:1145-1188):
   pixel -> ray, box entry, jitter, advance to the first occupied cell.
   Outputs, one entry per ray of the shard (any may be NULL):
   d_dir float[n*3], d_t float[n] (t after the advance), d_alive uint8[n], d_pixel uint32[n]. */
srf_status srf_generate_rays(srf_ctx* ctx, const srf_view_t* view, float* d_dir, float* d_t,
                             uint8_t* d_alive, uint32_t* d_pixel, void* stream);

/* OccupancySampler::generate_coords_from_rays (occupancy_sampler.cu:1190-1216), restructured:
   instead of <= 8 samples per ray per host iteration, the whole march of every ray is
   emitted at once into a compact buffer (the layout of the reference's training sampler,
   occupancy_sampler.cu:544-549: per ray a count and a base).
   Step 1 counts: d_counts uint32[n_rays].  The caller turns counts into bases (exclusive
   scan) or asks srf_sample_offsets to.  Step 2 emits into caller buffers:
   d_coords float[total*7] in the reference's Coordinate layout (pos.xyz, dt, dir.xyz;
   internal/utils/common.h:140-155); d_ordinal / d_cell (may be NULL) receive the march-step
   ordinal and the Morton cell index of every sample. */
srf_status srf_sample_count(srf_ctx* ctx, const srf_view_t* view, uint32_t* d_counts, void* stream);
srf_status srf_sample_offsets(srf_ctx* ctx, const uint32_t* d_counts, uint64_t n_rays,
                              uint64_t* d_offsets /* n_rays + 1 */, void* stream);
srf_status srf_sample_emit(srf_ctx* ctx, const srf_view_t* view, const uint64_t* d_offsets,
                           uint64_t capacity, float* d_coords, uint32_t* d_ordinal,
                           uint32_t* d_cell, void* stream);

/* NGPNetwork::inference_mixed_precision (internal/network/ngp_network.h:212-279):
   d_coords float[n*7] (Coordinate records) -> d_rgbsigma half[n*4] (r,g,b raw, sigma raw),
   column-major 4 x n as the reference requires. */
srf_status srf_network_inference(srf_ctx* ctx, const float* d_coords, uint64_t n,
                                 uint16_t* d_rgbsigma, void* stream);
/* NGPNetwork::density (ngp_network.h:281-310): positions float[n*3] -> half[n*16]. */
srf_status srf_network_density(srf_ctx* ctx, const float* d_positions, uint64_t n,
                               uint16_t* d_density_out, void* stream);

/* RayMarcher::volume_rendering (internal/render/ray_marcher.cu:204-282,376-415) over the
   compact sample layout: per ray front-to-back compositing with early termination.
   d_rgba float[n_rays*4] receives the premultiplied colour and opacity of every ray,
   d_n_composited uint32[n_rays] (may be NULL) the number of samples consumed. */
srf_status srf_volume_rendering(srf_ctx* ctx, const srf_view_t* view, const uint64_t* d_offsets,
                                uint64_t n_rays, const float* d_coords, const uint16_t* d_rgbsigma,
                                float* d_rgba, uint32_t* d_n_composited, void* stream);

/* ---- training-side sampler ---------------------------------------------------------------- */

/* The Dataset fields the sampler's training-side kernels read (OccupancySampler::init and
   sample_coords_from_dataset, internal/sampler/occupancy_sampler.cu:946-978,1090-1143).  All pointers are
   device pointers and have the reference's buffer layouts, so its own GPUMemory buffers can be passed as
   they are. */
typedef struct srf_train_views_t {
    uint32_t n_images;
    int32_t  width, height;                 /* image_resolution */
    float    focal_length[2];               /* in pixels */
    float    principal_point[2];            /* relative */
    const float*    d_xforms;               /* n_images x 12 floats: 3x4 camera matrices, column-major
                                               (Eigen::Matrix<float,3,4>'s default storage) */
    const uint16_t* d_images;               /* fp16 rgba, n_images * height * width * 4 (may be NULL for srf_sampler_init) */
    const uint16_t* d_sampling_probability; /* fp16, n_images * height * width; NULL = every pixel eligible */
} srf_train_views_t;

/* OccupancySampler::init (occupancy_sampler.cu:946-978): restarts the refresh counter and RNG stream (as
   srf_refresh_reset) and initialises the density grid: with a grid, `init_grid_with_mask` and the NGP warp,
   mark_untrained_density_grid (:12-102) writes 0 into cells some training view sees and -1 into the others;
   in every other case the grid is cleared.  The bitfield is not touched (the reference rebuilds it at the next
   refresh).  `views` may be NULL when no mask is asked for. */
srf_status srf_sampler_init(srf_ctx* ctx, const srf_train_views_t* views, int init_grid_with_mask,
                            uint64_t rng_seed, void* stream);

/* OccupancySampler::sample_coords_from_dataset / generate_training_samples_nerf (occupancy_sampler.cu:513-689,
   1090-1143): for each of n_rays training rays pick image and pixel (PCG32 state `rng_state`/`rng_inc`, stream
   position i*8 for ray i), march the ray and emit its occupied samples (at most maximum_marching_steps) as
   Coordinate records into one variable-length buffer.
     d_ray_counter[1]      rays kept                    d_numsteps_counter[1]  samples of all rays with samples,
     d_rays[kept*6]        origin, direction                                   including rays that found no room
     d_rays_rgba[kept*4]   the pixel's rgba             d_numsteps[kept*2]     per kept ray: sample count, base
     d_coords[n_coords*7]  samples, ray after ray
   A ray is kept when it has samples and base + count <= n_coords, where base is the number of samples of all
   earlier rays (kept or not).  The reference takes base and the ray slot from atomic counters, so its order
   depends on scheduling; this entry returns the order of a serial execution (ray 0, 1, 2, ...), reproducibly.
   The counters are set, not added to.  Totals must stay below 2^32. */
srf_status srf_sample_training_rays(srf_ctx* ctx, const srf_train_views_t* views, uint32_t n_rays,
                                    uint32_t n_rays_shift, uint32_t n_coords, uint64_t rng_state, uint64_t rng_inc,
                                    int snap_to_pixel_centers, uint32_t* d_ray_counter, uint32_t* d_numsteps_counter,
                                    float* d_rays, float* d_rays_rgba, uint32_t* d_numsteps, float* d_coords,
                                    void* stream);

/* Arguments of the training compositor that are not buffers. */
typedef struct srf_loss_params_t {
    uint32_t n_rays;                    /* rays of the batch (n_rays_per_batch): threads to run and the loss normaliser */
    uint32_t n_max_compacted_coords;    /* capacity of the compacted buffers, in samples */
    int32_t  loss_type;                 /* SRF_LOSS_* */
    float    loss_scale;
    int32_t  regularization_type;       /* SRF_REG_* */
    float    background_color[3];
    int32_t  color_space;               /* SRF_COLOR_* of the training images */
    int32_t  train_with_random_bg_color;/* draw the background from the RNG state below (one colour for the batch,
                                           as the reference's by-value rng gives) */
    uint64_t rng_state, rng_inc;
    uint32_t padded_output_width;       /* stride of d_dloss_doutput in halves (>= 4; NGPNetwork::padded_output_width) */
} srf_loss_params_t;

/* RayMarcher::volume_rendering_with_loss_and_gradient (internal/render/ray_marcher.cu:9-202,303-375): for
   each of the *d_n_rays_counter rays the training sampler kept, composite its samples front to back until the
   transmittance threshold, compare with the ray's training pixel, and write dL/d(network output) of the
   samples consumed, compacted ray after ray.
     in:  d_ray_coord_indices[n*2] (count, base per ray; srf_sample_training_rays' d_numsteps), d_rays_rgba[n*4],
          d_coords[*7], d_network_output half[*4] (srf_network_inference on d_coords)
     out: d_ray_coord_indices rewritten to (compacted count, compacted base); d_compacted_coords[*7];
          d_n_compacted_counter[1] = samples consumed by all rays (may exceed the capacity, as in the reference);
          d_dloss_doutput half[* padded_output_width] (first 4 of each row written);
          d_loss_output[n_rays] (may be NULL): mean loss of the ray / n_rays;
          d_reg_distortion[*2] (required for SRF_REG_DISTORTION, else NULL): running sums of w and w*m.
   Compacted bases are those of a serial execution in ray order (the reference's depend on scheduling). */
srf_status srf_volume_rendering_loss(srf_ctx* ctx, const srf_loss_params_t* params, const uint32_t* d_n_rays_counter,
                                     uint32_t* d_ray_coord_indices, const float* d_rays_rgba, const float* d_coords,
                                     const uint16_t* d_network_output, float* d_compacted_coords,
                                     uint32_t* d_n_compacted_counter, uint16_t* d_dloss_doutput, float* d_loss_output,
                                     float* d_reg_distortion, void* stream);

/* ---- whole frames ------------------------------------------------------------------------ */

/* Testbed::render_frame (internal/testbed.cu:479-606) for one sample-per-pixel pass of one
   view's shard.  d_out float[n_shard_rays*4]: the shard's pixels in shard order (row blocks
   concatenated), after shade, accumulate (running mean over spp_index) and tonemap.
   d_accum float[n_shard_rays*4] is the accumulate buffer the caller keeps between passes
   (ignored contents when spp_index == 0).  d_rgba_raw (may be NULL) receives the
   premultiplied pre-shade colour/opacity per ray, d_n_samples (may be NULL) the sampler's
   per-ray sample count.  `stats` (may be NULL) costs one stream synchronisation. */
srf_status srf_render_frame(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post,
                            float* d_out, float* d_accum, float* d_rgba_raw, uint32_t* d_n_samples,
                            srf_frame_stats_t* stats, void* stream);

/* The same frame with the output stage fused into the gather of a sharded render: the pixel of every ray
   of the shard is stored at its position in a whole-image buffer d_image float[height*width*4], which may
   live on another GPU of the box (a peer-mapped pointer: plain stores over NVLink, no collective).  Pixels
   outside the shard are not touched.  d_accum stays local and shard-indexed.  Replaces shade_kernel's
   scatter `frame_buffer[payload.idx] = ...` (internal/testbed.cu:476) across GPUs; the caller orders the
   stores against the consumer (a barrier or stream event after the call). */
srf_status srf_render_frame_scatter(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, float* d_image,
                                    float* d_accum, srf_frame_stats_t* stats, void* stream);

/* ---- several GPUs of one box, driven by one host process ------------------------------------------------------
   The reference renders on one GPU (internal/testbed.cu:479-606 loops over one device); its rays are independent
   (state = RayPayload + rgba, outputs keyed by payload.idx, :476), so a frame's rays shard.  The caller creates one
   context per device with the same configuration and uploads the same parameters and grid to each (replication).
   srf_comm_init enables peer access from every device to the first context's device and creates one stream per
   device.  No collective library is involved. */
typedef struct srf_comm srf_comm;
srf_status srf_comm_init(srf_ctx* const* ctx, uint32_t n, srf_comm** out);
void srf_comm_destroy(srf_comm* comm);
const char* srf_comm_last_error(const srf_comm* comm);   /* comm may be NULL: creation errors */

/* Testbed::render for n_views views of one resolution, each view's rays cut into blocks of shard_rows image rows that
   are dealt round-robin to the contexts (views[k].shard_count / shard_rank are set here).  Every context runs spp passes
   of srf_render_frame_scatter on its own device and stream and stores its finished pixels straight into the images on
   the first context's device (peer stores); stream events order those stores before the copy to the host.
   d_images: device buffer on the first context's device, n_views * height * width * 4 floats, or NULL to use an
   internal one.  h_images (may be NULL): the same, in host memory (pinned memory makes the copy asynchronous).
   stats (may be NULL): n entries, the counters of each context's last frame.  Synchronises. */
srf_status srf_render_frames_sharded(srf_comm* comm, const srf_view_t* views, uint32_t n_views, const srf_post_t* post,
                                     uint32_t spp, float* d_images, float* h_images, srf_frame_stats_t* stats);
/* Device time of the last srf_render_frames_sharded call on each context's stream (CUDA events), in ms: the time of
   the call is their maximum.  The reference times with std::chrono around its calls (internal/testbed.cu:179-196). */
srf_status srf_get_timings(const srf_comm* comm, float* ms_per_context, uint32_t n);

/* How srf_render_frame schedules a frame.  The reference alternates rounds of <= 8 march steps per ray with
   network evaluation, compositing and compaction of finished rays (internal/testbed.cu:523-583), so samples behind
   the point where a ray saturates are never evaluated.  Here a frame runs in a few large waves: wave k takes every
   unfinished ray steps[k] march steps further, the field and the compositor run on what was emitted, rays whose
   pixel is final are dropped; a last wave finishes whatever is left.  The image does not depend on the schedule.
   Default {128, 512, 2048, 8192}; n = 0 renders each frame in one pass.  (A call that asks srf_render_frame for per-ray
   sampler counts always runs in one pass.) */
srf_status srf_set_wave_schedule(srf_ctx* ctx, const uint32_t* steps, uint32_t n);

/* Memory the frame path may spend on cell-major copies of the leading hash-grid levels (for every cell of a level,
   the fp16 entries of its eight corners side by side: one 16*n_features_per_level-byte read per sample and level
   instead of eight scattered ones; NGPNetwork's grid encoding, internal/network/ngp_network.h:233-248, reads the
   entries one by one).  As many leading levels as fit are copied; the copies are rebuilt on the first frame after
   srf_upload_network.  Default 4 GiB (10 levels of the 16 x 2^19 grid); 0 switches them off.  Results do not change. */
srf_status srf_set_cell_table_budget(srf_ctx* ctx, uint64_t bytes);

/* Testbed::render (internal/python_api.cu:17-41): spp passes of srf_render_frame and the copy
   to a host image h_image float[height*width*4] (whole image; shard_count must be 1).
   Synchronises. */
srf_status srf_render(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, uint32_t spp,
                      float* h_image, srf_frame_stats_t* stats);

/* Parity tap: per-ray sample lists of rays [ray_first, ray_first + ray_count) of the shard,
   written to host arrays.  h_counts uint32[ray_count]; the other arrays hold the samples of
   all these rays back to back (capacity entries at most): h_pos_dt float[*4] (warped
   position, dt), h_ordinal, h_cell.  *n_total receives the number of samples.  Synchronises. */
srf_status srf_dump_samples(srf_ctx* ctx, const srf_view_t* view, uint64_t ray_first,
                            uint64_t ray_count, uint64_t capacity, uint32_t* h_counts,
                            float* h_pos_dt, uint32_t* h_ordinal, uint32_t* h_cell,
                            uint64_t* n_total);

/* Device-side error word of the context (the reference has none: its kernels cannot time out).  Bits: 1 = a
   ray hit the march loop's iteration bound, 2 = a wait on the tensor-core commit barrier expired, 4 = the
   sample pool ran out of chunks.  Frames enqueued without `stats` do not synchronise and therefore cannot
   report; the word stays set across frames until one of srf_render, srf_dump_samples, a frame with `stats`
   or this call has returned it as SRF_ERR_TIMEOUT / SRF_ERR_CAPACITY, which also clears it.  Synchronises
   `stream`.  `flags` (may be NULL) receives the raw word. */
srf_status srf_check_errors(srf_ctx* ctx, void* stream, uint32_t* flags);

/* Upper bound of live samples the context keeps scratch for; a frame with more samples is
   rendered in several batches.  0 = grow on demand (the default). */
srf_status srf_reserve(srf_ctx* ctx, uint64_t max_samples);

/* No counterpart in the reference.  srf_sample_offsets for callers that may not allocate device
   memory: programs that gave the whole GPU to their own pool at start-up, frame loops that must avoid
   the device-wide synchronisation cudaMalloc/cudaFree imply, hosts that forbid allocation after
   initialisation.  The tile sums of the scan live in a fixed array inside the library image instead of
   a context buffer, so this call performs no cudaMalloc/cudaFree and calls no allocating routine.
   Limits and rules:
     - at most 33 554 432 counts (16 384 tile sums of 2048 counts; 128 KiB held by every GPU that loads
       the library, until the process exits); more is refused with SRF_ERR_CAPACITY and a message;
     - the first call on a device looks the array's device address up (cudaGetSymbolAddress with that
       device current); make that first call before any stream capture begins;
     - all calls on a device share the array: calls whose kernels may overlap on the GPU (different
       streams without ordering) race and must be serialised by the caller.  Nothing has to be cleared
       between calls: each call overwrites every entry it later reads.
   `err`/`err_len` (may be NULL/0) receive the message of a failure.  Inputs and outputs are as in
   srf_sample_offsets; no context is needed. */
srf_status srf_sample_offsets_static(int device, const uint32_t* d_counts, uint64_t n_rays, uint64_t* d_offsets,
                                     void* stream, char* err, size_t err_len);

/* Evaluates the canonical elementary functions on the device (self-test tap):
   op 0 atan2(a,b), 1 asin(a), 2 cos(a), 3 sin(a), 4 exp(a), 5 log(a). */
srf_status srf_eval_math(int device, int op, const float* h_a, const float* h_b, float* h_out, size_t n);

#ifdef __cplusplus
}
#endif
#endif /* SRF_ABI_H_ */
