// srf_kernels.cuh -- launch wrappers of the device kernels (implemented in the .cu files of this
// directory) and the small structures they share with the context.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "srf_device.cuh"

namespace srf {

constexpr int kMaxLevels = 16;

// One level of the multiresolution hash grid.
struct LevelMeta {
    float scale;        // position scale: p = x * scale + 0.5
    uint32_t res;       // grid resolution
    uint32_t offset;    // first entry of the level (entries, not halves)
    uint32_t size;      // entries in the level
    uint32_t dense;     // 1: x + y*res + z*res^2, 0: spatial hash
};

struct NetMeta {
    LevelMeta level[kMaxLevels];
    uint32_t n_levels, n_features;
};

// Device counters of one frame; zeroed before the count kernel.
struct FrameCounters {
    unsigned long long n_alive, n_march_steps, n_samples, n_composited, n_hit;
    unsigned int error_flags;
    unsigned int pad;
};

// Per-ray record written by the count pass.
//   ray_dir_t: direction (xyz) and the ray parameter after the jitter (w)
//   ray_end:   RayEnd of the full march
void launch_ray_count(const DevCfg& g, const DevView& v, const uint8_t* bits, float4* ray_dir_t, uint8_t* ray_end,
                      uint32_t* counts, FrameCounters* counters, cudaStream_t stream);

// Exclusive scan of counts[0..n) into offsets[0..n] (offsets[n] = total). scratch: >= scan_scratch_bytes(n).
size_t scan_scratch_bytes(uint64_t n);
void launch_scan(const uint32_t* counts, uint64_t n, uint64_t* offsets, void* scratch, cudaStream_t stream);

// Emit pass over rays [ray_begin, ray_end): sample j of ray r goes to slot offsets[r] - offsets[ray_begin] + j.
//   pos_dt:     warped position (xyz) and step width (w)
//   sample_ray: the ray (shard index) of each sample
//   coords7:    alternatively the reference's Coordinate records (pos.xyz, dt, dir.xyz), 7 floats
//   ordinal/cell: optional march-step ordinal and Morton cell index (parity taps)
void launch_ray_emit(const DevCfg& g, const DevView& v, const uint8_t* bits, const float4* ray_dir_t,
                     const uint64_t* offsets, uint64_t ray_begin, uint64_t ray_end, float4* pos_dt,
                     uint32_t* sample_ray, float* coords7, uint32_t* ordinal, uint32_t* cell,
                     FrameCounters* counters, cudaStream_t stream);

// Frame path: single-pass paged sampler.  Samples of a ray live in a linked list of chunks of
// kChunkSamples records taken from a pool; see srf_sampler.cu.
constexpr uint32_t kChunkSamples = 16;
constexpr uint32_t kChunkShift = 4;
constexpr uint32_t kNoChunk = 0xffffffffu;
void launch_march_paged(const DevCfg& g, const DevView& v, const uint8_t* bits, uint64_t ray_begin, uint64_t ray_end,
                        float4* pool_pos_dt, uint32_t* chunk_ray, uint32_t* chunk_next, uint32_t pool_chunks,
                        uint32_t* chunk_cursor, float4* ray_dir_t, uint8_t* ray_end_out, uint32_t* ray_count,
                        uint32_t* ray_head, FrameCounters* counters, cudaStream_t stream, uint32_t wave = 0,
                        uint32_t pause_at = 0xffffffffu, uint32_t* ray_ordinal = nullptr, uint32_t* ray_total = nullptr,
                        uint4* ray_sh = nullptr);
//   wave / pause_at: rays are marched up to `pause_at` loop iterations in all; paused rays resume in the next wave from
//   ray_dir_t.w (t), ray_ordinal (loop iterations) and ray_total (samples so far).

// Rays only (generate_rays_from_camera_matrix): direction, t at the first occupied step, alive, pixel.
void launch_generate_rays(const DevCfg& g, const DevView& v, const uint8_t* bits, float* dir, float* t,
                          uint8_t* alive, uint32_t* pixel, cudaStream_t stream);

// Field evaluation on n samples.
//   network: hash-grid encoding + SH + density MLP + colour MLP -> (r,g,b,sigma) raw, 4 halves per sample.
//   dirs come either from ray_dir_t[sample_ray[i]] (compact layout) or from coords7 (Coordinate records).
void launch_field_network(const NetMeta& net, const __half* table, const __half* w_density, const __half* w_rgb,
                          const float4* pos_dt, const uint32_t* sample_ray, const float4* ray_dir_t,
                          const float* coords7, uint64_t n, uint2* rgbsigma, float4* shaded, const DevCfg* g,
                          const DevView* v, cudaStream_t stream, const uint32_t* n_chunks_dev = nullptr,
                          uint32_t ray_shift = 0);
//   the same on tcgen05 tensor cores with TMEM accumulators (srf_field_tc.cu); error_flags bit 1 reports an
//   expired wait on the MMA commit barrier.
//   Output: either rgbsigma (4 raw halves per sample, the reference's network output) or, on the frame path,
//   shaded (activated colour and step opacity, 4 floats per sample; needs g, v and pos_dt for dt).
void launch_field_network_tc(const NetMeta& net, const __half* table, const __half* w_density, const __half* w_rgb,
                             const float4* pos_dt, const uint32_t* sample_ray, const float4* ray_dir_t,
                             const float* coords7, uint64_t n, uint2* rgbsigma, float4* shaded, const DevCfg* g,
                             const DevView* v, unsigned int* error_flags, cudaStream_t stream,
                             const uint32_t* n_chunks_dev = nullptr, uint32_t ray_shift = 0, const uint4* ray_sh = nullptr,
                             const uint4* cell_table = nullptr, int n_cell_levels = 0,
                             const float* act_lut = nullptr);
//   act_lut (frame path, optional): the two activation functions tabulated over all fp16 arguments
//   (launch_build_activation_table: 2 x 65 536 floats).
void launch_build_activation_table(const DevCfg& g, float* lut, cudaStream_t stream);
//   cell_table (optional): cell-major copies of the leading n_cell_levels levels (launch_build_cell_tables;
//   cell_table_units gives the size in 16-byte units and the per-level offsets).
size_t cell_table_units(const NetMeta& net, int n_levels, unsigned long long* offsets);
void launch_build_cell_tables(const NetMeta& net, const __half* table, int n_levels, uint4* out, cudaStream_t stream);
//   ray_sh (frame path, optional): the 16 spherical-harmonics halves of every ray's direction, written by the sampler.
//   n_chunks_dev (frame path): the number of samples is *n_chunks_dev * kChunkSamples, read on the device, and
//   the ray of sample s is sample_ray[s >> ray_shift] (one entry per chunk).
//   density only: positions (3 floats, stride given in floats) -> 16 halves per position.
void launch_field_density(const NetMeta& net, const __half* table, const __half* w_density, const float* positions,
                          uint32_t stride, uint64_t n, __half* out16, cudaStream_t stream);
//   analytic blob field in fp32 -> (r,g,b logits, sigma), 4 floats per sample.
//   writes shaded samples (activated colour, step opacity).
void launch_field_blobs(const DevCfg& g, const DevView& v, const float* blobs, uint32_t n_blobs, const float* color_map,
                        const float4* pos_dt, uint64_t n, float4* shaded, cudaStream_t stream,
                        const uint32_t* n_chunks_dev = nullptr);

//   Normals render mode: (unit normal from the density MLP's input gradient, step opacity) per sample.
void launch_field_normals(const DevCfg& g, const NetMeta& net, const __half* table, const __half* w_density, const float4* pos_dt,
                          uint64_t n, float4* shaded, cudaStream_t stream, const uint32_t* n_chunks_dev = nullptr);

struct DevPost {
    float exposure_scale;      // 2^exposure
    float bg[4];               // background colour, already converted to the accumulation space
    int color_space, tonemap_curve, to_srgb;
};

// Compositing of rays [ray_begin, ray_end) over the compact layout, followed by shade, accumulate and
// tonemap of the ray's pixel.  shaded: per sample (activated r, g, b, step opacity) as the frame-path field
// kernels write it.  Any output may be null.
void launch_composite(const DevCfg& g, const DevView& v, const DevPost& post, const uint64_t* offsets,
                      uint64_t ray_begin, uint64_t ray_end, const float4* shaded, const uint8_t* ray_end_reason,
                      float4* out, float4* accum, float4* rgba_raw, uint32_t* n_composited, FrameCounters* counters,
                      cudaStream_t stream);

// The same over per-ray chunk lists (frame path).
void launch_composite_paged(const DevCfg& g, const DevView& v, const DevPost& post, uint64_t ray_begin, uint64_t ray_end,
                            const uint32_t* ray_head, const uint32_t* ray_count, const uint32_t* chunk_next,
                            const float4* pool_shaded, uint8_t* ray_end_reason, float4* out, float4* accum,
                            float4* rgba_raw, uint32_t* n_composited, FrameCounters* counters, cudaStream_t stream,
                            uint32_t wave = 0, float4* ray_rgba = nullptr, uint32_t* ray_ncomp = nullptr);
//   waves: a paused ray's running colour/opacity and consumed-sample count wait in ray_rgba / ray_ncomp; a ray whose
//   pixel has been written is marked RAY_END_DONE in ray_end_reason.

// Compositing over Coordinate records (stage entry srf_volume_rendering): no post stage.
void launch_composite_coords(const DevCfg& g, const DevView& v, const uint64_t* offsets, uint64_t n_rays,
                             const float* coords7, const uint2* rgbs_half, float4* rgba, uint32_t* n_composited,
                             cudaStream_t stream);

// Grid refresh pieces (srf_refresh.cu).
struct RefreshRng { uint64_t state, inc; };
// Density MLP weights the refresh needs, as fp32 (exact images of the fp16 parameters): layer 1 [64][32] and
// row 0 of layer 2.  Passed to the kernel by value (8.4 KB of its parameter block).
struct RefreshWeights { float w1[64 * 32]; float w2[64]; };
// One sampling pass: cell pick, jitter, encoding, density output 0, atomicMax into grid_current.
void launch_refresh_sample(const DevCfg& g, const NetMeta& net, const __half* table, const RefreshWeights& w,
                           const float* grid, float* grid_current, uint32_t n_elements, uint32_t step, RefreshRng rng,
                           float thresh, uint32_t aabb_scale, cudaStream_t stream);
// The whole refresh in two launches when every cell is sampled once, there is one cascade and no cell is masked.
void launch_refresh_fused(const DevCfg& g, const NetMeta& net, const __half* table, const RefreshWeights& w, float* grid,
                          uint32_t step, RefreshRng rng, float thresh, uint32_t aabb_scale, float decay, float* partial_a,
                          float* partial_b, float* mean, unsigned int* ticket, uint8_t* bits, float min_optical_thickness,
                          uint32_t* skip_shell, uint32_t* skip_yz, unsigned int* error_flags, cudaStream_t stream);
// Max-decay of every cell (when do_decay) and the mean of max(v,0) over the first `cells` entries.
void launch_decay_and_mean(float* grid, const float* grid_current, uint32_t total, uint32_t cells, float decay,
                           int do_decay, float* partial_a, float* partial_b, float* mean, cudaStream_t stream);
void launch_grid_to_bitfield(const DevCfg& g, const float* grid, uint8_t* bits, const float* mean,
                             float min_optical_thickness, cudaStream_t stream);

// Training views as the training-side kernels read them (device pointers; xforms are 3x4 column-major).
struct TrainViews {
    uint32_t n_images;
    int width, height;
    float focal_x, focal_y, pp_x, pp_y;
    const float* xforms;
    const __half* images;                   // rgba fp16 per pixel
    const __half* sampling_probability;     // fp16 per pixel, may be null (every pixel eligible)
};
// mark_untrained_density_grid: 0 for cells some training view sees, -1 for the others.
void launch_mark_untrained(const DevCfg& g, uint32_t aabb_scale, const TrainViews& tv, float* grid_out, cudaStream_t stream);
// generate_training_samples_nerf as count + scans + emit (srf_training.cu).
void launch_train_count(const DevCfg& g, const TrainViews& tv, const uint8_t* bits, uint32_t n_rays, uint32_t n_rays_shift,
                        uint32_t n_max_steps, RefreshRng rng, int snap, uint32_t* counts, uint32_t* flags, cudaStream_t stream);
void launch_train_emit(const DevCfg& g, const TrainViews& tv, const uint8_t* bits, uint32_t n_rays, uint32_t n_rays_shift,
                       uint32_t n_coords, RefreshRng rng, int snap, const uint32_t* counts, const uint64_t* offsets,
                       const uint64_t* ray_rank, uint32_t* ray_counter, uint32_t* numsteps_counter, float* rays_out,
                       float* rays_rgba, uint32_t* numsteps_out, float* coords_out, cudaStream_t stream);

// Training compositor (srf_loss.cu).  bg_linear: the background after srgb_to_linear; bg_final: the colour added
// behind a ray that ran through all its samples (bg_linear, or its sRGB encoding when not training in linear colour).
struct LossParams {
    uint32_t n_rays, n_max_compacted_coords, padded_output_width;
    int loss_type, color_space;
    float loss_scale, transmittance_threshold, min_optical_thickness;
    float bg_linear[3], bg_final[3];
};
void launch_loss_forward(const DevCfg& g, const LossParams& lp, const uint32_t* n_rays_counter, const uint32_t* ray_coord_indices,
                         const float* coords, const uint2* net_out, uint32_t* consumed, float4* ray_rgb, uint32_t n_slots,
                         cudaStream_t stream);
void launch_loss_backward(const DevCfg& g, const LossParams& lp, const uint32_t* n_rays_counter, uint32_t* ray_coord_indices,
                          const float* coords, const uint2* net_out, const float4* rays_rgba, const uint32_t* consumed,
                          const uint64_t* bases, const float4* ray_rgb, const float* mean_density, float* compacted_coords,
                          uint32_t* n_compacted_counter, __half* dloss_doutput, float* loss_output, float* reg_distortion,
                          uint32_t n_slots, cudaStream_t stream);

// Summaries of the bitfield used by the sampler's staged empty-space tests (N/32 and N*N/32 words).
void launch_build_skip_tables(const DevCfg& g, const uint8_t* bits, uint32_t* shell, uint32_t* yz, cudaStream_t stream);

void launch_eval_math(int op, const float* a, const float* b, float* out, size_t n, cudaStream_t stream);

}  // namespace srf
