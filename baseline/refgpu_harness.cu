// refgpu_harness.cu -- the REFERENCE's own CUDA kernels on the GPU, as a comparator.  NOT part of the library.
//
// baseline/build_refgpu.py cuts the kernels out of the reference's .cu files where they are mounted (the same line
// ranges as oracle/build_ref.py; nothing is copied into this repository), and nvcc compiles them for sm_100a with its
// default flags (-fmad=true, CUDA's math library) together with this file and the stand-in headers under
// oracle/ref_stub/ (Eigen, tiny-cuda-nn helpers) into baseline/_ref/libsrf_refgpu.so.  What runs on the GPU is
// therefore the reference's ray generation, occupancy-guided marching, compaction, compositing, shading, accumulation
// and tonemapping, launched in the reference's order with its host loop (one read-back of the alive counter per
// round, <= 8 samples per ray per round: internal/testbed.cu:479-606).  Two things are not the reference's:
//   * the network.  tiny-cuda-nn is not available; `network` is a function pointer with the signature of this
//     library's stage entry srf_network_inference (Coordinate records in global memory -> 4 halves per record in
//     global memory), which stands where NGPNetwork::inference_mixed_precision is called (:551-554);
//   * Eigen.  The stand-in keeps Eigen's reduction order; see oracle/ref_stub/Eigen/Dense.
// Uses: the same-GPU baseline of bench.py (--impl refgpu) and the parity tests that compare this library's frames
// with the reference's CUDA arithmetic (sample counts, composited RGBA, pixels).
#include "srf_cuda_on_host.h"

#include "internal/utils/common_device.h"
#include "internal/utils/loss.h"

#include "loss.inc"
#include "sampler_kernels.inc"
#include "marcher_kernels.inc"
#include "testbed_kernels.inc"
#include "render_buffer_kernels.inc"

#include "../include/srf_abi.h"

namespace {

constexpr uint32_t kMinSteps = 1, kMaxSteps = 8;       // RenderingBuffer::MIN/MAX_STEPS_INBETWEEN_COMPACTION
constexpr uint32_t kPaddedOutputWidth = 4;

// linear_kernel of tiny-cuda-nn: 128 threads per block, one thread per element
template <typename K, typename... Args>
void linear_launch(K kernel, cudaStream_t stream, uint32_t n_elements, Args... args) {
    if (n_elements == 0) return;
    kernel<<<(n_elements + 127) / 128, 128, 0, stream>>>(n_elements, args...);
}

// parity taps (this file's own kernels, launched only when a tap buffer is given)
__global__ void tap_samples_kernel(uint32_t n, const RayPayload* __restrict__ payloads, uint32_t* __restrict__ n_samples) {
    const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
    if (i >= n) return;
    n_samples[payloads[i].idx] += payloads[i].n_steps;
}
__global__ void tap_dead_kernel(uint32_t n, const RayPayload* __restrict__ payloads, const Eigen::Array4f* __restrict__ rgba,
                                float4* __restrict__ rgba_raw) {
    const uint32_t i = threadIdx.x + blockIdx.x * blockDim.x;
    if (i >= n || payloads[i].alive) return;
    rgba_raw[payloads[i].idx] = make_float4(rgba[i].x(), rgba[i].y(), rgba[i].z(), rgba[i].w());
}

struct Sampler {
    EWarpingType warping_type; BoundingBox aabb; bool use_grid;
    uint32_t n_grid_size, n_cascades; EGridDistType griddist_type; uint32_t n_max_steps;
    float cone_angle_constant, min_cone_stepsize, max_cone_stepsize, near_distance, far_distance;
    ESamplingType sampling_type; bool snap_rendering;
};

// OccupancySampler::OccupancySampler (internal/sampler/occupancy_sampler.cu:909-944)
Sampler make_sampler(const srf_config_t& c) {
    Sampler s;
    s.warping_type = (EWarpingType)c.warping_type;
    s.aabb = BoundingBox{Eigen::Vector3f::Constant(0.5f), Eigen::Vector3f::Constant(0.5f)};
    s.aabb.inflate(0.5f * c.aabb_scale);
    s.use_grid = c.use_grid != 0;
    s.n_grid_size = c.grid_size; s.n_cascades = c.num_cascades;
    s.griddist_type = (EGridDistType)c.grid_distribution_type;
    s.n_max_steps = c.maximum_marching_steps;
    s.cone_angle_constant = c.cone_angle_constant;
    const float sqrt3 = 1.73205080757f;
    s.min_cone_stepsize = c.min_cone_stepsize > 0.f ? c.min_cone_stepsize : sqrt3 / s.n_max_steps;
    s.max_cone_stepsize = c.max_cone_stepsize > 0.f ? c.max_cone_stepsize
                        : (s.use_grid ? (sqrt3 * (1 << (s.n_cascades - 1)) / s.n_grid_size) : s.min_cone_stepsize);
    s.near_distance = c.near_distance; s.far_distance = c.far_distance;
    s.sampling_type = (ESamplingType)c.sampling_type;
    s.snap_rendering = c.snap_to_pixel_centers_in_rendering != 0;
    return s;
}

}  // namespace

extern "C" {

typedef int (*refgpu_network_fn)(void* ctx, const float* d_coords, uint64_t n, uint16_t* d_rgbsigma, void* stream);

struct refgpu_ctx {
    srf_config_t cfg;
    Sampler s;
    int device;
    uint32_t n_elements = 0;                       // capacity in rays (next multiple of 256 of the pixel count)
    RayPayload* pay[2] = {nullptr, nullptr}; Eigen::Array4f* rgba[2] = {nullptr, nullptr};
    RayPayload* pay_hit = nullptr; Eigen::Array4f* rgba_hit = nullptr;
    Coordinate* coords = nullptr; __half* rgbsigma = nullptr;
    Eigen::Array4f* frame = nullptr;
    uint32_t* counters = nullptr;                  // [0] alive, [1] hit
    uint8_t* bits = nullptr; size_t n_bits = 0;
    SrfHostSurface* surface = nullptr;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    float last_ms = 0.f; uint32_t last_rounds = 0; uint64_t last_network_samples = 0;
};

static void free_buffers(refgpu_ctx* c) {
    void* p[] = {c->pay[0], c->pay[1], c->rgba[0], c->rgba[1], c->pay_hit, c->rgba_hit, c->coords, c->rgbsigma, c->frame};
    for (void* q : p) if (q) cudaFree(q);
    c->pay[0] = c->pay[1] = c->pay_hit = nullptr; c->rgba[0] = c->rgba[1] = c->rgba_hit = nullptr;
    c->coords = nullptr; c->rgbsigma = nullptr; c->frame = nullptr; c->n_elements = 0;
}

int refgpu_create(const srf_config_t* cfg, int device, const uint8_t* h_bitfield, size_t n_bytes, refgpu_ctx** out) {
    if (!cfg || !out) return 1;
    if (cudaSetDevice(device) != cudaSuccess) return 2;
    refgpu_ctx* c = new refgpu_ctx();
    c->cfg = *cfg; c->s = make_sampler(*cfg); c->device = device;
    bool ok = cudaStreamCreate(&c->stream) == cudaSuccess && cudaEventCreate(&c->ev0) == cudaSuccess && cudaEventCreate(&c->ev1) == cudaSuccess &&
              cudaMalloc((void**)&c->counters, 2 * sizeof(uint32_t)) == cudaSuccess && cudaMalloc((void**)&c->surface, sizeof(SrfHostSurface)) == cudaSuccess;
    if (ok && h_bitfield && n_bytes) {
        ok = cudaMalloc((void**)&c->bits, n_bytes) == cudaSuccess && cudaMemcpy(c->bits, h_bitfield, n_bytes, cudaMemcpyHostToDevice) == cudaSuccess;
        c->n_bits = n_bytes;
    }
    if (!ok) { delete c; return 2; }
    *out = c;
    return 0;
}

void refgpu_destroy(refgpu_ctx* c) {
    if (!c) return;
    cudaSetDevice(c->device);
    free_buffers(c);
    if (c->counters) cudaFree(c->counters);
    if (c->bits) cudaFree(c->bits);
    if (c->surface) cudaFree(c->surface);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

// Testbed::render_frame (internal/testbed.cu:479-606), one sample-per-pixel pass.  All buffers are device pointers:
//   d_out H*W*4 (tonemapped image), d_accum H*W*4 (kept by the caller between passes),
//   d_rgba_raw H*W*4 and d_n_samples H*W (optional parity taps; cost two small launches per round).
// Returns 0, or a CUDA error code + 100.  The time of the call (CUDA events on the harness's stream, host syncs
// included, as the reference's loop has them) is kept for refgpu_last_ms().
int refgpu_render_frame(refgpu_ctx* c, const srf_view_t* view, const srf_post_t* post, refgpu_network_fn network, void* network_ctx,
                        float* d_out, float* d_accum, float* d_rgba_raw, uint32_t* d_n_samples) {
    cudaSetDevice(c->device);
    const Sampler& s = c->s;
    cudaStream_t st = c->stream;
    const Eigen::Vector2i resolution((int)view->width, (int)view->height);
    const Eigen::Vector2f focal(resolution.x() * view->relative_focal_length[0], resolution.y() * view->relative_focal_length[1]);
    const Eigen::Vector2f pp(view->principal_point[0], view->principal_point[1]);
    Eigen::Matrix<float, 3, 4> cam;
    for (int r = 0; r < 3; ++r) for (int q = 0; q < 4; ++q) cam(r, q) = view->camera[r * 4 + q];
    const uint32_t n_pixels = view->width * view->height;
    const ERenderMode render_mode = (ERenderMode)view->render_mode;
    const uint32_t n_elements = tcnn::next_multiple(n_pixels, BATCH_SIZE_MULTIPLE);
    if (n_elements > c->n_elements) {                                        // Memory Allocation (:488-499)
        free_buffers(c);
        bool ok = true;
        for (int k = 0; k < 2; ++k) ok = ok && cudaMalloc((void**)&c->pay[k], sizeof(RayPayload) * n_elements) == cudaSuccess &&
                                             cudaMalloc((void**)&c->rgba[k], sizeof(Eigen::Array4f) * n_elements) == cudaSuccess;
        ok = ok && cudaMalloc((void**)&c->pay_hit, sizeof(RayPayload) * n_elements) == cudaSuccess &&
             cudaMalloc((void**)&c->rgba_hit, sizeof(Eigen::Array4f) * n_elements) == cudaSuccess &&
             cudaMalloc((void**)&c->coords, sizeof(Coordinate) * (size_t)n_elements * kMaxSteps) == cudaSuccess &&
             cudaMalloc((void**)&c->rgbsigma, sizeof(__half) * (size_t)n_elements * kMaxSteps * kPaddedOutputWidth) == cudaSuccess &&
             cudaMalloc((void**)&c->frame, sizeof(Eigen::Array4f) * n_elements) == cudaSuccess;
        if (!ok) { free_buffers(c); return 102; }
        cudaMemset(c->coords, 0, sizeof(Coordinate) * (size_t)n_elements * kMaxSteps);
        c->n_elements = n_elements;
    }
    cudaEventRecord(c->ev0, st);
    if (d_rgba_raw) cudaMemsetAsync(d_rgba_raw, 0, sizeof(float4) * n_pixels, st);
    if (d_n_samples) cudaMemsetAsync(d_n_samples, 0, sizeof(uint32_t) * n_pixels, st);
    // Clear Buffer & Generate Rays (:502-516)
    cudaMemsetAsync(c->frame, 0, sizeof(Eigen::Array4f) * n_pixels, st);
    cudaMemsetAsync(c->pay[0], 0, sizeof(RayPayload) * n_elements, st);
    {
        const dim3 threads = {16, 8, 1};
        const dim3 blocks = {(view->width + threads.x - 1) / threads.x, (view->height + threads.y - 1) / threads.y, 1};
        init_rays_with_payload_kernel_nerf<<<blocks, threads, 0, st>>>(resolution, focal, pp, cam, view->spp_index, s.snap_rendering, s.aabb, c->pay[0]);
        linear_launch(advance_pos_nerf, st, n_pixels, view->spp_index, c->pay[0], s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
                      s.griddist_type, s.use_grid ? (const uint8_t*)c->bits : (const uint8_t*)nullptr, s.n_max_steps, s.cone_angle_constant,
                      s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type);
    }
    cudaMemsetAsync(c->rgba[0], 0, sizeof(Eigen::Array4f) * n_elements, st);
    cudaMemsetAsync(c->counters + 1, 0, sizeof(uint32_t), st);               // n_hit_counter (:519)
    uint32_t i_steps_offset = 1, double_buffer_index = 0, n_alive = n_pixels, rounds = 0;
    uint64_t network_samples = 0;
    while (i_steps_offset < MARCH_ITER) {                                    // :523-583
        RayPayload* prev_p = c->pay[double_buffer_index % 2]; Eigen::Array4f* prev_c = c->rgba[double_buffer_index % 2];
        RayPayload* cur_p = c->pay[(double_buffer_index + 1) % 2]; Eigen::Array4f* cur_c = c->rgba[(double_buffer_index + 1) % 2];
        ++double_buffer_index;
        if (d_rgba_raw && rounds > 0) linear_launch(tap_dead_kernel, st, n_alive, (const RayPayload*)prev_p, (const Eigen::Array4f*)prev_c, (float4*)d_rgba_raw);
        cudaMemsetAsync(c->counters, 0, sizeof(uint32_t), st);
        linear_launch(compact_rays_kernel, st, n_alive, prev_p, prev_c, cur_p, cur_c, c->pay_hit, c->rgba_hit, c->counters, c->counters + 1);
        cudaMemcpyAsync(&n_alive, c->counters, sizeof(uint32_t), cudaMemcpyDeviceToHost, st);
        if (cudaStreamSynchronize(st) != cudaSuccess) return 100 + (int)cudaGetLastError();
        if (n_alive == 0) break;
        const uint32_t n_steps = tcnn::clamp(n_pixels / n_alive, kMinSteps, kMaxSteps);
        linear_launch(generate_coords_from_rays_regularly_kernel, st, n_alive, n_steps, s.warping_type, s.aabb, s.n_grid_size, s.n_cascades,
                      s.griddist_type, s.use_grid ? (const uint8_t*)c->bits : (const uint8_t*)nullptr, s.n_max_steps, s.cone_angle_constant,
                      s.min_cone_stepsize, s.max_cone_stepsize, s.near_distance, s.far_distance, s.sampling_type, cur_p, c->coords);
        if (d_n_samples) linear_launch(tap_samples_kernel, st, n_alive, (const RayPayload*)cur_p, d_n_samples);
        const uint32_t n_net = tcnn::next_multiple(n_alive * n_steps, BATCH_SIZE_MULTIPLE);
        if (network(network_ctx, (const float*)c->coords, n_net, (uint16_t*)c->rgbsigma, st) != 0) return 3;
        network_samples += n_net;
        linear_launch(volume_rendering_kernel, st, n_alive, n_steps, i_steps_offset, cur_p, cur_c, (const Coordinate*)c->coords,
                      (const precision_t*)c->rgbsigma, kPaddedOutputWidth, (EActivation)c->cfg.density_activation, (EActivation)c->cfg.rgb_activation,
                      render_mode, s.warping_type, s.aabb, s.n_cascades, s.min_cone_stepsize, cam, view->depth_scale, c->cfg.transmittance_threshold);
        i_steps_offset += n_steps;
        ++rounds;
    }
    uint32_t n_hit = 0;
    cudaMemcpyAsync(&n_hit, c->counters + 1, sizeof(uint32_t), cudaMemcpyDeviceToHost, st);
    cudaStreamSynchronize(st);
    linear_launch(shade_kernel, st, n_hit, (const Eigen::Array4f*)c->rgba_hit, (const RayPayload*)c->pay_hit, c->frame, render_mode,
                  c->cfg.train_in_linear_color != 0);
    // render_buffer.accumulate + tonemap (internal/utils/render_buffer.cu:204-236)
    if (view->spp_index == 0) cudaMemsetAsync(d_accum, 0, sizeof(float4) * n_pixels, st);
    {
        const dim3 threads = {16, 8, 1};
        const dim3 blocks = {(view->width + threads.x - 1) / threads.x, (view->height + threads.y - 1) / threads.y, 1};
        accumulate_kernel<<<blocks, threads, 0, st>>>(resolution, c->frame, (Eigen::Array4f*)d_accum, (float)view->spp_index, (EColorSpace)post->color_space);
        const SrfHostSurface surf = {reinterpret_cast<float4*>(d_out), (int)view->width};
        cudaMemcpyAsync(c->surface, &surf, sizeof(surf), cudaMemcpyHostToDevice, st);
        const Eigen::Array4f bg(post->background_color[0], post->background_color[1], post->background_color[2], post->background_color[3]);
        tonemap_kernel<<<blocks, threads, 0, st>>>(resolution, post->exposure, bg, (Eigen::Array4f*)d_accum, (EColorSpace)post->color_space,
                                                   post->to_srgb ? EColorSpace::SRGB : EColorSpace::Linear, (ETonemapCurve)post->tonemap_curve, c->surface);
    }
    cudaEventRecord(c->ev1, st);
    const cudaError_t e = cudaStreamSynchronize(st);                         // :605
    if (e != cudaSuccess) return 100 + (int)e;
    cudaEventElapsedTime(&c->last_ms, c->ev0, c->ev1);
    c->last_rounds = rounds; c->last_network_samples = network_samples;
    return 0;
}

float refgpu_last_ms(const refgpu_ctx* c) { return c->last_ms; }
uint32_t refgpu_last_rounds(const refgpu_ctx* c) { return c->last_rounds; }
uint64_t refgpu_last_network_samples(const refgpu_ctx* c) { return c->last_network_samples; }

}  // extern "C"
