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

// linear_kernel(...) of tiny-cuda-nn: one thread per element, 128 threads per block.
template <typename K, typename... Args>
void run_linear(K kernel, uint32_t n_elements, Args... args) {
    blockDim.x = 128; blockDim.y = blockDim.z = 1;
    for (uint32_t i = 0; i < n_elements; ++i) {
        blockIdx.x = i / 128; blockIdx.y = blockIdx.z = 0;
        threadIdx.x = i % 128; threadIdx.y = threadIdx.z = 0;
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

// The field a frame queries: Coordinate records (n x 7 floats) -> n x 4 halves (r, g, b, sigma raw).  Same
// signature as the oracle's srfo_network_inference, so that function can be passed directly.
typedef int (*refh_field_fn)(const void* cfg, const void* model, const float* coords, uint64_t n, uint16_t* rgbsigma);
// Positions (n x 3 floats) -> n x 16 halves (the density network's padded output); srfo_network_density's signature.
typedef int (*refh_density_fn)(const void* cfg, const void* model, const float* positions, uint64_t n, uint16_t* out16);
