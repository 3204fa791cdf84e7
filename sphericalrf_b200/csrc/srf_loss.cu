// srf_loss.cu -- volume rendering of training rays with loss and gradient
// (volume_rendering_with_loss_and_gradient_kernal, internal/render/ray_marcher.cu:9-202; the losses of
// internal/utils/loss.cu:18-101).
//
// The reference does everything for a ray in one kernel and reserves the ray's slots in the compacted
// buffers with atomicAdd, so the compacted order changes from run to run.  Here a forward kernel composites
// each ray and counts the samples it consumed, an exclusive scan turns the counts into bases in ray order
// (the bases a serial execution of the reference kernel would hand out), and a backward kernel writes the
// compacted coordinates, the loss and dL/d(network output).
#include "srf_kernels.cuh"

namespace srf {

namespace {

constexpr int kLossBlock = 128;

// One channel of loss_and_gradient (internal/utils/loss.cu:18-101).
__device__ __forceinline__ void loss_channel(int type, float target, float pred, float* loss, float* grad) {
    const float d = pred - target;
    switch (type) {
    case SRF_LOSS_RELATIVE_L2: {
        const float f = 1.f / (pred * pred + 1e-2f);
        *loss = d * d * f; *grad = 2.0f * d * f;
    } break;
    case SRF_LOSS_L1: *loss = fabsf(d); *grad = copysignf(1.0f, d); break;
    case SRF_LOSS_MAPE: {
        const float f = 1.f / (fabsf(pred) + 1e-2f);
        *loss = fabsf(d) * f; *grad = copysignf(f, d);
    } break;
    case SRF_LOSS_SMAPE: {
        const float f = 1.f / (0.5f * (fabsf(pred) + fabsf(target)) + 1e-2f);
        *loss = fabsf(d) * f; *grad = copysignf(f, d);
    } break;
    case SRF_LOSS_SMOOTH_L1: {
        const float a = 0.1f, ad = fabsf(d);
        const float sq = 0.5f / a * d * d;
        *loss = ad > a ? (ad - 0.5f * a) : sq;
        *grad = ad > a ? (d > 0.f ? 1.0f : -1.0f) : (d / a);
    } break;
    case SRF_LOSS_LOG_L1: {
        const float dv = fabsf(d) + 1.0f;
        *loss = srf_logf(dv); *grad = copysignf(1.f / dv, d);
    } break;
    default: *loss = d * d; *grad = 2.0f * d; break;     // L2
    }
}

struct Sample4 { float r, g, b, s; };
__device__ __forceinline__ Sample4 load_output(const uint2* out, uint64_t k) {
    const uint2 u = out[k];
    const __half2 a = *reinterpret_cast<const __half2*>(&u.x), b = *reinterpret_cast<const __half2*>(&u.y);
    return {__low2float(a), __high2float(a), __low2float(b), __high2float(b)};
}

// Both kernels give a warp to each ray.  The lanes load 32 consecutive samples of the ray at a time (coalesced)
// and evaluate the activations and the opacity of their own sample in parallel; the short recurrence over the
// samples (T, the colour sums) is then replayed in sample order by every lane from shuffled values, so each
// floating-point operation is the one the reference's single thread performs, in the same order.

// Forward pass (:57-80 and :113-116): composites until the transmittance threshold, records the number of
// samples consumed and the ray colour (background included when the ray ran through all its samples).
__global__ void __launch_bounds__(kLossBlock)
k_loss_forward(const DevCfg g, const LossParams lp, const uint32_t* __restrict__ n_rays_counter,
               const uint32_t* __restrict__ ray_coord_indices, const float* __restrict__ coords, const uint2* __restrict__ net_out,
               uint32_t* __restrict__ consumed, float4* __restrict__ ray_rgb, uint32_t n_slots) {
    const uint32_t i = (blockIdx.x * kLossBlock + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i >= n_slots) return;
    if (i >= *n_rays_counter) { if (lane == 0) consumed[i] = 0; return; }
    const uint32_t numsteps = ray_coord_indices[i * 2 + 0], base = ray_coord_indices[i * 2 + 1];
    float T = 1.f, r = 0.f, gg = 0.f, b = 0.f;
    uint32_t n = 0;
    bool stopped = false;
    for (uint32_t b0 = 0; b0 < numsteps && !stopped; b0 += 32) {
        float alpha = 0.f, cr = 0.f, cg = 0.f, cb = 0.f;
        if (b0 + lane < numsteps) {
            const uint64_t k = (uint64_t)base + b0 + lane;
            const Sample4 o = load_output(net_out, k);
            const float density = network_to_density(o.s, g.density_activation);
            alpha = 1.f - srf_expf(-density * coords[k * 7 + 3]);
            cr = network_to_rgb(o.r, g.rgb_activation);
            cg = network_to_rgb(o.g, g.rgb_activation);
            cb = network_to_rgb(o.b, g.rgb_activation);
        }
        const int cnt = (int)min(32u, numsteps - b0);
        for (int j = 0; j < cnt; ++j) {
            if (T < lp.transmittance_threshold) { stopped = true; break; }
            const float a_j = __shfl_sync(0xffffffffu, alpha, j);
            const float weight = a_j * T;
            r += weight * __shfl_sync(0xffffffffu, cr, j);
            gg += weight * __shfl_sync(0xffffffffu, cg, j);
            b += weight * __shfl_sync(0xffffffffu, cb, j);
            T *= (1.f - a_j);
            ++n;
        }
    }
    if (n == numsteps) { r += T * lp.bg_final[0]; gg += T * lp.bg_final[1]; b += T * lp.bg_final[2]; }
    if (lane == 0) {
        consumed[i] = n;
        ray_rgb[i] = make_float4(r, gg, b, T);
    }
}

// Loss and backward pass (:118-201).
__global__ void __launch_bounds__(kLossBlock)
k_loss_backward(const DevCfg g, const LossParams lp, const uint32_t* __restrict__ n_rays_counter,
                uint32_t* __restrict__ ray_coord_indices, const float* __restrict__ coords, const uint2* __restrict__ net_out,
                const float4* __restrict__ rays_rgba, const uint32_t* __restrict__ consumed, const uint64_t* __restrict__ bases,
                const float4* __restrict__ ray_rgb, const float* __restrict__ mean_density, float* __restrict__ compacted_coords,
                uint32_t* __restrict__ n_compacted_counter, __half* __restrict__ dloss_doutput, float* __restrict__ loss_output,
                float* __restrict__ reg_distortion, uint32_t n_slots) {
    const uint32_t i = (blockIdx.x * kLossBlock + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (i == 0 && lane == 0) *n_compacted_counter = (uint32_t)bases[n_slots];
    if (i >= n_slots || i >= *n_rays_counter) return;
    const uint32_t base = ray_coord_indices[i * 2 + 1];
    const uint32_t compacted_base = (uint32_t)bases[i];
    const uint32_t n_max = lp.n_max_compacted_coords;
    const uint32_t n = min(n_max - min(n_max, compacted_base), consumed[i]);                   // :122
    __syncwarp();                                      // every lane has read the old (count, base) pair
    if (lane == 0) {
        ray_coord_indices[i * 2 + 0] = n;
        ray_coord_indices[i * 2 + 1] = compacted_base;
    }
    if (n == 0) return;

    // ground-truth colour (:88-111)
    const float4 tex = rays_rgba[i];
    float target[3];
    if (g.train_in_linear_color || lp.color_space == SRF_COLOR_LINEAR) {
        target[0] = tex.x + (1.f - tex.w) * lp.bg_linear[0];
        target[1] = tex.y + (1.f - tex.w) * lp.bg_linear[1];
        target[2] = tex.z + (1.f - tex.w) * lp.bg_linear[2];
        if (!g.train_in_linear_color) for (int c = 0; c < 3; ++c) target[c] = linear_to_srgb(target[c]);
    } else if (lp.color_space == SRF_COLOR_SRGB) {
        const float t3[3] = {tex.x, tex.y, tex.z};
        for (int c = 0; c < 3; ++c)
            target[c] = tex.w > 0.f ? linear_to_srgb(t3[c] / tex.w) * tex.w + (1.f - tex.w) * lp.bg_final[c] : lp.bg_final[c];
    } else {
        target[0] = target[1] = target[2] = 0.f;          // the reference leaves rgbtarget unset for other colour spaces
    }
    const float4 rr = ray_rgb[i];
    const float rgb_ray[3] = {rr.x, rr.y, rr.z};
    float loss[3], grad[3];
    for (int c = 0; c < 3; ++c) loss_channel(lp.loss_type, target[c], rgb_ray[c], &loss[c], &grad[c]);
    const float n_rays_f = (float)lp.n_rays;
    if (loss_output && lane == 0) loss_output[i] = (loss[0] + (loss[1] + loss[2])) / 3.0f / n_rays_f;   // Eigen reduces three terms as t0 + (t1 + t2)
    const float loss_scale = lp.loss_scale / n_rays_f;
    const float output_l2_reg = g.rgb_activation == SRF_ACT_EXPONENTIAL ? 1e-4f : 0.0f;
    const float output_l1_reg_density = (g.use_grid && (*mean_density < lp.min_optical_thickness)) ? 1e-4f : 0.0f;

    float T = 1.f, r2[3] = {0.f, 0.f, 0.f};
    float sum_w = 0.f, sum_wp = 0.f;                       // distortion sums (:137-163; T stays 1 in that loop)
    for (uint32_t b0 = 0; b0 < n; b0 += 32) {
        const uint32_t j_mine = b0 + lane;
        const bool have = j_mine < n;
        const uint64_t k = (uint64_t)base + j_mine;
        Sample4 o = {0.f, 0.f, 0.f, 0.f};
        float dt = 0.f, alpha = 0.f, rgb[3] = {0.f, 0.f, 0.f};
        if (have) {
            o = load_output(net_out, k);
            dt = coords[k * 7 + 3];
            alpha = 1.f - srf_expf(-network_to_density(o.s, g.density_activation) * dt);
            rgb[0] = network_to_rgb(o.r, g.rgb_activation);
            rgb[1] = network_to_rgb(o.g, g.rgb_activation);
            rgb[2] = network_to_rgb(o.b, g.rgb_activation);
        }
        // replay the recurrence; lane j keeps the state right after its own sample
        float my_T = 0.f, my_w = 0.f, my_r2[3] = {0.f, 0.f, 0.f}, my_sw = 0.f, my_swp = 0.f;
        const int cnt = (int)min(32u, n - b0);
        for (int j = 0; j < cnt; ++j) {
            const float a_j = __shfl_sync(0xffffffffu, alpha, j);
            const float weight = a_j * T;
            r2[0] += weight * __shfl_sync(0xffffffffu, rgb[0], j);
            r2[1] += weight * __shfl_sync(0xffffffffu, rgb[1], j);
            r2[2] += weight * __shfl_sync(0xffffffffu, rgb[2], j);
            T *= (1.f - a_j);
            if (reg_distortion) {
                const float w1 = a_j * 1.f;
                sum_w += w1;
                sum_wp += w1 * (float)(b0 + j + 1) / (float)n;
            }
            if (j == lane) { my_T = T; my_w = weight; my_r2[0] = r2[0]; my_r2[1] = r2[1]; my_r2[2] = r2[2]; my_sw = sum_w; my_swp = sum_wp; }
        }
        // 28-byte coordinate records of these samples, copied by the whole warp
        {
            const float* src = coords + ((uint64_t)base + b0) * 7;
            float* dst = compacted_coords + ((uint64_t)compacted_base + b0) * 7;
            for (int q = lane; q < cnt * 7; q += 32) dst[q] = src[q];
        }
        if (have) {
            if (reg_distortion) {
                float* rd = reg_distortion + ((uint64_t)compacted_base + j_mine) * 2;
                rd[0] = my_sw; rd[1] = my_swp;
            }
            const float raw[3] = {o.r, o.g, o.b};
            float out[4], v[3];
            for (int c = 0; c < 3; ++c) {
                const float dloss_by_drgb = my_w * grad[c];
                out[c] = loss_scale * (dloss_by_drgb * network_to_rgb_derivative(raw[c], g.rgb_activation) + fmaxf(0.0f, output_l2_reg * raw[c]));
                v[c] = my_T * rgb[c] - (rgb_ray[c] - my_r2[c]);                               // T * rgb - suffix
            }
            const float dot = srf_dot3f(grad[0], v[0], grad[1], v[1], grad[2], v[2]);
            const float dloss_by_dmlp = network_to_density_derivative(o.s, g.density_activation) * (dt * dot);
            out[3] = loss_scale * dloss_by_dmlp + (o.s < 0.f ? -output_l1_reg_density : 0.0f);
            __half* d = dloss_doutput + ((uint64_t)compacted_base + j_mine) * lp.padded_output_width;
            const __half2 h01 = __floats2half2_rn(out[0], out[1]), h23 = __floats2half2_rn(out[2], out[3]);
            if ((lp.padded_output_width & 3u) == 0 && (reinterpret_cast<uintptr_t>(dloss_doutput) & 7u) == 0) {
                *reinterpret_cast<uint2*>(d) = make_uint2(*reinterpret_cast<const uint32_t*>(&h01), *reinterpret_cast<const uint32_t*>(&h23));
            } else {
                d[0] = __low2half(h01); d[1] = __high2half(h01); d[2] = __low2half(h23); d[3] = __high2half(h23);
            }
        }
    }
}

}  // namespace

void launch_loss_forward(const DevCfg& g, const LossParams& lp, const uint32_t* n_rays_counter, const uint32_t* ray_coord_indices,
                         const float* coords, const uint2* net_out, uint32_t* consumed, float4* ray_rgb, uint32_t n_slots,
                         cudaStream_t stream) {
    if (n_slots == 0) return;
    k_loss_forward<<<(unsigned int)(((uint64_t)n_slots * 32 + kLossBlock - 1) / kLossBlock), kLossBlock, 0, stream>>>(g, lp, n_rays_counter, ray_coord_indices, coords,
                                                                                      net_out, consumed, ray_rgb, n_slots);
}

void launch_loss_backward(const DevCfg& g, const LossParams& lp, const uint32_t* n_rays_counter, uint32_t* ray_coord_indices,
                          const float* coords, const uint2* net_out, const float4* rays_rgba, const uint32_t* consumed,
                          const uint64_t* bases, const float4* ray_rgb, const float* mean_density, float* compacted_coords,
                          uint32_t* n_compacted_counter, __half* dloss_doutput, float* loss_output, float* reg_distortion,
                          uint32_t n_slots, cudaStream_t stream) {
    if (n_slots == 0) return;
    k_loss_backward<<<(unsigned int)(((uint64_t)n_slots * 32 + kLossBlock - 1) / kLossBlock), kLossBlock, 0, stream>>>(
        g, lp, n_rays_counter, ray_coord_indices, coords, net_out, rays_rgba, consumed, bases, ray_rgb, mean_density, compacted_coords,
        n_compacted_counter, dloss_doutput, loss_output, reg_distortion, n_slots);
}

}  // namespace srf
