// srf_composite.cu -- front-to-back compositing and the per-pixel output stage.
//
// Replaces volume_rendering_kernel (internal/render/ray_marcher.cu:204-282), the hit/alive
// bookkeeping of compact_rays_kernel (internal/testbed.cu:423-446), shade_kernel (:448-477) and
// CudaRenderBuffer::accumulate / tonemap (internal/utils/render_buffer.cu:46-236).
//
// One warp per ray.  The warp streams the ray's contiguous samples 32 at a time (coalesced 8- or
// 16-byte loads); every lane turns its sample into (alpha, rgb) -- the exponentials and logistic
// functions, which are the expensive part -- and then the warp replays the reference's sequential
// recurrence  T = 1 - A; w = alpha*T; C += rgb*w; A += w  sample by sample through shuffles, so
// the accumulated colour, the opacity and the index at which  A > 1 - threshold  stops the ray are
// bit-identical to a scalar loop over the samples.  The last lane standing finishes the pixel.
#include "srf_kernels.cuh"

namespace srf {

namespace {

constexpr int kCompBlock = 256;                  // 8 rays per CTA

// tonemap(): internal/utils/render_buffer.cu:84-140
__device__ void tonemap3(float* x, int curve) {
    if (curve == SRF_TONEMAP_IDENTITY) return;
    for (int i = 0; i < 3; ++i) x[i] = fmaxf(x[i], 0.f);
    float k0, k1, k2, k3, k4, k5;
    if (curve == SRF_TONEMAP_ACES) {
        k0 = 0.6f * 0.6f * 2.51f; k1 = 0.6f * 0.03f; k2 = 0.0f; k3 = 0.6f * 0.6f * 2.43f; k4 = 0.6f * 0.59f; k5 = 0.14f;
    } else if (curve == SRF_TONEMAP_HABLE) {
        const float A = 0.15f, B = 0.50f, C = 0.10f, D = 0.20f, E = 0.02f, F = 0.30f;
        k0 = A * F - A * E; k1 = C * B * F - B * E; k2 = 0.0f; k3 = A * F; k4 = B * F; k5 = D * F * F;
        const float W = 11.2f;
        const float nom = k0 * (W * W) + k1 * W + k2;
        const float denom = k3 * (W * W) + k4 * W + k5;
        const float whiteScale = denom / nom;
        k0 = 4.0f * k0 * whiteScale; k1 = 2.0f * k1 * whiteScale; k2 = k2 * whiteScale; k3 = 4.0f * k3; k4 = 2.0f * k4;
    } else {
        const float Y = fmaf(0.0722f, x[2], fmaf(0.7152f, x[1], 0.2126f * x[0]));
        const float s = 1.f / (Y + 1.0f);
        for (int i = 0; i < 3; ++i) x[i] = x[i] * s;
        return;
    }
    for (int i = 0; i < 3; ++i) {
        const float sq = x[i] * x[i];
        const float nom = fmaf(k1, x[i], sq * k0) + k2;
        const float denom = fmaf(k4, x[i], k3 * sq) + k5;
        x[i] = nom / denom;
    }
}

// shade + accumulate + tonemap of one pixel.
__device__ void finish_pixel(const DevCfg& g, const DevView& v, const DevPost& post, bool hit, const float* rgba_in,
                             uint32_t n_steps_total, float4* accum, float4* out) {
    float fb[4] = {0.f, 0.f, 0.f, 0.f};
    if (hit) {
        float tmp[4] = {rgba_in[0], rgba_in[1], rgba_in[2], rgba_in[3]};
        if (v.render_mode == SRF_MODE_COST) {
            const float col = (float)n_steps_total / 128;
            tmp[0] = tmp[1] = tmp[2] = col; tmp[3] = 1.0f;
        }
        if (!g.train_in_linear_color && v.render_mode == SRF_MODE_SHADE)
            for (int i = 0; i < 3; ++i) tmp[i] = srgb_to_linear(tmp[i]);
        for (int i = 0; i < 4; ++i) fb[i] = tmp[i];
    }
    const float sc = (float)v.spp_index;
    float tmp[4] = {0.f, 0.f, 0.f, 0.f};
    if (v.spp_index != 0 && accum) { const float4 a = *accum; tmp[0] = a.x; tmp[1] = a.y; tmp[2] = a.z; tmp[3] = a.w; }
    float color[4] = {fb[0], fb[1], fb[2], fb[3]};
    switch (post.color_space) {
    case SRF_COLOR_VISPOSNEG: {
        const float val = color[0] - color[1];
        float tv = tmp[0] - tmp[1];
        tv = fmaf(tv, sc, val) / (sc + 1);
        tmp[0] = fmaxf(tv, 0.f); tmp[1] = fmaxf(-tv, 0.f);
    } break;
    case SRF_COLOR_SRGB:
        for (int i = 0; i < 3; ++i) color[i] = linear_to_srgb(color[i]);
        // fall through
    default:
        for (int i = 0; i < 3; ++i) tmp[i] = fmaf(tmp[i], sc, color[i]) / (sc + 1);
        break;
    }
    tmp[3] = fmaf(tmp[3], sc, color[3]) / (sc + 1);
    if (accum) *accum = make_float4(tmp[0], tmp[1], tmp[2], tmp[3]);
    if (!out) return;
    float c[4] = {tmp[0], tmp[1], tmp[2], tmp[3]};
    for (int i = 0; i < 3; ++i) c[i] *= post.exposure_scale;
    const float weight = (1 - c[3]) * post.bg[3];
    for (int i = 0; i < 3; ++i) c[i] = fmaf(post.bg[i], weight, c[i]);
    c[3] += weight;
    if (post.color_space == SRF_COLOR_SRGB) for (int i = 0; i < 3; ++i) c[i] = srgb_to_linear(c[i]);
    tonemap3(c, post.tonemap_curve);
    if (post.to_srgb) for (int i = 0; i < 3; ++i) c[i] = linear_to_srgb(c[i]);
    *out = make_float4(c[0], c[1], c[2], c[3]);
}

struct RayAccum { float r, g, b, a; uint32_t n; bool terminated; };

// The warp-synchronous compositing loop over samples [lo, hi).  load(i, raw4, dt, wpos) fetches sample i.
template <class Load>
__device__ __forceinline__ RayAccum composite_ray(const DevCfg& g, const DevView& v, uint64_t lo, uint64_t hi, Load load) {
    const int lane = threadIdx.x & 31;
    RayAccum acc = {0.f, 0.f, 0.f, 0.f, 0u, false};
    const V3 origin = mk3(v.cam[3], v.cam[7], v.cam[11]);
    const V3 cam_fwd = mk3(v.cam[2], v.cam[6], v.cam[10]);
    for (uint64_t base = lo; base < hi && !acc.terminated; base += 32) {
        const uint64_t i = base + lane;
        float alpha = 0.f, cr = 0.f, cg = 0.f, cb = 0.f;
        if (i < hi) {
            float raw[4], dt;
            V3 w;
            load(i, raw, &dt, &w);
            alpha = 1.f - srf_expf(-network_to_density(raw[3], g.density_activation) * dt);
            cr = network_to_rgb(raw[0], g.rgb_activation);
            cg = network_to_rgb(raw[1], g.rgb_activation);
            cb = network_to_rgb(raw[2], g.rgb_activation);
            if (v.render_mode == SRF_MODE_DEPTH || v.render_mode == SRF_MODE_DISTANCE) {
                const V3 p = unwarp_position(g, w);
                const float dx = p.x - origin.x, dy = p.y - origin.y, dz = p.z - origin.z;
                float zz;
                if (v.render_mode == SRF_MODE_DEPTH) zz = fmaf(cam_fwd.z, dz, fmaf(cam_fwd.y, dy, cam_fwd.x * dx)) * v.depth_scale;
                else zz = srf_norm3f(dx, dy, dz) * v.depth_scale;
                cr = cg = cb = zz;
            } else if (v.render_mode == SRF_MODE_AO) {
                cr = cg = cb = alpha;
            }
        }
        const int cnt = (int)((hi - base) < 32 ? (hi - base) : 32);
        for (int k = 0; k < cnt; ++k) {
            const float a_k = __shfl_sync(0xffffffffu, alpha, k);
            const float r_k = __shfl_sync(0xffffffffu, cr, k);
            const float g_k = __shfl_sync(0xffffffffu, cg, k);
            const float b_k = __shfl_sync(0xffffffffu, cb, k);
            const float T = 1.f - acc.a;
            const float wgt = a_k * T;
            acc.r = fmaf(r_k, wgt, acc.r);
            acc.g = fmaf(g_k, wgt, acc.g);
            acc.b = fmaf(b_k, wgt, acc.b);
            acc.a += wgt;
            ++acc.n;
            if (acc.a > g.transmittance_keep) { acc.terminated = true; break; }
        }
    }
    return acc;
}

template <bool HALF>
__global__ void __launch_bounds__(kCompBlock)
k_composite(const DevCfg g, const DevView v, const DevPost post, const uint64_t* __restrict__ offsets,
            uint64_t ray_begin, uint64_t ray_end, const float4* __restrict__ pos_dt,
            const uint2* __restrict__ rgbs_half, const float4* __restrict__ rgbs_float,
            const uint8_t* __restrict__ ray_end_reason, float4* __restrict__ out, float4* __restrict__ accum,
            float4* __restrict__ rgba_raw, uint32_t* __restrict__ n_composited, FrameCounters* __restrict__ counters) {
    __shared__ unsigned long long s_comp;
    __shared__ unsigned int s_hit;
    if (threadIdx.x == 0) { s_comp = 0ull; s_hit = 0u; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const uint64_t r = ray_begin + (uint64_t)blockIdx.x * (kCompBlock / 32) + (threadIdx.x >> 5);
    if (r < ray_end) {
        const uint64_t base = offsets[ray_begin];
        const uint64_t lo = offsets[r] - base, hi = offsets[r + 1] - base;
        const RayAccum acc = composite_ray(g, v, lo, hi, [&](uint64_t i, float* raw, float* dt, V3* w) {
            const float4 p = pos_dt[i];
            *dt = p.w;
            *w = mk3(p.x, p.y, p.z);
            if (HALF) {
                const uint2 q = rgbs_half[i];
                const __half2 h0 = *reinterpret_cast<const __half2*>(&q.x), h1 = *reinterpret_cast<const __half2*>(&q.y);
                raw[0] = __low2float(h0); raw[1] = __high2float(h0); raw[2] = __low2float(h1); raw[3] = __high2float(h1);
            } else {
                const float4 q = rgbs_float[i];
                raw[0] = q.x; raw[1] = q.y; raw[2] = q.z; raw[3] = q.w;
            }
        });
        if (lane == 0) {
            const uint32_t end = ray_end_reason[r];
            // A ray reaches the hit buffer when it stops being alive (terminated, left the box, or its
            // step size fell to 0 in empty space) and its opacity exceeds 0.001 (testbed.cu:438-445).
            // Rays that stay alive until the reference's loop bound leave their pixel untouched.
            const bool finished = acc.terminated || end == RAY_END_EXIT || end == RAY_END_DT0;
            const bool hit = finished && acc.a > 0.001f;
            const uint32_t n_steps_total = acc.terminated ? acc.n : 1u + acc.n;
            const float rgba[4] = {acc.r, acc.g, acc.b, acc.a};
            if (rgba_raw) rgba_raw[r] = make_float4(acc.r, acc.g, acc.b, acc.a);
            if (n_composited) n_composited[r] = acc.n;
            if (out || accum) finish_pixel(g, v, post, hit, rgba, n_steps_total, accum ? accum + r : nullptr, out ? out + r : nullptr);
            atomicAdd(&s_comp, (unsigned long long)acc.n);
            if (hit) atomicAdd(&s_hit, 1u);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && counters) {
        if (s_comp) atomicAdd(&counters->n_composited, s_comp);
        if (s_hit) atomicAdd(&counters->n_hit, (unsigned long long)s_hit);
    }
}

__global__ void __launch_bounds__(kCompBlock)
k_composite_coords(const DevCfg g, const DevView v, const uint64_t* __restrict__ offsets, uint64_t n_rays,
                   const float* __restrict__ coords7, const uint2* __restrict__ rgbs_half,
                   float4* __restrict__ rgba, uint32_t* __restrict__ n_composited) {
    const int lane = threadIdx.x & 31;
    const uint64_t r = (uint64_t)blockIdx.x * (kCompBlock / 32) + (threadIdx.x >> 5);
    if (r >= n_rays) return;
    const RayAccum acc = composite_ray(g, v, offsets[r], offsets[r + 1], [&](uint64_t i, float* raw, float* dt, V3* w) {
        const float* c = coords7 + i * 7;
        *w = mk3(c[0], c[1], c[2]);
        *dt = c[3];
        const uint2 q = rgbs_half[i];
        const __half2 h0 = *reinterpret_cast<const __half2*>(&q.x), h1 = *reinterpret_cast<const __half2*>(&q.y);
        raw[0] = __low2float(h0); raw[1] = __high2float(h0); raw[2] = __low2float(h1); raw[3] = __high2float(h1);
    });
    if (lane == 0) {
        if (rgba) rgba[r] = make_float4(acc.r, acc.g, acc.b, acc.a);
        if (n_composited) n_composited[r] = acc.n;
    }
}

}  // namespace

void launch_composite(const DevCfg& g, const DevView& v, const DevPost& post, const uint64_t* offsets,
                      uint64_t ray_begin, uint64_t ray_end, const float4* pos_dt, const uint2* rgbs_half,
                      const float4* rgbs_float, const uint8_t* ray_end_reason, float4* out, float4* accum,
                      float4* rgba_raw, uint32_t* n_composited, FrameCounters* counters, cudaStream_t stream) {
    if (ray_end <= ray_begin) return;
    const uint64_t n = ray_end - ray_begin;
    const unsigned int nb = (unsigned int)((n + kCompBlock / 32 - 1) / (kCompBlock / 32));
    if (rgbs_half)
        k_composite<true><<<nb, kCompBlock, 0, stream>>>(g, v, post, offsets, ray_begin, ray_end, pos_dt, rgbs_half,
                                                         rgbs_float, ray_end_reason, out, accum, rgba_raw, n_composited, counters);
    else
        k_composite<false><<<nb, kCompBlock, 0, stream>>>(g, v, post, offsets, ray_begin, ray_end, pos_dt, rgbs_half,
                                                          rgbs_float, ray_end_reason, out, accum, rgba_raw, n_composited, counters);
}

void launch_composite_coords(const DevCfg& g, const DevView& v, const uint64_t* offsets, uint64_t n_rays,
                             const float* coords7, const uint2* rgbs_half, float4* rgba, uint32_t* n_composited,
                             cudaStream_t stream) {
    if (n_rays == 0) return;
    const unsigned int nb = (unsigned int)((n_rays + kCompBlock / 32 - 1) / (kCompBlock / 32));
    k_composite_coords<<<nb, kCompBlock, 0, stream>>>(g, v, offsets, n_rays, coords7, rgbs_half, rgba, n_composited);
}

}  // namespace srf
