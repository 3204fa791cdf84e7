// srf_composite.cu -- front-to-back compositing and the per-pixel output stage.
//
// Replaces volume_rendering_kernel (internal/render/ray_marcher.cu:204-282), the hit/alive
// bookkeeping of compact_rays_kernel (internal/testbed.cu:423-446), shade_kernel (:448-477) and
// CudaRenderBuffer::accumulate / tonemap (internal/utils/render_buffer.cu:46-236).
//
// Frame path: the field kernels leave (activated colour, step opacity) per sample -- the exponentials
// and logistic functions are evaluated there, in parallel over samples -- and one thread per ray runs
// the reference's sequential recurrence  T = 1 - A; w = alpha*T; C += rgb*w; A += w  over its
// contiguous records, so colour, opacity and the index at which  A > 1 - threshold  stops the ray are
// bit-identical to a scalar loop.  The same thread then finishes the pixel.
// Stage entry srf_volume_rendering (raw fp16 network outputs in Coordinate order): one warp per ray,
// lanes evaluate the activations of 32 samples, the recurrence is replayed through shuffles.
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
        const float Y = srf_dot3f(0.2126f, x[0], 0.7152f, x[1], 0.0722f, x[2]);
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
        if (v.render_mode == SRF_MODE_NORMALS) {
            const float nn = srf_norm3f(tmp[0], tmp[1], tmp[2]);
            for (int i = 0; i < 3; ++i) tmp[i] = (0.5f * (nn > 0.f ? tmp[i] / nn : tmp[i]) + 0.5f) * tmp[3];
        } else if (v.render_mode == SRF_MODE_COST) {
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
    for (uint64_t base = lo; base < hi && !acc.terminated; base += 32) {
        const uint64_t i = base + lane;
        float alpha = 0.f, cr = 0.f, cg = 0.f, cb = 0.f;
        if (i < hi) {
            float raw[4], dt;
            V3 w;
            load(i, raw, &dt, &w);
            const float4 q = shade_sample(g, v, raw, dt, w);
            cr = q.x; cg = q.y; cb = q.z; alpha = q.w;
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

// Frame path: one thread per ray over samples the field kernels already turned into (colour, opacity).
// The recurrence is the reference's, statement for statement: T = 1 - A; w = alpha*T; C += c*w; A += w;
// stop once A > 1 - threshold.  Five arithmetic instructions per sample; each thread streams its
// ray's contiguous 16-byte records.
constexpr int kRayBlock = 128;

template <bool PAGED>
__global__ void __launch_bounds__(kRayBlock)
k_composite_rays(const DevCfg g, const DevView v, const DevPost post, const uint64_t* __restrict__ offsets,
                 const uint32_t* __restrict__ ray_head, const uint32_t* __restrict__ ray_count,
                 const uint32_t* __restrict__ chunk_next,
                 uint64_t ray_begin, uint64_t ray_end, const float4* __restrict__ shaded,
                 uint8_t* __restrict__ ray_end_reason, float4* __restrict__ out, float4* __restrict__ accum,
                 float4* __restrict__ rgba_raw, uint32_t* __restrict__ n_composited, FrameCounters* __restrict__ counters,
                 uint32_t wave, float4* __restrict__ ray_rgba, uint32_t* __restrict__ ray_ncomp) {
    const uint64_t r = ray_begin + (uint64_t)blockIdx.x * kRayBlock + threadIdx.x;
    unsigned long long comp = 0;
    unsigned int hits = 0;
    const uint32_t end = r < ray_end ? ray_end_reason[r] : (uint32_t)RAY_END_DONE;
    if (r < ray_end && !(wave > 0 && end == RAY_END_DONE)) {
        float R = 0.f, G = 0.f, B = 0.f, A = 0.f;
        uint32_t n = 0;
        if (wave > 0) {                                // the state an earlier wave left
            const float4 q = ray_rgba[r];
            R = q.x; G = q.y; B = q.z; A = q.w;
            n = ray_ncomp[r];
        }
        const uint32_t n_before = n;
        bool terminated = false;
        auto take = [&](const float4 q) {
            const float T = 1.f - A;
            const float wgt = q.w * T;
            R = fmaf(q.x, wgt, R);
            G = fmaf(q.y, wgt, G);
            B = fmaf(q.z, wgt, B);
            A += wgt;
            ++n;
            return A > g.transmittance_keep;
        };
        if (PAGED) {
            // Every lane walks its own chunk list, so a warp's load touches 32 different sectors and the kernel is bound
            // by L1 wavefronts, not by DRAM (ncu: l1tex 73 %, DRAM 42 %).  Two samples = one whole 32-byte sector per
            // 256-bit load halve the wavefronts (a chunk is 256-byte aligned, so pairs never straddle sectors; the slot
            // behind a ray's last sample exists and is read unused).  Four samples per 16-byte load each, with the link to
            // the next chunk fetched first, had measured the same as one at a time: 6.34 against 6.40 ms per frame.
            uint32_t left = ray_count[r], c = ray_head[r];
            while (left && !terminated) {
                const float4* p = shaded + (uint64_t)c * kChunkSamples;
                const uint32_t m = left < kChunkSamples ? left : kChunkSamples;
                for (uint32_t j = 0; j < m; j += 2) {
                    float4 q0, q1;
                    asm("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                        : "=f"(q0.x), "=f"(q0.y), "=f"(q0.z), "=f"(q0.w), "=f"(q1.x), "=f"(q1.y), "=f"(q1.z), "=f"(q1.w)
                        : "l"(p + j));
                    if (take(q0)) { terminated = true; break; }
                    if (j + 1 < m && take(q1)) { terminated = true; break; }
                }
                left -= m;
                c = chunk_next[c];
            }
        } else {
            const uint64_t base = offsets[ray_begin];
            const float4* p = shaded + (offsets[r] - base);
            const uint64_t cnt = offsets[r + 1] - offsets[r];
            for (uint64_t j = 0; j < cnt; ++j)
                if (take(__ldg(p + j))) { terminated = true; break; }
        }
        if (!terminated && end == RAY_END_PAUSED) {
            // more samples to come: keep the running sums, write no pixel yet
            ray_rgba[r] = make_float4(R, G, B, A);
            ray_ncomp[r] = n;
            comp = n - n_before;
        } else {
            // A ray reaches the hit buffer when it stops being alive (terminated, left the box, or its step
            // size fell to 0 in empty space) and its opacity exceeds 0.001 (testbed.cu:438-445).  Rays that
            // stay alive until the reference's loop bound leave their pixel untouched.
            const bool finished = terminated || end == RAY_END_EXIT || end == RAY_END_DT0;
            const bool hit = finished && A > 0.001f;
            const uint32_t n_steps_total = terminated ? n : 1u + n;
            const float rgba[4] = {R, G, B, A};
            if (rgba_raw) rgba_raw[r] = make_float4(R, G, B, A);
            if (n_composited) n_composited[r] = n;
            if (out || accum)
                finish_pixel(g, v, post, hit, rgba, n_steps_total, accum ? accum + r : nullptr,
                             out ? out + (v.out_by_pixel ? (uint64_t)shard_ray_pixel(v, r) : r) : nullptr);
            if (ray_rgba) ray_end_reason[r] = (uint8_t)RAY_END_DONE;
            comp = n - n_before;
            hits = hit ? 1u : 0u;
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        comp += __shfl_down_sync(0xffffffffu, comp, o);
        hits += __shfl_down_sync(0xffffffffu, hits, o);
    }
    if ((threadIdx.x & 31) == 0 && counters) {
        if (comp) atomicAdd(&counters->n_composited, comp);
        if (hits) atomicAdd(&counters->n_hit, (unsigned long long)hits);
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
                      uint64_t ray_begin, uint64_t ray_end, const float4* shaded, const uint8_t* ray_end_reason,
                      float4* out, float4* accum, float4* rgba_raw, uint32_t* n_composited, FrameCounters* counters,
                      cudaStream_t stream) {
    if (ray_end <= ray_begin) return;
    const uint64_t n = ray_end - ray_begin;
    const unsigned int nb = (unsigned int)((n + kRayBlock - 1) / kRayBlock);
    k_composite_rays<false><<<nb, kRayBlock, 0, stream>>>(g, v, post, offsets, nullptr, nullptr, nullptr, ray_begin, ray_end, shaded,
                                                          const_cast<uint8_t*>(ray_end_reason), out, accum, rgba_raw, n_composited,
                                                          counters, 0u, nullptr, nullptr);
}

void launch_composite_paged(const DevCfg& g, const DevView& v, const DevPost& post, uint64_t ray_begin, uint64_t ray_end,
                            const uint32_t* ray_head, const uint32_t* ray_count, const uint32_t* chunk_next,
                            const float4* pool_shaded, uint8_t* ray_end_reason, float4* out, float4* accum,
                            float4* rgba_raw, uint32_t* n_composited, FrameCounters* counters, cudaStream_t stream,
                            uint32_t wave, float4* ray_rgba, uint32_t* ray_ncomp) {
    if (ray_end <= ray_begin) return;
    const uint64_t n = ray_end - ray_begin;
    const unsigned int nb = (unsigned int)((n + kRayBlock - 1) / kRayBlock);
    k_composite_rays<true><<<nb, kRayBlock, 0, stream>>>(g, v, post, nullptr, ray_head, ray_count, chunk_next, ray_begin, ray_end,
                                                         pool_shaded, ray_end_reason, out, accum, rgba_raw, n_composited, counters,
                                                         wave, ray_rgba, ray_ncomp);
}

void launch_composite_coords(const DevCfg& g, const DevView& v, const uint64_t* offsets, uint64_t n_rays,
                             const float* coords7, const uint2* rgbs_half, float4* rgba, uint32_t* n_composited,
                             cudaStream_t stream) {
    if (n_rays == 0) return;
    const unsigned int nb = (unsigned int)((n_rays + kCompBlock / 32 - 1) / (kCompBlock / 32));
    k_composite_coords<<<nb, kCompBlock, 0, stream>>>(g, v, offsets, n_rays, coords7, rgbs_half, rgba, n_composited);
}

}  // namespace srf
