// srf_field.cu -- what a sample looks like: (r, g, b, sigma) from the network or from the analytic
// stand-in scene.
//
// Network path = NGPNetwork::inference_mixed_precision (internal/network/ngp_network.h:212-279):
// multiresolution hash encoding of the position (32 halves) and degree-4 spherical harmonics of
// the direction (16 halves); density MLP 32 -> 64 -> 16; colour MLP [density out(16), SH(16)] ->
// 64 -> 64 -> 3; output (r, g, b, density out[0]).  The reference runs six tiny-cuda-nn kernels
// with every intermediate in global memory and two glue kernels (grab_density_network_output,
// assemble_rgbd, :38-78); here one kernel keeps a tile of samples on chip from the table gathers
// to the four output halves.
//
// tiny-cuda-nn is not part of the reference tree; the arithmetic is the library's own statement of
// the published algorithm (Mueller et al. 2022): fp16 parameters and activations, fp32
// accumulation, one rounding to fp16 per layer; trilinear interpolation with fp32 weights in
// corner order 0..7 (bit d of the corner index selects the upper neighbour along axis d).
#include <cstring>
#include "srf_network.cuh"

namespace srf {

namespace {

template <int F>
__global__ void __launch_bounds__(kFieldBlock)
k_field_network(const NetMeta net, const __half* __restrict__ table, const __half* __restrict__ wd, const __half* __restrict__ wc,
                const float4* __restrict__ pos_dt, const uint32_t* __restrict__ sample_ray,
                const float4* __restrict__ ray_dir_t, const float* __restrict__ coords7, uint64_t n,
                uint2* __restrict__ rgbsigma, float4* __restrict__ shaded, const DevCfg cfg, const DevView view,
                const uint32_t* __restrict__ n_chunks_dev, uint32_t ray_shift) {
    if (n_chunks_dev) n = (uint64_t)(*n_chunks_dev) * kChunkSamples;
    __shared__ __align__(16) __half sW[kWeightHalves];
    __shared__ __align__(16) __half sRows[kFieldBlock * kRowLd];
    __shared__ EncMeta enc_meta;
    prepare_enc_meta(net, table, &enc_meta);
    load_weights(wd, wc, sW, true);
    __syncthreads();

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    __half* my_row = sRows + threadIdx.x * kRowLd;
    const __half* warp_rows = sRows + warp * 32 * kRowLd;
    const uint64_t n_tiles = (n + kFieldBlock - 1) / kFieldBlock;

    for (uint64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const uint64_t s = tile * kFieldBlock + threadIdx.x;
        // ---- encode: one thread per sample ----
        float x = 0.f, y = 0.f, z = 0.f, dx = 0.5f, dy = 0.5f, dz = 0.5f;
        if (s < n) {
            if (coords7) {
                const float* c = coords7 + s * 7;
                x = c[0]; y = c[1]; z = c[2]; dx = c[4]; dy = c[5]; dz = c[6];
            } else {
                const float4 p = pos_dt[s];
                const float4 d = ray_dir_t[sample_ray[s >> ray_shift]];
                x = p.x; y = p.y; z = p.z;
                dx = (d.x + 1.f) * 0.5f; dy = (d.y + 1.f) * 0.5f; dz = (d.z + 1.f) * 0.5f;   // warp_direction
            }
        }
        hash_encode<F>(&enc_meta, table, x, y, z, my_row);
        sh_encode(dx, dy, dz, my_row + 32);
        __syncwarp();

        // ---- density MLP: 32 -> 64 (ReLU) -> 16 ----
        uint32_t a_in[2][2][4];
        {
            uint32_t f0[2][4], f1[2][4];
            load_a_frag(warp_rows, 0, f0);
            load_a_frag(warp_rows, 16, f1);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int k = 0; k < 4; ++k) { a_in[mt][0][k] = f0[mt][k]; a_in[mt][1][k] = f1[mt][k]; }
        }
        uint32_t a_h[2][4][4];
        {
            float c1[2][8][4];
            mlp_layer<2, 8>(a_in, sW + kOffD1, kLd32, c1);
            acc_to_frag<4, true>(c1, a_h);
        }
        uint32_t a_rgb[2][2][4];
        uint32_t sigma_bits[2];     // density output 0 of rows g and g+8 (valid in lanes with t == 0)
        {
            float c2[2][2][4];
            mlp_layer<4, 2>(a_h, sW + kOffD2, kLd64, c2);
            uint32_t a_d[2][1][4];
            acc_to_frag<1, false>(c2, a_d);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt) {
#pragma unroll
                for (int k = 0; k < 4; ++k) a_rgb[mt][0][k] = a_d[mt][0][k];
                // a_d[mt][0][0] = (row g, cols 2t,2t+1), a_d[mt][0][1] = (row g+8, cols 2t,2t+1)
                sigma_bits[mt] = (a_d[mt][0][0] & 0xffffu) | (a_d[mt][0][1] << 16);
            }
            uint32_t f[2][4];
            load_a_frag(warp_rows, 32, f);      // SH occupies input rows 16..31 of the colour MLP
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int k = 0; k < 4; ++k) a_rgb[mt][1][k] = f[mt][k];
        }
        // ---- colour MLP: 32 -> 64 (ReLU) -> 64 (ReLU) -> 3 ----
        {
            float c1[2][8][4];
            mlp_layer<2, 8>(a_rgb, sW + kOffC1, kLd32, c1);
            acc_to_frag<4, true>(c1, a_h);
        }
        uint32_t a_h2[2][4][4];
        {
            float c2[2][8][4];
            mlp_layer<4, 8>(a_h, sW + kOffC2, kLd64, c2);
            acc_to_frag<4, true>(c2, a_h2);
        }
        float c3[2][1][4];
        mlp_layer<4, 1>(a_h2, sW + kOffC3, kLd64, c3);
        // c3[mt][0] = {(row g, col 2t), (row g, col 2t+1), (row g+8, col 2t), (row g+8, col 2t+1)}
        // lanes t == 0 hold r,g; lanes t == 1 hold b (col 2).
#pragma unroll
        for (int mt = 0; mt < 2; ++mt) {
            const float b_lo = __shfl_down_sync(0xffffffffu, c3[mt][0][0], 1);   // from lane t+1: col 2 of row g
            const float b_hi = __shfl_down_sync(0xffffffffu, c3[mt][0][2], 1);   // col 2 of row g+8
            if (t == 0) {
                const uint64_t base = tile * kFieldBlock + warp * 32 + mt * 16;
                const uint64_t s0 = base + g, s1 = base + g + 8;
                const uint32_t sg0 = sigma_bits[mt] & 0xffffu, sg1 = sigma_bits[mt] >> 16;
                const uint2 o0 = make_uint2(pack_half2(c3[mt][0][0], c3[mt][0][1]), (pack_half2(b_lo, 0.f) & 0xffffu) | (sg0 << 16));
                const uint2 o1 = make_uint2(pack_half2(c3[mt][0][2], c3[mt][0][3]), (pack_half2(b_hi, 0.f) & 0xffffu) | (sg1 << 16));
                const uint64_t ss[2] = {s0, s1};
                const uint2 oo[2] = {o0, o1};
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    if (ss[e] >= n) continue;
                    if (shaded) {
                        const __half2 h0 = *reinterpret_cast<const __half2*>(&oo[e].x), h1 = *reinterpret_cast<const __half2*>(&oo[e].y);
                        const float raw[4] = {__low2float(h0), __high2float(h0), __low2float(h1), __high2float(h1)};
                        const float4 p = pos_dt[ss[e]];
                        shaded[ss[e]] = shade_sample(cfg, view, raw, p.w, mk3(p.x, p.y, p.z));
                    } else {
                        rgbsigma[ss[e]] = oo[e];
                    }
                }
            }
        }
        __syncwarp();
    }
}

// Density only: positions -> 16 halves (NGPNetwork::density, ngp_network.h:281-310).
template <int F>
__global__ void __launch_bounds__(kFieldBlock)
k_field_density(const NetMeta net, const __half* __restrict__ table, const __half* __restrict__ wd, const float* __restrict__ positions,
                uint32_t stride, uint64_t n, __half* __restrict__ out16) {
    __shared__ __align__(16) __half sW[kOffC1];
    __shared__ __align__(16) __half sRows[kFieldBlock * kRowLd];
    __shared__ EncMeta enc_meta;
    prepare_enc_meta(net, table, &enc_meta);
    load_weights(wd, nullptr, sW, false);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    __half* my_row = sRows + threadIdx.x * kRowLd;
    const __half* warp_rows = sRows + warp * 32 * kRowLd;
    const uint64_t n_tiles = (n + kFieldBlock - 1) / kFieldBlock;
    for (uint64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        const uint64_t s = tile * kFieldBlock + threadIdx.x;
        float x = 0.f, y = 0.f, z = 0.f;
        if (s < n) { const float* p = positions + s * stride; x = p[0]; y = p[1]; z = p[2]; }
        hash_encode<F>(&enc_meta, table, x, y, z, my_row);
        __syncwarp();
        uint32_t a_in[2][2][4];
        {
            uint32_t f0[2][4], f1[2][4];
            load_a_frag(warp_rows, 0, f0);
            load_a_frag(warp_rows, 16, f1);
#pragma unroll
            for (int mt = 0; mt < 2; ++mt)
#pragma unroll
                for (int k = 0; k < 4; ++k) { a_in[mt][0][k] = f0[mt][k]; a_in[mt][1][k] = f1[mt][k]; }
        }
        uint32_t a_h[2][4][4];
        {
            float c1[2][8][4];
            mlp_layer<2, 8>(a_in, sW + kOffD1, kLd32, c1);
            acc_to_frag<4, true>(c1, a_h);
        }
        float c2[2][2][4];
        mlp_layer<4, 2>(a_h, sW + kOffD2, kLd64, c2);
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const uint64_t base = tile * kFieldBlock + warp * 32 + mt * 16;
                const uint64_t s0 = base + g, s1 = base + g + 8;
                const int col = nt * 8 + 2 * t;
                if (s0 < n) *reinterpret_cast<uint32_t*>(out16 + s0 * 16 + col) = pack_half2(c2[mt][nt][0], c2[mt][nt][1]);
                if (s1 < n) *reinterpret_cast<uint32_t*>(out16 + s1 * 16 + col) = pack_half2(c2[mt][nt][2], c2[mt][nt][3]);
            }
        __syncwarp();
    }
}

// Normals render mode (testbed.cu:557-559, ray_marcher.cu:250-255): per sample the density MLP's output 0 and its
// gradient with respect to the warped position, in the canonical fp32 form:
//   d enc[l,f] / d x_d = scale_l * sum over the 4 corner pairs along d of (w_a' * w_b') * (v_hi - v_lo);
//   g_h[j] = W2[0][j] where hidden unit j (fp16, ReLU) is positive; g_enc[k] = sum_j W1[j][k] g_h[j];
//   grad[d] = sum_k g_enc[k] * d enc[k] / d x_d.
// One thread per sample, fp32 accumulation in index order (a diagnostic mode: no tensor cores).  The record
// written is (unit normal, step opacity); the colour MLP is not evaluated.
template <int F>
__global__ void __launch_bounds__(128)
k_field_normals(const DevCfg g, const NetMeta net, const __half* __restrict__ table, const __half* __restrict__ wd,
                const float4* __restrict__ pos_dt, uint64_t n, float4* __restrict__ shaded, const uint32_t* __restrict__ n_chunks_dev) {
    __shared__ __align__(16) float sW1[64 * 32];
    __shared__ float sW2[64];
    for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) sW1[i] = __half2float(wd[i]);
    for (int i = threadIdx.x; i < 64; i += blockDim.x) sW2[i] = __half2float(wd[64 * 32 + i]);
    __syncthreads();
    if (n_chunks_dev) n = (uint64_t)(*n_chunks_dev) * kChunkSamples;
    const uint32_t* table32 = reinterpret_cast<const uint32_t*>(table);
    for (uint64_t s = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; s < n; s += (uint64_t)gridDim.x * blockDim.x) {
        const float4 p = pos_dt[s];
        const float x3[3] = {p.x, p.y, p.z};
        float enc[32], dydx[32][3];
        for (uint32_t l = 0; l < net.n_levels; ++l) {
            const LevelMeta L = net.level[l];
            float w[3]; uint32_t ig[3];
            for (int d = 0; d < 3; ++d) {
                const float q = fmaf(L.scale, x3[d], 0.5f);
                const float fl = floorf(q);
                w[d] = q - fl;
                ig[d] = (uint32_t)srf_f2i_rz(fl);
            }
            float v[8][F], acc[F];
#pragma unroll
            for (int f = 0; f < F; ++f) acc[f] = 0.f;
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
                const uint32_t gx = ig[0] + (c & 1u), gy = ig[1] + ((c >> 1) & 1u), gz = ig[2] + (c >> 2);
                const float wt = (((c & 1u) ? w[0] : 1.f - w[0]) * ((c & 2u) ? w[1] : 1.f - w[1])) * ((c & 4u) ? w[2] : 1.f - w[2]);
                uint32_t idx = L.dense ? gx + gy * L.res + gz * L.res * L.res : (gx ^ (gy * 2654435761u) ^ (gz * 805459861u));
                idx %= L.size;
                const uint32_t* e = table32 + (size_t)(L.offset + idx) * (F / 2);
#pragma unroll
                for (int f2 = 0; f2 < F / 2; ++f2) {
                    const uint32_t raw = __ldg(e + f2);
                    const __half2 h = *reinterpret_cast<const __half2*>(&raw);
                    v[c][2 * f2] = __low2float(h); v[c][2 * f2 + 1] = __high2float(h);
                }
#pragma unroll
                for (int f = 0; f < F; ++f) acc[f] = fmaf(wt, v[c][f], acc[f]);
            }
#pragma unroll
            for (int f = 0; f < F; ++f) enc[l * F + f] = __half2float(__float2half_rn(acc[f]));
#pragma unroll
            for (int d = 0; d < 3; ++d) {
                const int a = d == 0 ? 1 : 0, b = d == 2 ? 1 : 2;
#pragma unroll
                for (int f = 0; f < F; ++f) {
                    float gs = 0.f;
#pragma unroll
                    for (uint32_t c2 = 0; c2 < 4; ++c2) {
                        const uint32_t ba = c2 & 1u, bb = c2 >> 1;
                        const float wt = (ba ? w[a] : 1.f - w[a]) * (bb ? w[b] : 1.f - w[b]);
                        const uint32_t lo = (ba << a) | (bb << b), hi = lo | (1u << d);
                        gs = fmaf(wt, v[hi][f] - v[lo][f], gs);
                    }
                    dydx[l * F + f][d] = L.scale * gs;
                }
            }
        }
        float g_enc[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) g_enc[k] = 0.f;
        float out0 = 0.f;
        for (int o = 0; o < 64; ++o) {
            const float* wrow = sW1 + o * 32;
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) acc = fmaf(wrow[k], enc[k], acc);
            if (!(acc > 0.f)) acc = 0.f;
            const float h = __half2float(__float2half_rn(acc));
            out0 = fmaf(sW2[o], h, out0);
            const float gh = h > 0.f ? sW2[o] : 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) g_enc[k] = fmaf(wrow[k], gh, g_enc[k]);      // j ascending for every k
        }
        const float raw_sigma = __half2float(__float2half_rn(out0));
        float grad[3];
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            float acc = 0.f;
#pragma unroll
            for (int k = 0; k < 32; ++k) acc = fmaf(g_enc[k], dydx[k][d], acc);
            grad[d] = acc;
        }
        const float dd = -network_to_density_derivative(raw_sigma, g.density_activation);
        float nx = dd * grad[0], ny = dd * grad[1], nz = dd * grad[2];
        const float nn = srf_norm3f(nx, ny, nz);
        if (nn > 0.f) { nx /= nn; ny /= nn; nz /= nn; }
        const float alpha = 1.f - srf_expf(-network_to_density(raw_sigma, g.density_activation) * p.w);
        shaded[s] = make_float4(nx, ny, nz, alpha);
    }
}

// Analytic stand-in scene, fp32, one thread per sample.
__global__ void __launch_bounds__(256)
k_field_blobs(const DevCfg g, const DevView v, const float* __restrict__ blobs, uint32_t n_blobs, const float* __restrict__ cmap,
              const float4* __restrict__ pos_dt, uint64_t n, float4* __restrict__ out, const uint32_t* __restrict__ n_chunks_dev) {
    extern __shared__ float s_blobs[];
    for (uint32_t i = threadIdx.x; i < n_blobs * 5; i += blockDim.x) s_blobs[i] = blobs[i];
    __syncthreads();
    if (n_chunks_dev) n = (uint64_t)(*n_chunks_dev) * kChunkSamples;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const float4 p = pos_dt[i];
    const V3 x = unwarp_position(g, mk3(p.x, p.y, p.z));
    float sigma = 0.f;
    for (uint32_t b = 0; b < n_blobs; ++b) {
        const float* q = s_blobs + 5 * b;
        const float dx = x.x - q[0], dy = x.y - q[1], dz = x.z - q[2];
        const float d2 = fmaf(dz, dz, fmaf(dy, dy, dx * dx));
        const float inv = -0.5f / (q[3] * q[3]);
        sigma = fmaf(q[4], srf_expf(d2 * inv), sigma);
    }
    const float px = x.x - 0.5f, py = x.y - 0.5f, pz = x.z - 0.5f;
    const float raw[4] = {fmaf(cmap[2], pz, fmaf(cmap[1], py, cmap[0] * px)), fmaf(cmap[5], pz, fmaf(cmap[4], py, cmap[3] * px)),
                          fmaf(cmap[8], pz, fmaf(cmap[7], py, cmap[6] * px)), sigma};
    out[i] = shade_sample(g, v, raw, p.w, mk3(p.x, p.y, p.z));
    }
}

int field_grid(uint64_t n) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t tiles = (n + kFieldBlock - 1) / kFieldBlock;
    const uint64_t cap = (uint64_t)sms * 8;      // a multiple of the SM count; each CTA strides over tiles
    return (int)(tiles < cap ? tiles : cap);
}

}  // namespace

void launch_field_network(const NetMeta& net, const __half* table, const __half* w_density, const __half* w_rgb,
                          const float4* pos_dt, const uint32_t* sample_ray, const float4* ray_dir_t,
                          const float* coords7, uint64_t n, uint2* rgbsigma, float4* shaded, const DevCfg* g,
                          const DevView* v, cudaStream_t stream, const uint32_t* n_chunks_dev, uint32_t ray_shift) {
    if (n == 0 && !n_chunks_dev) return;
    const int grid = field_grid(n_chunks_dev ? ~0ull >> 8 : n);
    DevCfg g0; DevView v0;
    memset(&g0, 0, sizeof(g0)); memset(&v0, 0, sizeof(v0));
    if (g) g0 = *g;
    if (v) v0 = *v;
    if (net.n_features == 2)
        k_field_network<2><<<grid, kFieldBlock, 0, stream>>>(net, table, w_density, w_rgb, pos_dt, sample_ray, ray_dir_t, coords7, n, rgbsigma, shaded, g0, v0, n_chunks_dev, ray_shift);
    else
        k_field_network<4><<<grid, kFieldBlock, 0, stream>>>(net, table, w_density, w_rgb, pos_dt, sample_ray, ray_dir_t, coords7, n, rgbsigma, shaded, g0, v0, n_chunks_dev, ray_shift);
}

void launch_field_density(const NetMeta& net, const __half* table, const __half* w_density, const float* positions,
                          uint32_t stride, uint64_t n, __half* out16, cudaStream_t stream) {
    if (n == 0) return;
    const int grid = field_grid(n);
    if (net.n_features == 2)
        k_field_density<2><<<grid, kFieldBlock, 0, stream>>>(net, table, w_density, positions, stride, n, out16);
    else
        k_field_density<4><<<grid, kFieldBlock, 0, stream>>>(net, table, w_density, positions, stride, n, out16);
}

void launch_field_normals(const DevCfg& g, const NetMeta& net, const __half* table, const __half* w_density, const float4* pos_dt,
                          uint64_t n, float4* shaded, cudaStream_t stream, const uint32_t* n_chunks_dev) {
    if (n == 0 && !n_chunks_dev) return;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t want = n_chunks_dev ? ~0ull >> 8 : (n + 127) / 128;
    const uint64_t cap = (uint64_t)sms * 8;
    const unsigned int grid = (unsigned int)(want < cap ? want : cap);
    if (net.n_features == 2) k_field_normals<2><<<grid, 128, 0, stream>>>(g, net, table, w_density, pos_dt, n, shaded, n_chunks_dev);
    else k_field_normals<4><<<grid, 128, 0, stream>>>(g, net, table, w_density, pos_dt, n, shaded, n_chunks_dev);
}

void launch_field_blobs(const DevCfg& g, const DevView& v, const float* blobs, uint32_t n_blobs, const float* color_map,
                        const float4* pos_dt, uint64_t n, float4* shaded, cudaStream_t stream, const uint32_t* n_chunks_dev) {
    if (n == 0 && !n_chunks_dev) return;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t want = n_chunks_dev ? ~0ull >> 8 : (n + 255) / 256;
    const uint64_t cap = (uint64_t)sms * 16;
    k_field_blobs<<<(unsigned int)(want < cap ? want : cap), 256, n_blobs * 5 * sizeof(float), stream>>>(
        g, v, blobs, n_blobs, color_map, pos_dt, n, shaded, n_chunks_dev);
}

}  // namespace srf
