// srf_network.cuh -- device building blocks of the network: hash-grid encoding, spherical
// harmonics, and the warp-level MLP on mma.sync fragments.  See srf_field.cu for the data flow.
#pragma once

#include "srf_kernels.cuh"

namespace srf {

// ---- hash-grid encoding -------------------------------------------------------------------------
__device__ __forceinline__ uint32_t grid_index(uint32_t gx, uint32_t gy, uint32_t gz, const LevelMeta& L) {
    uint32_t idx;
    if (L.dense) {
        idx = gx + gy * L.res + gz * L.res * L.res;
        if (idx >= L.size) {                   // only cells on the upper faces wrap
            idx -= L.size;
            if (idx >= L.size) idx %= L.size;
        }
    } else {
        idx = (gx ^ (gy * 2654435761u) ^ (gz * 805459861u)) & (L.size - 1u);   // hashed levels hold 2^k entries
    }
    return idx;
}

// Encodes one position into 32 halves written to out[0..31] (stride 1).  F = features per level.
template <int F>
__device__ __forceinline__ void hash_encode(const NetMeta& net, const __half* __restrict__ table, float x, float y, float z, __half* out) {
    const int n_levels = 32 / F;
#pragma unroll 2
    for (int l = 0; l < n_levels; ++l) {
        const LevelMeta& L = net.level[l];
        const float px = fmaf(L.scale, x, 0.5f), py = fmaf(L.scale, y, 0.5f), pz = fmaf(L.scale, z, 0.5f);
        const float fx = floorf(px), fy = floorf(py), fz = floorf(pz);
        const float wx = px - fx, wy = py - fy, wz = pz - fz;
        const uint32_t ix = (uint32_t)srf_f2i_rz(fx), iy = (uint32_t)srf_f2i_rz(fy), iz = (uint32_t)srf_f2i_rz(fz);
        float acc[F];
#pragma unroll
        for (int f = 0; f < F; ++f) acc[f] = 0.f;
        // issue the eight gathers first, then interpolate
        uint32_t raw[8][F / 2];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const uint32_t gx = ix + (c & 1), gy = iy + ((c >> 1) & 1), gz = iz + ((c >> 2) & 1);
            const uint32_t idx = grid_index(gx, gy, gz, L);
            const uint32_t* e = reinterpret_cast<const uint32_t*>(table) + (size_t)(L.offset + idx) * (F / 2);
#pragma unroll
            for (int f = 0; f < F / 2; ++f) raw[c][f] = __ldg(e + f);
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float wt = (c & 1) ? wx : 1.f - wx;
            wt *= ((c >> 1) & 1) ? wy : 1.f - wy;
            wt *= ((c >> 2) & 1) ? wz : 1.f - wz;
#pragma unroll
            for (int f = 0; f < F / 2; ++f) {
                const __half2 h = *reinterpret_cast<const __half2*>(&raw[c][f]);
                acc[2 * f] = fmaf(wt, __low2float(h), acc[2 * f]);
                acc[2 * f + 1] = fmaf(wt, __high2float(h), acc[2 * f + 1]);
            }
        }
#pragma unroll
        for (int f = 0; f < F; ++f) out[l * F + f] = __float2half_rn(acc[f]);
    }
}

// Real spherical harmonics up to degree 3 of the direction 2*d - 1 (d = warped direction in [0,1]).
__device__ __forceinline__ void sh_encode(float dx, float dy, float dz, __half* out) {
    const float x = fmaf(dx, 2.f, -1.f), y = fmaf(dy, 2.f, -1.f), z = fmaf(dz, 2.f, -1.f);
    const float xy = x * y, xz = x * z, yz = y * z, x2 = x * x, y2 = y * y, z2 = z * z;
    out[0] = __float2half_rn(0.28209479177387814f);
    out[1] = __float2half_rn(-0.48860251190291987f * y);
    out[2] = __float2half_rn(0.48860251190291987f * z);
    out[3] = __float2half_rn(-0.48860251190291987f * x);
    out[4] = __float2half_rn(1.0925484305920792f * xy);
    out[5] = __float2half_rn(-1.0925484305920792f * yz);
    out[6] = __float2half_rn(fmaf(0.94617469575755997f, z2, -0.31539156525251999f));
    out[7] = __float2half_rn(-1.0925484305920792f * xz);
    out[8] = __float2half_rn(0.54627421529603959f * x2 - 0.54627421529603959f * y2);
    out[9] = __float2half_rn(0.59004358992664352f * y * (fmaf(-3.f, x2, y2)));
    out[10] = __float2half_rn(2.8906114426405538f * xy * z);
    out[11] = __float2half_rn(0.45704579946446572f * y * (fmaf(-5.f, z2, 1.f)));
    out[12] = __float2half_rn(0.3731763325901154f * z * (fmaf(5.f, z2, -3.f)));
    out[13] = __float2half_rn(0.45704579946446572f * x * (fmaf(-5.f, z2, 1.f)));
    out[14] = __float2half_rn(1.4453057213202769f * z * (x2 - y2));
    out[15] = __float2half_rn(0.59004358992664352f * x * (fmaf(3.f, y2, -x2)));
}

// ---- warp-level MLP on mma.sync m16n8k16 (fp16 in, fp32 accumulate) ------------------------------
// A warp owns 32 samples = two 16-row tiles.  Activations stay in registers between layers: the
// accumulator fragment of two neighbouring 8-column tiles is exactly the A fragment of one
// 16-deep k tile.
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// c[mt][nt] = sum_k a[mt][kt] * W[nt*8.., kt*16..]; W in shared memory, row-major [n][ldw].
template <int KT, int NT>
__device__ __forceinline__ void mlp_layer(const uint32_t (&a)[2][KT][4], const __half* sW, int ldw, float (&c)[2][NT][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
        for (int mt = 0; mt < 2; ++mt)
#pragma unroll
            for (int k = 0; k < 4; ++k) c[mt][nt][k] = 0.f;
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            const __half* w = sW + (nt * 8 + g) * ldw + kt * 16 + 2 * t;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(w);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(w + 8);
            mma16816(c[0][nt], a[0][kt], b0, b1);
            mma16816(c[1][nt], a[1][kt], b0, b1);
        }
    }
}

// Accumulators of 2*KT column tiles -> A fragments of KT k tiles, with optional ReLU.
template <int KT, bool RELU>
__device__ __forceinline__ void acc_to_frag(const float (&c)[2][2 * KT][4], uint32_t (&a)[2][KT][4]) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
        for (int kt = 0; kt < KT; ++kt) {
            float v[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) { v[k] = c[mt][2 * kt][k]; v[4 + k] = c[mt][2 * kt + 1][k]; }
            if (RELU) {
#pragma unroll
                for (int k = 0; k < 8; ++k) v[k] = v[k] > 0.f ? v[k] : 0.f;
            }
            a[mt][kt][0] = pack_half2(v[0], v[1]);
            a[mt][kt][1] = pack_half2(v[2], v[3]);
            a[mt][kt][2] = pack_half2(v[4], v[5]);
            a[mt][kt][3] = pack_half2(v[6], v[7]);
        }
}

// Shared-memory layout of the weights (halves). Row strides are padded so that the B-fragment
// loads of a warp fall into 32 distinct banks.
constexpr int kLd32 = 40;    // rows with 32 inputs
constexpr int kLd64 = 72;    // rows with 64 inputs
constexpr int kOffD1 = 0;                         // density layer 1: 64 x 32
constexpr int kOffD2 = kOffD1 + 64 * kLd32;       // density layer 2: 16 x 64
constexpr int kOffC1 = kOffD2 + 16 * kLd64;       // colour layer 1: 64 x 32
constexpr int kOffC2 = kOffC1 + 64 * kLd32;       // colour layer 2: 64 x 64
constexpr int kOffC3 = kOffC2 + 64 * kLd64;       // colour layer 3: 8 x 64 (rows 0..2 used)
constexpr int kWeightHalves = kOffC3 + 8 * kLd64;
constexpr int kRowLd = 56;                        // per-sample row: 32 encoding + 16 SH + 8 pad

constexpr int kFieldBlock = 128;                  // 4 warps, 128 samples per tile

__device__ __forceinline__ void load_weights(const __half* __restrict__ wd, const __half* __restrict__ wc, __half* sW,
                                             bool with_colour) {
    for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) sW[kOffD1 + (i / 32) * kLd32 + (i % 32)] = wd[i];
    for (int i = threadIdx.x; i < 16 * 64; i += blockDim.x) sW[kOffD2 + (i / 64) * kLd64 + (i % 64)] = wd[64 * 32 + i];
    if (with_colour) {
        for (int i = threadIdx.x; i < 64 * 32; i += blockDim.x) sW[kOffC1 + (i / 32) * kLd32 + (i % 32)] = wc[i];
        for (int i = threadIdx.x; i < 64 * 64; i += blockDim.x) sW[kOffC2 + (i / 64) * kLd64 + (i % 64)] = wc[64 * 32 + i];
        for (int i = threadIdx.x; i < 8 * 64; i += blockDim.x) sW[kOffC3 + (i / 64) * kLd64 + (i % 64)] = wc[64 * 32 + 64 * 64 + i];
    }
}

// A fragments of one 16-wide k tile from the warp's rows in shared memory.
__device__ __forceinline__ void load_a_frag(const __half* rows, int col0, uint32_t (&a)[2][4]) {
    const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int mt = 0; mt < 2; ++mt) {
        const __half* r0 = rows + (mt * 16 + g) * kRowLd + col0 + 2 * t;
        const __half* r1 = r0 + 8 * kRowLd;
        a[mt][0] = *reinterpret_cast<const uint32_t*>(r0);
        a[mt][1] = *reinterpret_cast<const uint32_t*>(r1);
        a[mt][2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
        a[mt][3] = *reinterpret_cast<const uint32_t*>(r1 + 8);
    }
}


}  // namespace srf
