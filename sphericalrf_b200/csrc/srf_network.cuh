// srf_network.cuh -- device building blocks of the network: hash-grid encoding, spherical
// harmonics, and the warp-level MLP on mma.sync fragments.  See srf_field.cu for the data flow.
#pragma once

#include "srf_kernels.cuh"

namespace srf {

// ---- hash-grid encoding -------------------------------------------------------------------------
// Trilinear interpolation of F fp16 features per level over the eight corners of the sample's cell
// (Mueller et al. 2022).  Corner c takes the upper neighbour along axis d when bit d of c is set; its
// weight is ((wx' * wy') * wz') in fp32; features accumulate in fp32 in corner order 0..7 with one
// fused multiply-add per corner and feature, and are rounded to fp16 once.
// Index of a corner: dense level  x + y*res + z*res^2 (mod size);  hashed level
// (x ^ y*2654435761 ^ z*805459861) & (size-1)  (hashed levels hold 2^k entries).
//
// Shape of the code (measured on a B200 with real sample positions, 27 M samples): the dense levels
// and the hashed levels run in two separate loops so that neither body carries the other's index
// arithmetic, and the per-level constants are read from a small shared-memory table rather than from
// the kernel's parameter block with a dynamic index -- 12.7 G samples/s against 9.2 for a single loop
// over a parameter-block table; full unrolling and fp16 accumulation bought less than that.

struct EncLevel {
    float scale;
    uint32_t res, r2, size, mask, pad;   // mask = size - 1 (hashed levels hold 2^k entries)
    const uint32_t* base;                // first entry of the level, as 32-bit words
};
struct __align__(16) EncCellLevel {      // what a read from a level's cell-major copy needs: one 16-byte load
    float scale;
    uint32_t res;
    const uint4* cells;                  // record of cell (0, 0, 0)
};
struct EncMeta {
    EncLevel level[kMaxLevels];
    EncCellLevel cell[kMaxLevels];
    int n_levels, n_dense;               // levels [0, n_dense) are dense, the rest hashed
    int n_staged;                        // levels [0, n_staged) were copied to shared memory (their base points there)
    int n_cell;                          // levels [0, n_cell) have a cell-major copy
};

// Cell-major copies of the leading levels (optional): for every cell (cx, cy, cz) of a level, cx + res*(cy + res*cz),
// the fp16 entries of its eight corners in corner order, so that a sample reads one 16*F-byte record per level instead
// of eight scattered entries.  Same numbers as the table: the copy is rebuilt whenever the table is uploaded.
struct CellTables {
    const uint4* base;
    unsigned long long offset[kMaxLevels];     // first record of the level, in uint4 units
    int n_levels;
};

// Filled once per CTA (all threads call it, followed by a barrier the caller provides).
// Dense levels always precede hashed ones: the resolution grows with the level.
__device__ __forceinline__ void prepare_enc_meta(const NetMeta& net, const __half* __restrict__ table, EncMeta* m) {
    const uint32_t words_per_entry = net.n_features / 2;
    const int t = threadIdx.x;
    if (t < (int)net.n_levels) {
        const LevelMeta& L = net.level[t];
        m->level[t].scale = L.scale; m->level[t].res = L.res; m->level[t].r2 = L.res * L.res;
        m->level[t].size = L.size; m->level[t].mask = L.size - 1u; m->level[t].pad = 0u;
        m->level[t].base = reinterpret_cast<const uint32_t*>(table) + (size_t)L.offset * words_per_entry;
        m->cell[t].scale = L.scale; m->cell[t].res = L.res; m->cell[t].cells = nullptr;
    }
    if (t == 0) {
        int d = 0;
        while (d < (int)net.n_levels && net.level[d].dense) ++d;
        m->n_levels = (int)net.n_levels;
        m->n_dense = d;
        m->n_staged = 0;
        m->n_cell = 0;
    }
}

// After prepare_enc_meta and a barrier: points the leading levels at their cell-major copies.
__device__ __forceinline__ void attach_cell_tables(const CellTables& ct, EncMeta* m) {
    const int t = threadIdx.x;
    if (ct.base && t < ct.n_levels) m->cell[t].cells = ct.base + ct.offset[t];
    if (ct.base && t == 0) m->n_cell = ct.n_levels;
}

// Index of corner (x, y, z) in a level, as the encoder computes it.
__device__ __forceinline__ uint32_t corner_index(const LevelMeta& L, uint32_t x, uint32_t y, uint32_t z) {
    if (L.dense) {
        uint32_t i = x + y * L.res + z * L.res * L.res;
        if (i >= L.size) i %= L.size;
        return i;
    }
    return (x ^ (y * 2654435761u) ^ (z * 805459861u)) & (L.size - 1u);
}

struct LevelCell {
    uint32_t ix, iy, iz;     // lower corner of the cell
    float wx, wy, wz;        // position inside the cell
};

__device__ __forceinline__ LevelCell level_cell(float scale, float x, float y, float z) {
    LevelCell c;
    const float px = fmaf(scale, x, 0.5f), py = fmaf(scale, y, 0.5f), pz = fmaf(scale, z, 0.5f);
    const float fx = floorf(px), fy = floorf(py), fz = floorf(pz);
    c.wx = px - fx; c.wy = py - fy; c.wz = pz - fz;
    c.ix = (uint32_t)srf_f2i_rz(fx); c.iy = (uint32_t)srf_f2i_rz(fy); c.iz = (uint32_t)srf_f2i_rz(fz);
    return c;
}

// One entry of the table (F halves) through the read-only path.
template <int F>
__device__ __forceinline__ void load_entry(const uint32_t* base, uint32_t idx, uint32_t (&raw)[F / 2]) {
    const uint32_t* e = base + (size_t)idx * (F / 2);
#pragma unroll
    for (int f = 0; f < F / 2; ++f) raw[f] = __ldg(e + f);
}

template <int F>
__device__ __forceinline__ void level_interpolate(const LevelCell& c, const uint32_t (&raw)[8][F / 2], float (&acc)[F]) {
    const float ux = 1.f - c.wx, uy = 1.f - c.wy, uz = 1.f - c.wz;
    const float wxy[4] = {ux * uy, c.wx * uy, ux * c.wy, c.wx * c.wy};
#pragma unroll
    for (int f = 0; f < F; ++f) acc[f] = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float wt = wxy[k & 3] * ((k & 4) ? c.wz : uz);
#pragma unroll
        for (int f = 0; f < F / 2; ++f) {
            const __half2 h = *reinterpret_cast<const __half2*>(&raw[k][f]);
            acc[2 * f] = fmaf(wt, __low2float(h), acc[2 * f]);
            acc[2 * f + 1] = fmaf(wt, __high2float(h), acc[2 * f + 1]);
        }
    }
}

// `out(i, word)` receives packed pair i (features 2i, 2i+1 of the 32-half encoding) of every level: an array in
// registers or local memory (ArraySink), or a store straight into the place the encoding is needed.
struct ArraySink {
    uint32_t (&a)[16];
    __device__ __forceinline__ void operator()(int i, uint32_t w) const { a[i] = w; }
};

template <int F, class Sink>
__device__ __forceinline__ void level_finish(const LevelCell& c, const uint32_t (&raw)[8][F / 2], int l, const Sink& out) {
    float acc[F];
    level_interpolate<F>(c, raw, acc);
#pragma unroll
    for (int f = 0; f < F / 2; ++f) {
        const __half2 h = __floats2half2_rn(acc[2 * f], acc[2 * f + 1]);
        out(l * (F / 2) + f, *reinterpret_cast<const uint32_t*>(&h));
    }
}

// One dense level.  STAGED: the level's entries were copied to shared memory and `base` points there (plain loads);
// otherwise they are read from global memory through the read-only path.
template <int F, bool STAGED, class Sink>
__device__ __forceinline__ void dense_level(const EncMeta* m, int l, float x, float y, float z, const Sink& out) {
    const EncLevel L = m->level[l];
    const uint32_t* base = L.base;
    const LevelCell c = level_cell(L.scale, x, y, z);
    const uint32_t y0 = c.iy * L.res, z0 = c.iz * L.r2;
    const uint32_t xy[4] = {c.ix + y0, c.ix + 1u + y0, c.ix + y0 + L.res, c.ix + 1u + y0 + L.res};
    uint32_t raw[8][F / 2];
    // Fast path when the largest of the eight indices is inside the level (almost always).  The test must hold in
    // exact arithmetic, not modulo 2^32: a position far outside [0,1] gives cell coordinates near 2^32 whose sum
    // wraps back below the level size; cell coordinates below 4096 cannot wrap (dense levels have res <= 256).
    if ((c.ix | c.iy | c.iz) < 4096u && xy[3] + z0 + L.r2 < L.size) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t i = xy[k & 3] + ((k & 4) ? z0 + L.r2 : z0);
            if constexpr (STAGED) {
#pragma unroll
                for (int f = 0; f < F / 2; ++f) raw[k][f] = base[(size_t)i * (F / 2) + f];
            } else {
                load_entry<F>(base, i, raw[k]);
            }
        }
    } else {                                 // cells touching the upper faces of a dense level
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            uint32_t i = xy[k & 3] + ((k & 4) ? z0 + L.r2 : z0);
            if (i >= L.size) {
                i -= L.size;
                if (i >= L.size) i %= L.size;
            }
            if constexpr (STAGED) {
#pragma unroll
                for (int f = 0; f < F / 2; ++f) raw[k][f] = base[(size_t)i * (F / 2) + f];
            } else {
                load_entry<F>(base, i, raw[k]);
            }
        }
    }
    level_finish<F>(c, raw, l, out);
}

// One level read from its cell-major copy.  Cells outside the level (positions outside [0,1]) take the scattered path.
template <int F, class Sink>
__device__ __forceinline__ void cell_level(const EncMeta* m, int l, float x, float y, float z, const Sink& out) {
    const EncCellLevel C = m->cell[l];
    const LevelCell c = level_cell(C.scale, x, y, z);
    uint32_t raw[8][F / 2];
    if (c.ix < C.res && c.iy < C.res && c.iz < C.res) {
        const uint4* e = C.cells + ((size_t)(c.iz * C.res + c.iy) * C.res + c.ix) * (size_t)F;     // 8 * F/2 words = F uint4
        if constexpr (F == 2) {                   // one 32-byte record: a single 256-bit load
            uint32_t* r = &raw[0][0];
            asm("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(e));
        } else {
#pragma unroll
            for (int q = 0; q < F; ++q) {
                const uint4 v = __ldg(e + q);
                uint32_t* r = &raw[0][0] + 4 * q;
                r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
            }
        }
    } else {
        const EncLevel L = m->level[l];
        const bool dense = l < m->n_dense;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t cx = c.ix + (k & 1), cy = c.iy + ((k >> 1) & 1), cz = c.iz + (k >> 2);
            uint32_t i;
            if (dense) { i = cx + cy * L.res + cz * L.r2; if (i >= L.size) i %= L.size; }
            else i = (cx ^ (cy * 2654435761u) ^ (cz * 805459861u)) & L.mask;
            load_entry<F>(L.base, i, raw[k]);
        }
    }
    level_finish<F>(c, raw, l, out);
}

// B consecutive levels read from their cell-major copies with the B loads issued back to back (no branch between
// them: the cell coordinates are clamped into the level for the load, and a level whose cell was outside is read
// again through the scattered path afterwards, which positions inside [0,1] never need).
constexpr int kCellBatch = 2;          // 1: 139.0, 2: 132.0, 3: 140.4 ms per benchmark frame (3 spills at 64 registers)
// (Leaving the second read out on the frame path, whose positions always lie inside [0,1]^3, measured slower: 135.9
// against 131.8 ms per benchmark frame.)
template <int F, int B, class Sink>
__device__ __forceinline__ void cell_levels(const EncMeta* m, int l, float x, float y, float z, const Sink& out) {
    LevelCell c[B];
    uint32_t raw[B][8][F / 2];
    bool inside[B];
    bool all_inside = true;
#pragma unroll
    for (int b = 0; b < B; ++b) {
        const EncCellLevel C = m->cell[l + b];
        c[b] = level_cell(C.scale, x, y, z);
        inside[b] = c[b].ix < C.res && c[b].iy < C.res && c[b].iz < C.res;
        all_inside = all_inside && inside[b];
        const uint32_t hi = C.res - 1u;
        const uint32_t cx = min(c[b].ix, hi), cy = min(c[b].iy, hi), cz = min(c[b].iz, hi);
        const uint4* e = C.cells + ((size_t)(cz * C.res + cy) * C.res + cx) * (size_t)F;
        if constexpr (F == 2) {
            uint32_t* r = &raw[b][0][0];
            asm("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "l"(e));
        } else {
#pragma unroll
            for (int q = 0; q < F; ++q) {
                const uint4 v = __ldg(e + q);
                uint32_t* r = &raw[b][0][0] + 4 * q;
                r[0] = v.x; r[1] = v.y; r[2] = v.z; r[3] = v.w;
            }
        }
    }
    if (!all_inside) {
#pragma unroll
        for (int b = 0; b < B; ++b) {
            if (inside[b]) continue;
            const EncLevel L = m->level[l + b];
            const bool dense = l + b < m->n_dense;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const uint32_t cx = c[b].ix + (k & 1), cy = c[b].iy + ((k >> 1) & 1), cz = c[b].iz + (k >> 2);
                uint32_t i;
                if (dense) { i = cx + cy * L.res + cz * L.r2; if (i >= L.size) i %= L.size; }
                else i = (cx ^ (cy * 2654435761u) ^ (cz * 805459861u)) & L.mask;
                load_entry<F>(L.base, i, raw[b][k]);
            }
        }
    }
#pragma unroll
    for (int b = 0; b < B; ++b) level_finish<F>(c[b], raw[b], l + b, out);
}

// Encodes levels [l_begin, l_end) of one position into the packed pairs out[l*F/2 ...] (pair i = features
// 2i, 2i+1 of the 32-half encoding).  `m` lives in shared memory (prepare_enc_meta).  Callers that want to
// interleave the encoding with other work call it on successive level ranges.
// CELLS: the caller attaches cell-major copies (attach_cell_tables); callers that never do compile without that path.
template <int F, bool CELLS, class Sink>
__device__ __forceinline__ void hash_encode_range(const EncMeta* m, const __half* __restrict__ table, float x, float y,
                                                  float z, int l_begin, int l_end, const Sink& out) {
    (void)table;                                  // the level bases in `m` were derived from it
    const int n_dense = m->n_dense;
    if constexpr (CELLS) {
        const int cell_end = l_end < m->n_cell ? l_end : m->n_cell;
        int l = l_begin;
#pragma unroll 1
        for (; l + kCellBatch <= cell_end; l += kCellBatch) cell_levels<F, kCellBatch>(m, l, x, y, z, out);
#pragma unroll 1
        for (; l < cell_end; ++l) cell_level<F>(m, l, x, y, z, out);
        if (l_begin < cell_end) l_begin = cell_end;
    }
    const int dense_end = l_end < n_dense ? l_end : n_dense;
    const int staged_end = dense_end < m->n_staged ? dense_end : m->n_staged;
#pragma unroll 1
    for (int l = l_begin; l < staged_end; ++l) dense_level<F, true>(m, l, x, y, z, out);
#pragma unroll 1
    for (int l = l_begin > staged_end ? l_begin : staged_end; l < dense_end; ++l) dense_level<F, false>(m, l, x, y, z, out);
#pragma unroll 3
    for (int l = l_begin > n_dense ? l_begin : n_dense; l < l_end; ++l) {
        const float scale = m->level[l].scale;
        const uint32_t mask = m->level[l].mask;
        const uint32_t* base = m->level[l].base;
        const LevelCell c = level_cell(scale, x, y, z);
        const uint32_t y0 = c.iy * 2654435761u, y1 = y0 + 2654435761u;
        const uint32_t z0 = c.iz * 805459861u, z1 = z0 + 805459861u;
        const uint32_t xy[4] = {c.ix ^ y0, (c.ix + 1u) ^ y0, c.ix ^ y1, (c.ix + 1u) ^ y1};
        uint32_t raw[8][F / 2];
#pragma unroll
        for (int k = 0; k < 8; ++k) load_entry<F>(base, (xy[k & 3] ^ ((k & 4) ? z1 : z0)) & mask, raw[k]);
        level_finish<F>(c, raw, l, out);
    }
}

// Encodes one position into 32 halves, returned as 16 packed pairs.
template <int F, bool CELLS = false>
__device__ __forceinline__ void hash_encode_packed(const EncMeta* m, const __half* __restrict__ table, float x, float y,
                                                   float z, uint32_t (&out)[16]) {
    hash_encode_range<F, CELLS>(m, table, x, y, z, 0, m->n_levels, ArraySink{out});
}

// Same, written as 32 consecutive halves.
template <int F>
__device__ __forceinline__ void hash_encode(const EncMeta* m, const __half* __restrict__ table, float x, float y, float z, __half* out) {
    uint32_t packed[16];
    hash_encode_packed<F>(m, table, x, y, z, packed);
#pragma unroll
    for (int i = 0; i < 16; ++i) *reinterpret_cast<uint32_t*>(out + 2 * i) = packed[i];
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
