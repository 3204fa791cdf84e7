// srf_refresh.cu -- density-grid refresh: Testbed::train_prep_nerf (internal/testbed.cu:203-239).
//
// The reference runs generate_grid_samples_nerf_nonuniform twice, the density network (hash
// encoding + MLP as separate tiny-cuda-nn kernels with all 16 outputs), a memset, the splat,
// the max-decay, a reduce_sum, grid_to_bitfield and the max-pool: eleven launches with every
// intermediate (positions, indices, encodings, network outputs) in global memory
// (internal/sampler/occupancy_sampler.cu:104-285,980-1088).  Here one kernel goes from the cell
// hash to the splat -- it draws the jittered position, gathers the encoding, evaluates the one
// network output that is consumed and does the atomicMax -- and one kernel does the max-decay
// together with the first level of the mean's summation tree.
//
// Bit-exactness: everything the refresh produces is compared bit for bit, so the MLP here is
// evaluated with scalar fp32 fused multiply-adds in input order (fp16 parameters and activations,
// one rounding to fp16 per layer), not on the tensor cores whose accumulation order is not
// specified; and the mean is a fixed summation tree (chunks of 1024, stride halving).
#include "srf_network.cuh"

namespace srf {

namespace {

constexpr int kRefreshBlock = 128;

// generate_grid_samples_nerf_nonuniform (:104-185) + hash encoding + density MLP output 0 for sample index i of one
// sampling pass: returns the optical thickness the splat (:187-212) writes and, in *idx_out, the cell it goes to.
template <int F>
__device__ __forceinline__ float refresh_sample(const DevCfg& g, const EncMeta* enc_meta, const RefreshWeights& W,
                                                const __half* __restrict__ table, const float* __restrict__ grid_in, uint32_t i,
                                                uint32_t n_elements, uint32_t step, const Pcg& rng0, float thresh,
                                                uint32_t aabb_scale, uint32_t* idx_out) {
    Pcg rng = rng0;
    if (i < (1u << 30)) pcg_jump(rng, i * 4u);             // rng.advance(i*4), :125
    else pcg_advance(rng, (uint64_t)i * 4u);
    const uint32_t nc = g.n_cascades, N = g.grid_size;
    const uint32_t level = (uint32_t)(pcg_next_float(rng) * (float)nc) % nc;
    uint32_t idx = 0;
    for (uint32_t j = 0; j < 10; ++j) {
        idx = ((i + step * n_elements) * 56924617u + j * 19349663u + 96925573u) % g.cells;
        idx += level * g.cells;
        if (grid_in[idx] > thresh) break;
    }
    *idx_out = idx;
    const uint32_t pos_idx = idx % g.cells;
    const uint32_t cx = morton3D_invert(pos_idx >> 0), cy = morton3D_invert(pos_idx >> 1), cz = morton3D_invert(pos_idx >> 2);
    const float u0 = pcg_next_float(rng), u1 = pcg_next_float(rng), u2 = pcg_next_float(rng);
    const float fn = (float)N;
    const float p0 = ((float)cx + u0) / fn - 0.5f, p1 = ((float)cy + u1) / fn - 0.5f, p2 = ((float)cz + u2) / fn - 0.5f;
    V3 pos;
    switch (g.grid_dist) {
    case SRF_GRID_WARPED_EXP: {
        const float s = scalbnf(1.0f, -(int)(nc - level - 1));
        pos = mk3(p0 * s + 0.5f, p1 * s + 0.5f, p2 * s + 0.5f);
    } break;
    case SRF_GRID_WARPED_RECIPROCAL: {
        const float s = 1.f / (float)(nc - level);
        pos = mk3(p0 * s + 0.5f, p1 * s + 0.5f, p2 * s + 0.5f);
    } break;
    case SRF_GRID_METRIC_EXP: {
        const float s = scalbnf((float)aabb_scale, -(int)(nc - level - 1));
        pos = warp_position(g, mk3(p0 * s + 0.5f, p1 * s + 0.5f, p2 * s + 0.5f));
    } break;
    default: {
        const float s = (float)aabb_scale / (float)(nc - level);
        pos = warp_position(g, mk3(p0 * s + 0.5f, p1 * s + 0.5f, p2 * s + 0.5f));
    } break;
    }

    uint32_t enc[16];
    hash_encode_packed<F>(enc_meta, table, pos.x, pos.y, pos.z, enc);
    float x[32];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const __half2 h = *reinterpret_cast<const __half2*>(&enc[k]);
        x[2 * k] = __low2float(h); x[2 * k + 1] = __high2float(h);
    }
    // The 2 112 weights the MLP needs arrive in the kernel's parameter block (constant bank): with the loops
    // below fully unrolled every multiply-add names its weight as a constant operand, so the layer costs no
    // load instructions at all (a shared-memory copy of the matrix made this kernel L1/shared-memory bound).
    float out0 = 0.f;
#pragma unroll
    for (int o = 0; o < 64; ++o) {
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) acc = fmaf(W.w1[o * 32 + k], x[k], acc);
        if (!(acc > 0.f)) acc = 0.f;
        const float h = __half2float(__float2half_rn(acc));
        out0 = fmaf(W.w2[o], h, out0);
    }
    const float raw = __half2float(__float2half_rn(out0));
    return network_to_density(raw, g.density_activation) * g.min_step;
}

// Which sample index lands, at its first try, in cell c: the reference gives thread i the cell
// ((i + step*n) * 56924617 + 96925573) mod cells, a bijection of [0, cells) when the cell count is a power of two and n
// a multiple of it; inv_mult is the inverse of 56924617 modulo 2^32.
__device__ __forceinline__ uint32_t sample_index_of_cell(uint32_t tid, uint32_t cells, uint32_t n_elements, uint32_t step, uint32_t inv_mult) {
    const uint32_t q = tid / cells, c = tid % cells;
    const uint32_t v = (c - 96925573u) * inv_mult;                    // (i + step*n) mod cells
    return q * cells + ((v - step * n_elements) & (cells - 1u));
}

// One of the two sampling passes followed by splat_grid_samples_nerf_max_nearest_neighbor (:187-212).
template <int F>
__global__ void __launch_bounds__(kRefreshBlock)
k_refresh_sample(const DevCfg g, const NetMeta net, const __grid_constant__ RefreshWeights W, const __half* __restrict__ table,
                 const float* __restrict__ grid_in, float* __restrict__ grid_current, uint32_t n_elements,
                 uint32_t step, Pcg rng0, float thresh, uint32_t aabb_scale, uint32_t inv_mult) {
    __shared__ EncMeta enc_meta;
    prepare_enc_meta(net, table, &enc_meta);
    __syncthreads();
    const uint32_t tid = blockIdx.x * kRefreshBlock + threadIdx.x;
    if (tid >= n_elements) return;
    // The result does not depend on which thread handles which sample index (the splat is an atomic max), so when the
    // cell map is a bijection thread t takes the index whose first-try cell is t: neighbouring threads then work on
    // neighbouring Morton cells and their gathers share table lines.
    const uint32_t i = inv_mult ? sample_index_of_cell(tid, g.cells, n_elements, step, inv_mult) : tid;
    uint32_t idx;
    const float thickness = refresh_sample<F>(g, &enc_meta, W, table, grid_in, i, n_elements, step, rng0, thresh, aabb_scale, &idx);
    // positive floats order like their bit patterns (:209-211)
    atomicMax(reinterpret_cast<unsigned int*>(grid_current + idx), __float_as_uint(thickness));
}

// stride-halving sum of 1024 values held one per thread; result valid in thread 0.
__device__ __forceinline__ float block_tree_sum_1024(float v, float* smem /* 1024 */) {
    const int t = threadIdx.x;
    smem[t] = v;
    __syncthreads();
    for (int h = 512; h >= 32; h >>= 1) {
        if (t < h) smem[t] = smem[t] + smem[t + h];
        __syncthreads();
    }
    float x = 0.f;              // the first warp finishes in registers: strides 16 .. 1
    if (t < 32) {
        x = smem[t];
        for (int h = 16; h >= 1; h >>= 1) {
            const float y = __shfl_down_sync(0xffffffffu, x, h);
            x = x + y;
        }
    }
    return x;
}

// A chunk of 1024 cells per block of kFusedBlock threads (the chunk is the unit of the mean's summation tree, so it cannot
// be split over blocks).  Measured on a B200, 128^3 grid, 64 refreshes: 0.637 ms with 128 threads, 0.521 with 256, 0.555
// with 512, 0.619 with 1024 -- against 0.501 ms for the multi-launch path (memset, k_refresh_sample, k_decay_and_partial,
// two k_tree_sum, k_grid_to_bitfield, two memsets, k_build_skip_tables).  The refresh is ~95 % the per-cell encoding and
// MLP arithmetic; what fusing saves (an 8 MB memset, the 24 MB decay pass, seven launch gaps of a few microseconds) is
// less than what the coarse 1024-cell work items lose to wave quantisation (2 048 blocks over 148 x 4 resident = 3.46
// waves) and to the per-thread serial loop.  The fused pair is therefore kept as an option (SRF_B200_FUSED_REFRESH=1,
// bit-identical, tested) and the multi-launch path stays the default.
#ifndef SRF_FUSED_BLOCK
#define SRF_FUSED_BLOCK 256
#endif
constexpr int kFusedBlock = SRF_FUSED_BLOCK;

// The stride-halving sum of 1024 values in shared memory by a block of kFusedBlock threads: the same additions in the
// same order as block_tree_sum_1024 (within a stride every addition is independent), so the same bits.  Result in smem[0].
__device__ __forceinline__ void tree_sum_1024_by_block(float* smem /* 1024, filled, synchronised */) {
    const int t = threadIdx.x;
    for (int h = 512; h >= 1; h >>= 1) {
        for (int k = t; k < h; k += kFusedBlock) smem[k] = smem[k] + smem[k + h];
        __syncthreads();
    }
}

// The whole refresh in one kernel for the common case -- every cell sampled once (the first 256 training steps),
// one cascade, no cell masked as never seen: then the reference's pseudo-random cell map is a bijection, the sample whose
// first try is cell c is the only writer of cell c, and sample -> encode -> MLP -> splat -> max-decay collapse into
// "compute, compare with the decayed old value, store" with no atomics, no scratch grid and no separate decay pass
// (generate_grid_samples_nerf_nonuniform, splat_grid_samples_nerf_max_nearest_neighbor, ema_grid_samples_nerf:
// internal/sampler/occupancy_sampler.cu:104-238).  A block owns a chunk of 1024 Morton-consecutive cells and leaves the
// chunk's term of the mean's summation tree; the block that finishes last (a ticket from one atomic counter: no block
// ever waits for another) folds the upper levels of the tree and writes the mean.  Block 0 also clears the sampler's
// skip tables, which the bit-packing kernel that follows fills.
template <int F>
__global__ void __launch_bounds__(kFusedBlock)
k_refresh_fused(const DevCfg g, const NetMeta net, const __grid_constant__ RefreshWeights W, const __half* __restrict__ table,
                float* __restrict__ grid, uint32_t step, Pcg rng0, float thresh, uint32_t aabb_scale, uint32_t inv_mult, float decay,
                float* __restrict__ partial_a, float* __restrict__ partial_b, float* __restrict__ mean, unsigned int* __restrict__ ticket,
                uint32_t* __restrict__ skip_shell, uint32_t* __restrict__ skip_yz, unsigned int* __restrict__ error_flags) {
    __shared__ EncMeta enc_meta;
    __shared__ float smem[1024];
    __shared__ unsigned int s_last;
    prepare_enc_meta(net, table, &enc_meta);
    __syncthreads();
    const uint32_t cells = g.cells;
    if (blockIdx.x == 0 && skip_shell) {
        const uint32_t N = g.grid_size;
        for (uint32_t k = threadIdx.x; k < (N + 31) / 32; k += kFusedBlock) skip_shell[k] = 0u;
        for (uint32_t k = threadIdx.x; k < (N * N + 31) / 32; k += kFusedBlock) skip_yz[k] = 0u;
    }
    const uint32_t chunk0 = blockIdx.x * 1024u;
    bool masked = false;
#pragma unroll 1
    for (uint32_t it = 0; it < 1024u / kFusedBlock; ++it) {
        const uint32_t c = chunk0 + it * kFusedBlock + threadIdx.x;
        float contrib = 0.f;
        if (c < cells) {
            const float prev = grid[c];
            masked |= !(prev > thresh);                    // such a cell's sample goes elsewhere: the host must not pick this path
            const uint32_t i = sample_index_of_cell(c, cells, cells, step, inv_mult);
            uint32_t idx;
            const float thickness = refresh_sample<F>(g, &enc_meta, W, table, grid, i, cells, step, rng0, thresh, aabb_scale, &idx);
            const float v = (prev < 0.f) ? prev : fmaxf(prev * decay, thickness);      // ema_grid_samples_nerf, :235-237
            grid[c] = v;
            contrib = fmaxf(v, 0.f) / (float)cells;
        }
        smem[it * kFusedBlock + threadIdx.x] = contrib;
    }
    if (masked && error_flags) atomicOr(error_flags, 8u);
    __syncthreads();
    tree_sum_1024_by_block(smem);
    if (threadIdx.x == 0) {
        partial_a[blockIdx.x] = smem[0];
        __threadfence();
        s_last = atomicAdd(ticket, 1u) == gridDim.x - 1u ? 1u : 0u;
    }
    __syncthreads();
    if (!s_last) return;
    // last block: the upper levels of the tree (chunks of 1024 partial sums, zero padded), as k_tree_sum runs them
    __threadfence();
    uint32_t n = gridDim.x;
    const float* in = partial_a;
    float* out = partial_b;
    for (;;) {
        const uint32_t nb = (n + 1023u) / 1024u;
        for (uint32_t b = 0; b < nb; ++b) {
            for (uint32_t k = threadIdx.x; k < 1024u; k += kFusedBlock) {
                const uint32_t j = b * 1024u + k;
                smem[k] = j < n ? __ldcg(in + j) : 0.f;
            }
            __syncthreads();
            tree_sum_1024_by_block(smem);
            if (threadIdx.x == 0) (nb == 1 ? mean : out)[b] = smem[0];
            __syncthreads();
        }
        if (nb == 1) break;
        n = nb;
        const float* t = in; in = out; out = const_cast<float*>(t);
        __threadfence_block();
    }
    if (threadIdx.x == 0) *ticket = 0u;                     // ready for the next refresh
}

// grid_to_bitfield (:240-260) for one cascade and k_build_skip_tables in one pass: a thread packs 32 Morton-consecutive
// cells into one word of the bitfield and marks the word's radial / latitude indices in the skip tables (cleared by
// k_refresh_fused).
__global__ void __launch_bounds__(256)
k_bits_and_skip(const float* __restrict__ grid, uint32_t* __restrict__ bits32, uint32_t n_words, uint32_t n_grid_size,
                const float* __restrict__ mean, float min_optical_thickness, uint32_t* __restrict__ shell, uint32_t* __restrict__ yz) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_words) return;
    const float m = *mean;
    const float thresh = (m < min_optical_thickness) ? m : min_optical_thickness;   // std::min(min_thickness, mean)
    const float4* p = reinterpret_cast<const float4*>(grid) + (size_t)i * 8;
    uint32_t b = 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float4 a = p[k];
        b |= (a.x > thresh ? 1u : 0u) << (4 * k);
        b |= (a.y > thresh ? 1u : 0u) << (4 * k + 1);
        b |= (a.z > thresh ? 1u : 0u) << (4 * k + 2);
        b |= (a.w > thresh ? 1u : 0u) << (4 * k + 3);
    }
    bits32[i] = b;
    if (!b || !shell) return;
    const uint32_t m0 = i * 32u;
    const uint32_t y_base = morton3D_invert(m0 >> 1), z_base = morton3D_invert(m0 >> 2);
#pragma unroll
    for (uint32_t zl = 0; zl < 2; ++zl) {
        bool any_z = false;
#pragma unroll
        for (uint32_t yl = 0; yl < 4; ++yl) {
            const uint32_t o = ((yl & 1u) << 1) | (zl << 2) | ((yl >> 1) << 4);
            const uint32_t mask = (1u << o) | (1u << (o | 1u)) | (1u << (o | 8u)) | (1u << (o | 9u));
            if (b & mask) {
                any_z = true;
                const uint32_t k = (z_base + zl) * n_grid_size + (y_base + yl), kb = 1u << (k & 31u);
                if (!(yz[k >> 5] & kb)) atomicOr(yz + (k >> 5), kb);
            }
        }
        if (any_z) {
            const uint32_t z = z_base + zl, sb = 1u << (z & 31u);
            if (!(shell[z >> 5] & sb)) atomicOr(shell + (z >> 5), sb);
        }
    }
}

// ema_grid_samples_nerf (:214-238) over all cells, plus level 0 of the mean's summation tree
// over the first `cells` entries: partial[b] = tree sum of max(v,0)/cells over chunk b.
__global__ void __launch_bounds__(1024)
k_decay_and_partial(float* __restrict__ grid, const float* __restrict__ current, uint32_t total, uint32_t cells,
                    float decay, int do_decay, float* __restrict__ partial) {
    __shared__ float smem[1024];
    const uint32_t i = blockIdx.x * 1024u + threadIdx.x;
    float v = 0.f;
    if (i < total) {
        v = grid[i];
        if (do_decay) {
            const float prev = v;
            v = (prev < 0.f) ? prev : fmaxf(prev * decay, current[i]);
            grid[i] = v;
        }
    }
    const float contrib = (i < cells) ? fmaxf(v, 0.f) / (float)cells : 0.f;
    if (blockIdx.x * 1024u < cells) {           // uniform per block
        const float s = block_tree_sum_1024(contrib, smem);
        if (threadIdx.x == 0) partial[blockIdx.x] = s;
    }
}

__global__ void __launch_bounds__(1024)
k_tree_sum(const float* __restrict__ in, uint32_t n, float* __restrict__ out) {
    __shared__ float smem[1024];
    const uint32_t i = blockIdx.x * 1024u + threadIdx.x;
    const float s = block_tree_sum_1024(i < n ? in[i] : 0.f, smem);
    if (threadIdx.x == 0) out[blockIdx.x] = s;
}

// grid_to_bitfield (:240-260)
__global__ void k_grid_to_bitfield(const float* __restrict__ grid, uint8_t* __restrict__ bits, uint32_t n_bytes,
                                   const float* __restrict__ mean, float min_optical_thickness) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_bytes) return;
    const float m = *mean;
    const float thresh = (m < min_optical_thickness) ? m : min_optical_thickness;   // std::min(min_thickness, mean)
    const float4 a = reinterpret_cast<const float4*>(grid)[2 * i], b = reinterpret_cast<const float4*>(grid)[2 * i + 1];
    uint32_t r = 0;
    r |= a.x > thresh ? 1u : 0u;   r |= a.y > thresh ? 2u : 0u;   r |= a.z > thresh ? 4u : 0u;   r |= a.w > thresh ? 8u : 0u;
    r |= b.x > thresh ? 16u : 0u;  r |= b.y > thresh ? 32u : 0u;  r |= b.z > thresh ? 64u : 0u;  r |= b.w > thresh ? 128u : 0u;
    bits[i] = (uint8_t)r;
}

// bitfield_max_pool (:262-285)
__global__ void k_bitfield_max_pool(uint32_t n_elements, uint32_t n_grid_size, const uint8_t* __restrict__ prev_level,
                                    uint8_t* __restrict__ next_level) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_elements) return;
    uint8_t bits = 0;
    for (uint32_t j = 0; j < 8; ++j) bits |= prev_level[i * 8 + j] > 0 ? (uint8_t)(1u << j) : 0;
    const uint32_t x = morton3D_invert(i >> 0) + n_grid_size / 8;
    const uint32_t y = morton3D_invert(i >> 1) + n_grid_size / 8;
    const uint32_t z = morton3D_invert(i >> 2) + n_grid_size / 8;
    next_level[morton3D(x, y, z)] |= bits;
}

// Summaries of the level-0 bitfield for the sampler's staged empty-space tests: which radial indices z, and
// which (z, y) index pairs, have at least one occupied cell.  One thread per 32-bit word of the bitfield: 32
// Morton-consecutive cells are a block of 4 x 4 x 2 cells (bit layout of the low Morton bits: x0 y0 z0 x1 y1),
// so a word contributes at most two z values and eight (z, y) pairs.
__global__ void k_build_skip_tables(const uint32_t* __restrict__ bits32, uint32_t n_words, uint32_t n_grid_size,
                                    uint32_t* __restrict__ shell, uint32_t* __restrict__ yz) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_words) return;
    const uint32_t b = bits32[i];
    if (!b) return;
    const uint32_t m0 = i * 32u;
    const uint32_t y_base = morton3D_invert(m0 >> 1), z_base = morton3D_invert(m0 >> 2);
#pragma unroll
    for (uint32_t zl = 0; zl < 2; ++zl) {
        bool any_z = false;
#pragma unroll
        for (uint32_t yl = 0; yl < 4; ++yl) {
            // the four cells x = 0..3 of this (y, z): Morton offsets with bits x0 (1) and x1 (8)
            const uint32_t o = ((yl & 1u) << 1) | (zl << 2) | ((yl >> 1) << 4);
            const uint32_t mask = (1u << o) | (1u << (o | 1u)) | (1u << (o | 8u)) | (1u << (o | 9u));
            if (b & mask) {
                any_z = true;
                const uint32_t k = (z_base + zl) * n_grid_size + (y_base + yl), kb = 1u << (k & 31u);
                if (!(yz[k >> 5] & kb)) atomicOr(yz + (k >> 5), kb);          // mostly already set: read first
            }
        }
        if (any_z) {
            const uint32_t z = z_base + zl, sb = 1u << (z & 31u);
            if (!(shell[z >> 5] & sb)) atomicOr(shell + (z >> 5), sb);
        }
    }
}

}  // namespace

void launch_build_skip_tables(const DevCfg& g, const uint8_t* bits, uint32_t* shell, uint32_t* yz, cudaStream_t stream) {
    const uint32_t N = g.grid_size;
    cudaMemsetAsync(shell, 0, ((N + 31) / 32) * sizeof(uint32_t), stream);
    cudaMemsetAsync(yz, 0, ((size_t)N * N + 31) / 32 * sizeof(uint32_t), stream);
    const uint32_t n_words = g.cells / 32;          // grid_size is a power of two >= 8: whole words
    k_build_skip_tables<<<(n_words + 255) / 256, 256, 0, stream>>>(reinterpret_cast<const uint32_t*>(bits), n_words, N, shell, yz);
}

void launch_refresh_sample(const DevCfg& g, const NetMeta& net, const __half* table, const RefreshWeights& w,
                           const float* grid, float* grid_current, uint32_t n_elements, uint32_t step, RefreshRng rng,
                           float thresh, uint32_t aabb_scale, cudaStream_t stream) {
    if (n_elements == 0) return;
    const unsigned int nb = (n_elements + kRefreshBlock - 1) / kRefreshBlock;
    Pcg r = {rng.state, rng.inc};
    uint32_t inv_mult = 0;
    if ((g.cells & (g.cells - 1u)) == 0 && n_elements % g.cells == 0) {
        inv_mult = 1;                                      // inverse of 56924617 modulo 2^32 (Newton iteration)
        for (int it = 0; it < 6; ++it) inv_mult *= 2u - 56924617u * inv_mult;
    }
    if (net.n_features == 2)
        k_refresh_sample<2><<<nb, kRefreshBlock, 0, stream>>>(g, net, w, table, grid, grid_current, n_elements, step, r, thresh, aabb_scale, inv_mult);
    else
        k_refresh_sample<4><<<nb, kRefreshBlock, 0, stream>>>(g, net, w, table, grid, grid_current, n_elements, step, r, thresh, aabb_scale, inv_mult);
}

// The refresh as two launches (k_refresh_fused, k_bits_and_skip).  Preconditions, checked by the caller: one cascade,
// a power-of-two cell count, every cell sampled once, no cell of `grid` below `thresh`.
void launch_refresh_fused(const DevCfg& g, const NetMeta& net, const __half* table, const RefreshWeights& w, float* grid,
                          uint32_t step, RefreshRng rng, float thresh, uint32_t aabb_scale, float decay, float* partial_a,
                          float* partial_b, float* mean, unsigned int* ticket, uint8_t* bits, float min_optical_thickness,
                          uint32_t* skip_shell, uint32_t* skip_yz, unsigned int* error_flags, cudaStream_t stream) {
    uint32_t inv_mult = 1;                                 // inverse of 56924617 modulo 2^32 (Newton iteration)
    for (int it = 0; it < 6; ++it) inv_mult *= 2u - 56924617u * inv_mult;
    const unsigned int nb = (g.cells + 1023u) / 1024u;
    Pcg r = {rng.state, rng.inc};
    if (net.n_features == 2)
        k_refresh_fused<2><<<nb, kFusedBlock, 0, stream>>>(g, net, w, table, grid, step, r, thresh, aabb_scale, inv_mult, decay, partial_a,
                                                             partial_b, mean, ticket, skip_shell, skip_yz, error_flags);
    else
        k_refresh_fused<4><<<nb, kFusedBlock, 0, stream>>>(g, net, w, table, grid, step, r, thresh, aabb_scale, inv_mult, decay, partial_a,
                                                             partial_b, mean, ticket, skip_shell, skip_yz, error_flags);
    const uint32_t n_words = g.cells / 32;
    k_bits_and_skip<<<(n_words + 255) / 256, 256, 0, stream>>>(grid, reinterpret_cast<uint32_t*>(bits), n_words, g.grid_size, mean,
                                                              min_optical_thickness, skip_shell, skip_yz);
}

// Max-decay (optional) + mean.  partial_a / partial_b: ceil(cells/1024) floats each.
void launch_decay_and_mean(float* grid, const float* grid_current, uint32_t total, uint32_t cells, float decay,
                           int do_decay, float* partial_a, float* partial_b, float* mean, cudaStream_t stream) {
    const unsigned int nb = (total + 1023u) / 1024u;
    k_decay_and_partial<<<nb, 1024, 0, stream>>>(grid, grid_current, total, cells, decay, do_decay, partial_a);
    uint32_t n = (cells + 1023u) / 1024u;
    float* in = partial_a;
    float* out = partial_b;
    while (true) {
        const uint32_t nb2 = (n + 1023u) / 1024u;
        k_tree_sum<<<nb2, 1024, 0, stream>>>(in, n, nb2 == 1 ? mean : out);
        if (nb2 == 1) break;
        n = nb2;
        float* t = in; in = out; out = t;
    }
}

void launch_grid_to_bitfield(const DevCfg& g, const float* grid, uint8_t* bits, const float* mean,
                             float min_optical_thickness, cudaStream_t stream) {
    const uint32_t n_bytes = g.cells * g.n_cascades / 8;
    k_grid_to_bitfield<<<(n_bytes + 255) / 256, 256, 0, stream>>>(grid, bits, n_bytes, mean, min_optical_thickness);
    if (g.grid_dist == SRF_GRID_WARPED_EXP || g.grid_dist == SRF_GRID_METRIC_EXP) {
        for (uint32_t level = 1; level < g.n_cascades; ++level) {
            const uint32_t n = g.cells / 64;
            k_bitfield_max_pool<<<(n + 255) / 256, 256, 0, stream>>>(n, g.grid_size, bits + (size_t)g.cells * (level - 1) / 8,
                                                                    bits + (size_t)g.cells * level / 8);
        }
    }
}

}  // namespace srf
