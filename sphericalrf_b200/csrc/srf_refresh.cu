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

// generate_grid_samples_nerf_nonuniform (:104-185) + hash encoding + density MLP output 0 +
// splat_grid_samples_nerf_max_nearest_neighbor (:187-212) for one of the two sampling passes.
template <int F>
__global__ void __launch_bounds__(kRefreshBlock)
k_refresh_sample(const DevCfg g, const NetMeta net, const __grid_constant__ RefreshWeights W, const __half* __restrict__ table,
                 const float* __restrict__ grid_in, float* __restrict__ grid_current, uint32_t n_elements,
                 uint32_t step, Pcg rng0, float thresh, uint32_t aabb_scale, uint32_t inv_mult) {
    // The 2 112 weights the MLP needs arrive in the kernel's parameter block (constant bank): with the loops
    // below fully unrolled every multiply-add names its weight as a constant operand, so the layer costs no
    // load instructions at all (a shared-memory copy of the matrix made this kernel L1/shared-memory bound).
    __shared__ EncMeta enc_meta;
    prepare_enc_meta(net, table, &enc_meta);
    __syncthreads();
    const uint32_t tid = blockIdx.x * kRefreshBlock + threadIdx.x;
    if (tid >= n_elements) return;
    // Which sample index i this thread takes.  The reference gives thread i the cell
    // ((i + step*n) * 56924617 + 96925573) mod cells: a pseudo-random cell, so neighbouring threads gather from
    // unrelated table lines.  The result does not depend on which thread handles which i (the splat is an
    // atomic max), so when the map is a bijection (power-of-two cell count, n a multiple of it: inv_mult != 0)
    // thread t takes the i whose first-try cell is t: neighbouring threads then work on neighbouring Morton cells
    // and their gathers share lines.
    uint32_t i = tid;
    if (inv_mult) {
        const uint32_t q = tid / g.cells, c = tid % g.cells;
        const uint32_t v = (c - 96925573u) * inv_mult;                    // (i + step*n) mod cells
        i = q * g.cells + ((v - step * n_elements) & (g.cells - 1u));
    }

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
    hash_encode_packed<F>(&enc_meta, table, pos.x, pos.y, pos.z, enc);
    float x[32];
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        const __half2 h = *reinterpret_cast<const __half2*>(&enc[k]);
        x[2 * k] = __low2float(h); x[2 * k + 1] = __high2float(h);
    }
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
    const float thickness = network_to_density(raw, g.density_activation) * g.min_step;
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
