// srf_field_tc.cu -- the network field on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// Same data flow as srf_field.cu (NGPNetwork::inference_mixed_precision,
// internal/network/ngp_network.h:212-279), different engine for the five dense layers.  A CTA of
// 1024 threads -- one per SM -- is eight independent groups of 128 threads; a group owns a tile of 128
// samples: thread
// r gathers and interpolates the hash-grid features of sample r straight into the shared-memory
// image of the MMA's A operand; the group's first thread issues tcgen05.mma (M = 128 samples,
// N = 64 or 16 neurons, K = 16 per instruction) with the fp32 accumulator in tensor memory; after
// the commit barrier every thread reads its own sample's row back with tcgen05.ld, applies ReLU,
// rounds to fp16 and writes the next layer's A operand.  Weights (20 KB) sit in shared memory in the
// B-operand layout for the lifetime of the CTA and are shared by all groups.
//
// Operand layout (no swizzle, K-major): a matrix of R rows x K halves is stored as K/8 column
// blocks; block j holds, for every row, the 8 halves k = 8j..8j+7 as one 16-byte unit, rows
// consecutive: offset(row, k) = (k/8)*R*16 + row*16 + (k%8)*2.  In the tensor core's terms the
// 8-row x 16-byte core matrices are contiguous (128 B), the stride between 8-row groups (SBO) is
// 128 B and the stride between the two core matrices along K of one instruction (LBO) is R*16 B.
//
// One 16 KB activation region per group is enough: each layer's output overwrites the region its
// input was read from, which is safe once the layer's commit barrier has completed (the tensor core
// has finished reading shared memory by then).  The spherical harmonics of the direction are the same for
// every sample of a ray: on the frame path the sampler writes them once per ray and this kernel reads the 32
// bytes when the colour network's input is assembled (stage entry points compute them per sample).
//
// Tensor memory: 64 columns per group (all 64 for the 64-wide layers, the first 16 for the 16-wide
// ones): the CTA allocates all 512 columns of its SM.  Its 1024 threads at 64 registers take the whole
// register file and its 148 KB of shared memory more than half of the SM's, so a second CTA can never be
// resident and the allocation never has to wait.
//
// Why one large CTA instead of four of 256 threads: the gathers of the encoding live on L1 hits
// (neighbouring samples share cells), and L1 is what the unified 256 KB array has left after shared
// memory.  Four CTAs carried four copies of the 20 KB weight images (208 KB of shared memory, ~48 KB of
// L1); one CTA carries one copy (148 KB, ~92 KB of L1).  Measured on the benchmark frame: 208 -> 183 ms.
//
// Every wait on a commit barrier is bounded; on expiry the group raises an error flag and leaves its
// tile loop; the CTA frees its tensor memory and returns.
#include <cstdlib>
#include <cstring>
#include "srf_network.cuh"

namespace srf {

namespace {

constexpr int kGroups = 8;                      // groups of 128 threads per CTA (6 groups at 80 registers: 146 ms per
                                                // benchmark frame against 132)
constexpr int kGroup = 128;
constexpr int kTcBlock = kGroup * kGroups;
constexpr uint32_t kTmemCols = 64 * kGroups;      // 64 per group: the whole tensor memory of the SM
constexpr uint32_t kWaitLimit = 1u << 20;
// (Sets of two or four groups sharing one commit round trip per layer were slower: 159.5 and 181.9 ms per benchmark
// frame against 153.1 with every group on its own.)

// shared-memory map (bytes)
constexpr int kSmW_D1 = 0;                        // [4][64][8]
constexpr int kSmW_D2 = kSmW_D1 + 4 * 64 * 16;    // [8][16][8]
constexpr int kSmW_C1 = kSmW_D2 + 8 * 16 * 16;    // [4][64][8]
constexpr int kSmW_C2 = kSmW_C1 + 4 * 64 * 16;    // [8][64][8]
constexpr int kSmW_C3 = kSmW_C2 + 8 * 64 * 16;    // [8][16][8]
constexpr int kSmAct = kSmW_C3 + 8 * 16 * 16;     // kGroups x [8][128][8]: the activation regions
constexpr int kActBytes = 8 * 128 * 16;
constexpr int kSmBar = kSmAct + kGroups * kActBytes;   // kGroups mbarriers + tensor-memory base (4 B)
constexpr int kSmEnc = kSmBar + kGroups * 8 + 16;  // per-level constants of the encoding
constexpr int kSmDesc = (kSmEnc + (int)sizeof(EncMeta) + 15) / 16 * 16;    // operand descriptors: [group][layer][k step] x (A, B)
constexpr int kSmStage = kSmDesc + kGroups * 5 * 4 * 16;                    // coarse levels of the hash table (optional, dynamic size)
constexpr int kSmTotal = kSmStage;                // without staged levels
constexpr int kSmLimit = 227 * 1024;
static_assert(kTmemCols == 512, "the CTA owns the SM's tensor memory");
static_assert(kSmTotal > 227 * 1024 / 2, "a second CTA must not fit: it would wait for tensor memory forever");
static_assert(kSmTotal <= kSmLimit, "shared memory of one SM");
static_assert(kSmEnc % 16 == 0 && kSmBar % 8 == 0, "EncMeta holds 16-byte records, the barriers are 8-byte objects");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// K-major, no-swizzle shared-memory matrix descriptor.
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
    d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
    d |= (uint64_t)1 << 46;                      // descriptor version of this architecture
    return d;                                    // base offset 0, layout type 0 (no swizzle)
}

// kind::f16 instruction descriptor: fp16 A and B (K-major), fp32 accumulator, M = 128.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((128u >> 4) << 24);
}

// tcgen05.mma, kind::f16, one CTA; the accumulate flag is fixed at compile time (no predicate to compute at run time).
template <bool ACCUMULATE>
__device__ __forceinline__ void mma_f16_fixed(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    if (ACCUMULATE)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                     :: "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 0, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                     :: "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Bounded wait on the commit barrier; false when the bound expired.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t"
            ".reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t"
            "}\n"
            : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

// Weights W[n][k] (row-major, global) -> B-operand image [(k/8)][n][k%8] in shared memory.
__device__ __forceinline__ void load_weight_image(const __half* __restrict__ w, int n_rows, int k_cols, unsigned char* dst) {
    const int units = n_rows * (k_cols / 8);                 // 16-byte units
    for (int u = threadIdx.x; u < units; u += kTcBlock) {
        const int n = u / (k_cols / 8), j = u % (k_cols / 8);
        const uint4 v = *reinterpret_cast<const uint4*>(w + n * k_cols + j * 8);
        *reinterpret_cast<uint4*>(dst + ((size_t)j * n_rows + n) * 16) = v;
    }
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// 16 fp32 accumulators (as bits) -> two 16-byte units of fp16, optional ReLU; written as column
// blocks j0, j0+1 of an A image with 128 rows.
template <bool RELU>
__device__ __forceinline__ void store_units(const uint32_t (&acc)[16], unsigned char* image, int j0, int row) {
    uint32_t h[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float lo = __uint_as_float(acc[2 * k]), hi = __uint_as_float(acc[2 * k + 1]);
        if (RELU) asm("cvt.rn.relu.f16x2.f32 %0, %1, %2;" : "=r"(h[k]) : "f"(hi), "f"(lo));   // round and clamp at 0 in one instruction
        else h[k] = pack2(lo, hi);
    }
    const uint4 u0 = make_uint4(h[0], h[1], h[2], h[3]);
    const uint4 u1 = make_uint4(h[4], h[5], h[6], h[7]);
    *reinterpret_cast<uint4*>(image + ((size_t)j0 * 128 + row) * 16) = u0;
    *reinterpret_cast<uint4*>(image + ((size_t)(j0 + 1) * 128 + row) * 16) = u1;
}

// group-local named barriers 1..kGroups (id 0 is __syncthreads)
__device__ __forceinline__ void group_sync(int group) {
    asm volatile("bar.sync %0, 128;" :: "r"(group + 1) : "memory");
}
__device__ __forceinline__ bool group_any(int group, bool v) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbar.red.or.pred q, %2, 128, p;\n\tselp.u32 %0, 1, 0, q;\n\t}\n"
                 : "=r"(r) : "r"((uint32_t)v), "r"(group + 1) : "memory");
    return r != 0;
}

// FRAME: the frame path's argument set (paged pool records in, per-ray SH table, shaded records out), fixed at compile
// time so that the stage entry points' alternatives cost it neither branches nor registers.
template <int F, bool FRAME>
__global__ void __launch_bounds__(kTcBlock, 1)
k_field_network_tc(const NetMeta net, const __half* __restrict__ table, const __half* __restrict__ wd,
                   const __half* __restrict__ wc, const float4* __restrict__ pos_dt,
                   const uint32_t* __restrict__ sample_ray, const float4* __restrict__ ray_dir_t,
                   const float* __restrict__ coords7, uint64_t n, uint2* __restrict__ rgbsigma,
                   float4* __restrict__ shaded, const DevCfg g, const DevView v,
                   unsigned int* __restrict__ error_flags, const uint32_t* __restrict__ n_chunks_dev, uint32_t ray_shift,
                   const uint4* __restrict__ ray_sh, int n_staged, const CellTables cells,
                   const float* __restrict__ act_lut) {
    if (n_chunks_dev) n = (uint64_t)(*n_chunks_dev) * kChunkSamples;        // frame path: the sampler's chunk count
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5;
    const int group = tid >> 7, row = tid & 127;
    uint64_t* bar_ptr = reinterpret_cast<uint64_t*>(smem + kSmBar) + group;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + kSmBar + kGroups * 8);
    const uint32_t bar = smem_u32(bar_ptr);

    EncMeta* enc_meta = reinterpret_cast<EncMeta*>(smem + kSmEnc);
    prepare_enc_meta(net, table, enc_meta);
    attach_cell_tables(cells, enc_meta);
    load_weight_image(wd, 64, 32, smem + kSmW_D1);
    load_weight_image(wd + 64 * 32, 16, 64, smem + kSmW_D2);
    load_weight_image(wc, 64, 32, smem + kSmW_C1);
    load_weight_image(wc + 64 * 32, 64, 64, smem + kSmW_C2);
    load_weight_image(wc + 64 * 32 + 64 * 64, 16, 64, smem + kSmW_C3);
    if (tid < kGroups * 20) {                      // operand descriptors: [group][layer][k step] = (A, B)
        const int gq = tid / 20, layer = (tid % 20) / 4, kk = tid % 4;
        const uint32_t b_img = smem_u32(smem + (layer == 0 ? kSmW_D1 : layer == 1 ? kSmW_D2 : layer == 2 ? kSmW_C1 : layer == 3 ? kSmW_C2 : kSmW_C3));
        const uint32_t n_out = (layer == 1 || layer == 4) ? 16u : 64u;
        const uint32_t a_img = smem_u32(smem + kSmAct + gq * kActBytes);
        ulonglong2 d;
        d.x = make_desc(a_img + (uint32_t)kk * 2u * (128u * 16u), 128u * 16u, 128u);
        d.y = make_desc(b_img + (uint32_t)kk * 2u * n_out * 16u, n_out * 16u, 128u);
        reinterpret_cast<ulonglong2*>(smem + kSmDesc)[tid] = d;
    }
    if (row == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" :: "r"(bar) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(tmem_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (n_staged > 0) {
        // Coarse dense levels are read by every sample and are small: copy them into shared memory once per CTA and
        // point the level table there.
        uint32_t* stage = reinterpret_cast<uint32_t*>(smem + kSmStage);
        uint32_t off = 0;
        for (int l = 0; l < n_staged; ++l) {
            const uint32_t words = net.level[l].size * (F / 2);
            const uint32_t* src = reinterpret_cast<const uint32_t*>(table) + (size_t)net.level[l].offset * (F / 2); 
            for (uint32_t i = tid; i < words; i += kTcBlock) stage[off + i] = __ldg(src + i);
            if (tid == 0) enc_meta->level[l].base = stage + off;
            off += words;
        }
        if (tid == 0) enc_meta->n_staged = n_staged;
        __syncthreads();
    }
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_group = tmem_base + (uint32_t)group * 64u;                      // this group's columns
    const uint32_t tmem_row = tmem_group + ((uint32_t)((warp & 3) * 32) << 16);          // this warp's quarter of the lanes

    unsigned char* act = smem + kSmAct + group * kActBytes;
    constexpr uint32_t kIdesc64 = make_idesc(64), kIdesc16 = make_idesc(16);

    // One dense layer: K/16 instructions over the A image in the activation region and the layer's B image.  The
    // operand descriptors were computed once per CTA (desc_tab, filled below the weight images): the issuing thread
    // is one thread among 32 busy warps, and every instruction it spends here is time its whole group waits (the
    // issue took 420-670 cycles per layer with the descriptors built on the spot).
    const ulonglong2* my_desc = reinterpret_cast<const ulonglong2*>(smem + kSmDesc) + group * 20;
    auto issue_layer = [&](int layer, int k16, uint32_t idesc) {
        if (row == 0) {
            tc_fence_after();
            const ulonglong2* d = my_desc + layer * 4;
            const ulonglong2 d0 = d[0], d1 = d[1];
            if (k16 == 4) {
                const ulonglong2 d2 = d[2], d3 = d[3];
                mma_f16_fixed<false>(tmem_group, d0.x, d0.y, idesc);
                mma_f16_fixed<true>(tmem_group, d1.x, d1.y, idesc);
                mma_f16_fixed<true>(tmem_group, d2.x, d2.y, idesc);
                mma_f16_fixed<true>(tmem_group, d3.x, d3.y, idesc);
            } else {
                mma_f16_fixed<false>(tmem_group, d0.x, d0.y, idesc);
                mma_f16_fixed<true>(tmem_group, d1.x, d1.y, idesc);
            }
            mma_commit(bar);
        }
    };
    // Epilogue of a 64-wide layer: my row -> ReLU -> fp16 -> 8 units of the activation region.
    auto hidden_epilogue = [&]() {
        uint32_t acc[16];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            tmem_ld16(tmem_row + q * 16, acc);
            tmem_ld_wait();
            store_units<true>(acc, act, 2 * q, row);
        }
    };

    uint32_t phase = 0;
    bool failed = false;
    // Only the group's first warp polls the commit barrier; the other three sleep in the hardware
    // barrier of group_any() instead of spending issue slots on a spin loop.
    auto wait_layer = [&]() -> bool {
        bool expired = false;
        if ((warp & 3) == 0) expired = !mbar_wait(bar, phase);
        phase ^= 1;
        return !group_any(group, expired);
    };
    const uint64_t n_tiles = (n + kGroup - 1) / kGroup;
    const uint64_t tile_stride = (uint64_t)gridDim.x * kGroups;
    for (uint64_t tile = (uint64_t)blockIdx.x * kGroups + group; tile < n_tiles; tile += tile_stride) {
        const uint64_t s = tile * kGroup + row;
        // ---- encode: one thread per sample, written as 16-byte units of the A image ----
        float x = 0.f, y = 0.f, z = 0.f, dx = 0.5f, dy = 0.5f, dz = 0.5f;
        uint32_t ray = 0;
        if (s < n) {
            if (!FRAME && coords7) {
                const float* c = coords7 + s * 7;
                x = c[0]; y = c[1]; z = c[2]; dx = c[4]; dy = c[5]; dz = c[6];
            } else {
                const float4 p = pos_dt[s];
                x = p.x; y = p.y; z = p.z;
                ray = sample_ray[s >> ray_shift];
                if (!FRAME && !ray_sh) {
                    const float4 d = ray_dir_t[ray];
                    dx = (d.x + 1.f) * 0.5f; dy = (d.y + 1.f) * 0.5f; dz = (d.z + 1.f) * 0.5f;   // warp_direction
                }
            }
        }
        {
            // The 16 packed pairs are collected in an array indexed by the level (it lives in local memory, which L1
            // serves) and stored as four 16-byte units; storing each pair straight into the A image (sixteen 4-byte
            // stores, four-way bank conflicts) measured 134.9 ms per benchmark frame against 132.0.
            uint32_t enc[16];
                        hash_encode_packed<F, true>(enc_meta, table, x, y, z, enc);
#pragma unroll
            for (int j = 0; j < 4; ++j)
                *reinterpret_cast<uint4*>(act + ((size_t)j * 128 + row) * 16) =
                    make_uint4(enc[4 * j], enc[4 * j + 1], enc[4 * j + 2], enc[4 * j + 3]);
        }
        // Spherical harmonics of the direction: read later from the per-ray table the sampler wrote (frame path), or
        // computed here and kept in registers (stage entry points).
        const bool sh_from_ray = FRAME || (ray_sh && !coords7);
        uint4 sh0 = make_uint4(0u, 0u, 0u, 0u), sh1 = sh0;
        if (!sh_from_ray) {
            __align__(16) __half sh[16];
            sh_encode(dx, dy, dz, sh);
            sh0 = *reinterpret_cast<const uint4*>(sh);
            sh1 = *reinterpret_cast<const uint4*>(sh + 8);
        }
        fence_async_smem();
        group_sync(group);

        // ---- density layer 1: 32 -> 64, ReLU ----
        issue_layer(0, 2, kIdesc64);
        if (FRAME) {                                  // hint only: bring the next tile's records into L2
            const uint64_t sn = s + tile_stride * kGroup;
            if (sn < n) {
                asm volatile("prefetch.global.L2 [%0];" :: "l"(pos_dt + sn));
                if ((row & 15) == 0) asm volatile("prefetch.global.L2 [%0];" :: "l"(sample_ray + (sn >> ray_shift)));
            }
        }
        if (!wait_layer()) { failed = true; break; }
        tc_fence_after();
        hidden_epilogue();
        tc_fence_before();
        fence_async_smem();
        group_sync(group);
        // ---- density layer 2: 64 -> 16 ----
        issue_layer(1, 4, kIdesc16);
        if (!wait_layer()) { failed = true; break; }
        tc_fence_after();
        uint32_t sigma_half;
        {
            uint32_t acc[16];
            tmem_ld16(tmem_row, acc);
            tmem_ld_wait();
            store_units<false>(acc, act, 0, row);         // colour input rows 0..15 = density output
            sigma_half = pack2(__uint_as_float(acc[0]), 0.f) & 0xffffu;
        }
        if (sh_from_ray) {
            sh0 = __ldg(ray_sh + 2 * (size_t)ray);
            sh1 = __ldg(ray_sh + 2 * (size_t)ray + 1);
        }
        *reinterpret_cast<uint4*>(act + ((size_t)2 * 128 + row) * 16) = sh0;   // rows 16..31 = SH
        *reinterpret_cast<uint4*>(act + ((size_t)3 * 128 + row) * 16) = sh1;
        tc_fence_before();
        fence_async_smem();
        group_sync(group);
        // ---- colour layer 1: 32 -> 64, ReLU ----
        issue_layer(2, 2, kIdesc64);
        if (!wait_layer()) { failed = true; break; }
        tc_fence_after();
        hidden_epilogue();
        tc_fence_before();
        fence_async_smem();
        group_sync(group);
        // ---- colour layer 2: 64 -> 64, ReLU ----
        issue_layer(3, 4, kIdesc64);
        if (!wait_layer()) { failed = true; break; }
        tc_fence_after();
        hidden_epilogue();
        tc_fence_before();
        fence_async_smem();
        group_sync(group);
        // ---- colour layer 3: 64 -> 16 (3 used) ----
        issue_layer(4, 4, kIdesc16);
        if (!wait_layer()) { failed = true; break; }
        tc_fence_after();
        {
            uint32_t acc[16];
            tmem_ld16(tmem_row, acc);
            tmem_ld_wait();
            if (s < n) {
                const uint32_t rg = pack2(__uint_as_float(acc[0]), __uint_as_float(acc[1]));
                const uint32_t bs = (pack2(__uint_as_float(acc[2]), 0.f) & 0xffffu) | (sigma_half << 16);
                if (FRAME || shaded) {
                    // frame path: activations evaluated here, on the fp16-rounded network outputs
                    const float4 p = pos_dt[s];                      // re-read (L2) instead of holding four registers
                    if (act_lut) {
                        shaded[s] = shade_sample_lut(g, v, act_lut, rg & 0xffffu, rg >> 16, bs & 0xffffu, sigma_half, p.w,
                                                     mk3(p.x, p.y, p.z));
                    } else {
                        const __half2 h0 = *reinterpret_cast<const __half2*>(&rg), h1 = *reinterpret_cast<const __half2*>(&bs);
                        const float raw[4] = {__low2float(h0), __high2float(h0), __low2float(h1), __high2float(h1)};
                        shaded[s] = shade_sample(g, v, raw, p.w, mk3(p.x, p.y, p.z));
                    }
                } else {
                    rgbsigma[s] = make_uint2(rg, bs);
                }
            }
        }
        // (Measured and left as they are, in ms per benchmark frame against 132.0: no barrier here -- the one after the
        // next tile's gather orders the same accesses -- 131.4-132.4; two tcgen05.ld in flight in the epilogues 134.0;
        // every warp polling the commit barrier itself, agreement at the end of the tile, 131.2-144.0.)
        tc_fence_before();
        group_sync(group);
    }
    if (failed && row == 0 && error_flags) atomicOr(error_flags, 2u);
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_base), "r"(kTmemCols) : "memory");
}

__global__ void k_build_activation_table(const DevCfg g, float* __restrict__ lut) {
    const uint32_t h = blockIdx.x * blockDim.x + threadIdx.x;
    if (h >= 65536u) return;
    const float x = __half2float(__ushort_as_half((unsigned short)h));
    lut[h] = network_to_rgb(x, g.rgb_activation);
    lut[65536 + h] = network_to_density(x, g.density_activation);
}

// One thread per cell of level l: the entries of the cell's eight corners, in corner order.
template <int F>
__global__ void k_build_cell_table(const NetMeta net, const __half* __restrict__ table, int l, uint4* __restrict__ out) {
    const LevelMeta L = net.level[l];
    const uint32_t* words = reinterpret_cast<const uint32_t*>(table) + (size_t)L.offset * (F / 2);
    const uint64_t n_cells = (uint64_t)L.res * L.res * L.res;
    for (uint64_t c = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; c < n_cells; c += (uint64_t)gridDim.x * blockDim.x) {
        const uint32_t cx = (uint32_t)(c % L.res), cy = (uint32_t)((c / L.res) % L.res), cz = (uint32_t)(c / ((uint64_t)L.res * L.res));
        uint32_t w[8 * (F / 2)];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const uint32_t i = corner_index(L, cx + (k & 1), cy + ((k >> 1) & 1), cz + (k >> 2));
#pragma unroll
            for (int f = 0; f < F / 2; ++f) w[k * (F / 2) + f] = words[(size_t)i * (F / 2) + f];
        }
#pragma unroll
        for (int q = 0; q < F; ++q) out[c * F + q] = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
    }
}

}  // namespace

size_t cell_table_units(const NetMeta& net, int n_levels, unsigned long long* offsets) {
    size_t units = 0;
    for (int l = 0; l < n_levels && l < (int)net.n_levels; ++l) {
        if (offsets) offsets[l] = units;
        units += (size_t)net.level[l].res * net.level[l].res * net.level[l].res * net.n_features;
    }
    return units;
}

void launch_build_cell_tables(const NetMeta& net, const __half* table, int n_levels, uint4* out, cudaStream_t stream) {
    unsigned long long off[kMaxLevels];
    cell_table_units(net, n_levels, off);
    for (int l = 0; l < n_levels && l < (int)net.n_levels; ++l) {
        if (net.n_features == 2) k_build_cell_table<2><<<148 * 8, 256, 0, stream>>>(net, table, l, out + off[l]);
        else k_build_cell_table<4><<<148 * 8, 256, 0, stream>>>(net, table, l, out + off[l]);
    }
}

void launch_build_activation_table(const DevCfg& g, float* lut, cudaStream_t stream) {
    k_build_activation_table<<<256, 256, 0, stream>>>(g, lut);
}

void launch_field_network_tc(const NetMeta& net, const __half* table, const __half* w_density, const __half* w_rgb,
                             const float4* pos_dt, const uint32_t* sample_ray, const float4* ray_dir_t,
                             const float* coords7, uint64_t n, uint2* rgbsigma, float4* shaded, const DevCfg* g,
                             const DevView* v, unsigned int* error_flags, cudaStream_t stream,
                             const uint32_t* n_chunks_dev, uint32_t ray_shift, const uint4* ray_sh,
                             const uint4* cell_table, int n_cell_levels, const float* act_lut) {
    if (n == 0 && !n_chunks_dev) return;
    // Staged levels: as many leading dense levels as fit into `stage_budget` bytes of shared memory (default: none).
    // Shared memory taken here is L1 taken from the gathers of the other levels.
    static const long stage_budget = [] { const char* e = getenv("SRF_B200_STAGE_BYTES"); return e ? atol(e) : 0l; }();
    int n_staged = 0;
    size_t stage_bytes = 0;
    for (uint32_t l = 0; l < net.n_levels && net.level[l].dense; ++l) {
        const size_t b = (size_t)net.level[l].size * net.n_features * sizeof(__half);
        if ((long)(stage_bytes + b) > stage_budget || kSmTotal + stage_bytes + b > (size_t)kSmLimit) break;
        stage_bytes += b; ++n_staged;
    }
    const int smem_bytes = kSmTotal + (int)stage_bytes;
    // per device and cheap: set on every launch rather than cached per process
    // no more shared memory than the CTA needs: the rest of the unified array serves the gathers as L1
    const int carveout = (smem_bytes * 100 + 228 * 1024 - 1) / (228 * 1024);
    const void* kernels[] = {(const void*)k_field_network_tc<2, true>, (const void*)k_field_network_tc<2, false>,
                             (const void*)k_field_network_tc<4, true>, (const void*)k_field_network_tc<4, false>};
    for (const void* k : kernels) {
        cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
        cudaFuncSetAttribute(k, cudaFuncAttributePreferredSharedMemoryCarveout, carveout);
    }
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const uint64_t tiles = (n + kTcBlock - 1) / kTcBlock;    // kGroups 128-sample tiles per CTA and sweep
    const uint64_t cap = (uint64_t)sms;                      // one resident CTA per SM
    const int grid = n_chunks_dev ? (int)cap : (int)(tiles < cap ? tiles : cap);
    DevCfg g0; DevView v0;
    memset(&g0, 0, sizeof(g0)); memset(&v0, 0, sizeof(v0));
    if (g) g0 = *g;
    if (v) v0 = *v;
    const bool frame = shaded && ray_sh && pos_dt && sample_ray && !coords7;
    CellTables ct;
    memset(&ct, 0, sizeof(ct));
    if (cell_table && n_cell_levels > 0) {
        ct.base = cell_table;
        ct.n_levels = n_cell_levels < (int)net.n_levels ? n_cell_levels : (int)net.n_levels;
        cell_table_units(net, ct.n_levels, ct.offset);
    }
#define SRF_TC_LAUNCH(FEAT, FRAME)                                                                                          \
    k_field_network_tc<FEAT, FRAME><<<grid, kTcBlock, smem_bytes, stream>>>(net, table, w_density, w_rgb, pos_dt, sample_ray, \
        ray_dir_t, coords7, n, rgbsigma, shaded, g0, v0, error_flags, n_chunks_dev, ray_shift, ray_sh, n_staged, ct, act_lut)
    if (net.n_features == 2) { if (frame) SRF_TC_LAUNCH(2, true); else SRF_TC_LAUNCH(2, false); }
    else { if (frame) SRF_TC_LAUNCH(4, true); else SRF_TC_LAUNCH(4, false); }
#undef SRF_TC_LAUNCH
}

}  // namespace srf
