// srf_sampler.cu -- the sampler: ray generation, occupancy-guided marching, sample compaction.
//
// Replaces init_rays_with_payload_kernel_nerf, advance_pos_nerf and
// generate_coords_from_rays_regularly_kernel (internal/sampler/occupancy_sampler.cu:691-863) and
// the host-driven compaction loop around them (internal/testbed.cu:523-583).  Instead of up to
// 8 samples per ray per host iteration, each ray is marched to its end in one kernel: a count
// pass sizes a compact per-ray-contiguous sample buffer, an exclusive scan places the rays, an
// emit pass fills it.
#include <cooperative_groups.h>

#include "srf_network.cuh"

namespace cg = cooperative_groups;

namespace srf {

namespace {

constexpr int kBlock = 128;

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

__global__ void __launch_bounds__(kBlock)
k_ray_count(const DevCfg g, const DevView v, const uint8_t* __restrict__ bits, float4* __restrict__ ray_dir_t,
            uint8_t* __restrict__ ray_end, uint32_t* __restrict__ counts, FrameCounters* __restrict__ counters) {
    const uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x;
    unsigned long long alive = 0, steps = 0, samples = 0;
    unsigned int err = 0;
    if (i < v.n_rays) {
        const uint32_t pixel = shard_ray_pixel(v, i);
        const RayInit r = init_ray(g, v, pixel);
        uint32_t n = 0, end = RAY_END_BORN_DEAD, n_steps = 0;
        if (r.alive) {
            end = march_ray(g, bits, r.o, r.d, r.t, &n_steps,
                            [&](const V3&, float, uint32_t, uint32_t, float) { ++n; return true; });
            alive = 1;
            if (end == RAY_END_LIMIT) err = 1u;
        }
        ray_dir_t[i] = make_float4(r.d.x, r.d.y, r.d.z, r.t);
        ray_end[i] = (uint8_t)end;
        counts[i] = n;
        steps = n_steps;
        samples = n;
    }
    alive = warp_sum_u64(alive);
    steps = warp_sum_u64(steps);
    samples = warp_sum_u64(samples);
    err = __any_sync(0xffffffffu, err != 0);
    if ((threadIdx.x & 31) == 0) {
        if (alive) atomicAdd(&counters->n_alive, alive);
        if (steps) atomicAdd(&counters->n_march_steps, steps);
        if (samples) atomicAdd(&counters->n_samples, samples);
        if (err) atomicOr(&counters->error_flags, 1u);
    }
}

template <bool COORDS>
__global__ void __launch_bounds__(kBlock)
k_ray_emit(const DevCfg g, const DevView v, const uint8_t* __restrict__ bits, const float4* __restrict__ ray_dir_t,
           const uint64_t* __restrict__ offsets, uint64_t ray_begin, uint64_t ray_end, float4* __restrict__ pos_dt,
           uint32_t* __restrict__ sample_ray, float* __restrict__ coords7, uint32_t* __restrict__ ordinal_out,
           uint32_t* __restrict__ cell_out) {
    const uint64_t i = ray_begin + (uint64_t)blockIdx.x * kBlock + threadIdx.x;
    if (i >= ray_end) return;
    const uint64_t lo = offsets[i], hi = offsets[i + 1];
    if (hi == lo) return;
    const uint64_t base = offsets[ray_begin];
    const float4 dt4 = ray_dir_t[i];
    const V3 o = mk3(v.cam[3], v.cam[7], v.cam[11]);
    const V3 d = mk3(dt4.x, dt4.y, dt4.z);
    const V3 wd = mk3((d.x + 1.f) * 0.5f, (d.y + 1.f) * 0.5f, (d.z + 1.f) * 0.5f);   // warp_direction
    uint64_t slot = lo - base;
    const uint64_t slot_end = hi - base;
    uint32_t n_steps;
    march_ray(g, bits, o, d, dt4.w, &n_steps, [&](const V3& w, float dt, uint32_t ord, uint32_t cell, float) {
        if (COORDS) {
            float* c = coords7 + slot * 7;
            c[0] = w.x; c[1] = w.y; c[2] = w.z; c[3] = dt; c[4] = wd.x; c[5] = wd.y; c[6] = wd.z;
        } else {
            pos_dt[slot] = make_float4(w.x, w.y, w.z, dt);
            sample_ray[slot] = (uint32_t)i;
        }
        if (ordinal_out) ordinal_out[slot] = ord;
        if (cell_out) cell_out[slot] = cell;
        ++slot;
        return slot < slot_end;     // never writes past the slots the count pass reserved
    });
}

// Single-pass sampler of the frame path.  Each thread marches its ray once and appends the live
// samples to the ray's own list of fixed-size chunks (kChunkSamples records) taken from a pool.  Chunks
// are handed out by one atomicAdd per group of lanes that need one at the same time (the lanes of a
// warp march neighbouring pixels in near lockstep, so they usually run out of room together).  There is
// no counting pass, no scan and no read-back: the field kernel later walks the pool densely, the
// compositor walks each ray's chunk list.
//
// Waves.  A frame may run the sampler several times: a wave takes every running ray up to `pause_at` march
// steps in all and leaves the rest of the march for the next wave (RAY_END_PAUSED; t in ray_dir_t.w, loop iterations and samples so far
// in ray_ordinal / ray_total).  Between waves the field and the compositor run on what was emitted, and rays the
// compositor has finished (RAY_END_DONE) are not marched further -- the counterpart of the reference's
// rounds of <= 8 steps with compaction of dead rays (testbed.cu:523-583), with round sizes that keep the
// kernels large.  The arithmetic of a ray does not depend on where it is paused.
__global__ void __launch_bounds__(kBlock)
k_march_paged(const DevCfg g, const DevView v, const uint8_t* __restrict__ bits, uint64_t ray_begin, uint64_t ray_end,
              float4* __restrict__ pool_pos_dt, uint32_t* __restrict__ chunk_ray, uint32_t* __restrict__ chunk_next,
              uint32_t pool_chunks, uint32_t* __restrict__ chunk_cursor, float4* __restrict__ ray_dir_t,
              uint8_t* __restrict__ ray_end_out, uint32_t* __restrict__ ray_count, uint32_t* __restrict__ ray_head,
              FrameCounters* __restrict__ counters, uint32_t wave, uint32_t pause_at, uint32_t* __restrict__ ray_ordinal,
              uint32_t* __restrict__ ray_total, uint4* __restrict__ ray_sh) {
    const uint64_t i = ray_begin + (uint64_t)blockIdx.x * kBlock + threadIdx.x;
    unsigned long long alive = 0, steps = 0, samples = 0;
    unsigned int err = 0;
    if (i < ray_end) {
        V3 o, d;
        MarchState st = {0.f, 0u, 0u};
        uint32_t end = RAY_END_BORN_DEAD;
        bool run = false;
        if (wave == 0) {
            const uint32_t pixel = shard_ray_pixel(v, i);
            const RayInit r = init_ray(g, v, pixel);
            o = r.o; d = r.d; st.t = r.t;
            run = r.alive;
            alive = r.alive ? 1 : 0;
            if (ray_sh && r.alive) {                // the direction encoding is the same for every sample of the ray
                __align__(16) __half sh[16];
                sh_encode((d.x + 1.f) * 0.5f, (d.y + 1.f) * 0.5f, (d.z + 1.f) * 0.5f, sh);      // warp_direction
                ray_sh[2 * i] = *reinterpret_cast<const uint4*>(sh);
                ray_sh[2 * i + 1] = *reinterpret_cast<const uint4*>(sh + 8);
            }
        } else {
            end = ray_end_out[i];
            if (end == RAY_END_PAUSED) {
                const float4 q = ray_dir_t[i];
                o = mk3(v.cam[3], v.cam[7], v.cam[11]);
                d = mk3(q.x, q.y, q.z);
                st.t = q.w; st.ordinal = ray_ordinal[i]; st.n = ray_total[i];
                run = true;
            }
        }
        uint32_t n = 0, head = kNoChunk;
        const uint32_t steps_before = st.ordinal;
        if (run) {
            uint32_t chunk = kNoChunk, fill = kChunkSamples;
            end = march_ray_from(g, bits, o, d, st, pause_at, [&](const V3& w, float dt, uint32_t, uint32_t, float) {
                if (fill == kChunkSamples) {
                    const cg::coalesced_group lanes = cg::coalesced_threads();
                    uint32_t base = 0;
                    if (lanes.thread_rank() == 0) base = atomicAdd(chunk_cursor, lanes.size());
                    const uint32_t c = lanes.shfl(base, 0) + lanes.thread_rank();
                    if (c >= pool_chunks) { err = 4u; return false; }      // the pool is sized so that this cannot happen
                    chunk_ray[c] = (uint32_t)i;
                    chunk_next[c] = kNoChunk;
                    if (chunk == kNoChunk) head = c; else chunk_next[chunk] = c;
                    chunk = c;
                    fill = 0;
                }
                pool_pos_dt[(uint64_t)chunk * kChunkSamples + fill] = make_float4(w.x, w.y, w.z, dt);
                ++fill;
                ++n;
                return true;
            });
            if (end == RAY_END_LIMIT) err |= 1u;
        }
        if (wave == 0 || run) {
            ray_dir_t[i] = make_float4(d.x, d.y, d.z, st.t);
            ray_end_out[i] = (uint8_t)end;
            if (ray_ordinal) { ray_ordinal[i] = st.ordinal; ray_total[i] = st.n; }
        }
        ray_count[i] = n;
        ray_head[i] = head;
        steps = st.ordinal - steps_before;
        samples = n;
    }
    alive = warp_sum_u64(alive);
    steps = warp_sum_u64(steps);
    samples = warp_sum_u64(samples);
    for (int o = 16; o > 0; o >>= 1) err |= __shfl_down_sync(0xffffffffu, err, o);
    if ((threadIdx.x & 31) == 0) {
        if (alive) atomicAdd(&counters->n_alive, alive);
        if (steps) atomicAdd(&counters->n_march_steps, steps);
        if (samples) atomicAdd(&counters->n_samples, samples);
        if (err) atomicOr(&counters->error_flags, err);
    }
}

__global__ void __launch_bounds__(kBlock)
k_generate_rays(const DevCfg g, const DevView v, const uint8_t* __restrict__ bits, float* __restrict__ dir,
                float* __restrict__ t_out, uint8_t* __restrict__ alive_out, uint32_t* __restrict__ pixel_out) {
    const uint64_t i = (uint64_t)blockIdx.x * kBlock + threadIdx.x;
    if (i >= v.n_rays) return;
    const uint32_t pixel = shard_ray_pixel(v, i);
    const RayInit r = init_ray(g, v, pixel);
    bool alive = false;
    float t = 0.f;
    if (r.alive) {
        uint32_t n_steps;
        DevCfg g1 = g;
        g1.sample_cap = 1;
        march_ray(g1, bits, r.o, r.d, r.t, &n_steps, [&](const V3&, float, uint32_t, uint32_t, float ts) {
            alive = true; t = ts; return false;
        });
    }
    if (dir) { dir[3 * i] = r.d.x; dir[3 * i + 1] = r.d.y; dir[3 * i + 2] = r.d.z; }
    if (t_out) t_out[i] = t;
    if (alive_out) alive_out[i] = alive ? 1 : 0;
    if (pixel_out) pixel_out[i] = pixel;
}

// ---- exclusive scan (u32 counts -> u64 offsets) ---------------------------------------------------
constexpr int kScanBlock = 256;
constexpr int kScanItems = 8;                     // per thread
constexpr int kScanTile = kScanBlock * kScanItems;

__device__ __forceinline__ unsigned long long block_exclusive_scan(unsigned long long v, unsigned long long* total,
                                                                    unsigned long long* smem /* 8 */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    unsigned long long x = v;
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    if (lane == 31) smem[wid] = x;
    __syncthreads();
    if (wid == 0) {
        unsigned long long w = lane < kScanBlock / 32 ? smem[lane] : 0ull;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long y = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += y;
        }
        if (lane < kScanBlock / 32) smem[lane] = w;
    }
    __syncthreads();
    const unsigned long long warp_base = wid ? smem[wid - 1] : 0ull;
    *total = smem[kScanBlock / 32 - 1];
    __syncthreads();
    return warp_base + x - v;
}

__global__ void __launch_bounds__(kScanBlock)
k_scan_tile_sums(const uint32_t* __restrict__ counts, uint64_t n, unsigned long long* __restrict__ tile_sums) {
    __shared__ unsigned long long smem[8];
    const uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
    unsigned long long s = 0;
    for (int k = 0; k < kScanItems; ++k) if (base + k < n) s += counts[base + k];
    unsigned long long total;
    block_exclusive_scan(s, &total, smem);
    if (threadIdx.x == 0) tile_sums[blockIdx.x] = total;
}

__global__ void __launch_bounds__(kScanBlock)
k_scan_tiles(unsigned long long* __restrict__ tile_sums, uint32_t n_tiles) {
    __shared__ unsigned long long smem[8];
    unsigned long long carry = 0;
    for (uint32_t base = 0; base < n_tiles; base += kScanBlock) {
        const uint32_t i = base + threadIdx.x;
        const unsigned long long v = i < n_tiles ? tile_sums[i] : 0ull;
        unsigned long long total;
        const unsigned long long ex = block_exclusive_scan(v, &total, smem);
        if (i < n_tiles) tile_sums[i] = carry + ex;
        carry += total;
    }
}

__global__ void __launch_bounds__(kScanBlock)
k_scan_final(const uint32_t* __restrict__ counts, uint64_t n, const unsigned long long* __restrict__ tile_sums,
             uint64_t* __restrict__ offsets) {
    __shared__ unsigned long long smem[8];
    const uint64_t base = (uint64_t)blockIdx.x * kScanTile + (uint64_t)threadIdx.x * kScanItems;
    uint32_t c[kScanItems];
    unsigned long long s = 0;
    for (int k = 0; k < kScanItems; ++k) { c[k] = base + k < n ? counts[base + k] : 0u; s += c[k]; }
    unsigned long long total;
    unsigned long long ex = block_exclusive_scan(s, &total, smem) + tile_sums[blockIdx.x];
    for (int k = 0; k < kScanItems; ++k) {
        if (base + k < n) offsets[base + k] = ex;
        ex += c[k];
        if (base + k + 1 == n) offsets[n] = ex;
    }
}

__global__ void k_eval_math(int op, const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float r = 0.f;
    switch (op) {
    case 0: r = srf_atan2f(a[i], b[i]); break;
    case 1: r = srf_asinf(a[i]); break;
    case 2: r = srf_cosf(a[i]); break;
    case 3: r = srf_sinf(a[i]); break;
    case 4: r = srf_expf(a[i]); break;
    case 5: r = srf_logf(a[i]); break;
    default: break;
    }
    out[i] = r;
}

inline unsigned int blocks_for(uint64_t n, int block) { return (unsigned int)((n + block - 1) / block); }

}  // namespace

void launch_ray_count(const DevCfg& g, const DevView& v, const uint8_t* bits, float4* ray_dir_t, uint8_t* ray_end,
                      uint32_t* counts, FrameCounters* counters, cudaStream_t stream) {
    if (v.n_rays == 0) return;
    k_ray_count<<<blocks_for(v.n_rays, kBlock), kBlock, 0, stream>>>(g, v, bits, ray_dir_t, ray_end, counts, counters);
}

size_t scan_scratch_bytes(uint64_t n) { return ((n + kScanTile - 1) / kScanTile + 1) * sizeof(unsigned long long); }

void launch_scan(const uint32_t* counts, uint64_t n, uint64_t* offsets, void* scratch, cudaStream_t stream) {
    if (n == 0) { cudaMemsetAsync(offsets, 0, sizeof(uint64_t), stream); return; }
    const uint32_t n_tiles = (uint32_t)((n + kScanTile - 1) / kScanTile);
    unsigned long long* tile_sums = (unsigned long long*)scratch;
    k_scan_tile_sums<<<n_tiles, kScanBlock, 0, stream>>>(counts, n, tile_sums);
    k_scan_tiles<<<1, kScanBlock, 0, stream>>>(tile_sums, n_tiles);
    k_scan_final<<<n_tiles, kScanBlock, 0, stream>>>(counts, n, tile_sums, offsets);
}

void launch_ray_emit(const DevCfg& g, const DevView& v, const uint8_t* bits, const float4* ray_dir_t,
                     const uint64_t* offsets, uint64_t ray_begin, uint64_t ray_end, float4* pos_dt,
                     uint32_t* sample_ray, float* coords7, uint32_t* ordinal, uint32_t* cell,
                     FrameCounters* counters, cudaStream_t stream) {
    (void)counters;
    if (ray_end <= ray_begin) return;
    const unsigned int nb = blocks_for(ray_end - ray_begin, kBlock);
    if (coords7)
        k_ray_emit<true><<<nb, kBlock, 0, stream>>>(g, v, bits, ray_dir_t, offsets, ray_begin, ray_end, pos_dt,
                                                    sample_ray, coords7, ordinal, cell);
    else
        k_ray_emit<false><<<nb, kBlock, 0, stream>>>(g, v, bits, ray_dir_t, offsets, ray_begin, ray_end, pos_dt,
                                                     sample_ray, coords7, ordinal, cell);
}

void launch_march_paged(const DevCfg& g, const DevView& v, const uint8_t* bits, uint64_t ray_begin, uint64_t ray_end,
                        float4* pool_pos_dt, uint32_t* chunk_ray, uint32_t* chunk_next, uint32_t pool_chunks,
                        uint32_t* chunk_cursor, float4* ray_dir_t, uint8_t* ray_end_out, uint32_t* ray_count,
                        uint32_t* ray_head, FrameCounters* counters, cudaStream_t stream, uint32_t wave, uint32_t pause_at,
                        uint32_t* ray_ordinal, uint32_t* ray_total, uint4* ray_sh) {
    if (ray_end <= ray_begin) return;
    k_march_paged<<<blocks_for(ray_end - ray_begin, kBlock), kBlock, 0, stream>>>(
        g, v, bits, ray_begin, ray_end, pool_pos_dt, chunk_ray, chunk_next, pool_chunks, chunk_cursor, ray_dir_t, ray_end_out,
        ray_count, ray_head, counters, wave, pause_at, ray_ordinal, ray_total, ray_sh);
}

void launch_generate_rays(const DevCfg& g, const DevView& v, const uint8_t* bits, float* dir, float* t,
                          uint8_t* alive, uint32_t* pixel, cudaStream_t stream) {
    if (v.n_rays == 0) return;
    k_generate_rays<<<blocks_for(v.n_rays, kBlock), kBlock, 0, stream>>>(g, v, bits, dir, t, alive, pixel);
}

void launch_eval_math(int op, const float* a, const float* b, float* out, size_t n, cudaStream_t stream) {
    if (n == 0) return;
    k_eval_math<<<blocks_for(n, 256), 256, 0, stream>>>(op, a, b, out, n);
}

// ---- srf_sample_offsets_static: the exclusive scan with its scratch inside the library ----------
//
// Some callers of the scan cannot allocate device memory at all: a renderer embedded in an
// application that handed the whole GPU to its own memory pool at start-up, a frame loop that must
// never hit the implicit device synchronisation of cudaMalloc/cudaFree, or a plug-in host that
// forbids allocation after initialisation.  srf_sample_offsets() keeps its tile sums in a buffer the
// context allocates (and grows) on demand; this variant keeps them in a fixed array that is part of
// the library image instead, so the call itself never allocates.
//
// The price: the array is sized for a stated maximum, every GPU that loads the library carries it
// until the process exits, and all calls on one device share it (see the header for the rules).
namespace {

constexpr uint64_t kStaticScanMaxTiles = 16384;                                  // 128 KiB of tile sums
constexpr uint64_t kStaticScanMaxRays = kStaticScanMaxTiles * (uint64_t)kScanTile;   // 33 554 432 counts

static __device__ __align__(256) unsigned long long g_static_scan_tile_sums[kStaticScanMaxTiles + 1];

constexpr int kMaxDevices = 64;
// Device address of the array above, per device.  In host code the array's NAME is only a handle for
// the runtime, not a device address; each device has its own copy at its own address, found once with
// cudaGetSymbolAddress while that device is current.
void* g_static_scan_ptr[kMaxDevices] = {};

void write_error(char* err, size_t err_len, const char* msg) {
    if (!err || err_len == 0) return;
    size_t i = 0;
    for (; msg[i] && i + 1 < err_len; ++i) err[i] = msg[i];
    err[i] = 0;
}

}  // namespace
}  // namespace srf

extern "C" srf_status srf_sample_offsets_static(int device, const uint32_t* d_counts, uint64_t n_rays,
                                                uint64_t* d_offsets, void* stream, char* err, size_t err_len) {
    using namespace srf;
    if (!d_counts || !d_offsets) { write_error(err, err_len, "srf_sample_offsets_static: NULL buffer"); return SRF_ERR_ARG; }
    if (device < 0 || device >= kMaxDevices) { write_error(err, err_len, "srf_sample_offsets_static: device index out of range"); return SRF_ERR_ARG; }
    if (n_rays > kStaticScanMaxRays) {
        write_error(err, err_len, "srf_sample_offsets_static: more than 33554432 counts; the built-in scratch holds "
                                  "16384 tile sums of 2048 counts each - use srf_sample_offsets");
        return SRF_ERR_CAPACITY;
    }
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) { write_error(err, err_len, "srf_sample_offsets_static: cudaGetDevice failed"); return SRF_ERR_CUDA; }
    if (prev != device && cudaSetDevice(device) != cudaSuccess) {
        write_error(err, err_len, "srf_sample_offsets_static: cudaSetDevice failed");
        return SRF_ERR_CUDA;
    }
    srf_status st = SRF_OK;
    if (!g_static_scan_ptr[device]) {
        // first call on this device: look the array's device address up (no allocation; the array is
        // part of the loaded module)
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scan_tile_sums);
        if (e != cudaSuccess || !p) {
            write_error(err, err_len, cudaGetErrorString(e));
            st = SRF_ERR_CUDA;
        } else {
            g_static_scan_ptr[device] = p;
        }
    }
    if (st == SRF_OK) {
        // every tile sum the later kernels read is written by the first kernel of this call, so
        // nothing left over from an earlier call needs clearing
        launch_scan(d_counts, n_rays, d_offsets, g_static_scan_ptr[device], (cudaStream_t)stream);
        const cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) { write_error(err, err_len, cudaGetErrorString(e)); st = SRF_ERR_CUDA; }
    }
    if (prev != device) cudaSetDevice(prev);
    return st;
}
