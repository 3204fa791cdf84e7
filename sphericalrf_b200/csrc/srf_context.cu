// srf_context.cu -- the C-ABI of libsrf_b200.so (include/srf_abi.h): context, parameter upload,
// stage entry points and the frame loop that replaces Testbed::render_frame
// (internal/testbed.cu:479-606).
//
// Frame loop.  The reference alternates compaction, <= 8 samples per ray, the network and
// compositing under host control, reading a counter back every iteration.  Here a frame is, per
// batch of rays: single-pass march into a paged sample pool -> field over the pool -> per-ray
// compositing + output stage.  Nothing is read back: the field kernel takes the number of chunks the
// sampler used from device memory.  Batches exist only to bound the pool (every ray of a batch is
// given room for the most samples its step-size law allows).  The count -> scan -> emit kernels serve
// the stage entry points and the parity tap, which need the compact ray-major layout.
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <thread>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "srf_kernels.cuh"

using namespace srf;

namespace {

thread_local std::string g_create_error;

constexpr uint64_t kAutoSampleCapacity = 512ull << 20;  // default upper bound of the sample pool (32 B per slot)

struct DevBuf {
    void* p = nullptr;
    size_t bytes = 0;
};

}  // namespace

struct srf_ctx {
    srf_config_t cfg;
    DevCfg g;
    NetMeta net;
    int device = 0;
    std::string err;
    uint32_t n_table_entries = 0;
    float min_optical_thickness = 0.01f;

    // model
    float* grid = nullptr;
    float* grid_current = nullptr;
    float* partial_a = nullptr;
    float* partial_b = nullptr;
    float* mean = nullptr;
    uint8_t* bits = nullptr;
    uint32_t* skip_shell = nullptr;          // summaries of the bitfield for the sampler (see march_ray)
    uint32_t* skip_yz = nullptr;
    bool skip_capable = false;
    __half* table = nullptr;
    uint4* cell_table = nullptr;         // cell-major copies of the leading levels of the table (see CellTables)
    int n_cell_levels = 0;               // levels the allocation covers
    uint64_t cell_budget = 4ull << 30;   // bytes the copies may take (srf_set_cell_table_budget); 0: none
    int cell_levels_forced = -1;         // SRF_B200_CELL_LEVELS, when set
    bool cell_dirty = true;              // the table changed since the copies were built
    float* act_lut = nullptr;            // both activations tabulated over all fp16 arguments
    __half* w_density = nullptr;
    __half* w_rgb = nullptr;
    bool have_net = false;
    float* blobs = nullptr;
    float* cmap = nullptr;
    uint32_t n_blobs = 0;

    // per-frame scratch
    DevBuf train_flags, train_rank, loss_rgb;
    DevBuf ray_sh;                                             // 16 SH halves per ray (frame path, network field)
    DevBuf ray_ordinal, ray_total, ray_rgba, ray_ncomp;        // per-ray state between the waves of a frame
    uint32_t wave_budget[8] = {128, 512, 2048, 8192, 0, 0, 0, 0};   // march steps per ray in waves 0, 1, ...; a final unlimited wave follows
    uint32_t n_wave_budgets = 4;
    DevBuf ray_dir_t, ray_end, counts, offsets, scan_scratch;
    DevBuf pos_dt, sample_ray, rgbs;
    DevBuf pool_pos, pool_shaded, chunk_ray, chunk_next, ray_head;   // paged frame path
    uint32_t* d_chunk_cursor = nullptr;
    unsigned int* d_ticket = nullptr;        // last-block ticket of the fused refresh (zero between launches)
    bool fused_refresh = false;              // SRF_B200_FUSED_REFRESH=1: the two-launch refresh (same bits; measured 4 % slower, see srf_refresh.cu)
    bool grid_may_hold_masked_cells = false; // a negative cell was uploaded or written by the never-seen mask
    DevBuf img_out, img_accum;
    FrameCounters* d_counters = nullptr;
    FrameCounters* h_counters = nullptr;     // pinned
    uint64_t reserve_samples = 0;

    // refresh
    uint32_t refresh_step = 0;
    RefreshRng rng = {0, 0};
    RefreshWeights refresh_w;                // fp32 images of the density MLP weights the refresh reads

    // which engine runs the MLPs of the render path: tcgen05/TMEM (default) or the mma.sync kernel
    bool use_tcgen05 = true;

    // timing
    bool timing = false;
    cudaEvent_t ev[8] = {};
};

namespace {

#define SRF_CK(ctx, call)                                                                      \
    do {                                                                                       \
        cudaError_t e_ = (call);                                                               \
        if (e_ != cudaSuccess) {                                                               \
            (ctx)->err = std::string(#call) + ": " + cudaGetErrorString(e_);                   \
            return SRF_ERR_CUDA;                                                               \
        }                                                                                      \
    } while (0)

srf_status fail(srf_ctx* ctx, srf_status st, const std::string& msg) {
    if (ctx) ctx->err = msg; else g_create_error = msg;
    return st;
}

srf_status ensure(srf_ctx* ctx, DevBuf& b, size_t bytes) {
    if (bytes <= b.bytes) return SRF_OK;
    if (b.p) SRF_CK(ctx, cudaFree(b.p));
    b.p = nullptr; b.bytes = 0;
    const size_t want = bytes + bytes / 8;           // grow with slack
    SRF_CK(ctx, cudaMalloc(&b.p, want));
    b.bytes = want;
    return SRF_OK;
}

float resolved_per_level_scale(const srf_config_t& c) {
    float pls = c.per_level_scale;
    if (pls <= 0.f && c.n_levels > 1)
        pls = std::exp(std::log(c.desired_resolution / (float)c.base_resolution) / (float)(c.n_levels - 1));
    return pls;
}

// Level geometry of the hash grid (Mueller et al. 2022): scale_l = base * b^l - 1,
// resolution_l = ceil(scale_l) + 1, entries_l = min(2^T, round_up(res^3, 8)).
void build_net_meta(const srf_config_t& c, NetMeta* net) {
    memset(net, 0, sizeof(*net));
    net->n_levels = c.n_levels;
    net->n_features = c.n_features_per_level;
    const float pls = resolved_per_level_scale(c);
    const uint64_t T = 1ull << c.log2_hashmap_size;
    uint32_t off = 0;
    for (uint32_t l = 0; l < c.n_levels; ++l) {
        const double s = (double)c.base_resolution * std::pow((double)pls, (double)l) - 1.0;
        const float sf = (float)s;
        const uint32_t res = (uint32_t)std::ceil(sf) + 1u;
        const uint64_t dense = (uint64_t)res * res * res;
        uint64_t n = (dense + 7ull) / 8ull * 8ull;
        if (n > T) n = T;
        net->level[l].scale = sf;
        net->level[l].res = res;
        net->level[l].offset = off;
        net->level[l].size = (uint32_t)n;
        net->level[l].dense = dense <= n ? 1u : 0u;
        off += (uint32_t)n;
    }
}

uint32_t table_entries(const NetMeta& net) {
    const LevelMeta& L = net.level[net.n_levels - 1];
    return L.offset + L.size;
}

srf_status validate(const srf_config_t* c, std::string* why) {
    auto bad = [&](const char* m) { *why = m; return SRF_ERR_ARG; };
    if (!c) return bad("config is NULL");
    if (c->struct_size != sizeof(srf_config_t)) return bad("srf_config_t.struct_size does not match this library");
    if (c->version != SRF_ABI_VERSION) return bad("srf_config_t.version does not match this library");
    if (c->warping_type < 0 || c->warping_type > SRF_WARP_SINUSOIDAL) return bad("Unknown warping type.");
    if (c->sampling_type < 0 || c->sampling_type > SRF_SAMPLING_LOG) return bad("Unknown sampling type.");
    if (c->grid_distribution_type < 0 || c->grid_distribution_type > SRF_GRID_METRIC_RECIPROCAL)
        return bad("Unknown grid distribution type.");
    if (c->grid_size < 8 || c->grid_size > 1024 || (c->grid_size & (c->grid_size - 1))) return bad("grid_size must be a power of two in [8, 1024]");
    if (c->num_cascades < 1 || c->num_cascades > 8) return bad("num_cascades must be in [1, 8]");
    if ((uint64_t)c->grid_size * c->grid_size * c->grid_size * c->num_cascades > (1ull << 31)) return bad("grid too large");
    if (c->maximum_marching_steps == 0) return bad("maximum_marching_steps must be positive");
    if (c->aabb_scale == 0) return bad("aabb_scale must be positive");
    if (c->field_type == SRF_FIELD_NETWORK) {
        if (c->n_levels * c->n_features_per_level != 32) return bad("n_levels * n_features_per_level must be 32");
        if (c->n_features_per_level != 2 && c->n_features_per_level != 4) return bad("n_features_per_level must be 2 or 4");
        if (c->log2_hashmap_size < 10 || c->log2_hashmap_size > 24) return bad("log2_hashmap_size must be in [10, 24]");
        if (c->base_resolution < 2) return bad("base_resolution must be >= 2");
    } else if (c->field_type != SRF_FIELD_BLOBS) {
        return bad("unknown field_type");
    }
    if (c->density_activation < 0 || c->density_activation > 3 || c->rgb_activation < 0 || c->rgb_activation > 3)
        return bad("unknown activation");
    return SRF_OK;
}

void resolve(const srf_config_t& c, DevCfg* g, float* min_thick) {
    memset(g, 0, sizeof(*g));
    g->warping_type = c.warping_type;
    g->grid_dist = c.grid_distribution_type;
    g->sampling_type = c.sampling_type;
    g->use_grid = c.use_grid;
    g->grid_size = c.grid_size;
    g->n_cascades = c.num_cascades;
    g->cells = c.grid_size * c.grid_size * c.grid_size;
    const float amount = 0.5f * (float)c.aabb_scale;
    g->box_min = 0.5f - amount;
    g->box_max = 0.5f + amount;
    g->box_diag = g->box_max - g->box_min;
    const float sqrt3 = 1.73205080757f;
    g->min_step = c.min_cone_stepsize > 0.f ? c.min_cone_stepsize : sqrt3 / (float)c.maximum_marching_steps;
    g->max_step = c.max_cone_stepsize > 0.f ? c.max_cone_stepsize
                : (c.use_grid ? (sqrt3 * (float)(1u << (c.num_cascades - 1)) / (float)c.grid_size) : g->min_step);
    g->cone_angle = c.cone_angle_constant;
    g->near_distance = c.near_distance;
    g->far_distance = c.far_distance;
    g->ds = 1.f / (float)c.maximum_marching_steps;
    if (c.sampling_type == SRF_SAMPLING_LOG) {
        g->g_far = srf_logf(c.far_distance);
        g->g_near = srf_logf(c.near_distance);
    } else {
        g->g_far = 1.f / c.far_distance;
        g->g_near = 1.f / c.near_distance;
    }
    g->g_diff = g->g_far - g->g_near;
    uint32_t cap = c.march_iter ? c.march_iter - 1 : 9999u;
    if (c.max_samples_per_ray && c.max_samples_per_ray < cap) cap = c.max_samples_per_ray;
    g->sample_cap = cap;
    g->step_limit = 1u << 24;
    g->snap = c.snap_to_pixel_centers_in_rendering;
    g->transmittance_keep = 1.0f - c.transmittance_threshold;
    g->density_activation = c.density_activation;
    g->rgb_activation = c.rgb_activation;
    g->train_in_linear_color = c.train_in_linear_color;
    g->field_type = c.field_type;
    *min_thick = c.min_optical_thickness;
}

// Upper bound of the samples one ray can emit, from the step-size law alone (every sample is a march
// step): used to size the sample pool per ray so that the single-pass sampler can never run out of chunks.
uint32_t ray_sample_bound(const srf_config_t& c, const DevCfg& g) {
    const double cap = g.sample_cap;
    double b = cap;
    const double ds = 1.0 / (double)c.maximum_marching_steps;
    switch (c.sampling_type) {
    case SRF_SAMPLING_ORIGINAL:       // dt >= min_step; the path inside the cube is at most sqrt(3) * edge
        if (g.min_step > 0.f) b = 1.7320508 * (double)g.box_diag / (double)g.min_step + 16.0;
        break;
    case SRF_SAMPLING_DISPARITY: {    // 1/t falls from <= 1/0.05 by ds*(1/near - 1/far) per step, then one jump to far
        const double delta = ds * ((double)g.g_near - (double)g.g_far);
        if (delta > 0.0) b = 20.0 / delta * 1.001 + 16.0;
    } break;
    case SRF_SAMPLING_LOG: {          // log t grows from >= log 0.05 by ds*(log far - log near) per step up to log far
        const double delta = ds * ((double)g.g_far - (double)g.g_near);
        if (delta > 0.0 && c.far_distance > 0.05f) b = (std::log((double)c.far_distance) - std::log(0.05)) / delta * 1.001 + 16.0;
    } break;
    default: break;
    }
    if (!(b < cap)) b = cap;
    if (b < 1.0) b = 1.0;
    return (uint32_t)std::ceil(b);
}

uint64_t shard_rows_total(const srf_view_t& v) {
    const uint32_t sr = v.shard_rows ? v.shard_rows : 8, sc = v.shard_count ? v.shard_count : 1;
    const uint32_t n_blocks = (v.height + sr - 1) / sr;
    uint64_t rows = 0;
    for (uint32_t b = v.shard_rank; b < n_blocks; b += sc) rows += std::min(sr, v.height - b * sr);
    return rows;
}

srf_status make_view(srf_ctx* ctx, const srf_view_t* view, DevView* v) {
    if (!view) return fail(ctx, SRF_ERR_ARG, "view is NULL");
    if (view->width == 0 || view->height == 0) return fail(ctx, SRF_ERR_ARG, "empty image");
    const uint32_t sc = view->shard_count ? view->shard_count : 1;
    if (view->shard_rank >= sc) return fail(ctx, SRF_ERR_ARG, "shard_rank >= shard_count");
    if (view->render_mode == SRF_MODE_NORMALS && ctx->cfg.field_type != SRF_FIELD_NETWORK)
        return fail(ctx, SRF_ERR_ARG, "render mode Normals needs the network field (it renders the density MLP's input gradient)");
    if (view->render_mode < 0 || view->render_mode > SRF_MODE_COST) return fail(ctx, SRF_ERR_ARG, "unknown render mode");
    memset(v, 0, sizeof(*v));
    memcpy(v->cam, view->camera, sizeof(v->cam));
    v->width = view->width; v->height = view->height;
    v->rw = (float)view->width; v->rh = (float)view->height;
    v->fx = v->rw * view->relative_focal_length[0];          // testbed.cu:483
    v->fy = v->rh * view->relative_focal_length[1];
    v->ppx = view->principal_point[0]; v->ppy = view->principal_point[1];
    v->spp_index = view->spp_index;
    const bool snap = ctx ? ctx->cfg.snap_to_pixel_centers_in_rendering != 0 : true;
    ld_random_pixel_offset_host(snap ? 0u : view->spp_index, &v->off_x, &v->off_y);   // common_device.h:152
    v->render_mode = view->render_mode;
    v->depth_scale = view->depth_scale;
    v->shard_rows = view->shard_rows ? view->shard_rows : 8;
    v->shard_count = sc;
    v->shard_rank = view->shard_rank;
    v->n_rays = shard_rows_total(*view) * view->width;
    return SRF_OK;
}

float host_powf(float x, float y) { return x > 0.f ? srf_expf(y * srf_logf(x)) : 0.f; }
float host_linear_to_srgb(float l) { return l < 0.0031308f ? 12.92f * l : 1.055f * host_powf(l, 0.41666f) - 0.055f; }
float host_srgb_to_linear(float s) { return s <= 0.04045f ? s / 12.92f : host_powf((s + 0.055f) / 1.055f, 2.4f); }

void make_post(const srf_post_t* post, DevPost* p) {
    srf_post_t def;
    memset(&def, 0, sizeof(def));
    def.background_color[3] = 1.f;
    if (!post) post = &def;
    p->exposure_scale = host_powf(2.0f, post->exposure);      // render_buffer.cu:155
    for (int i = 0; i < 4; ++i) p->bg[i] = post->background_color[i];
    if (post->color_space != SRF_COLOR_SRGB) for (int i = 0; i < 3; ++i) p->bg[i] = host_srgb_to_linear(p->bg[i]);   // :160-162
    p->color_space = post->color_space;
    p->tonemap_curve = post->tonemap_curve;
    p->to_srgb = post->to_srgb;
}

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (prev != dev) cudaSetDevice(dev); else prev = -1; }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// NVTX range for the lifetime of the object: names the library's stages in a timeline profiler (a few nanoseconds
// when no tool is attached).
struct NvtxRange {
    explicit NvtxRange(const char* name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange&) = delete;
    NvtxRange& operator=(const NvtxRange&) = delete;
};

srf_status ensure_ray_buffers(srf_ctx* ctx, uint64_t n_rays) {
    srf_status st;
    if ((st = ensure(ctx, ctx->ray_dir_t, n_rays * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->ray_end, n_rays)) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->counts, n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->offsets, (n_rays + 1) * sizeof(uint64_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->scan_scratch, scan_scratch_bytes(n_rays))) != SRF_OK) return st;
    return SRF_OK;
}

srf_status ensure_sample_buffers(srf_ctx* ctx, uint64_t n_samples) {
    srf_status st;
    if ((st = ensure(ctx, ctx->pos_dt, n_samples * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->sample_ray, n_samples * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->rgbs, n_samples * sizeof(float4))) != SRF_OK) return st;   // shaded samples
    return SRF_OK;
}

// Zeroes the per-frame counters.  The error word behind them is NOT cleared here: it stays set until a
// call that synchronises anyway (srf_render, srf_dump_samples, a frame with stats, srf_check_errors) has
// reported it, so a truncated frame whose caller asked for no statistics cannot pass for a good one.
cudaError_t reset_frame_counters(srf_ctx* ctx, cudaStream_t s) {
    return cudaMemsetAsync(ctx->d_counters, 0, offsetof(FrameCounters, error_flags), s);
}

// Turns the device error word into a status and clears it (the caller has synchronised `s` after copying
// the word to ctx->h_counters->error_flags).
srf_status report_error_flags(srf_ctx* ctx, uint32_t flags, cudaStream_t s) {
    if (!flags) return SRF_OK;
    cudaMemsetAsync(&ctx->d_counters->error_flags, 0, sizeof(unsigned int), s);
    if (flags & 1u) return fail(ctx, SRF_ERR_TIMEOUT, "a ray hit the march loop's iteration bound");
    if (flags & 2u) return fail(ctx, SRF_ERR_TIMEOUT, "a wait on the tensor-core commit barrier expired");
    if (flags & 4u) return fail(ctx, SRF_ERR_CAPACITY, "the sample pool ran out of chunks");
    if (flags & 8u) return fail(ctx, SRF_ERR_STATE, "the fused grid refresh met a masked cell (the grid was changed behind the context)");
    return fail(ctx, SRF_ERR_CUDA, "unknown device error flag");
}

// Reads the error word back (synchronises `s`) and reports it.
srf_status check_error_flags(srf_ctx* ctx, cudaStream_t s, uint32_t* flags_out) {
    SRF_CK(ctx, cudaMemcpyAsync(&ctx->h_counters->error_flags, &ctx->d_counters->error_flags, sizeof(unsigned int),
                                cudaMemcpyDeviceToHost, s));
    SRF_CK(ctx, cudaStreamSynchronize(s));
    const uint32_t flags = ctx->h_counters->error_flags;
    if (flags_out) *flags_out = flags;
    return report_error_flags(ctx, flags, s);
}

srf_status check_ready(srf_ctx* ctx) {
    if (ctx->cfg.field_type == SRF_FIELD_NETWORK && !ctx->have_net)
        return fail(ctx, SRF_ERR_STATE, "network parameters were not uploaded (srf_upload_network)");
    if (ctx->cfg.field_type == SRF_FIELD_BLOBS && ctx->n_blobs == 0)
        return fail(ctx, SRF_ERR_STATE, "blob scene was not uploaded (srf_upload_blobs)");
    return SRF_OK;
}

// count + scan for a view; leaves per-ray records in the context.
srf_status count_and_scan(srf_ctx* ctx, const DevView& v, cudaStream_t s) {
    srf_status st = ensure_ray_buffers(ctx, v.n_rays);
    if (st != SRF_OK) return st;
    SRF_CK(ctx, reset_frame_counters(ctx, s));
    launch_ray_count(ctx->g, v, ctx->cfg.use_grid ? ctx->bits : nullptr, (float4*)ctx->ray_dir_t.p, (uint8_t*)ctx->ray_end.p,
                     (uint32_t*)ctx->counts.p, ctx->d_counters, s);
    launch_scan((const uint32_t*)ctx->counts.p, v.n_rays, (uint64_t*)ctx->offsets.p, ctx->scan_scratch.p, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

}  // namespace

// =====================================================================================================
extern "C" {

void srf_config_default(srf_config_t* c) {
    memset(c, 0, sizeof(*c));
    c->struct_size = sizeof(*c);
    c->version = SRF_ABI_VERSION;
    c->warping_type = SRF_WARP_NGP;
    c->aabb_scale = 1;
    c->use_grid = 1;
    c->grid_size = 128;
    c->num_cascades = 1;
    c->ema_decay = 0.95f;
    c->grid_distribution_type = SRF_GRID_WARPED_EXP;
    c->maximum_marching_steps = 1024;
    c->near_distance = 0.2f;
    c->far_distance = 100.f;
    c->sampling_type = SRF_SAMPLING_ORIGINAL;
    c->snap_to_pixel_centers_in_rendering = 1;
    c->min_optical_thickness = 0.01f;
    c->transmittance_threshold = 1e-4f;
    c->n_levels = 16;
    c->n_features_per_level = 2;
    c->log2_hashmap_size = 19;
    c->base_resolution = 16;
    c->desired_resolution = 2048.f;
    c->density_activation = SRF_ACT_EXPONENTIAL;
    c->rgb_activation = SRF_ACT_LOGISTIC;
    c->field_type = SRF_FIELD_NETWORK;
    c->march_iter = 10000;
}

const char* srf_last_error(const srf_ctx* ctx) { return ctx ? ctx->err.c_str() : g_create_error.c_str(); }

srf_status srf_create(const srf_config_t* cfg, int device, srf_ctx** out) {
    if (!out) return fail(nullptr, SRF_ERR_ARG, "out is NULL");
    *out = nullptr;
    std::string why;
    srf_status st = validate(cfg, &why);
    if (st != SRF_OK) return fail(nullptr, st, why);
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        return fail(nullptr, SRF_ERR_CUDA, "no CUDA device: this library has no CPU path");
    if (device < 0 || device >= n_dev) return fail(nullptr, SRF_ERR_ARG, "device index out of range");
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, device) != cudaSuccess) return fail(nullptr, SRF_ERR_CUDA, "cudaGetDeviceProperties failed");
    if (prop.major != 10) return fail(nullptr, SRF_ERR_CUDA, "this library is built for sm_100a (B200) only");
    srf_ctx* ctx = new (std::nothrow) srf_ctx();
    if (!ctx) return fail(nullptr, SRF_ERR_CUDA, "out of host memory");
    ctx->cfg = *cfg;
    ctx->device = device;
    resolve(*cfg, &ctx->g, &ctx->min_optical_thickness);
    if (const char* e = getenv("SRF_B200_MLP")) ctx->use_tcgen05 = std::string(e) != "mma_sync";
    DeviceGuard guard(device);
    auto cleanup = [&](srf_status s) { g_create_error = ctx->err; srf_destroy(ctx); return s; };
#define CK_CREATE(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { ctx->err = std::string(#call) + ": " + cudaGetErrorString(e_); return cleanup(SRF_ERR_CUDA); } } while (0)
    const size_t total = (size_t)ctx->g.cells * ctx->g.n_cascades;
    CK_CREATE(cudaMalloc((void**)&ctx->grid, total * sizeof(float)));
    CK_CREATE(cudaMalloc((void**)&ctx->grid_current, total * sizeof(float)));
    const size_t n_partial = (ctx->g.cells + 1023) / 1024 + 1;
    CK_CREATE(cudaMalloc((void**)&ctx->partial_a, n_partial * sizeof(float)));
    CK_CREATE(cudaMalloc((void**)&ctx->partial_b, n_partial * sizeof(float)));
    CK_CREATE(cudaMalloc((void**)&ctx->mean, sizeof(float)));
    CK_CREATE(cudaMalloc((void**)&ctx->bits, total / 8));
    CK_CREATE(cudaMemset(ctx->grid, 0, total * sizeof(float)));
    CK_CREATE(cudaMemset(ctx->bits, 0, total / 8));
    CK_CREATE(cudaMemset(ctx->mean, 0, sizeof(float)));
    // staged empty-space tests apply to the configuration every shipped config uses: sinusoidal ("ERP") warp,
    // one cascade, grid laid out in warped space
    ctx->skip_capable = cfg->use_grid && cfg->num_cascades == 1 &&
                        (cfg->warping_type == SRF_WARP_ERP || cfg->warping_type == SRF_WARP_SINUSOIDAL) &&
                        (cfg->grid_distribution_type == SRF_GRID_WARPED_EXP || cfg->grid_distribution_type == SRF_GRID_WARPED_RECIPROCAL);
    if (const char* e = getenv("SRF_B200_WAVES")) {      // "0" = one pass per frame; "64,256" = march steps of the leading waves
        ctx->n_wave_budgets = 0;
        for (const char* q = e; *q && ctx->n_wave_budgets < 8;) {
            char* endp = nullptr;
            const unsigned long b = strtoul(q, &endp, 10);
            if (endp == q) break;
            if (b > 0) ctx->wave_budget[ctx->n_wave_budgets++] = (uint32_t)b;
            q = *endp ? endp + 1 : endp;
        }
    }
    if (const char* e = getenv("SRF_B200_SKIP_TABLES")) if (std::string(e) == "0") ctx->skip_capable = false;
    if (ctx->skip_capable) {
        const size_t N = cfg->grid_size;
        CK_CREATE(cudaMalloc((void**)&ctx->skip_shell, ((N + 31) / 32) * sizeof(uint32_t)));
        CK_CREATE(cudaMalloc((void**)&ctx->skip_yz, ((N * N + 31) / 32) * sizeof(uint32_t)));
        CK_CREATE(cudaMemset(ctx->skip_shell, 0, ((N + 31) / 32) * sizeof(uint32_t)));
        CK_CREATE(cudaMemset(ctx->skip_yz, 0, ((N * N + 31) / 32) * sizeof(uint32_t)));
        ctx->g.skip_shell = ctx->skip_shell;
        ctx->g.skip_yz = ctx->skip_yz;
    }
    if (cfg->field_type == SRF_FIELD_NETWORK) {
        build_net_meta(*cfg, &ctx->net);
        ctx->n_table_entries = table_entries(ctx->net);
        CK_CREATE(cudaMalloc((void**)&ctx->table, (size_t)ctx->n_table_entries * cfg->n_features_per_level * sizeof(__half)));
        if (const char* e = getenv("SRF_B200_CELL_LEVELS")) ctx->cell_levels_forced = atoi(e);
        const char* lut_env = getenv("SRF_B200_ACT_LUT");
        if (!lut_env || atoi(lut_env) != 0) {
            CK_CREATE(cudaMalloc((void**)&ctx->act_lut, 2 * 65536 * sizeof(float)));
            launch_build_activation_table(ctx->g, ctx->act_lut, 0);
            CK_CREATE(cudaDeviceSynchronize());
        }
        CK_CREATE(cudaMalloc((void**)&ctx->w_density, (64 * 32 + 16 * 64) * sizeof(__half)));
        CK_CREATE(cudaMalloc((void**)&ctx->w_rgb, (64 * 32 + 64 * 64 + 16 * 64) * sizeof(__half)));
    }
    CK_CREATE(cudaMalloc((void**)&ctx->d_counters, sizeof(FrameCounters)));
    CK_CREATE(cudaMemset(ctx->d_counters, 0, sizeof(FrameCounters)));
    CK_CREATE(cudaMalloc((void**)&ctx->d_chunk_cursor, sizeof(uint32_t)));
    CK_CREATE(cudaMalloc((void**)&ctx->d_ticket, sizeof(unsigned int)));
    CK_CREATE(cudaMemset(ctx->d_ticket, 0, sizeof(unsigned int)));
    if (const char* e = getenv("SRF_B200_FUSED_REFRESH")) ctx->fused_refresh = std::string(e) == "1";
    CK_CREATE(cudaMallocHost((void**)&ctx->h_counters, sizeof(FrameCounters)));
    for (int i = 0; i < 8; ++i) CK_CREATE(cudaEventCreate(&ctx->ev[i]));
#undef CK_CREATE
    // OccupancySampler::init (occupancy_sampler.cu:956-957): Testbed seeds its generator with 43 and
    // hands the sampler default_rng_t{rng.next_uint()}; srf_refresh_reset overrides.
    srf_refresh_reset(ctx, 43);
    *out = ctx;
    return SRF_OK;
}

void srf_destroy(srf_ctx* ctx) {
    if (!ctx) return;
    DeviceGuard guard(ctx->device);
    void* ptrs[] = {ctx->grid, ctx->grid_current, ctx->partial_a, ctx->partial_b, ctx->mean, ctx->bits, ctx->table, ctx->cell_table, ctx->act_lut,
                    ctx->w_density, ctx->w_rgb, ctx->skip_shell, ctx->skip_yz, ctx->train_flags.p, ctx->train_rank.p, ctx->loss_rgb.p, ctx->ray_sh.p, ctx->ray_ordinal.p, ctx->ray_total.p, ctx->ray_rgba.p, ctx->ray_ncomp.p, ctx->blobs, ctx->cmap, ctx->d_counters, ctx->ray_dir_t.p, ctx->ray_end.p,
                    ctx->counts.p, ctx->offsets.p, ctx->scan_scratch.p, ctx->pos_dt.p, ctx->sample_ray.p, ctx->rgbs.p,
                    ctx->img_out.p, ctx->img_accum.p, ctx->pool_pos.p, ctx->pool_shaded.p, ctx->chunk_ray.p, ctx->chunk_next.p,
                    ctx->ray_head.p, ctx->d_chunk_cursor, ctx->d_ticket};
    for (void* p : ptrs) if (p) cudaFree(p);
    if (ctx->h_counters) cudaFreeHost(ctx->h_counters);
    for (int i = 0; i < 8; ++i) if (ctx->ev[i]) cudaEventDestroy(ctx->ev[i]);
    delete ctx;
}

srf_status srf_set_timing(srf_ctx* ctx, int enabled) {
    if (!ctx) return SRF_ERR_ARG;
    ctx->timing = enabled != 0;
    return SRF_OK;
}

srf_status srf_hashgrid_layout(const srf_config_t* cfg, uint32_t* offsets, uint32_t* resolutions, float* scales) {
    if (!cfg || cfg->n_levels == 0 || cfg->n_levels > (uint32_t)kMaxLevels) return fail(nullptr, SRF_ERR_ARG, "bad n_levels");
    NetMeta net;
    build_net_meta(*cfg, &net);
    for (uint32_t l = 0; l < cfg->n_levels; ++l) {
        if (offsets) offsets[l] = net.level[l].offset;
        if (resolutions) resolutions[l] = net.level[l].res;
        if (scales) scales[l] = net.level[l].scale;
    }
    if (offsets) offsets[cfg->n_levels] = table_entries(net);
    return SRF_OK;
}

srf_status srf_upload_network(srf_ctx* ctx, const uint16_t* h_table, size_t n_table, const uint16_t* h_d, size_t n_d,
                              const uint16_t* h_c, size_t n_c) {
    if (!ctx) return SRF_ERR_ARG;
    if (ctx->cfg.field_type != SRF_FIELD_NETWORK) return fail(ctx, SRF_ERR_STATE, "context was created without a network field");
    if (!h_table || !h_d || !h_c) return fail(ctx, SRF_ERR_ARG, "NULL parameter array");
    if (n_table != (size_t)ctx->n_table_entries * ctx->cfg.n_features_per_level)
        return fail(ctx, SRF_ERR_ARG, "hash table size does not match srf_hashgrid_layout");
    if (n_d != 64 * 32 + 16 * 64) return fail(ctx, SRF_ERR_ARG, "density MLP must hold 64x32 + 16x64 halves");
    if (n_c != 64 * 32 + 64 * 64 + 16 * 64) return fail(ctx, SRF_ERR_ARG, "colour MLP must hold 64x32 + 64x64 + 16x64 halves");
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpy(ctx->table, h_table, n_table * sizeof(__half), cudaMemcpyHostToDevice));
    ctx->cell_dirty = true;
    SRF_CK(ctx, cudaMemcpy(ctx->w_density, h_d, n_d * sizeof(__half), cudaMemcpyHostToDevice));
    SRF_CK(ctx, cudaMemcpy(ctx->w_rgb, h_c, n_c * sizeof(__half), cudaMemcpyHostToDevice));
    for (int i = 0; i < 64 * 32; ++i) ctx->refresh_w.w1[i] = __half2float(__ushort_as_half(h_d[i]));
    for (int i = 0; i < 64; ++i) ctx->refresh_w.w2[i] = __half2float(__ushort_as_half(h_d[64 * 32 + i]));
    ctx->have_net = true;
    return SRF_OK;
}

srf_status srf_upload_blobs(srf_ctx* ctx, const float* h_blobs, uint32_t n_blobs, const float* h_cmap) {
    if (!ctx) return SRF_ERR_ARG;
    if (!h_blobs || !h_cmap || n_blobs == 0) return fail(ctx, SRF_ERR_ARG, "empty blob scene");
    if (n_blobs > 2048) return fail(ctx, SRF_ERR_CAPACITY, "at most 2048 blobs");
    DeviceGuard guard(ctx->device);
    if (ctx->blobs) { cudaFree(ctx->blobs); ctx->blobs = nullptr; }
    if (!ctx->cmap) SRF_CK(ctx, cudaMalloc((void**)&ctx->cmap, 9 * sizeof(float)));
    SRF_CK(ctx, cudaMalloc((void**)&ctx->blobs, (size_t)n_blobs * 5 * sizeof(float)));
    SRF_CK(ctx, cudaMemcpy(ctx->blobs, h_blobs, (size_t)n_blobs * 5 * sizeof(float), cudaMemcpyHostToDevice));
    SRF_CK(ctx, cudaMemcpy(ctx->cmap, h_cmap, 9 * sizeof(float), cudaMemcpyHostToDevice));
    ctx->n_blobs = n_blobs;
    return SRF_OK;
}

// ---- grid ------------------------------------------------------------------------------------------
srf_status srf_upload_density_grid(srf_ctx* ctx, const float* h, size_t n, void* stream) {
    if (!ctx || !h) return SRF_ERR_ARG;
    if (n != (size_t)ctx->g.cells * ctx->g.n_cascades) return fail(ctx, SRF_ERR_ARG, "density grid size mismatch");
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpyAsync(ctx->grid, h, n * sizeof(float), cudaMemcpyHostToDevice, (cudaStream_t)stream));
    SRF_CK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    bool masked = false;
    for (size_t i = 0; i < n && !masked; ++i) masked = !(h[i] > -0.01f);
    ctx->grid_may_hold_masked_cells = masked;
    return SRF_OK;
}
srf_status srf_download_density_grid(srf_ctx* ctx, float* h, size_t n, void* stream) {
    if (!ctx || !h) return SRF_ERR_ARG;
    if (n != (size_t)ctx->g.cells * ctx->g.n_cascades) return fail(ctx, SRF_ERR_ARG, "density grid size mismatch");
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpyAsync(h, ctx->grid, n * sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SRF_CK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return SRF_OK;
}
srf_status srf_upload_bitfield(srf_ctx* ctx, const uint8_t* h, size_t n, void* stream) {
    if (!ctx || !h) return SRF_ERR_ARG;
    if (n != (size_t)ctx->g.cells * ctx->g.n_cascades / 8) return fail(ctx, SRF_ERR_ARG, "bitfield size mismatch");
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpyAsync(ctx->bits, h, n, cudaMemcpyHostToDevice, (cudaStream_t)stream));
    if (ctx->skip_capable) launch_build_skip_tables(ctx->g, ctx->bits, ctx->skip_shell, ctx->skip_yz, (cudaStream_t)stream);
    SRF_CK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return SRF_OK;
}
srf_status srf_download_bitfield(srf_ctx* ctx, uint8_t* h, size_t n, void* stream) {
    if (!ctx || !h) return SRF_ERR_ARG;
    if (n != (size_t)ctx->g.cells * ctx->g.n_cascades / 8) return fail(ctx, SRF_ERR_ARG, "bitfield size mismatch");
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpyAsync(h, ctx->bits, n, cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SRF_CK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return SRF_OK;
}
srf_status srf_download_grid_mean(srf_ctx* ctx, float* h_mean, void* stream) {
    if (!ctx || !h_mean) return SRF_ERR_ARG;
    DeviceGuard guard(ctx->device);
    SRF_CK(ctx, cudaMemcpyAsync(h_mean, ctx->mean, sizeof(float), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    SRF_CK(ctx, cudaStreamSynchronize((cudaStream_t)stream));
    return SRF_OK;
}

srf_status srf_update_grid_bitfield(srf_ctx* ctx, void* stream) {
    if (!ctx) return SRF_ERR_ARG;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t total = ctx->g.cells * ctx->g.n_cascades;
    launch_decay_and_mean(ctx->grid, ctx->grid_current, total, ctx->g.cells, 0.f, 0, ctx->partial_a, ctx->partial_b, ctx->mean, s);
    launch_grid_to_bitfield(ctx->g, ctx->grid, ctx->bits, ctx->mean, ctx->min_optical_thickness, s);
    if (ctx->skip_capable) launch_build_skip_tables(ctx->g, ctx->bits, ctx->skip_shell, ctx->skip_yz, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

static void host_pcg_step(RefreshRng& r) { r.state = r.state * 0x5851f42d4c957f2dULL + r.inc; }
static void host_pcg_advance(RefreshRng& r, uint64_t delta) {
    uint64_t cur_mult = 0x5851f42d4c957f2dULL, cur_plus = r.inc, acc_mult = 1u, acc_plus = 0u;
    while (delta > 0) {
        if (delta & 1) { acc_mult *= cur_mult; acc_plus = acc_plus * cur_mult + cur_plus; }
        cur_plus = (cur_mult + 1) * cur_plus;
        cur_mult *= cur_mult;
        delta >>= 1;
    }
    r.state = acc_mult * r.state + acc_plus;
}

srf_status srf_refresh_reset(srf_ctx* ctx, uint64_t seed) {
    if (!ctx) return SRF_ERR_ARG;
    // PCG32 seeding (O'Neill): state = 0, inc = (seq << 1) | 1 with seq = 1, step, add the seed, step.
    ctx->rng.state = 0;
    ctx->rng.inc = (1ull << 1) | 1ull;
    host_pcg_step(ctx->rng);
    ctx->rng.state += seed;
    host_pcg_step(ctx->rng);
    ctx->refresh_step = 0;
    return SRF_OK;
}

srf_status srf_refresh_grid(srf_ctx* ctx, uint32_t training_step, void* stream) {
    NvtxRange nvtx_range("srf_refresh_grid");
    if (!ctx) return SRF_ERR_ARG;
    if (ctx->cfg.field_type != SRF_FIELD_NETWORK) return fail(ctx, SRF_ERR_STATE, "the grid refresh queries the network field");
    srf_status st = check_ready(ctx);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t total = ctx->g.cells * ctx->g.n_cascades;
    const uint32_t n_uniform = training_step >= 256 ? total / 4 : total;          // testbed.cu:206
    const uint32_t n_nonuniform = training_step >= 256 ? total / 4 : 0;           // testbed.cu:207
    // One kernel for sample -> encode -> MLP -> splat -> max-decay -> mean, one for the bits, where the cell map is a
    // bijection with a single writer per cell: every cell sampled once, one cascade, power-of-two cell count, no cell
    // masked as never seen (a masked cell's sample is redirected to another cell).
    const bool fused = ctx->fused_refresh && n_nonuniform == 0 && ctx->g.n_cascades == 1 && (ctx->g.cells & (ctx->g.cells - 1u)) == 0 &&
                       !ctx->grid_may_hold_masked_cells;
    if (fused) {
        launch_refresh_fused(ctx->g, ctx->net, ctx->table, ctx->refresh_w, ctx->grid, ctx->refresh_step, ctx->rng, (float)-0.01,
                             ctx->cfg.aabb_scale, ctx->cfg.ema_decay, ctx->partial_a, ctx->partial_b, ctx->mean, ctx->d_ticket, ctx->bits,
                             ctx->min_optical_thickness, ctx->skip_capable ? ctx->skip_shell : nullptr,
                             ctx->skip_capable ? ctx->skip_yz : nullptr, &ctx->d_counters->error_flags, s);
        host_pcg_advance(ctx->rng, 1ull << 32);                                    // rng.advance() after each of the two
        host_pcg_advance(ctx->rng, 1ull << 32);                                    // sampling launches, :1009,1028
        ++ctx->refresh_step;
        SRF_CK(ctx, cudaGetLastError());
        return SRF_OK;
    }
    SRF_CK(ctx, cudaMemsetAsync(ctx->grid_current, 0, (size_t)total * sizeof(float), s));   // occupancy_sampler.cu:1039
    launch_refresh_sample(ctx->g, ctx->net, ctx->table, ctx->refresh_w, ctx->grid, ctx->grid_current, n_uniform,
                          ctx->refresh_step, ctx->rng, (float)-0.01, ctx->cfg.aabb_scale, s);
    host_pcg_advance(ctx->rng, 1ull << 32);                                        // rng.advance(), :1009
    launch_refresh_sample(ctx->g, ctx->net, ctx->table, ctx->refresh_w, ctx->grid, ctx->grid_current, n_nonuniform,
                          ctx->refresh_step, ctx->rng, ctx->min_optical_thickness, ctx->cfg.aabb_scale, s);
    host_pcg_advance(ctx->rng, 1ull << 32);                                        // :1028
    launch_decay_and_mean(ctx->grid, ctx->grid_current, total, ctx->g.cells, ctx->cfg.ema_decay, 1, ctx->partial_a,
                          ctx->partial_b, ctx->mean, s);
    ++ctx->refresh_step;                                                            // :1060
    launch_grid_to_bitfield(ctx->g, ctx->grid, ctx->bits, ctx->mean, ctx->min_optical_thickness, s);
    if (ctx->skip_capable) launch_build_skip_tables(ctx->g, ctx->bits, ctx->skip_shell, ctx->skip_yz, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

// ---- training-side sampler -------------------------------------------------------------------------

static srf_status make_train_views(srf_ctx* ctx, const srf_train_views_t* in, bool need_images, TrainViews* tv) {
    if (!in) return fail(ctx, SRF_ERR_ARG, "training views are required");
    if (in->n_images == 0 || in->width <= 0 || in->height <= 0) return fail(ctx, SRF_ERR_ARG, "training views: empty image set");
    if (!(in->focal_length[0] > 0.f) || !(in->focal_length[1] > 0.f)) return fail(ctx, SRF_ERR_ARG, "training views: focal length must be positive");
    if (!in->d_xforms) return fail(ctx, SRF_ERR_ARG, "training views: camera matrices missing");
    if (need_images && !in->d_images) return fail(ctx, SRF_ERR_ARG, "training views: images missing");
    tv->n_images = in->n_images; tv->width = in->width; tv->height = in->height;
    tv->focal_x = in->focal_length[0]; tv->focal_y = in->focal_length[1];
    tv->pp_x = in->principal_point[0]; tv->pp_y = in->principal_point[1];
    tv->xforms = in->d_xforms;
    tv->images = reinterpret_cast<const __half*>(in->d_images);
    tv->sampling_probability = reinterpret_cast<const __half*>(in->d_sampling_probability);
    return SRF_OK;
}

srf_status srf_sampler_init(srf_ctx* ctx, const srf_train_views_t* views, int init_grid_with_mask, uint64_t rng_seed, void* stream) {
    if (!ctx) return SRF_ERR_ARG;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    srf_refresh_reset(ctx, rng_seed);
    const size_t total = (size_t)ctx->g.cells * ctx->g.n_cascades;
    if (ctx->cfg.use_grid && init_grid_with_mask && ctx->cfg.warping_type == SRF_WARP_NGP) {
        TrainViews tv;
        srf_status st = make_train_views(ctx, views, false, &tv);
        if (st != SRF_OK) return st;
        launch_mark_untrained(ctx->g, ctx->cfg.aabb_scale, tv, ctx->grid, s);
        SRF_CK(ctx, cudaGetLastError());
        ctx->grid_may_hold_masked_cells = true;
    } else {
        SRF_CK(ctx, cudaMemsetAsync(ctx->grid, 0, total * sizeof(float), s));
        ctx->grid_may_hold_masked_cells = false;
    }
    return SRF_OK;
}

srf_status srf_sample_training_rays(srf_ctx* ctx, const srf_train_views_t* views, uint32_t n_rays, uint32_t n_rays_shift,
                                    uint32_t n_coords, uint64_t rng_state, uint64_t rng_inc, int snap_to_pixel_centers,
                                    uint32_t* d_ray_counter, uint32_t* d_numsteps_counter, float* d_rays, float* d_rays_rgba,
                                    uint32_t* d_numsteps, float* d_coords, void* stream) {
    NvtxRange nvtx_range("srf_sample_training_rays");
    if (!ctx || !d_ray_counter || !d_numsteps_counter || !d_rays || !d_rays_rgba || !d_numsteps || !d_coords) return SRF_ERR_ARG;
    if (n_rays == 0) return fail(ctx, SRF_ERR_ARG, "n_rays must be positive");
    TrainViews tv;
    srf_status st = make_train_views(ctx, views, true, &tv);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    if ((st = ensure(ctx, ctx->counts, (size_t)n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->train_flags, (size_t)n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->offsets, ((size_t)n_rays + 1) * sizeof(uint64_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->train_rank, ((size_t)n_rays + 1) * sizeof(uint64_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->scan_scratch, scan_scratch_bytes(n_rays))) != SRF_OK) return st;
    uint32_t* counts = (uint32_t*)ctx->counts.p;
    uint32_t* flags = (uint32_t*)ctx->train_flags.p;
    uint64_t* offsets = (uint64_t*)ctx->offsets.p;
    uint64_t* rank = (uint64_t*)ctx->train_rank.p;
    const RefreshRng rng = {rng_state, rng_inc};
    launch_train_count(ctx->g, tv, ctx->bits, n_rays, n_rays_shift, ctx->cfg.maximum_marching_steps, rng, snap_to_pixel_centers,
                       counts, flags, s);
    launch_scan(counts, n_rays, offsets, ctx->scan_scratch.p, s);
    launch_scan(flags, n_rays, rank, ctx->scan_scratch.p, s);
    SRF_CK(ctx, cudaMemsetAsync(d_ray_counter, 0, sizeof(uint32_t), s));
    launch_train_emit(ctx->g, tv, ctx->bits, n_rays, n_rays_shift, n_coords, rng, snap_to_pixel_centers, counts, offsets, rank,
                      d_ray_counter, d_numsteps_counter, d_rays, d_rays_rgba, d_numsteps, d_coords, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

static uint32_t host_pcg_next_uint(RefreshRng& r) {
    const uint64_t old = r.state;
    r.state = old * 0x5851f42d4c957f2dULL + r.inc;
    const uint32_t xorshifted = (uint32_t)(((old >> 18u) ^ old) >> 27u);
    const uint32_t rot = (uint32_t)(old >> 59u);
    return (xorshifted >> rot) | (xorshifted << ((~rot + 1u) & 31));
}
static float host_pcg_next_float(RefreshRng& r) {
    const uint32_t u = (host_pcg_next_uint(r) >> 9) | 0x3f800000u;
    float f;
    memcpy(&f, &u, 4);
    return f - 1.0f;
}

srf_status srf_volume_rendering_loss(srf_ctx* ctx, const srf_loss_params_t* p, const uint32_t* d_n_rays_counter,
                                     uint32_t* d_ray_coord_indices, const float* d_rays_rgba, const float* d_coords,
                                     const uint16_t* d_network_output, float* d_compacted_coords, uint32_t* d_n_compacted_counter,
                                     uint16_t* d_dloss_doutput, float* d_loss_output, float* d_reg_distortion, void* stream) {
    NvtxRange nvtx_range("srf_volume_rendering_loss");
    if (!ctx || !p || !d_n_rays_counter || !d_ray_coord_indices || !d_rays_rgba || !d_coords || !d_network_output ||
        !d_compacted_coords || !d_n_compacted_counter || !d_dloss_doutput)
        return SRF_ERR_ARG;
    if (p->n_rays == 0) return fail(ctx, SRF_ERR_ARG, "n_rays must be positive");
    if (p->padded_output_width < 4) return fail(ctx, SRF_ERR_ARG, "padded_output_width must be at least 4");
    if (p->loss_type < SRF_LOSS_L2 || p->loss_type > SRF_LOSS_RELATIVE_L2) return fail(ctx, SRF_ERR_ARG, "Unknown loss type.");
    if (p->regularization_type != SRF_REG_NONE && p->regularization_type != SRF_REG_DISTORTION)
        return fail(ctx, SRF_ERR_ARG, "Unknown regularization type.");
    if (p->regularization_type == SRF_REG_DISTORTION && !d_reg_distortion)
        return fail(ctx, SRF_ERR_ARG, "distortion regularisation needs d_reg_distortion");
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    LossParams lp;
    lp.n_rays = p->n_rays; lp.n_max_compacted_coords = p->n_max_compacted_coords; lp.padded_output_width = p->padded_output_width;
    lp.loss_type = p->loss_type; lp.color_space = p->color_space; lp.loss_scale = p->loss_scale;
    lp.transmittance_threshold = ctx->cfg.transmittance_threshold;
    lp.min_optical_thickness = ctx->min_optical_thickness;
    float bg[3] = {p->background_color[0], p->background_color[1], p->background_color[2]};
    if (p->train_with_random_bg_color) {                     // ray_marcher.cu:83-85: the same three draws for every ray
        RefreshRng r = {p->rng_state, p->rng_inc};
        for (int c = 0; c < 3; ++c) bg[c] = host_pcg_next_float(r);
    }
    for (int c = 0; c < 3; ++c) {
        lp.bg_linear[c] = host_srgb_to_linear(bg[c]);         // :86
        lp.bg_final[c] = ctx->cfg.train_in_linear_color ? lp.bg_linear[c] : host_linear_to_srgb(lp.bg_linear[c]);   // :95-100
    }
    if (!ctx->cfg.train_in_linear_color && p->color_space != SRF_COLOR_LINEAR && p->color_space != SRF_COLOR_SRGB)
        for (int c = 0; c < 3; ++c) lp.bg_final[c] = lp.bg_linear[c];
    const uint32_t n = p->n_rays;
    srf_status st;
    if ((st = ensure(ctx, ctx->counts, (size_t)n * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->offsets, ((size_t)n + 1) * sizeof(uint64_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->loss_rgb, (size_t)n * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->scan_scratch, scan_scratch_bytes(n))) != SRF_OK) return st;
    uint32_t* consumed = (uint32_t*)ctx->counts.p;
    uint64_t* bases = (uint64_t*)ctx->offsets.p;
    launch_loss_forward(ctx->g, lp, d_n_rays_counter, d_ray_coord_indices, d_coords, (const uint2*)d_network_output, consumed,
                        (float4*)ctx->loss_rgb.p, n, s);
    launch_scan(consumed, n, bases, ctx->scan_scratch.p, s);
    launch_loss_backward(ctx->g, lp, d_n_rays_counter, d_ray_coord_indices, d_coords, (const uint2*)d_network_output,
                         (const float4*)d_rays_rgba, consumed, bases, (const float4*)ctx->loss_rgb.p, ctx->mean, d_compacted_coords,
                         d_n_compacted_counter, (__half*)d_dloss_doutput, d_loss_output,
                         p->regularization_type == SRF_REG_DISTORTION ? d_reg_distortion : nullptr, n, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

// ---- stages ------------------------------------------------------------------------------------------
srf_status srf_shard_ray_count(const srf_view_t* view, uint64_t* n_rays) {
    if (!view || !n_rays) return SRF_ERR_ARG;
    *n_rays = shard_rows_total(*view) * view->width;
    return SRF_OK;
}

srf_status srf_generate_rays(srf_ctx* ctx, const srf_view_t* view, float* d_dir, float* d_t, uint8_t* d_alive,
                             uint32_t* d_pixel, void* stream) {
    if (!ctx) return SRF_ERR_ARG;
    DevView v;
    srf_status st = make_view(ctx, view, &v);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    launch_generate_rays(ctx->g, v, ctx->cfg.use_grid ? ctx->bits : nullptr, d_dir, d_t, d_alive, d_pixel, (cudaStream_t)stream);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

srf_status srf_sample_count(srf_ctx* ctx, const srf_view_t* view, uint32_t* d_counts, void* stream) {
    if (!ctx || !d_counts) return SRF_ERR_ARG;
    DevView v;
    srf_status st = make_view(ctx, view, &v);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    if ((st = ensure_ray_buffers(ctx, v.n_rays)) != SRF_OK) return st;
    SRF_CK(ctx, reset_frame_counters(ctx, s));
    launch_ray_count(ctx->g, v, ctx->cfg.use_grid ? ctx->bits : nullptr, (float4*)ctx->ray_dir_t.p, (uint8_t*)ctx->ray_end.p,
                     d_counts, ctx->d_counters, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

srf_status srf_sample_offsets(srf_ctx* ctx, const uint32_t* d_counts, uint64_t n_rays, uint64_t* d_offsets, void* stream) {
    if (!ctx || !d_counts || !d_offsets) return SRF_ERR_ARG;
    DeviceGuard guard(ctx->device);
    srf_status st = ensure(ctx, ctx->scan_scratch, scan_scratch_bytes(n_rays));
    if (st != SRF_OK) return st;
    launch_scan(d_counts, n_rays, d_offsets, ctx->scan_scratch.p, (cudaStream_t)stream);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

srf_status srf_sample_emit(srf_ctx* ctx, const srf_view_t* view, const uint64_t* d_offsets, uint64_t capacity,
                           float* d_coords, uint32_t* d_ordinal, uint32_t* d_cell, void* stream) {
    if (!ctx || !d_offsets || !d_coords) return SRF_ERR_ARG;
    DevView v;
    srf_status st = make_view(ctx, view, &v);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    if (ctx->ray_dir_t.bytes < v.n_rays * sizeof(float4))
        return fail(ctx, SRF_ERR_STATE, "srf_sample_emit must follow srf_sample_count of the same view");
    uint64_t total = 0;
    SRF_CK(ctx, cudaMemcpyAsync(&total, d_offsets + v.n_rays, sizeof(uint64_t), cudaMemcpyDeviceToHost, s));
    SRF_CK(ctx, cudaStreamSynchronize(s));
    if (total > capacity) return fail(ctx, SRF_ERR_CAPACITY, "coordinate buffer too small for the samples of this view");
    launch_ray_emit(ctx->g, v, ctx->cfg.use_grid ? ctx->bits : nullptr, (const float4*)ctx->ray_dir_t.p, d_offsets, 0, v.n_rays,
                    nullptr, nullptr, d_coords, d_ordinal, d_cell, ctx->d_counters, s);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

// Cell-major copies of as many leading levels as the budget allows, (re)built on `stream` when the table changed.
static srf_status ensure_cell_tables(srf_ctx* ctx, cudaStream_t stream) {
    int want = 0;
    if (ctx->use_tcgen05) {
        for (int l = 1; l <= (int)ctx->net.n_levels; ++l) {
            if (ctx->cell_levels_forced >= 0 ? l > ctx->cell_levels_forced
                                             : cell_table_units(ctx->net, l, nullptr) * sizeof(uint4) > ctx->cell_budget) break;
            want = l;
        }
    }
    if (want != ctx->n_cell_levels) {
        if (ctx->cell_table) { SRF_CK(ctx, cudaFree(ctx->cell_table)); ctx->cell_table = nullptr; }
        ctx->n_cell_levels = 0;
        // The copies are an optimisation: when the device cannot spare the memory, take fewer levels (or none)
        // instead of failing the frame.
        const int asked = want;
        while (want > 0) {
            if (cudaMalloc((void**)&ctx->cell_table, cell_table_units(ctx->net, want, nullptr) * sizeof(uint4)) == cudaSuccess) break;
            cudaGetLastError();
            ctx->cell_table = nullptr;
            --want;
        }
        if (want < asked) {                       // remember what fitted, so that later frames do not try again
            ctx->cell_budget = cell_table_units(ctx->net, want, nullptr) * sizeof(uint4);
            if (ctx->cell_levels_forced >= 0) ctx->cell_levels_forced = want;
        }
        if (want > 0) {
            ctx->n_cell_levels = want;
            ctx->cell_dirty = true;
        }
    }
    if (ctx->cell_dirty && ctx->n_cell_levels > 0) {
        launch_build_cell_tables(ctx->net, ctx->table, ctx->n_cell_levels, ctx->cell_table, stream);
        SRF_CK(ctx, cudaGetLastError());
    }
    ctx->cell_dirty = false;
    return SRF_OK;
}

srf_status srf_set_cell_table_budget(srf_ctx* ctx, uint64_t bytes) {
    if (!ctx) return SRF_ERR_ARG;
    ctx->cell_budget = bytes;
    return SRF_OK;
}

srf_status srf_network_inference(srf_ctx* ctx, const float* d_coords, uint64_t n, uint16_t* d_rgbsigma, void* stream) {
    if (!ctx || (!d_coords && n) || (!d_rgbsigma && n)) return SRF_ERR_ARG;
    if (ctx->cfg.field_type != SRF_FIELD_NETWORK) return fail(ctx, SRF_ERR_STATE, "context has no network field");
    srf_status st = check_ready(ctx);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    // The cell-major level copies are used when a frame has built them since the last upload; this entry point does not
    // build them itself (a trainer that uploads parameters before every batch would pay the rebuild each time).
    if (ctx->use_tcgen05)
        launch_field_network_tc(ctx->net, ctx->table, ctx->w_density, ctx->w_rgb, nullptr, nullptr, nullptr, d_coords, n,
                                (uint2*)d_rgbsigma, nullptr, nullptr, nullptr, &ctx->d_counters->error_flags, (cudaStream_t)stream,
                                nullptr, 0, nullptr, ctx->cell_table, ctx->cell_dirty ? 0 : ctx->n_cell_levels);
    else
        launch_field_network(ctx->net, ctx->table, ctx->w_density, ctx->w_rgb, nullptr, nullptr, nullptr, d_coords, n,
                             (uint2*)d_rgbsigma, nullptr, nullptr, nullptr, (cudaStream_t)stream);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

srf_status srf_network_density(srf_ctx* ctx, const float* d_positions, uint64_t n, uint16_t* d_out, void* stream) {
    if (!ctx || (!d_positions && n) || (!d_out && n)) return SRF_ERR_ARG;
    if (ctx->cfg.field_type != SRF_FIELD_NETWORK) return fail(ctx, SRF_ERR_STATE, "context has no network field");
    srf_status st = check_ready(ctx);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    launch_field_density(ctx->net, ctx->table, ctx->w_density, d_positions, 3, n, (__half*)d_out, (cudaStream_t)stream);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

srf_status srf_volume_rendering(srf_ctx* ctx, const srf_view_t* view, const uint64_t* d_offsets, uint64_t n_rays,
                                const float* d_coords, const uint16_t* d_rgbsigma, float* d_rgba, uint32_t* d_n_composited,
                                void* stream) {
    if (!ctx || !d_offsets || !d_coords || !d_rgbsigma) return SRF_ERR_ARG;
    DevView v;
    srf_status st = make_view(ctx, view, &v);
    if (st != SRF_OK) return st;
    DeviceGuard guard(ctx->device);
    launch_composite_coords(ctx->g, v, d_offsets, n_rays, d_coords, (const uint2*)d_rgbsigma, (float4*)d_rgba, d_n_composited,
                            (cudaStream_t)stream);
    SRF_CK(ctx, cudaGetLastError());
    return SRF_OK;
}

// ---- frames -------------------------------------------------------------------------------------------
static srf_status render_frame_impl(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, float* d_out, float* d_accum,
                                    float* d_rgba_raw, uint32_t* d_n_samples, srf_frame_stats_t* stats, void* stream,
                                    int out_by_pixel) {
    NvtxRange nvtx_range("srf_render_frame");
    if (!ctx) return SRF_ERR_ARG;
    srf_status st = check_ready(ctx);
    if (st != SRF_OK) return st;
    DevView v;
    if ((st = make_view(ctx, view, &v)) != SRF_OK) return st;
    v.out_by_pixel = out_by_pixel;
    DevPost dp;
    make_post(post, &dp);
    DeviceGuard guard(ctx->device);
    cudaStream_t s = (cudaStream_t)stream;
    if (stats) memset(stats, 0, sizeof(*stats));
    if (v.n_rays == 0) return SRF_OK;
    const bool tm = ctx->timing && stats;
    float ms_sampler = 0.f, ms_field = 0.f, ms_comp = 0.f;
    auto lap = [&](int a, int b, float* acc) {
        float ms = 0.f;
        cudaEventSynchronize(ctx->ev[b]);
        cudaEventElapsedTime(&ms, ctx->ev[a], ctx->ev[b]);
        *acc += ms;
    };

    // Sample pool: every ray of a batch is given room for the most samples its step-size law allows, so the
    // single-pass sampler cannot run out of chunks and nothing has to be read back before the field runs.
    const uint32_t bound = ray_sample_bound(ctx->cfg, ctx->g);
    const uint64_t per_ray_slots = ((uint64_t)bound + kChunkSamples - 1) / kChunkSamples * kChunkSamples + kChunkSamples;
    const uint64_t limit = ctx->reserve_samples ? ctx->reserve_samples : kAutoSampleCapacity;
    uint64_t rays_per_batch = limit / per_ray_slots;
    if (rays_per_batch == 0) return fail(ctx, SRF_ERR_CAPACITY, "srf_reserve limit is smaller than the samples one ray may emit");
    if (rays_per_batch >= v.n_rays) {
        rays_per_batch = v.n_rays;
    } else {
        // equal batches (no small tail batch), in multiples of 128 rays
        if (rays_per_batch > 128) rays_per_batch -= rays_per_batch % 128;
        const uint64_t n_b = (v.n_rays + rays_per_batch - 1) / rays_per_batch;
        const uint64_t even = ((v.n_rays + n_b - 1) / n_b + 127) / 128 * 128;
        if (even < rays_per_batch) rays_per_batch = even;
    }
    const uint64_t pool_slots = rays_per_batch * per_ray_slots;
    if (pool_slots / kChunkSamples >= 0xffffffffull) return fail(ctx, SRF_ERR_CAPACITY, "sample pool exceeds 2^32 chunks");
    const uint32_t pool_chunks = (uint32_t)(pool_slots / kChunkSamples);
    if ((st = ensure(ctx, ctx->ray_dir_t, v.n_rays * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->ray_end, v.n_rays)) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->counts, v.n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->ray_head, v.n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->pool_pos, pool_slots * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->pool_shaded, pool_slots * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->chunk_ray, (size_t)pool_chunks * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->chunk_next, (size_t)pool_chunks * sizeof(uint32_t))) != SRF_OK) return st;
    SRF_CK(ctx, reset_frame_counters(ctx, s));

    const bool blobs = ctx->cfg.field_type == SRF_FIELD_BLOBS;
    const uint8_t* bits = ctx->cfg.use_grid ? ctx->bits : nullptr;
    const bool sh_per_ray = !blobs && ctx->use_tcgen05 && v.render_mode != SRF_MODE_NORMALS;
    if (sh_per_ray && (st = ensure(ctx, ctx->ray_sh, v.n_rays * 2 * sizeof(uint4))) != SRF_OK) return st;
    if (!blobs && (st = ensure_cell_tables(ctx, s)) != SRF_OK) return st;
    uint32_t n_batches = 0;
    // Waves: the leading waves take every ray a limited number of march steps further, so that rays the compositor
    // finishes early never have the rest of their samples generated or evaluated; the last wave is unlimited.  A
    // caller who asks for the sampler's per-ray counts gets the whole march in one wave.
    uint32_t budgets[9];                       // pause_at of each wave: cumulative march steps
    uint32_t n_waves = 0;
    if (!d_n_samples) {
        uint64_t total_steps = 0;
        for (uint32_t k = 0; k < ctx->n_wave_budgets; ++k) {
            total_steps += ctx->wave_budget[k];
            if (total_steps < ctx->g.step_limit) budgets[n_waves++] = (uint32_t)total_steps;
        }
    }
    budgets[n_waves++] = 0xffffffffu;
    const bool waves = n_waves > 1;
    if (waves) {
        if ((st = ensure(ctx, ctx->ray_ordinal, v.n_rays * sizeof(uint32_t))) != SRF_OK) return st;
        if ((st = ensure(ctx, ctx->ray_total, v.n_rays * sizeof(uint32_t))) != SRF_OK) return st;
        if ((st = ensure(ctx, ctx->ray_rgba, v.n_rays * sizeof(float4))) != SRF_OK) return st;
        if ((st = ensure(ctx, ctx->ray_ncomp, v.n_rays * sizeof(uint32_t))) != SRF_OK) return st;
    }
    for (uint64_t r0 = 0; r0 < v.n_rays; r0 += rays_per_batch) {
        const uint64_t r1 = std::min<uint64_t>(r0 + rays_per_batch, v.n_rays);
        for (uint32_t wave = 0; wave < n_waves; ++wave) {
            SRF_CK(ctx, cudaMemsetAsync(ctx->d_chunk_cursor, 0, sizeof(uint32_t), s));
            if (tm) cudaEventRecord(ctx->ev[2], s);
            nvtxRangePushA("srf sampler");
            launch_march_paged(ctx->g, v, bits, r0, r1, (float4*)ctx->pool_pos.p, (uint32_t*)ctx->chunk_ray.p,
                               (uint32_t*)ctx->chunk_next.p, pool_chunks, ctx->d_chunk_cursor, (float4*)ctx->ray_dir_t.p,
                               (uint8_t*)ctx->ray_end.p, (uint32_t*)ctx->counts.p, (uint32_t*)ctx->ray_head.p, ctx->d_counters, s,
                               wave, budgets[wave], waves ? (uint32_t*)ctx->ray_ordinal.p : nullptr,
                               waves ? (uint32_t*)ctx->ray_total.p : nullptr, sh_per_ray ? (uint4*)ctx->ray_sh.p : nullptr);
            nvtxRangePop();
            if (tm) cudaEventRecord(ctx->ev[3], s);
            nvtxRangePushA("srf field");
            if (blobs)
                launch_field_blobs(ctx->g, v, ctx->blobs, ctx->n_blobs, ctx->cmap, (const float4*)ctx->pool_pos.p, 0,
                                   (float4*)ctx->pool_shaded.p, s, ctx->d_chunk_cursor);
            else if (v.render_mode == SRF_MODE_NORMALS)
                launch_field_normals(ctx->g, ctx->net, ctx->table, ctx->w_density, (const float4*)ctx->pool_pos.p, 0,
                                     (float4*)ctx->pool_shaded.p, s, ctx->d_chunk_cursor);
            else if (ctx->use_tcgen05)
                launch_field_network_tc(ctx->net, ctx->table, ctx->w_density, ctx->w_rgb, (const float4*)ctx->pool_pos.p,
                                        (const uint32_t*)ctx->chunk_ray.p, (const float4*)ctx->ray_dir_t.p, nullptr, 0, nullptr,
                                        (float4*)ctx->pool_shaded.p, &ctx->g, &v, &ctx->d_counters->error_flags, s,
                                        ctx->d_chunk_cursor, kChunkShift, sh_per_ray ? (const uint4*)ctx->ray_sh.p : nullptr,
                                        ctx->cell_table, ctx->n_cell_levels, ctx->act_lut);
            else
                launch_field_network(ctx->net, ctx->table, ctx->w_density, ctx->w_rgb, (const float4*)ctx->pool_pos.p,
                                     (const uint32_t*)ctx->chunk_ray.p, (const float4*)ctx->ray_dir_t.p, nullptr, 0, nullptr,
                                     (float4*)ctx->pool_shaded.p, &ctx->g, &v, s, ctx->d_chunk_cursor, kChunkShift);
            nvtxRangePop();
            if (tm) cudaEventRecord(ctx->ev[4], s);
            NvtxRange composite_range("srf composite");
            launch_composite_paged(ctx->g, v, dp, r0, r1, (const uint32_t*)ctx->ray_head.p, (const uint32_t*)ctx->counts.p,
                                   (const uint32_t*)ctx->chunk_next.p, (const float4*)ctx->pool_shaded.p, (uint8_t*)ctx->ray_end.p,
                                   (float4*)d_out, (float4*)d_accum, (float4*)d_rgba_raw, nullptr, ctx->d_counters, s, wave,
                                   waves ? (float4*)ctx->ray_rgba.p : nullptr, waves ? (uint32_t*)ctx->ray_ncomp.p : nullptr);
            if (tm) {
                cudaEventRecord(ctx->ev[5], s);
                lap(2, 3, &ms_sampler); lap(3, 4, &ms_field); lap(4, 5, &ms_comp);
            }
        }
        ++n_batches;
    }
    if (d_n_samples) SRF_CK(ctx, cudaMemcpyAsync(d_n_samples, ctx->counts.p, v.n_rays * sizeof(uint32_t), cudaMemcpyDeviceToDevice, s));
    SRF_CK(ctx, cudaGetLastError());
    if (stats) {
        SRF_CK(ctx, cudaMemcpyAsync(ctx->h_counters, ctx->d_counters, sizeof(FrameCounters), cudaMemcpyDeviceToHost, s));
        SRF_CK(ctx, cudaStreamSynchronize(s));
        stats->n_rays = v.n_rays;
        stats->n_rays_alive = ctx->h_counters->n_alive;
        stats->n_march_steps = ctx->h_counters->n_march_steps;
        stats->n_samples = ctx->h_counters->n_samples;
        stats->n_samples_composited = ctx->h_counters->n_composited;
        stats->n_rays_hit = ctx->h_counters->n_hit;
        stats->n_batches = n_batches;
        stats->n_waves = n_waves;
        stats->error_flags = ctx->h_counters->error_flags;
        stats->ms_sampler = ms_sampler; stats->ms_field = ms_field; stats->ms_composite = ms_comp; stats->ms_post = 0.f;
        if ((st = report_error_flags(ctx, stats->error_flags, s)) != SRF_OK) return st;
    }
    return SRF_OK;
}

srf_status srf_set_wave_schedule(srf_ctx* ctx, const uint32_t* steps, uint32_t n) {
    if (!ctx) return SRF_ERR_ARG;
    if (n > 8) return fail(ctx, SRF_ERR_ARG, "at most 8 leading waves");
    if (n && !steps) return fail(ctx, SRF_ERR_ARG, "steps is NULL");
    for (uint32_t k = 0; k < n; ++k)
        if (steps[k] == 0) return fail(ctx, SRF_ERR_ARG, "a wave must advance by at least one march step");
    for (uint32_t k = 0; k < n; ++k) ctx->wave_budget[k] = steps[k];
    ctx->n_wave_budgets = n;
    return SRF_OK;
}

srf_status srf_render_frame(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, float* d_out, float* d_accum,
                            float* d_rgba_raw, uint32_t* d_n_samples, srf_frame_stats_t* stats, void* stream) {
    return render_frame_impl(ctx, view, post, d_out, d_accum, d_rgba_raw, d_n_samples, stats, stream, 0);
}

srf_status srf_render_frame_scatter(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, float* d_image,
                                    float* d_accum, srf_frame_stats_t* stats, void* stream) {
    if (!d_image) return fail(ctx, SRF_ERR_ARG, "d_image is NULL");
    return render_frame_impl(ctx, view, post, d_image, d_accum, nullptr, nullptr, stats, stream, 1);
}

srf_status srf_render(srf_ctx* ctx, const srf_view_t* view, const srf_post_t* post, uint32_t spp, float* h_image,
                      srf_frame_stats_t* stats) {
    NvtxRange nvtx_range("srf_render");
    if (!ctx || !view || !h_image) return SRF_ERR_ARG;
    if ((view->shard_count ? view->shard_count : 1) != 1) return fail(ctx, SRF_ERR_ARG, "srf_render renders whole images: shard_count must be 1");
    if (spp == 0) return fail(ctx, SRF_ERR_ARG, "spp must be positive");
    DeviceGuard guard(ctx->device);
    const size_t n = (size_t)view->width * view->height;
    srf_status st;
    if ((st = ensure(ctx, ctx->img_out, n * sizeof(float4))) != SRF_OK) return st;
    if ((st = ensure(ctx, ctx->img_accum, n * sizeof(float4))) != SRF_OK) return st;
    srf_view_t v = *view;
    for (uint32_t i = 0; i < spp; ++i) {          // python_api.cu:22-27
        v.spp_index = i;
        st = srf_render_frame(ctx, &v, post, (float*)ctx->img_out.p, (float*)ctx->img_accum.p, nullptr, nullptr,
                              i + 1 == spp ? stats : nullptr, nullptr);
        if (st != SRF_OK) return st;
    }
    SRF_CK(ctx, cudaMemcpy(h_image, ctx->img_out.p, n * sizeof(float4), cudaMemcpyDeviceToHost));   // :30-38
    if (!stats && (st = check_error_flags(ctx, nullptr, nullptr)) != SRF_OK) return st;   // with stats the last pass reported
    return SRF_OK;
}

// ---- several GPUs of one box, one host process ---------------------------------------------------------------------------
// Rays shard, everything else is replicated: the caller creates one context per device and uploads the same arrays to
// each.  A frame's row blocks are dealt round-robin to the contexts; every context's output stage stores its pixels straight
// into the image on the first context's device (plain 16-byte peer stores over NVLink from k_composite_rays; no collective,
// no staging tile).  Hand-off is by stream events: every device's stream records an event when its part is enqueued, the
// first device's stream waits for all of them before the image is copied out.  No device-side waiting anywhere.
struct srf_comm {
    std::vector<srf_ctx*> ctx;
    std::vector<cudaStream_t> stream;
    std::vector<cudaEvent_t> begin, done;
    cudaEvent_t go = nullptr;                 // recorded on the first device; every stream starts after it
    float* d_images = nullptr;                // on the first device, when the caller passes none
    size_t d_images_bytes = 0;
    std::vector<float> ms;                    // device time of the last call, per context
    std::string err;
};

static srf_status comm_fail(srf_comm* c, srf_status st, const std::string& msg) {
    if (c) c->err = msg;
    g_create_error = msg;
    return st;
}

srf_status srf_comm_init(srf_ctx* const* ctx, uint32_t n, srf_comm** out) {
    if (!out) return comm_fail(nullptr, SRF_ERR_ARG, "out is NULL");
    *out = nullptr;
    if (!ctx || n == 0) return comm_fail(nullptr, SRF_ERR_ARG, "no contexts");
    for (uint32_t i = 0; i < n; ++i) {
        if (!ctx[i]) return comm_fail(nullptr, SRF_ERR_ARG, "a context is NULL");
        for (uint32_t j = 0; j < i; ++j)
            if (ctx[j]->device == ctx[i]->device) return comm_fail(nullptr, SRF_ERR_ARG, "two contexts share a device: one context per GPU");
        if (memcmp(&ctx[i]->cfg, &ctx[0]->cfg, sizeof(srf_config_t)) != 0)
            return comm_fail(nullptr, SRF_ERR_ARG, "the contexts were created with different configurations");
    }
    srf_comm* c = new (std::nothrow) srf_comm();
    if (!c) return comm_fail(nullptr, SRF_ERR_CUDA, "out of host memory");
    c->ctx.assign(ctx, ctx + n);
    c->stream.assign(n, nullptr); c->begin.assign(n, nullptr); c->done.assign(n, nullptr); c->ms.assign(n, 0.f);
    const int root = ctx[0]->device;
    for (uint32_t i = 0; i < n; ++i) {
        DeviceGuard guard(ctx[i]->device);
        cudaError_t e = cudaSuccess;
        if (i > 0) {
            int can = 0;
            e = cudaDeviceCanAccessPeer(&can, ctx[i]->device, root);
            if (e == cudaSuccess && !can) { srf_comm_destroy(c); return comm_fail(nullptr, SRF_ERR_CUDA, "a device cannot access the first device's memory (no peer access)"); }
            if (e == cudaSuccess) {
                e = cudaDeviceEnablePeerAccess(root, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) { cudaGetLastError(); e = cudaSuccess; }
            }
        }
        if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&c->stream[i], cudaStreamNonBlocking);
        if (e == cudaSuccess) e = cudaEventCreate(&c->begin[i]);
        if (e == cudaSuccess) e = cudaEventCreate(&c->done[i]);
        if (e == cudaSuccess && i == 0) e = cudaEventCreateWithFlags(&c->go, cudaEventDisableTiming);
        if (e != cudaSuccess) {
            const std::string msg = std::string("srf_comm_init: ") + cudaGetErrorString(e);
            srf_comm_destroy(c);
            return comm_fail(nullptr, SRF_ERR_CUDA, msg);
        }
    }
    *out = c;
    return SRF_OK;
}

void srf_comm_destroy(srf_comm* c) {
    if (!c) return;
    for (size_t i = 0; i < c->ctx.size(); ++i) {
        DeviceGuard guard(c->ctx[i]->device);
        if (c->stream[i]) { cudaStreamSynchronize(c->stream[i]); cudaStreamDestroy(c->stream[i]); }
        if (c->begin[i]) cudaEventDestroy(c->begin[i]);
        if (c->done[i]) cudaEventDestroy(c->done[i]);
        if (i == 0) {
            if (c->go) cudaEventDestroy(c->go);
            if (c->d_images) cudaFree(c->d_images);
        }
    }
    delete c;
}

const char* srf_comm_last_error(const srf_comm* c) { return c ? c->err.c_str() : g_create_error.c_str(); }

srf_status srf_render_frames_sharded(srf_comm* c, const srf_view_t* views, uint32_t n_views, const srf_post_t* post, uint32_t spp,
                                     float* d_images, float* h_images, srf_frame_stats_t* stats) {
    NvtxRange nvtx_range("srf_render_frames_sharded");
    if (!c || !views || n_views == 0) return comm_fail(c, SRF_ERR_ARG, "no views");
    if (spp == 0) return comm_fail(c, SRF_ERR_ARG, "spp must be positive");
    const uint32_t n = (uint32_t)c->ctx.size();
    const size_t px = (size_t)views[0].width * views[0].height;
    for (uint32_t k = 0; k < n_views; ++k)
        if (views[k].width != views[0].width || views[k].height != views[0].height)
            return comm_fail(c, SRF_ERR_ARG, "the views of one call share a resolution");
    const size_t bytes = px * n_views * sizeof(float4);
    srf_ctx* root = c->ctx[0];
    if (!d_images) {
        DeviceGuard guard(root->device);
        if (bytes > c->d_images_bytes) {
            if (c->d_images) cudaFree(c->d_images);
            c->d_images = nullptr; c->d_images_bytes = 0;
            if (cudaMalloc((void**)&c->d_images, bytes) != cudaSuccess) { cudaGetLastError(); return comm_fail(c, SRF_ERR_CUDA, "cannot allocate the image buffer"); }
            c->d_images_bytes = bytes;
        }
        d_images = c->d_images;
    }
    {   // every stream starts after this point of the first device's stream
        DeviceGuard guard(root->device);
        if (cudaEventRecord(c->go, c->stream[0]) != cudaSuccess) return comm_fail(c, SRF_ERR_CUDA, "cudaEventRecord failed");
    }
    // One host thread per device enqueues that device's frames: a frame is a few dozen launches, a batch of views
    // more than a stream's launch queue holds, and a single enqueuing thread would block on the first device's queue
    // while the others sit idle.
    std::vector<srf_status> status(n, SRF_OK);
    std::vector<std::string> message(n);
    auto enqueue = [&](uint32_t r) {
        srf_ctx* ctx = c->ctx[r];
        DeviceGuard guard(ctx->device);
        if (r > 0 && cudaStreamWaitEvent(c->stream[r], c->go, 0) != cudaSuccess) {
            status[r] = SRF_ERR_CUDA; message[r] = "cudaStreamWaitEvent failed";
            return;
        }
        cudaEventRecord(c->begin[r], c->stream[r]);
        for (uint32_t k = 0; k < n_views && status[r] == SRF_OK; ++k) {
            srf_view_t v = views[k];
            v.shard_rows = v.shard_rows ? v.shard_rows : 8;
            v.shard_count = n;
            v.shard_rank = r;
            const uint64_t n_local = shard_rows_total(v) * v.width;
            srf_status st = ensure(ctx, ctx->img_accum, (size_t)std::max<uint64_t>(n_local, 1) * sizeof(float4));
            for (uint32_t i = 0; i < spp && st == SRF_OK; ++i) {
                v.spp_index = i;
                st = srf_render_frame_scatter(ctx, &v, post, d_images + (size_t)k * px * 4, (float*)ctx->img_accum.p, nullptr, c->stream[r]);
            }
            if (st != SRF_OK) { status[r] = st; message[r] = ctx->err; }
        }
        cudaEventRecord(c->done[r], c->stream[r]);
    };
    {
        std::vector<std::thread> workers;
        uint32_t started = 1;                       // devices [1, started) have a thread of their own
        try {
            for (; started < n; ++started) workers.emplace_back(enqueue, started);
        } catch (...) {                             // no more threads to be had: this thread does the rest
        }
        enqueue(0);
        for (uint32_t r = started; r < n; ++r) enqueue(r);
        for (std::thread& w : workers) w.join();
    }
    for (uint32_t r = 0; r < n; ++r)
        if (status[r] != SRF_OK) {
            for (uint32_t q = 0; q < n; ++q) {           // leave no work of this call in flight
                DeviceGuard guard(c->ctx[q]->device);
                cudaStreamSynchronize(c->stream[q]);
            }
            return comm_fail(c, status[r], message[r]);
        }
    {   // the image is complete when every device's part is: the first device's stream waits for all of them
        DeviceGuard guard(root->device);
        for (uint32_t r = 1; r < n; ++r)
            if (cudaStreamWaitEvent(c->stream[0], c->done[r], 0) != cudaSuccess) return comm_fail(c, SRF_ERR_CUDA, "cudaStreamWaitEvent failed");
        if (h_images && cudaMemcpyAsync(h_images, d_images, bytes, cudaMemcpyDeviceToHost, c->stream[0]) != cudaSuccess)
            return comm_fail(c, SRF_ERR_CUDA, "copy of the image to the host failed");
        const cudaError_t e = cudaStreamSynchronize(c->stream[0]);
        if (e != cudaSuccess) return comm_fail(c, SRF_ERR_CUDA, std::string("srf_render_frames_sharded: ") + cudaGetErrorString(e));
    }
    for (uint32_t r = 0; r < n; ++r) {
        srf_ctx* ctx = c->ctx[r];
        DeviceGuard guard(ctx->device);
        cudaEventSynchronize(c->done[r]);
        cudaEventElapsedTime(&c->ms[r], c->begin[r], c->done[r]);
        uint32_t flags = 0;
        const srf_status st = check_error_flags(ctx, c->stream[r], &flags);
        if (stats) {
            // counters of the context's last frame (its shard of the last view and pass)
            memset(&stats[r], 0, sizeof(srf_frame_stats_t));
            if (cudaMemcpy(ctx->h_counters, ctx->d_counters, offsetof(FrameCounters, error_flags), cudaMemcpyDeviceToHost) == cudaSuccess) {
                stats[r].n_rays_alive = ctx->h_counters->n_alive; stats[r].n_march_steps = ctx->h_counters->n_march_steps;
                stats[r].n_samples = ctx->h_counters->n_samples; stats[r].n_samples_composited = ctx->h_counters->n_composited;
                stats[r].n_rays_hit = ctx->h_counters->n_hit;
            }
            stats[r].error_flags = flags;
        }
        if (st != SRF_OK) return comm_fail(c, st, ctx->err);
    }
    return SRF_OK;
}

srf_status srf_get_timings(const srf_comm* c, float* ms_per_context, uint32_t n) {
    if (!c || !ms_per_context) return SRF_ERR_ARG;
    for (uint32_t r = 0; r < n && r < c->ms.size(); ++r) ms_per_context[r] = c->ms[r];
    return SRF_OK;
}

srf_status srf_dump_samples(srf_ctx* ctx, const srf_view_t* view, uint64_t ray_first, uint64_t ray_count, uint64_t capacity,
                            uint32_t* h_counts, float* h_pos_dt, uint32_t* h_ordinal, uint32_t* h_cell, uint64_t* n_total) {
    if (!ctx || !h_counts) return SRF_ERR_ARG;
    DevView v;
    srf_status st = make_view(ctx, view, &v);
    if (st != SRF_OK) return st;
    if (ray_first + ray_count > v.n_rays) return fail(ctx, SRF_ERR_ARG, "ray range exceeds the shard");
    DeviceGuard guard(ctx->device);
    cudaStream_t s = nullptr;
    if ((st = count_and_scan(ctx, v, s)) != SRF_OK) return st;
    std::vector<uint64_t> off(ray_count + 1);
    SRF_CK(ctx, cudaMemcpy(off.data(), (const uint64_t*)ctx->offsets.p + ray_first, (ray_count + 1) * sizeof(uint64_t), cudaMemcpyDeviceToHost));
    SRF_CK(ctx, cudaMemcpy(h_counts, (const uint32_t*)ctx->counts.p + ray_first, ray_count * sizeof(uint32_t), cudaMemcpyDeviceToHost));
    const uint64_t total = off[ray_count] - off[0];
    if (n_total) *n_total = total;
    if (total > capacity) return fail(ctx, SRF_ERR_CAPACITY, "sample arrays too small");
    if (total == 0) return SRF_OK;
    if ((st = ensure_sample_buffers(ctx, total)) != SRF_OK) return st;
    DevBuf ord, cell;
    if ((st = ensure(ctx, ord, total * sizeof(uint32_t))) != SRF_OK) return st;
    if ((st = ensure(ctx, cell, total * sizeof(uint32_t))) != SRF_OK) { cudaFree(ord.p); return st; }
    launch_ray_emit(ctx->g, v, ctx->cfg.use_grid ? ctx->bits : nullptr, (const float4*)ctx->ray_dir_t.p, (const uint64_t*)ctx->offsets.p,
                    ray_first, ray_first + ray_count, (float4*)ctx->pos_dt.p, (uint32_t*)ctx->sample_ray.p, nullptr,
                    (uint32_t*)ord.p, (uint32_t*)cell.p, ctx->d_counters, s);
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && h_pos_dt) e = cudaMemcpy(h_pos_dt, ctx->pos_dt.p, total * sizeof(float4), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && h_ordinal) e = cudaMemcpy(h_ordinal, ord.p, total * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && h_cell) e = cudaMemcpy(h_cell, cell.p, total * sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaFree(ord.p);
    cudaFree(cell.p);
    if (e != cudaSuccess) { ctx->err = std::string("srf_dump_samples: ") + cudaGetErrorString(e); return SRF_ERR_CUDA; }
    return check_error_flags(ctx, s, nullptr);
}

srf_status srf_check_errors(srf_ctx* ctx, void* stream, uint32_t* flags) {
    if (!ctx) return SRF_ERR_ARG;
    DeviceGuard guard(ctx->device);
    return check_error_flags(ctx, (cudaStream_t)stream, flags);
}

srf_status srf_reserve(srf_ctx* ctx, uint64_t max_samples) {
    if (!ctx) return SRF_ERR_ARG;
    ctx->reserve_samples = max_samples;
    return SRF_OK;
}

srf_status srf_eval_math(int device, int op, const float* h_a, const float* h_b, float* h_out, size_t n) {
    if (!h_a || !h_out || op < 0 || op > 5) return fail(nullptr, SRF_ERR_ARG, "bad arguments");
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || device < 0 || device >= n_dev) return fail(nullptr, SRF_ERR_CUDA, "no such CUDA device");
    DeviceGuard guard(device);
    float *a = nullptr, *b = nullptr, *o = nullptr;
    cudaError_t e = cudaMalloc((void**)&a, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&b, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc((void**)&o, n * sizeof(float));
    if (e == cudaSuccess) e = cudaMemcpy(a, h_a, n * sizeof(float), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = h_b ? cudaMemcpy(b, h_b, n * sizeof(float), cudaMemcpyHostToDevice) : cudaMemset(b, 0, n * sizeof(float));
    if (e == cudaSuccess) { launch_eval_math(op, a, b, o, n, nullptr); e = cudaGetLastError(); }
    if (e == cudaSuccess) e = cudaMemcpy(h_out, o, n * sizeof(float), cudaMemcpyDeviceToHost);
    cudaFree(a); cudaFree(b); cudaFree(o);
    if (e != cudaSuccess) return fail(nullptr, SRF_ERR_CUDA, cudaGetErrorString(e));
    return SRF_OK;
}

}  // extern "C"
