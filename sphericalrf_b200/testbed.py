"""Host-side mirror of the reference's Python surface, on top of the C-ABI.

`Renderer` is a thin, explicit wrapper (numpy / torch in and out) used by tests and the benchmark.
`Testbed` mirrors the parts of `pyngp.Testbed` the reference's drivers use for inference
(internal/python_api.cu:84-133; experiment/*/python/run.py:128-250): `load_model_config`,
`render`, `set_nerf_camera_matrix`, `fov`, `fov_xy`, `background_color`, `color_space`,
`density_activation`, `rgb_activation`, `rendering_buffer.*`.  All arithmetic happens in
libsrf_b200.so on the GPU; torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C
import json
import math
from pathlib import Path

import numpy as np

from . import abi


def _np_ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Renderer:
    """One library context on one GPU."""

    def __init__(self, cfg: abi.Config, device: int = 0, lib=None):
        self.lib = abi.load() if lib is None else lib      # `lib`: another build of the same C-ABI (tests)
        self.cfg = cfg
        self.device = device
        self.ctx = C.c_void_p()
        st = self.lib.srf_create(C.byref(cfg), device, C.byref(self.ctx))
        if st != abi.OK:
            msg = self.lib.srf_last_error(None)
            raise abi.SrfError(st, msg.decode() if msg else "")

    def close(self):
        if getattr(self, "ctx", None):
            self.lib.srf_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _ck(self, st):
        if st != abi.OK:
            msg = self.lib.srf_last_error(self.ctx)
            raise abi.SrfError(st, msg.decode() if msg else "")

    # ---- parameters ----
    def upload_network(self, table, density_mlp, rgb_mlp):
        t = np.ascontiguousarray(table, np.float16)
        d = np.ascontiguousarray(density_mlp, np.float16)
        c = np.ascontiguousarray(rgb_mlp, np.float16)
        self._ck(self.lib.srf_upload_network(self.ctx, _np_ptr(t), t.size, _np_ptr(d), d.size, _np_ptr(c), c.size))

    def upload_blobs(self, blobs, color_map):
        b = np.ascontiguousarray(blobs, np.float32)
        m = np.ascontiguousarray(color_map, np.float32)
        self._ck(self.lib.srf_upload_blobs(self.ctx, _np_ptr(b), b.shape[0], _np_ptr(m)))

    def upload_density_grid(self, grid):
        g = np.ascontiguousarray(grid, np.float32)
        self._ck(self.lib.srf_upload_density_grid(self.ctx, _np_ptr(g), g.size, None))

    def download_density_grid(self):
        n = self.cfg.grid_size ** 3 * self.cfg.num_cascades
        g = np.zeros(n, np.float32)
        self._ck(self.lib.srf_download_density_grid(self.ctx, _np_ptr(g), n, None))
        return g

    def upload_bitfield(self, bits):
        b = np.ascontiguousarray(bits, np.uint8)
        self._ck(self.lib.srf_upload_bitfield(self.ctx, _np_ptr(b), b.size, None))

    def download_bitfield(self):
        n = self.cfg.grid_size ** 3 * self.cfg.num_cascades // 8
        b = np.zeros(n, np.uint8)
        self._ck(self.lib.srf_download_bitfield(self.ctx, _np_ptr(b), n, None))
        return b

    def grid_mean(self):
        m = np.zeros(1, np.float32)
        self._ck(self.lib.srf_download_grid_mean(self.ctx, _np_ptr(m), None))
        return m[0]

    def update_grid_bitfield(self, stream=None):
        self._ck(self.lib.srf_update_grid_bitfield(self.ctx, stream))

    def refresh_reset(self, seed):
        self._ck(self.lib.srf_refresh_reset(self.ctx, seed))

    def refresh_grid(self, training_step=0, stream=None):
        self._ck(self.lib.srf_refresh_grid(self.ctx, training_step, stream))

    def reserve(self, max_samples):
        self._ck(self.lib.srf_reserve(self.ctx, max_samples))

    def check_errors(self, stream=None):
        """srf_check_errors: raises if a frame enqueued since the last check was cut short on the device."""
        self._ck(self.lib.srf_check_errors(self.ctx, stream, None))

    def set_timing(self, on=True):
        self._ck(self.lib.srf_set_timing(self.ctx, 1 if on else 0))

    # ---- frames ----
    def n_rays(self, view):
        n = C.c_uint64(0)
        self._ck(self.lib.srf_shard_ray_count(C.byref(view), C.byref(n)))
        return n.value

    def render_frame_device(self, view, post, out, accum, rgba_raw=None, n_samples=None, stats=None, stream=None):
        """All buffers are torch CUDA tensors (or None). Enqueues on `stream` (a raw cudaStream_t or None)."""
        p = lambda t: None if t is None else C.c_void_p(t.data_ptr())
        self._ck(self.lib.srf_render_frame(self.ctx, C.byref(view), C.byref(post), p(out), p(accum), p(rgba_raw),
                                           p(n_samples), None if stats is None else C.byref(stats), stream))

    def render_frame_scatter_device(self, view, post, image, accum, stats=None, stream=None):
        """Writes the shard's pixels at their positions of the whole-image tensor `image` (H*W, 4), which may be
        a peer GPU's buffer; `accum` is the local shard-indexed accumulate buffer."""
        self._ck(self.lib.srf_render_frame_scatter(self.ctx, C.byref(view), C.byref(post), C.c_void_p(image.data_ptr()),
                                                   None if accum is None else C.c_void_p(accum.data_ptr()),
                                                   None if stats is None else C.byref(stats), stream))

    def render_frame(self, view, post, accum=None, want_raw=False, want_counts=False, want_stats=False):
        """Convenience path for tests: allocates device buffers with torch, returns numpy arrays."""
        import torch
        n = self.n_rays(view)
        dev = torch.device("cuda", self.device)
        out = torch.zeros((n, 4), dtype=torch.float32, device=dev)
        acc = torch.zeros((n, 4), dtype=torch.float32, device=dev) if accum is None else torch.as_tensor(accum, device=dev).contiguous()
        raw = torch.zeros((n, 4), dtype=torch.float32, device=dev) if want_raw else None
        cnt = torch.zeros(n, dtype=torch.int32, device=dev) if want_counts else None
        stats = abi.FrameStats() if want_stats else None
        self.render_frame_device(view, post, out, acc, raw, cnt, stats, None)
        torch.cuda.synchronize(dev)
        res = dict(out=out.cpu().numpy(), accum=acc.cpu().numpy())
        if want_raw:
            res["rgba_raw"] = raw.cpu().numpy()
        if want_counts:
            res["n_samples"] = cnt.cpu().numpy().astype(np.uint32)
        if want_stats:
            res["stats"] = stats.as_dict()
        return res

    def render(self, view, post, spp=1, want_stats=False):
        """srf_render: host image (H, W, 4) float32."""
        img = np.zeros((view.height, view.width, 4), np.float32)
        stats = abi.FrameStats() if want_stats else None
        self._ck(self.lib.srf_render(self.ctx, C.byref(view), C.byref(post), spp, _np_ptr(img),
                                     None if stats is None else C.byref(stats)))
        return (img, stats.as_dict()) if want_stats else img

    def set_wave_schedule(self, steps):
        """March steps per ray of the leading waves of a frame ([] = one pass); see srf_set_wave_schedule."""
        a = (C.c_uint32 * max(len(steps), 1))(*steps)
        self._ck(self.lib.srf_set_wave_schedule(self.ctx, a, len(steps)))

    def network_inference(self, coords):
        """srf_network_inference on host Coordinate records (n, 7) float32 -> (n, 4) float16 raw (r, g, b, sigma)."""
        import torch
        dev = torch.device("cuda", self.device)
        c = torch.from_numpy(np.ascontiguousarray(coords, np.float32)).to(dev)
        out = torch.zeros((c.shape[0], 4), dtype=torch.float16, device=dev)
        self._ck(self.lib.srf_network_inference(self.ctx, C.c_void_p(c.data_ptr()), c.shape[0], C.c_void_p(out.data_ptr()), None))
        torch.cuda.synchronize(dev)
        return out.cpu().numpy()

    # -- training-side sampler --
    def _device_views(self, views: dict):
        """srf_train_views_t over torch device copies of dict(n_images, width, height, focal_length,
        principal_point, xforms (n,12) column-major, images (n,H,W,4) fp16 | None, sampling_probability | None)."""
        import torch
        dev = torch.device("cuda", self.device)
        keep = [torch.from_numpy(np.ascontiguousarray(views["xforms"], np.float32)).to(dev),
                None if views.get("images") is None else torch.from_numpy(np.ascontiguousarray(views["images"], np.float16)).to(dev),
                None if views.get("sampling_probability") is None else
                torch.from_numpy(np.ascontiguousarray(views["sampling_probability"], np.float16)).to(dev)]
        tv = abi.TrainViews()
        tv.n_images, tv.width, tv.height = int(views["n_images"]), int(views["width"]), int(views["height"])
        tv.focal_length[:] = [float(x) for x in views["focal_length"]]
        tv.principal_point[:] = [float(x) for x in views["principal_point"]]
        tv.d_xforms = keep[0].data_ptr()
        tv.d_images = None if keep[1] is None else keep[1].data_ptr()
        tv.d_sampling_probability = None if keep[2] is None else keep[2].data_ptr()
        return tv, keep

    def sampler_init(self, views, init_grid_with_mask=False, rng_seed=0):
        """OccupancySampler::init: restart the refresh stream, mask or clear the density grid."""
        import torch
        tv, keep = (None, None) if views is None else self._device_views(views)
        self._ck(self.lib.srf_sampler_init(self.ctx, None if tv is None else C.byref(tv), 1 if init_grid_with_mask else 0,
                                           rng_seed, None))
        torch.cuda.synchronize(self.device)

    def sample_training_rays(self, views, n_rays, n_rays_shift, n_coords, rng_state, rng_inc, snap=True):
        """srf_sample_training_rays with device buffers from torch; returns numpy arrays (kept rays only)."""
        import torch
        dev = torch.device("cuda", self.device)
        tv, keep = self._device_views(views)
        counters = torch.zeros(2, dtype=torch.int32, device=dev)
        rays = torch.zeros((n_rays, 6), dtype=torch.float32, device=dev)
        rgba = torch.zeros((n_rays, 4), dtype=torch.float32, device=dev)
        numsteps = torch.zeros((n_rays, 2), dtype=torch.int32, device=dev)
        coords = torch.zeros((n_coords, 7), dtype=torch.float32, device=dev)
        self._ck(self.lib.srf_sample_training_rays(self.ctx, C.byref(tv), n_rays, n_rays_shift, n_coords, rng_state, rng_inc,
                                                   1 if snap else 0, C.c_void_p(counters.data_ptr()),
                                                   C.c_void_p(counters.data_ptr() + 4), C.c_void_p(rays.data_ptr()),
                                                   C.c_void_p(rgba.data_ptr()), C.c_void_p(numsteps.data_ptr()),
                                                   C.c_void_p(coords.data_ptr()), None))
        torch.cuda.synchronize(dev)
        c = counters.cpu().numpy().astype(np.uint32)
        k = int(c[0])
        return dict(n_rays=k, n_samples_total=int(c[1]), rays=rays[:k].cpu().numpy(), rgba=rgba[:k].cpu().numpy(),
                    numsteps=numsteps[:k].cpu().numpy().astype(np.uint32), coords=coords.cpu().numpy())

    def volume_rendering_loss(self, params, n_rays_kept, ray_coord_indices, rays_rgba, coords, network_output):
        """srf_volume_rendering_loss on host arrays (uploaded and read back through torch)."""
        import torch
        dev = torch.device("cuda", self.device)
        up = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a, dt)).to(dev)
        cap, w, n = int(params.n_max_compacted_coords), int(params.padded_output_width), int(params.n_rays)
        kept = torch.tensor([n_rays_kept], dtype=torch.int32, device=dev)
        idx = up(np.asarray(ray_coord_indices).astype(np.int32), np.int32)
        rgba, co, no = up(rays_rgba, np.float32), up(coords, np.float32), up(network_output, np.float16)
        cc = torch.zeros((cap, 7), dtype=torch.float32, device=dev)
        dl = torch.zeros((cap, w), dtype=torch.float16, device=dev)
        loss = torch.zeros(n, dtype=torch.float32, device=dev)
        reg = torch.zeros((cap, 2), dtype=torch.float32, device=dev)
        n_comp = torch.zeros(1, dtype=torch.int32, device=dev)
        ptr = lambda t: C.c_void_p(t.data_ptr())
        self._ck(self.lib.srf_volume_rendering_loss(self.ctx, C.byref(params), ptr(kept), ptr(idx), ptr(rgba), ptr(co), ptr(no), ptr(cc),
                                                    ptr(n_comp), ptr(dl), ptr(loss),
                                                    ptr(reg) if params.regularization_type == abi.REG_DISTORTION else None, None))
        torch.cuda.synchronize(dev)
        return dict(indices=idx.cpu().numpy().astype(np.uint32), compacted_coords=cc.cpu().numpy(), n_compacted=int(n_comp.item()),
                    dloss=dl.cpu().numpy(), loss=loss.cpu().numpy(), reg=reg.cpu().numpy())

    def dump_samples(self, view, ray_first, ray_count, capacity):
        counts = np.zeros(ray_count, np.uint32)
        pos_dt = np.zeros((capacity, 4), np.float32)
        ordinal = np.zeros(capacity, np.uint32)
        cell = np.zeros(capacity, np.uint32)
        n_total = C.c_uint64(0)
        self._ck(self.lib.srf_dump_samples(self.ctx, C.byref(view), ray_first, ray_count, capacity, _np_ptr(counts),
                                           _np_ptr(pos_dt), _np_ptr(ordinal), _np_ptr(cell), C.byref(n_total)))
        n = n_total.value
        return counts, pos_dt[:n], ordinal[:n], cell[:n]


def eval_math(op, a, b=None, device=0):
    lib = abi.load()
    a = np.ascontiguousarray(a, np.float32)
    b = None if b is None else np.ascontiguousarray(b, np.float32)
    out = np.zeros_like(a)
    abi.check(lib.srf_eval_math(device, op, _np_ptr(a), _np_ptr(b), _np_ptr(out), a.size))
    return out


# ---- configuration parsing (the reference's JSON keys, including the "samlper" spelling) --------
_WARPS = {"ngp": abi.WARP_NGP, "mipnerf360": abi.WARP_MIPNERF360, "donerf": abi.WARP_DONERF, "sigmoid": abi.WARP_SIGMOID,
          "erp": abi.WARP_ERP, "sinusoidalprojection": abi.WARP_SINUSOIDAL}
_SAMPLINGS = {"original": abi.SAMPLING_ORIGINAL, "disparity": abi.SAMPLING_DISPARITY, "log": abi.SAMPLING_LOG}
_GRIDS = {"warpedspace_exp": abi.GRID_WARPED_EXP, "warpedspace_reciprocal": abi.GRID_WARPED_RECIPROCAL,
          "metricspace_exp": abi.GRID_METRIC_EXP, "metricspace_reciprocal": abi.GRID_METRIC_RECIPROCAL}


def config_from_json(model_config: dict) -> abi.Config:
    """Reads the sections the reference reads (internal/testbed.cu:65-76) with its defaults
    (internal/sampler/occupancy_sampler.cu:909-944, internal/render/ray_marcher.cu:294-301,
    internal/network/ngp_network.h:597-637) and its error messages."""
    c = abi.default_config()
    s = model_config["samlper"]
    try:
        c.warping_type = _WARPS[str(s.get("warping_type", "NGP")).lower()]
    except KeyError:
        raise RuntimeError("Unknown warping type.")
    c.aabb_scale = int(s.get("aabb_scale", 1))
    c.use_grid = 1 if s.get("use_grid", True) else 0
    if c.use_grid:
        c.grid_size = int(s.get("grid_size", 128))
        c.num_cascades = int(s.get("num_cascades", 1))
        c.ema_decay = float(s.get("ema_decay", 0.95))
        try:
            c.grid_distribution_type = _GRIDS[str(s.get("grid_distribution_type", "Exp")).lower()]
        except KeyError:
            raise RuntimeError("Unknown grid distribution type.")   # the reference's default "Exp" throws as well
    c.maximum_marching_steps = int(s.get("maximum_marching_steps", 1024))
    c.cone_angle_constant = float(s.get("cone_angle_constant", 0.0))
    c.min_cone_stepsize = float(s.get("min_cone_stepsize", 0.0))
    c.max_cone_stepsize = float(s.get("max_cone_stepsize", 0.0))
    c.near_distance = float(s.get("near_distance", 0.2))
    c.far_distance = float(s.get("far_distance", 100.0))
    try:
        c.sampling_type = _SAMPLINGS[str(s.get("sampling_type", "Original")).lower()]
    except KeyError:
        raise RuntimeError("Unknown sampling type.")
    c.snap_to_pixel_centers_in_rendering = 1 if s.get("snap_to_pixel_centers_in_rendering", True) else 0
    c.min_optical_thickness = float(s.get("min_optical_thickness", 0.01))
    r = model_config.get("render", {})
    c.transmittance_threshold = float(r.get("transmittance_threshold", 1e-4))
    c.train_in_linear_color = 1 if r.get("train_in_linear_color", False) else 0
    enc = model_config["network"]["encoding"]
    fpl = int(enc.get("n_features_per_level", 2))
    n_levels = int(enc.get("n_levels", 16))
    if enc.get("n_features", 0):
        n_levels = int(enc["n_features"]) // fpl
    c.n_levels, c.n_features_per_level = n_levels, fpl
    c.log2_hashmap_size = int(enc.get("log2_hashmap_size", 15))
    base = int(enc.get("base_resolution", 0))
    c.base_resolution = base if base else 1 << (c.log2_hashmap_size // 3)
    c.desired_resolution = float(enc.get("desired_resolution", 2048.0))
    c.per_level_scale = float(enc.get("per_level_scale", 0.0))
    for key in ("network", "rgb_network"):
        net = model_config["network"][key]
        if int(net.get("n_neurons", 64)) != 64:
            raise RuntimeError("this library implements the 64-neuron MLPs every shipped config uses")
    if int(model_config["network"]["network"].get("n_hidden_layers", 1)) != 1 or \
       int(model_config["network"]["rgb_network"].get("n_hidden_layers", 2)) != 2:
        raise RuntimeError("this library implements 1 hidden density layer and 2 hidden colour layers")
    if int(model_config["network"]["dir_encoding"].get("degree", 4)) != 4:
        raise RuntimeError("this library implements spherical harmonics of degree 4")
    return c


class _RenderingBuffer:
    """Testbed::RenderingBuffer fields exposed to Python (internal/python_api.cu:123-133)."""

    def __init__(self):
        self.render_mode = abi.MODE_SHADE
        self.tonemap_curve = abi.TONEMAP_IDENTITY
        self.exposure = 0.0
        self.fov_axis = 1
        self.relative_focal_length = [1.0, 1.0]
        self.principal_point = [0.5, 0.5]
        self.MIN_STEPS_INBETWEEN_COMPACTION = 1   # kept for compatibility; the frame loop has no compaction rounds
        self.MAX_STEPS_INBETWEEN_COMPACTION = 8


class Testbed:
    """Inference-side mirror of `pyngp.Testbed`."""

    def __init__(self, device: int = 0):
        self.device = device
        self.renderer = None
        self.density_activation = abi.ACT_EXPONENTIAL       # testbed.h:115-116
        self.rgb_activation = abi.ACT_LOGISTIC
        self.background_color = [0.0, 0.0, 0.0, 1.0]        # testbed.h:117
        self.color_space = abi.COLOR_LINEAR
        self.rendering_buffer = _RenderingBuffer()
        self.scene_scale = 1.0
        self.scene_offset = np.array([0.5, 0.5, 0.5], np.float32)
        self._camera = np.zeros((3, 4), np.float32)
        self.model_config = None
        self.cfg = None

    # -- configuration --
    def load_model_config(self, config_path: str):
        p = Path(config_path)
        if not str(config_path) or not p.exists():
            raise RuntimeError("The model config must exist.")
        if p.suffix.lower() == ".msgpack":
            from .snapshot import _msgpack
            with open(p, "rb") as f:
                self.load_model_config_dict(_msgpack().unpackb(f.read(), raw=False, strict_map_key=False))
            return
        if p.suffix.lower() != ".json":
            raise RuntimeError("The model config must be a .json or .msgpack file.")
        with open(p) as f:
            text = "\n".join(line.split("//")[0] for line in f.read().splitlines())   # the reference parses with comments allowed
        self.load_model_config_dict(json.loads(text))

    def load_model_config_dict(self, model_config: dict):
        self.model_config = model_config
        self.cfg = config_from_json(model_config)
        self.cfg.density_activation = self.density_activation
        self.cfg.rgb_activation = self.rgb_activation
        if self.renderer is not None:
            self.renderer.close()
        self.renderer = Renderer(self.cfg, self.device)

    def load_parameters(self, hash_table, density_mlp, rgb_mlp, density_grid, scene_scale=1.0, scene_offset=(0.5, 0.5, 0.5)):
        """What load_snapshot restores (internal/testbed.cu:151-171), from arrays: network parameters,
        density grid (followed by update_grid_bitfield), scene scale and offset."""
        self.renderer.upload_network(hash_table, density_mlp, rgb_mlp)
        self.renderer.upload_density_grid(density_grid)
        self.renderer.update_grid_bitfield()
        self.scene_scale = float(scene_scale)
        self.scene_offset = np.asarray(scene_offset, np.float32)

    def load_snapshot(self, snapshot_path: str):
        """Testbed::load_snapshot (internal/testbed.cu:151-171): configuration, scene scale and offset, density
        grid (+ update_grid_bitfield) and network parameters from one .msgpack file."""
        from . import snapshot
        self.load_model_config(snapshot_path)
        if "snapshot" not in self.model_config:
            raise RuntimeError("ERROR in loading snapshot.")
        snap = snapshot.read_snapshot(snapshot_path)
        want = snapshot.table_entries(self.cfg)
        if snap["hash_table"].size != want:
            raise RuntimeError(f"snapshot holds {snap['hash_table'].size} hash-grid parameters, the configuration needs {want}")
        self.load_parameters(snap["hash_table"], snap["density_mlp"], snap["rgb_mlp"], snap["density_grid"],
                             snap["scene_scale"], snap["scene_offset"])

    # -- camera (internal/testbed.h:73-89, internal/utils/common_device.h:105-141) --
    @property
    def fov(self):
        fl = np.float32(self.rendering_buffer.relative_focal_length[self.rendering_buffer.fov_axis])
        return float(180.0 * (2.0 / math.pi) * np.arctan(np.float32(1.0) / (fl * np.float32(2.0))))   # degrees

    @fov.setter
    def fov(self, rad):
        f = float(np.float32(0.5) / np.float32(math.tan(0.5 * float(rad))))                            # radians in
        self.rendering_buffer.relative_focal_length = [f, f]

    @property
    def fov_xy(self):
        return [float(180.0 * (2.0 / math.pi) * np.arctan(np.float32(1.0) / (np.float32(f) * np.float32(2.0))))
                for f in self.rendering_buffer.relative_focal_length]

    @fov_xy.setter
    def fov_xy(self, rads):
        self.rendering_buffer.relative_focal_length = [float(np.float32(0.5) / np.float32(math.tan(0.5 * float(r)))) for r in rads]

    def set_nerf_camera_matrix(self, cam):
        m = np.asarray(cam, np.float32).reshape(3, 4).copy()
        m[:, 1] *= -1.0
        m[:, 2] *= -1.0
        m[:, 3] = m[:, 3] * np.float32(self.scene_scale) + self.scene_offset
        self._camera = m

    # -- rendering (internal/python_api.cu:17-41) --
    def render(self, width=1920, height=1080, spp=1, to_srgb=True):
        if self.renderer is None:
            raise RuntimeError("load_model_config first")
        rb = self.rendering_buffer
        view = abi.make_view(self._camera, width, height, rb.relative_focal_length, rb.principal_point, 0,
                             int(rb.render_mode), 1.0 / self.scene_scale)
        post = abi.default_post()
        post.exposure = float(rb.exposure)
        post.background_color[:] = [float(x) for x in self.background_color]
        post.color_space = int(self.color_space)
        post.tonemap_curve = int(rb.tonemap_curve)
        post.to_srgb = 1 if to_srgb else 0
        return self.renderer.render(view, post, spp)
