"""ctypes helpers above the C-ABI for tests and the benchmark.

`Renderer` is a thin, explicit wrapper of one library context (numpy / torch in and out).  The reference's Python
surface (`pyngp.Testbed`: internal/python_api.cu:84-133) is the compiled module `sphericalrf_b200.pyngp`, built from
the C++ host in include/srf_testbed.hpp; nothing of it lives here.  All arithmetic happens in libsrf_b200.so on the
GPU; torch is used for device memory and streams only.
"""
from __future__ import annotations

import ctypes as C

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

    def set_cell_table_budget(self, n_bytes):
        """Bytes the frame path may spend on cell-major copies of the leading hash-grid levels (0 = none)."""
        self._ck(self.lib.srf_set_cell_table_budget(self.ctx, int(n_bytes)))

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


class Comm:
    """srf_comm over several Renderers of one process (one per GPU, same configuration and uploads)."""

    def __init__(self, renderers):
        self.renderers = list(renderers)
        self.lib = self.renderers[0].lib
        arr = (C.c_void_p * len(self.renderers))(*[r.ctx for r in self.renderers])
        self.comm = C.c_void_p()
        st = self.lib.srf_comm_init(arr, len(self.renderers), C.byref(self.comm))
        if st != abi.OK:
            msg = self.lib.srf_comm_last_error(None)
            raise abi.SrfError(st, msg.decode() if msg else "")

    def close(self):
        if getattr(self, "comm", None):
            self.lib.srf_comm_destroy(self.comm)
            self.comm = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def render(self, views, post, spp=1, host_images=None, want_stats=False, device_images=None):
        """srf_render_frames_sharded: images (n_views, H, W, 4) float32 in host memory (a pinned torch tensor may be
        passed as `host_images`; it is filled and returned as numpy)."""
        n = len(views)
        arr = (abi.View * n)(*views)
        h, w = views[0].height, views[0].width
        if host_images is False:                       # leave the images on the first GPU
            out, hp = None, None
        elif host_images is None:
            out = np.zeros((n, h, w, 4), np.float32)
            hp = _np_ptr(out)
        else:
            out = host_images
            hp = C.c_void_p(host_images.data_ptr())
        stats = (abi.FrameStats * len(self.renderers))() if want_stats else None
        st = self.lib.srf_render_frames_sharded(self.comm, arr, n, C.byref(post), spp,
                                                None if device_images is None else C.c_void_p(device_images.data_ptr()), hp, stats)
        if st != abi.OK:
            msg = self.lib.srf_comm_last_error(self.comm)
            raise abi.SrfError(st, msg.decode() if msg else "")
        return (out, [s.as_dict() for s in stats]) if want_stats else out

    def timings(self):
        ms = (C.c_float * len(self.renderers))()
        self.lib.srf_get_timings(self.comm, ms, len(self.renderers))
        return [float(x) for x in ms]


def eval_math(op, a, b=None, device=0):
    lib = abi.load()
    a = np.ascontiguousarray(a, np.float32)
    b = None if b is None else np.ascontiguousarray(b, np.float32)
    out = np.zeros_like(a)
    abi.check(lib.srf_eval_math(device, op, _np_ptr(a), _np_ptr(b), _np_ptr(out), a.size))
    return out


def config_from_json(model_config: dict) -> abi.Config:
    """The configuration structure the C++ host (include/srf_testbed.hpp, srf_host::parse_config) derives from a
    parsed model configuration: the reference's keys, defaults and error messages."""
    from . import pyngp
    return abi.Config.from_buffer_copy(pyngp.parse_config(model_config))
