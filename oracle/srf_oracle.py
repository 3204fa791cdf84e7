"""ctypes binding of the CPU oracle (oracle/libsrf_oracle.so).  TEST INFRASTRUCTURE.

Imported only by tests/, by __graft_entry__.smoke() and by bench.py's CPU-baseline legs; the
library and the package never import it.  PARITY UNPINNED: see oracle/srf_oracle.h.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

from sphericalrf_b200 import abi

HERE = Path(__file__).resolve().parent
LIB = HERE / "libsrf_oracle.so"


class Model(C.Structure):
    _fields_ = [("hash_table", C.c_void_p), ("density_mlp", C.c_void_p), ("rgb_mlp", C.c_void_p),
                ("blobs", C.c_void_p), ("n_blobs", C.c_uint32), ("color_map", C.c_void_p)]


class Rng(C.Structure):
    _fields_ = [("state", C.c_uint64), ("inc", C.c_uint64)]


LIB_PLAIN = HERE / "libsrf_oracle_plain.so"


def build(force=False):
    srcs = [HERE / "srf_oracle.cpp", HERE / "srf_oracle.h", HERE / "Makefile", HERE.parent / "include" / "srf_abi.h",
            HERE.parent / "include" / "srf_canon_math.h"]
    for target in (LIB, LIB_PLAIN):
        if force or not target.exists() or any(s.stat().st_mtime > target.stat().st_mtime for s in srcs):
            subprocess.run(["make", "-C", str(HERE)] + (["-B"] if force else []), check=True, capture_output=True)
            break
    return LIB


_libs = {}
_plain = False


def lib():
    """The oracle library: the canonical one, or inside `plain_arithmetic()` the build with the C library's
    elementary functions and no fused multiply-adds (comparable bit for bit with oracle/srf_ref.py)."""
    if _plain not in _libs:
        build()
        l = C.CDLL(str(LIB_PLAIN if _plain else LIB))
        l.srfo_shard_ray_count.restype = C.c_uint64
        _libs[_plain] = l
    return _libs[_plain]


class plain_arithmetic:
    """Context manager: every oracle call inside runs in the plain-arithmetic build."""

    def __enter__(self):
        global _plain
        self._old = _plain
        _plain = True
        return self

    def __exit__(self, *exc):
        global _plain
        _plain = self._old
        return False


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    """Holds a configuration, a bitfield and model arrays; numpy in, numpy out."""

    def __init__(self, cfg: abi.Config, bitfield=None, hash_table=None, density_mlp=None, rgb_mlp=None,
                 blobs=None, color_map=None):
        self.cfg = cfg
        self.bitfield = None if bitfield is None else np.ascontiguousarray(bitfield, dtype=np.uint8)
        self._keep = [np.ascontiguousarray(a) if a is not None else None
                      for a in (hash_table, density_mlp, rgb_mlp, blobs, color_map)]
        ht, dm, rm, bl, cm = self._keep
        self.model = Model()
        self.model.hash_table = None if ht is None else ht.ctypes.data
        self.model.density_mlp = None if dm is None else dm.ctypes.data
        self.model.rgb_mlp = None if rm is None else rm.ctypes.data
        self.model.blobs = None if bl is None else bl.ctypes.data
        self.model.n_blobs = 0 if bl is None else bl.shape[0]
        self.model.color_map = None if cm is None else cm.ctypes.data

    def n_rays(self, view):
        return int(lib().srfo_shard_ray_count(C.byref(view)))

    def generate_rays(self, view):
        n = self.n_rays(view)
        d = np.zeros((n, 3), np.float32); t = np.zeros(n, np.float32)
        alive = np.zeros(n, np.uint8); pixel = np.zeros(n, np.uint32)
        rc = lib().srfo_generate_rays(C.byref(self.cfg), C.byref(view), _p(self.bitfield), _p(d), _p(t), _p(alive), _p(pixel))
        assert rc == 0
        return d, t, alive, pixel

    def march(self, view, ray_first, ray_count, capacity):
        counts = np.zeros(ray_count, np.uint32)
        pos_dt = np.zeros((capacity, 4), np.float32)
        ordinal = np.zeros(capacity, np.uint32); cell = np.zeros(capacity, np.uint32)
        n_total = C.c_uint64(0); n_steps = C.c_uint64(0)
        rc = lib().srfo_march(C.byref(self.cfg), C.byref(view), _p(self.bitfield), C.c_uint64(ray_first),
                              C.c_uint64(ray_count), C.c_uint64(capacity), _p(counts), _p(pos_dt), _p(ordinal),
                              _p(cell), C.byref(n_total), C.byref(n_steps))
        if rc != 0:
            raise RuntimeError(f"oracle march: capacity {capacity} < {n_total.value}")
        n = n_total.value
        return counts, pos_dt[:n], ordinal[:n], cell[:n], n_steps.value

    def network_inference(self, coords):
        coords = np.ascontiguousarray(coords, np.float32)
        n = coords.shape[0]
        out = np.zeros((n, 4), np.float16)
        rc = lib().srfo_network_inference(C.byref(self.cfg), C.byref(self.model), _p(coords), C.c_uint64(n), _p(out))
        assert rc == 0
        return out

    def network_density(self, positions):
        positions = np.ascontiguousarray(positions, np.float32)
        n = positions.shape[0]
        out = np.zeros((n, 16), np.float16)
        rc = lib().srfo_network_density(C.byref(self.cfg), C.byref(self.model), _p(positions), C.c_uint64(n), _p(out))
        assert rc == 0
        return out

    def render_frame(self, view, post, ray_first=0, ray_count=0, accum=None):
        n = self.n_rays(view)
        out = np.zeros((n, 4), np.float32)
        accum = np.zeros((n, 4), np.float32) if accum is None else accum
        raw = np.zeros((n, 4), np.float32)
        ns = np.zeros(n, np.uint32); nc = np.zeros(n, np.uint32)
        stats = abi.FrameStats()
        rc = lib().srfo_render_frame(C.byref(self.cfg), C.byref(view), C.byref(post), _p(self.bitfield),
                                     C.byref(self.model), C.c_uint64(ray_first), C.c_uint64(ray_count), _p(out),
                                     _p(accum), _p(raw), _p(ns), _p(nc), C.byref(stats))
        assert rc == 0
        return dict(out=out, accum=accum, rgba_raw=raw, n_samples=ns, n_composited=nc, stats=stats.as_dict())

    def update_grid_bitfield(self, grid):
        grid = np.ascontiguousarray(grid, np.float32)
        bits = np.zeros(grid.shape[0] // 8, np.uint8)
        mean = C.c_float(0)
        rc = lib().srfo_update_grid_bitfield(C.byref(self.cfg), _p(grid), _p(bits), C.byref(mean))
        assert rc == 0
        return bits, np.float32(mean.value)

    def refresh(self, grid, refresh_step, training_step, rng: Rng):
        """In-place max-decay refresh of `grid`; returns (bitfield, mean, next refresh_step)."""
        assert grid.dtype == np.float32 and grid.flags.c_contiguous
        bits = np.zeros(grid.shape[0] // 8, np.uint8)
        mean = C.c_float(0)
        step = C.c_uint32(refresh_step)
        rc = lib().srfo_refresh_grid(C.byref(self.cfg), C.byref(self.model), _p(grid), _p(bits), C.byref(mean),
                                     C.byref(step), C.c_uint32(training_step), C.byref(rng))
        assert rc == 0
        return bits, np.float32(mean.value), step.value


def rng_seed(seed) -> Rng:
    r = Rng()
    lib().srfo_rng_seed(C.byref(r), C.c_uint64(seed))
    return r


def eval_math(op, a, b=None):
    a = np.ascontiguousarray(a, np.float32)
    b = np.zeros_like(a) if b is None else np.ascontiguousarray(b, np.float32)
    out = np.zeros_like(a)
    rc = lib().srfo_eval_math(C.c_int(op), _p(a), _p(b), _p(out), C.c_size_t(a.size))
    assert rc == 0
    return out


def warp_position(cfg, pos, inverse=False):
    pos = np.ascontiguousarray(pos, np.float32)
    out = np.zeros_like(pos)
    lib().srfo_warp_position(C.byref(cfg), _p(pos), _p(out), C.c_size_t(pos.shape[0]), C.c_int(1 if inverse else 0))
    return out


def calc_dt(cfg, t):
    t = np.ascontiguousarray(t, np.float32)
    out = np.zeros_like(t)
    lib().srfo_calc_dt(C.byref(cfg), _p(t), _p(out), C.c_size_t(t.size))
    return out


def grid_index(cfg, pos):
    pos = np.ascontiguousarray(pos, np.float32)
    level = np.zeros(pos.shape[0], np.uint32); idx = np.zeros(pos.shape[0], np.uint32)
    lib().srfo_grid_index(C.byref(cfg), _p(pos), _p(level), _p(idx), C.c_size_t(pos.shape[0]))
    return level, idx


def pixel_offset(spp):
    out = np.zeros(2, np.float32)
    lib().srfo_pixel_offset(C.c_uint32(spp), _p(out))
    return out


def tonemap(rgb, curve):
    rgb = np.ascontiguousarray(rgb, np.float32)
    out = np.zeros_like(rgb)
    lib().srfo_tonemap(_p(rgb), _p(out), C.c_size_t(rgb.shape[0]), C.c_int(curve))
    return out


def srgb(x, to_linear):
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros_like(x)
    lib().srfo_srgb(_p(x), _p(out), C.c_size_t(x.size), C.c_int(1 if to_linear else 0))
    return out


def loss(target, prediction, loss_type):
    t = np.ascontiguousarray(target, np.float32); p = np.ascontiguousarray(prediction, np.float32)
    l = np.zeros_like(t); g = np.zeros_like(t)
    lib().srfo_loss(_p(t), _p(p), _p(l), _p(g), C.c_size_t(t.shape[0]), C.c_int(loss_type))
    return l, g


def hashgrid_layout(cfg):
    off = np.zeros(cfg.n_levels + 1, np.uint32); res = np.zeros(cfg.n_levels, np.uint32)
    sc = np.zeros(cfg.n_levels, np.float32)
    lib().srfo_hashgrid_layout(C.byref(cfg), _p(off), _p(res), _p(sc))
    return off, res, sc


def num_threads():
    return int(lib().srfo_num_threads())


def set_num_threads(n=0):
    """OpenMP threads of the oracle (0: one per core this process may run on)."""
    import os
    if n <= 0:
        n = len(os.sched_getaffinity(0))
    lib().srfo_set_num_threads(C.c_int(n))
    return num_threads()


def _host_views(views: dict):
    """srf_train_views_t with host pointers from dict(n_images, width, height, focal_length, principal_point,
    xforms (n,12) float32 column-major, images (n,H,W,4) float16 or None, sampling_probability (n,H,W) float16 or
    None).  Returns (struct, keep-alive list)."""
    keep = [np.ascontiguousarray(views["xforms"], np.float32),
            None if views.get("images") is None else np.ascontiguousarray(views["images"], np.float16),
            None if views.get("sampling_probability") is None else np.ascontiguousarray(views["sampling_probability"], np.float16)]
    tv = abi.TrainViews()
    tv.n_images, tv.width, tv.height = int(views["n_images"]), int(views["width"]), int(views["height"])
    tv.focal_length[:] = [float(x) for x in views["focal_length"]]
    tv.principal_point[:] = [float(x) for x in views["principal_point"]]
    tv.d_xforms = keep[0].ctypes.data
    tv.d_images = None if keep[1] is None else keep[1].ctypes.data
    tv.d_sampling_probability = None if keep[2] is None else keep[2].ctypes.data
    return tv, keep


def mark_untrained(cfg: abi.Config, views: dict):
    tv, keep = _host_views(views)
    grid = np.zeros(cfg.grid_size ** 3 * cfg.num_cascades, np.float32)
    rc = lib().srfo_mark_untrained(C.byref(cfg), C.byref(tv), _p(grid))
    assert rc == 0
    return grid


def sample_training_rays(cfg: abi.Config, views: dict, bitfield, n_rays, n_rays_shift, n_coords, rng: Rng, snap=True):
    """Returns dict(n_rays, n_samples_total, rays (k,6), rgba (k,4), numsteps (k,2), coords (n_coords,7))."""
    tv, keep = _host_views(views)
    bits = None if bitfield is None else np.ascontiguousarray(bitfield, np.uint8)
    rc_, nc_ = C.c_uint32(0), C.c_uint32(0)
    rays = np.zeros((n_rays, 6), np.float32); rgba = np.zeros((n_rays, 4), np.float32)
    numsteps = np.zeros((n_rays, 2), np.uint32); coords = np.zeros((n_coords, 7), np.float32)
    rc = lib().srfo_sample_training_rays(C.byref(cfg), C.byref(tv), _p(bits), C.c_uint32(n_rays), C.c_uint32(n_rays_shift),
                                         C.c_uint32(n_coords), C.byref(rng), C.c_int(1 if snap else 0), C.byref(rc_),
                                         C.byref(nc_), _p(rays), _p(rgba), _p(numsteps), _p(coords))
    assert rc == 0
    k = rc_.value
    return dict(n_rays=k, n_samples_total=nc_.value, rays=rays[:k], rgba=rgba[:k], numsteps=numsteps[:k], coords=coords)


def volume_rendering_loss(cfg: abi.Config, params: "abi.LossParams", n_rays_kept, ray_coord_indices, rays_rgba, coords,
                          network_output, mean_density):
    """Serial execution of the training compositor.  Returns dict(indices (n,2), compacted_coords, n_compacted,
    dloss (capacity, width) float16, loss (n_rays,), reg (capacity, 2))."""
    idx = np.ascontiguousarray(ray_coord_indices, np.uint32).copy()
    rgba = np.ascontiguousarray(rays_rgba, np.float32)
    co = np.ascontiguousarray(coords, np.float32)
    no = np.ascontiguousarray(network_output, np.float16)
    cap, w = int(params.n_max_compacted_coords), int(params.padded_output_width)
    cc = np.zeros((cap, 7), np.float32); dl = np.zeros((cap, w), np.float16)
    loss = np.zeros(int(params.n_rays), np.float32); reg = np.zeros((cap, 2), np.float32)
    n_comp = C.c_uint32(0)
    rc = lib().srfo_volume_rendering_loss(C.byref(cfg), C.byref(params), C.c_uint32(n_rays_kept), _p(idx), _p(rgba), _p(co), _p(no),
                                          C.c_float(mean_density), _p(cc), C.byref(n_comp), _p(dl), _p(loss), _p(reg))
    assert rc == 0
    return dict(indices=idx, compacted_coords=cc, n_compacted=n_comp.value, dloss=dl, loss=loss, reg=reg)
