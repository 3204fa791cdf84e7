"""ctypes binding of oracle/_ref/libsrf_ref.so: the reference's own kernels compiled for the host.

TEST INFRASTRUCTURE.  Built by oracle/build_ref.py from the reference's sources where they are mounted; the
shared object travels with the repository (git-ignored), the sources do not.  `available()` tells whether the
library can be had here; tests that need it skip otherwise.  The field of a frame and the density of a refresh
are supplied by the CPU oracle (function pointers into libsrf_oracle*.so): the network itself lives in
tiny-cuda-nn, which is not available anywhere.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from sphericalrf_b200 import abi

from . import build_ref, srf_oracle

_libs = {}


def available(fma: bool = False) -> bool:
    try:
        return build_ref.build(fma=fma) is not None
    except Exception:
        return False


def lib(fma: bool = False):
    if fma not in _libs:
        path = build_ref.build(fma=fma)
        if path is None:
            raise RuntimeError("the reference is not mounted and oracle/_ref holds no earlier build")
        l = C.CDLL(str(path))
        l.refh_ld_random_val.restype = C.c_float
        l.refh_ld_random_val.argtypes = [C.c_uint32, C.c_uint32, C.c_uint32]
        l.refh_sobol.restype = C.c_uint32
        l.refh_sobol.argtypes = [C.c_uint32, C.c_uint32]
        _libs[fma] = l
    return _libs[fma]


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def set_num_threads(n=0):
    """OpenMP threads of the per-ray kernels (0: one per core this process may run on); returns the count in force."""
    import os
    if n <= 0:
        n = len(os.sched_getaffinity(0))
    return int(lib().refh_set_num_threads(C.c_int(n)))


def ld_random_val(index, seed, dim, fma=False):
    return np.float32(lib(fma).refh_ld_random_val(index, seed, dim))


def sobol(index, dim):
    return int(lib().refh_sobol(index, dim))


def ld_random_pixel_offset(spp, x=0, y=0):
    out = np.zeros(2, np.float32)
    lib().refh_ld_random_pixel_offset(C.c_uint32(spp), C.c_uint32(x), C.c_uint32(y), _p(out))
    return out


def warp_position(cfg, pos, inverse=False, fma=False):
    pos = np.ascontiguousarray(pos, np.float32)
    out = np.zeros_like(pos)
    lib(fma).refh_warp_position(C.byref(cfg), _p(pos), _p(out), C.c_size_t(pos.shape[0]), C.c_int(1 if inverse else 0))
    return out


def calc_dt(cfg, t, fma=False):
    t = np.ascontiguousarray(t, np.float32)
    out = np.zeros_like(t)
    lib(fma).refh_calc_dt(C.byref(cfg), _p(t), _p(out), C.c_size_t(t.size))
    return out


def grid_index(cfg, pos, fma=False):
    pos = np.ascontiguousarray(pos, np.float32)
    level = np.zeros(pos.shape[0], np.uint32); idx = np.zeros(pos.shape[0], np.uint32)
    lib(fma).refh_grid_index(C.byref(cfg), _p(pos), _p(level), _p(idx), C.c_size_t(pos.shape[0]))
    return level, idx


def tonemap(rgb, curve):
    rgb = np.ascontiguousarray(rgb, np.float32)
    out = np.zeros_like(rgb)
    lib().refh_tonemap(_p(rgb), _p(out), C.c_size_t(rgb.shape[0]), C.c_int(curve))
    return out


def srgb(x, to_linear):
    x = np.ascontiguousarray(x, np.float32)
    out = np.zeros_like(x)
    lib().refh_srgb(_p(x), _p(out), C.c_size_t(x.size), C.c_int(1 if to_linear else 0))
    return out


def loss(target, prediction, loss_type):
    t = np.ascontiguousarray(target, np.float32); p = np.ascontiguousarray(prediction, np.float32)
    l = np.zeros_like(t); g = np.zeros_like(t)
    lib().refh_loss(_p(t), _p(p), _p(l), _p(g), C.c_size_t(t.shape[0]), C.c_int(loss_type))
    return l, g


def generate_rays(cfg, view, bitfield, fma=False):
    n = view.width * view.height
    d = np.zeros((n, 3), np.float32); t = np.zeros(n, np.float32); alive = np.zeros(n, np.uint8)
    bits = None if bitfield is None else np.ascontiguousarray(bitfield, np.uint8)
    rc = lib(fma).refh_generate_rays(C.byref(cfg), C.byref(view), _p(bits), _p(d), _p(t), _p(alive))
    assert rc == 0
    return d, t, alive


def _empty_field():
    """A field that answers "nothing here": colour logits 0 and the most negative finite half as raw density, which
    the default Exponential density activation turns into density 0.  No sample has any opacity, so no ray
    saturates and every ray marches to its end (sampler parity); no pixel is hit."""
    proto = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p)
    pattern = np.array([0, 0, 0, 0xFBFF], np.uint16).tobytes()       # (0, 0, 0, -65504) as halves

    def fn(cfg, model, coords, n, out):
        C.memmove(out, pattern * int(n), 8 * int(n))
        return 0
    return proto(fn)


def render_frame(cfg, view, post, bitfield, oracle: "srf_oracle.Oracle | None", accum=None, capture=(0, 0), capacity=0,
                 fma=False):
    """Testbed::render_frame through the reference's kernels.  `oracle` supplies the network field (its model and
    whichever oracle build is active); None renders with an empty field (sampler parity: every ray runs to its
    end; needs the Exponential density activation).  Returns per-pixel arrays and, for pixels [capture[0], capture[0]+capture[1]), the emitted samples."""
    n = view.width * view.height
    out = np.zeros((n, 4), np.float32)
    acc = np.zeros((n, 4), np.float32) if accum is None else np.ascontiguousarray(accum, np.float32).copy()
    raw = np.zeros((n, 4), np.float32); ns = np.zeros(n, np.uint32); hit = np.zeros(n, np.uint8)
    cap_first, cap_count = capture
    cap_counts = np.zeros(max(cap_count, 1), np.uint32)
    cap_pos = np.zeros((max(capacity, 1), 4), np.float32)
    total = C.c_uint64(0); rounds = C.c_uint64(0)
    bits = None if bitfield is None else np.ascontiguousarray(bitfield, np.uint8)
    if oracle is None:
        keep = _empty_field()
        field, fcfg, fmodel = C.cast(keep, C.c_void_p), None, None
    else:
        keep = None
        field = C.cast(srf_oracle.lib().srfo_network_inference, C.c_void_p)
        fcfg, fmodel = C.cast(C.pointer(oracle.cfg), C.c_void_p), C.cast(C.pointer(oracle.model), C.c_void_p)
    rc = lib(fma).refh_render_frame(C.byref(cfg), C.byref(view), C.byref(post), _p(bits), field, fcfg, fmodel, _p(out), _p(acc),
                                    _p(raw), _p(ns), _p(hit), C.c_uint32(cap_first), C.c_uint32(cap_count), C.c_uint64(capacity),
                                    _p(cap_counts), _p(cap_pos), C.byref(total), C.byref(rounds))
    assert rc == 0, f"refh_render_frame returned {rc} (capture capacity {capacity}, needed {total.value})"
    return dict(out=out, accum=acc, rgba_raw=raw, n_samples=ns, hit=hit, rounds=rounds.value,
                cap_counts=cap_counts[:cap_count], cap_pos_dt=cap_pos[:total.value])


def update_grid(cfg, grid, n_uniform, n_nonuniform, rng: "srf_oracle.Rng", i_step, oracle: "srf_oracle.Oracle"):
    """sample_positions_from_grid + density + update_grid, in place on `grid`.  Returns (positions, indices, i_step)."""
    assert grid.dtype == np.float32 and grid.flags.c_contiguous
    n = n_uniform + n_nonuniform
    pos = np.zeros((n, 3), np.float32); idx = np.zeros(n, np.uint32)
    st, inc, step = C.c_uint64(rng.state), C.c_uint64(rng.inc), C.c_uint32(i_step)
    density = C.cast(srf_oracle.lib().srfo_network_density, C.c_void_p)
    rc = lib().refh_update_grid(C.byref(cfg), _p(grid), C.c_uint32(n_uniform), C.c_uint32(n_nonuniform), C.byref(st), C.byref(inc),
                                C.byref(step), density, C.cast(C.pointer(oracle.cfg), C.c_void_p),
                                C.cast(C.pointer(oracle.model), C.c_void_p), _p(pos), _p(idx))
    assert rc == 0
    rng.state, rng.inc = st.value, inc.value
    return pos, idx, step.value


def grid_to_bitfield(cfg, grid, mean):
    grid = np.ascontiguousarray(grid, np.float32)
    bits = np.zeros(grid.shape[0] // 8, np.uint8)
    rc = lib().refh_grid_to_bitfield(C.byref(cfg), _p(grid), C.c_float(mean), _p(bits))
    assert rc == 0
    return bits


def mark_untrained(cfg, views: dict):
    x = np.ascontiguousarray(views["xforms"], np.float32)
    grid = np.zeros(cfg.grid_size ** 3 * cfg.num_cascades, np.float32)
    focal = np.asarray(views["focal_length"], np.float32)
    rc = lib().refh_mark_untrained(C.byref(cfg), C.c_uint32(int(views["n_images"])), C.c_int(int(views["width"])),
                                   C.c_int(int(views["height"])), _p(focal), _p(x), _p(grid))
    assert rc == 0
    return grid


def sample_training_rays(cfg, views: dict, bitfield, n_rays, n_rays_shift, n_coords, rng: "srf_oracle.Rng", snap=True):
    """generate_training_samples_nerf with threads in index order; same result layout as the oracle's function."""
    x = np.ascontiguousarray(views["xforms"], np.float32)
    img = np.ascontiguousarray(views["images"], np.float16)
    prob = views.get("sampling_probability")
    if prob is None:
        prob = np.ones((int(views["n_images"]), int(views["height"]), int(views["width"])), np.float16)   # the reference always reads one
    prob = np.ascontiguousarray(prob, np.float16)
    bits = None if bitfield is None else np.ascontiguousarray(bitfield, np.uint8)
    focal = np.asarray(views["focal_length"], np.float32); pp = np.asarray(views["principal_point"], np.float32)
    rc_, nc_ = C.c_uint32(0), C.c_uint32(0)
    rays = np.zeros((n_rays, 6), np.float32); rgba = np.zeros((n_rays, 4), np.float32)
    numsteps = np.zeros((n_rays, 2), np.uint32); coords = np.zeros((n_coords, 7), np.float32)
    rc = lib().refh_sample_training_rays(C.byref(cfg), _p(bits), C.c_uint32(n_rays), C.c_uint32(n_rays_shift), C.c_uint32(n_coords),
                                         C.c_uint32(int(views["n_images"])), C.c_int(int(views["width"])), C.c_int(int(views["height"])),
                                         _p(focal), _p(pp), _p(x), _p(img), _p(prob), C.c_uint64(rng.state), C.c_uint64(rng.inc),
                                         C.c_int(1 if snap else 0), C.byref(rc_), C.byref(nc_), _p(rays), _p(rgba), _p(numsteps),
                                         _p(coords))
    assert rc == 0
    k = rc_.value
    return dict(n_rays=k, n_samples_total=nc_.value, rays=rays[:k], rgba=rgba[:k], numsteps=numsteps[:k], coords=coords)


def volume_rendering_loss(cfg, params, n_rays_kept, ray_coord_indices, rays_rgba, coords, network_output, mean_density):
    """volume_rendering_with_loss_and_gradient_kernal with threads in index order; the oracle's result layout."""
    idx = np.ascontiguousarray(ray_coord_indices, np.uint32).copy()
    rgba = np.ascontiguousarray(rays_rgba, np.float32)
    co = np.ascontiguousarray(coords, np.float32)
    no = np.ascontiguousarray(network_output, np.float16)
    cap, w = int(params.n_max_compacted_coords), int(params.padded_output_width)
    cc = np.zeros((cap, 7), np.float32); dl = np.zeros((cap, w), np.float16)
    loss_out = np.zeros(int(params.n_rays), np.float32); reg = np.zeros((cap, 2), np.float32)
    n_comp = C.c_uint32(0)
    rc = lib().refh_volume_rendering_loss(C.byref(cfg), C.byref(params), C.c_uint32(n_rays_kept), _p(idx), _p(rgba), _p(co), _p(no),
                                          C.c_float(mean_density), _p(cc), C.byref(n_comp), _p(dl), _p(loss_out), _p(reg))
    assert rc == 0
    return dict(indices=idx, compacted_coords=cc, n_compacted=n_comp.value, dloss=dl, loss=loss_out, reg=reg)
