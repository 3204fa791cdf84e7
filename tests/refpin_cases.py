"""Cases that pin the CPU oracle to the reference's own source.

Every case is computed twice: by `backend="reference"` -- the reference's kernels compiled for the host
(oracle/srf_ref.py, built from the reference's sources where they are mounted) -- and by `backend="oracle"` -- the
oracle in its plain-arithmetic build (the C library's elementary functions, no fused multiply-adds), which is the
arithmetic such a host compile performs.  The two must agree bit for bit.  tests/golden/make_ref_golden.py stores
the reference side as a fixture (large arrays as CRC-32 digests), so the comparison also runs where the reference
is not mounted.
"""
import ctypes as C
import zlib

import numpy as np

from helpers import make_oracle, small_scene
from sphericalrf_b200 import abi, synth


def digest(a):
    """CRC-32 of an array's bytes plus its length, as a small uint64 array."""
    a = np.ascontiguousarray(a)
    return np.array([zlib.crc32(a.tobytes()), a.size], dtype=np.uint64)


SAMPLER_CASES = {
    "disparity_erp": dict(sampling="Disparity", warp=abi.WARP_ERP),
    "original_erp": dict(sampling="Original", warp=abi.WARP_ERP, radius=4.0),
    "log_sinusoidal": dict(sampling="Log", warp=abi.WARP_SINUSOIDAL, aabb_scale=64),
    "original_ngp": dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.2),
    "original_mipnerf360": dict(sampling="Original", warp=abi.WARP_MIPNERF360, aabb_scale=8, radius=1.5),
    "original_donerf": dict(sampling="Original", warp=abi.WARP_DONERF, aabb_scale=4, radius=1.5),
    "original_sigmoid": dict(sampling="Original", warp=abi.WARP_SIGMOID, aabb_scale=8, radius=2.0),
    "ngp_3cascades_exp": dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=3, grid_dist=abi.GRID_WARPED_EXP),
    "ngp_2cascades_metric_reciprocal": dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=2,
                                            grid_dist=abi.GRID_METRIC_RECIPROCAL),
    "ngp_2cascades_metric_exp": dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=2,
                                     grid_dist=abi.GRID_METRIC_EXP),
    "erp_2cascades_reciprocal": dict(sampling="Disparity", warp=abi.WARP_ERP, cascades=2, grid_dist=abi.GRID_WARPED_RECIPROCAL),
}


def _scene(case, kind="net"):
    kw = dict(case)
    sampling = kw.pop("sampling")
    sc = small_scene(kind=kind, sampling="Disparity" if sampling == "Log" else sampling, **kw)
    if sampling == "Log":
        sc["cfg"].sampling_type = abi.SAMPLING_LOG
        sc["cfg"].far_distance = 100.0
    return sc


def _bitfield(oracle_mod, sc):
    """Input preparation (same bytes for both backends): the canonical oracle's thresholding of the grid."""
    return make_oracle(oracle_mod, sc, None).update_grid_bitfield(sc["grid"])[0]


def sampler_case(name, backend, oracle_mod, ref_mod):
    """Rays (direction, t, alive) and every sample of every ray (count, warped position, dt)."""
    sc = _scene(SAMPLER_CASES[name])
    cfg, view = sc["cfg"], sc["view"]
    bits = _bitfield(oracle_mod, sc)
    n = view.width * view.height
    cap = 1 << 23
    if backend == "reference":
        d, t, alive = ref_mod.generate_rays(cfg, view, bits)
        res = ref_mod.render_frame(cfg, view, abi.default_post(), bits, None, capture=(0, n), capacity=cap)
        counts, pos_dt = res["cap_counts"], res["cap_pos_dt"]
        # A ray whose step width reaches 0 inside an occupied cell emits zero-width samples until the reference's
        # frame loop gives up (MARCH_ITER); the oracle ends such a ray at its first zero-width step.  Zero-width
        # samples carry no opacity, so they are dropped here before comparing.
        ray_of = np.repeat(np.arange(n), counts)
        keep = pos_dt[:, 3] != 0
        counts = np.bincount(ray_of[keep], minlength=n).astype(np.uint32)
        pos_dt = pos_dt[keep]
    else:
        with oracle_mod.plain_arithmetic():
            orc = make_oracle(oracle_mod, sc, bits)
            d, t, alive, _ = orc.generate_rays(view)
            counts, pos_dt, _, _, _ = orc.march(view, 0, n, cap)
    live = alive > 0
    return {"alive": alive, "dir": digest(d[live]), "t": digest(t[live]), "counts": counts.astype(np.uint32),
            "pos_dt": digest(pos_dt)}


FRAME_CASES = {
    # name: (scene kwargs, config overrides, view overrides, post overrides, spp passes)
    "shade": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, {}, {}, 1),
    "shade_linear_training": (dict(sampling="Disparity", warp=abi.WARP_ERP), dict(train_in_linear_color=1), {}, {}, 1),
    "depth": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, dict(render_mode=abi.MODE_DEPTH, depth_scale=0.5), {}, 1),
    "distance": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, dict(render_mode=abi.MODE_DISTANCE, depth_scale=0.25), {}, 1),
    "ao": (dict(sampling="Original", warp=abi.WARP_ERP, radius=4.0), {}, dict(render_mode=abi.MODE_AO), {}, 1),
    "cost": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, dict(render_mode=abi.MODE_COST), {}, 1),
    "early_termination": (dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.2),
                          dict(transmittance_threshold=0.2, density_activation=abi.ACT_EXPONENTIAL), {}, {}, 1),
    "relu_none_activations": (dict(sampling="Disparity", warp=abi.WARP_ERP),
                              dict(density_activation=abi.ACT_RELU, rgb_activation=abi.ACT_NONE), {}, {}, 1),
    "exp_rgb_logistic_density": (dict(sampling="Disparity", warp=abi.WARP_ERP),
                                 dict(density_activation=abi.ACT_LOGISTIC, rgb_activation=abi.ACT_EXPONENTIAL), {}, {}, 1),
    "spp3_jittered": (dict(sampling="Disparity", warp=abi.WARP_ERP), dict(snap_to_pixel_centers_in_rendering=0), {}, {}, 3),
    "aces_srgb_out": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, {},
                      dict(tonemap_curve=abi.TONEMAP_ACES, to_srgb=1, exposure=0.7, background_color=(0.3, 0.6, 0.1, 1.0)), 1),
    "hable": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, {},
              dict(tonemap_curve=abi.TONEMAP_HABLE, exposure=-0.4, background_color=(1.0, 1.0, 1.0, 0.5)), 1),
    "reinhard_srgb_space": (dict(sampling="Disparity", warp=abi.WARP_ERP), {}, {},
                            dict(tonemap_curve=abi.TONEMAP_REINHARD, color_space=abi.COLOR_SRGB, to_srgb=1), 2),
    "visposneg": (dict(sampling="Disparity", warp=abi.WARP_ERP), dict(snap_to_pixel_centers_in_rendering=0), {},
                  dict(color_space=abi.COLOR_VISPOSNEG), 3),
}


def frame_case(name, backend, oracle_mod, ref_mod):
    """A rendered frame: pre-shade premultiplied RGBA per pixel, emitted samples per pixel, the output image after
    `spp` accumulated passes."""
    skw, cfg_over, view_over, post_over, spp = FRAME_CASES[name]
    sc = _scene(skw)
    cfg = sc["cfg"]
    for k, v in cfg_over.items():
        setattr(cfg, k, v)
    bits = _bitfield(oracle_mod, sc)
    post = abi.default_post()
    for k, v in post_over.items():
        if k == "background_color":
            post.background_color[:] = list(v)
        else:
            setattr(post, k, v)
    v0 = sc["view"]
    cam = [v0.camera[i] for i in range(12)]
    out = {}
    accum = None
    with oracle_mod.plain_arithmetic():
        orc = make_oracle(oracle_mod, sc, bits)          # also the field of the reference backend
        for i in range(spp):
            view = abi.make_view(cam, v0.width, v0.height, (v0.relative_focal_length[0], v0.relative_focal_length[1]),
                                 spp_index=i, render_mode=view_over.get("render_mode", abi.MODE_SHADE),
                                 depth_scale=view_over.get("depth_scale", 1.0))
            if backend == "reference":
                res = ref_mod.render_frame(cfg, view, post, bits, orc, accum=accum)
            else:
                res = orc.render_frame(view, post, accum=accum)
            accum = res["accum"]
            out[f"rgba_raw_{i}"] = res["rgba_raw"].copy()
            out[f"out_{i}"] = res["out"].copy()
            if backend == "reference":
                out[f"hit_{i}"] = np.array([int(res["hit"].sum())], np.uint64)
            else:
                out[f"hit_{i}"] = np.array([int(res["stats"]["n_rays_hit"])], np.uint64)
    return out


REFRESH_CASES = {
    # name: (scene kwargs, [training_step of each consecutive refresh])
    "all_cells_erp": (dict(sampling="Disparity", warp=abi.WARP_ERP, grid_size=16), [0, 16, 32]),
    "quarter_mode_erp": (dict(sampling="Disparity", warp=abi.WARP_ERP, grid_size=16), [0, 256, 272]),
    "ngp_2cascades_metric_exp": (dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=2,
                                      grid_dist=abi.GRID_METRIC_EXP, grid_size=16), [0, 300]),
    "ngp_2cascades_warped_reciprocal": (dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=2,
                                             grid_dist=abi.GRID_WARPED_RECIPROCAL, grid_size=16), [0, 300]),
}


def refresh_case(name, backend, oracle_mod, ref_mod):
    """Consecutive density-grid refreshes: the grid after every step, and the bitfield the reference's bit-packing
    kernels make of it for the oracle's mean (the mean's summation order belongs to tiny-cuda-nn)."""
    skw, steps = REFRESH_CASES[name]
    sc = _scene(skw)
    cfg = sc["cfg"]
    grid = (sc["grid"] * np.float32(0.002)).astype(np.float32)      # optical-thickness units, straddling the 0.01 threshold
    grid[::97] = -1.0                                                # cells a mask marked as never seen
    rng = oracle_mod.rng_seed(3001)
    total = grid.shape[0]
    out = {}
    with oracle_mod.plain_arithmetic():
        orc = make_oracle(oracle_mod, sc, None)
        i_step = 0
        for k, tstep in enumerate(steps):
            if backend == "reference":
                n_uni = total // 4 if tstep >= 256 else total
                n_non = total // 4 if tstep >= 256 else 0
                _, _, i_step = ref_mod.update_grid(cfg, grid, n_uni, n_non, rng, i_step, orc)
                _, mean = orc.update_grid_bitfield(grid)             # the oracle's mean of the reference's grid
                bits = ref_mod.grid_to_bitfield(cfg, grid, float(mean))
            else:
                bits, mean, i_step = orc.refresh(grid, i_step, tstep, rng)
            out[f"grid_{k}"] = grid.copy()
            out[f"bits_{k}"] = bits.copy()
            out[f"rng_{k}"] = np.array([rng.state, rng.inc], np.uint64)
    return out


TRAIN_CASES = {
    "erp_disparity": dict(warp=abi.WARP_ERP, sampling="Disparity"),
    "ngp_original_cascades": dict(warp=abi.WARP_NGP, sampling="Original", cascades=2, grid_dist=abi.GRID_WARPED_EXP, aabb_scale=4),
    "no_grid": dict(warp=abi.WARP_ERP, sampling="Disparity", use_grid=False),
}


def training_case(name, backend, oracle_mod, ref_mod):
    """Training rays (kept rays, counts and bases, pixel colours, every Coordinate) followed by the loss/gradient
    compositor on them, for two losses."""
    kw = dict(TRAIN_CASES[name])
    use_grid = kw.pop("use_grid", True)
    sampling = kw["sampling"]
    sc = small_scene(kind="net", radius=0.5 if sampling == "Disparity" else 4.0, **kw)
    cfg = sc["cfg"]
    cfg.use_grid = 1 if use_grid else 0
    cfg.maximum_marching_steps = 96
    views = synth.training_views(31, n_images=5, width=28, height=20, radius=0.4 if sampling == "Disparity" else 3.0)
    bits = _bitfield(oracle_mod, sc)
    n_rays, n_coords = 200, 9000                                     # small enough that late rays find no room
    rng = oracle_mod.rng_seed(5)
    out = {}
    with oracle_mod.plain_arithmetic():
        orc = make_oracle(oracle_mod, sc, bits)
        mod = ref_mod if backend == "reference" else oracle_mod
        s = mod.sample_training_rays(cfg, views, bits, n_rays, 3, n_coords, rng, snap=True)
        k = s["n_rays"]
        used = int(min(s["n_samples_total"], n_coords))
        out["n_rays"] = np.array([k, s["n_samples_total"]], np.uint64)
        out["rays"] = s["rays"].copy(); out["rgba"] = s["rgba"].copy(); out["numsteps"] = s["numsteps"].copy()
        kept = int((s["numsteps"][:, 0].astype(np.int64)).sum())
        out["coords"] = digest(s["coords"][:kept] if k and int(s["numsteps"][:, 1].max()) < kept else s["coords"])
        net = orc.network_inference(s["coords"][:max(used, 1)])
        for loss_type, space, reg in ((abi.LOSS_L2, abi.COLOR_LINEAR, abi.REG_NONE), (abi.LOSS_SMOOTH_L1, abi.COLOR_SRGB, abi.REG_DISTORTION)):
            p = abi.LossParams()
            p.n_rays, p.n_max_compacted_coords, p.loss_type, p.loss_scale = n_rays, 6000, loss_type, 128.0
            p.regularization_type = reg
            p.background_color[:] = [0.2, 0.5, 0.9]
            p.color_space = space
            p.train_with_random_bg_color = 1 if reg == abi.REG_DISTORTION else 0
            p.rng_state, p.rng_inc = 0x853c49e6748fea9b, 0xda3e39cb94b95bdb
            p.padded_output_width = 4
            r = mod.volume_rendering_loss(cfg, p, k, s["numsteps"], s["rgba"], s["coords"], net, 0.004)
            m = min(r["n_compacted"], 6000)
            tag = f"loss{loss_type}"
            out[tag + "_indices"] = r["indices"][:k].copy()
            out[tag + "_n"] = np.array([r["n_compacted"]], np.uint64)
            out[tag + "_coords"] = digest(r["compacted_coords"][:m])
            out[tag + "_dloss"] = digest(r["dloss"][:m])
            out[tag + "_dloss_head"] = r["dloss"][:min(m, 256)].view(np.uint16).copy()
            out[tag + "_loss"] = r["loss"][:k].copy()
            if reg == abi.REG_DISTORTION:
                out[tag + "_reg"] = digest(r["reg"][:m])
                out[tag + "_reg_head"] = r["reg"][:min(m, 256)].copy()
    return out


def mask_case(name, backend, oracle_mod, ref_mod):
    """mark_untrained_density_grid for the four grid distributions."""
    dist = {"warped_exp": abi.GRID_WARPED_EXP, "warped_reciprocal": abi.GRID_WARPED_RECIPROCAL,
            "metric_exp": abi.GRID_METRIC_EXP, "metric_reciprocal": abi.GRID_METRIC_RECIPROCAL}[name]
    sc = small_scene(kind="blobs", sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, cascades=2, grid_dist=dist, grid_size=16)
    views = synth.training_views(32, n_images=3, width=28, height=20, radius=2.5)
    with oracle_mod.plain_arithmetic():
        grid = (ref_mod if backend == "reference" else oracle_mod).mark_untrained(sc["cfg"], views)
    return {"grid": grid}


def taps_case(name, backend, oracle_mod, ref_mod):
    """Scalar functions on seeded inputs: the low-discrepancy jitter, the warps and their inverses, the three step-size
    laws, cell indices, tonemap curves, the sRGB pair."""
    rng = np.random.default_rng(11)
    out = {}
    if name == "jitter":
        idx = rng.integers(0, 2 ** 32, 300, dtype=np.uint64)
        seeds = rng.integers(0, 2 ** 32, 300, dtype=np.uint64)
        if backend == "reference":
            out["ld0"] = np.array([ref_mod.ld_random_val(int(i), int(s), 0) for i, s in zip(idx, seeds)], np.float32)
            out["ld1"] = np.array([ref_mod.ld_random_val(int(i), int(s), 1) for i, s in zip(idx, seeds)], np.float32)
            out["sobol1"] = np.array([ref_mod.sobol(int(i), 1) for i in idx], np.uint32)
            out["offset"] = np.stack([ref_mod.ld_random_pixel_offset(s) for s in range(8)])
        else:
            L = oracle_mod.lib()
            L.srfo_ld_random_val.restype = C.c_float
            L.srfo_sobol.restype = C.c_uint32
            out["ld0"] = np.array([L.srfo_ld_random_val(C.c_uint32(int(i)), C.c_uint32(int(s)), C.c_uint32(0)) for i, s in zip(idx, seeds)], np.float32)
            out["ld1"] = np.array([L.srfo_ld_random_val(C.c_uint32(int(i)), C.c_uint32(int(s)), C.c_uint32(1)) for i, s in zip(idx, seeds)], np.float32)
            out["sobol1"] = np.array([L.srfo_sobol(C.c_uint32(int(i)), C.c_uint32(1)) for i in idx], np.uint32)
            out["offset"] = np.stack([oracle_mod.pixel_offset(s) for s in range(8)])
        return out
    if name == "warps":
        pos = (rng.random((1200, 3)) * 6 - 2.5).astype(np.float32)
        unit = rng.random((1200, 3)).astype(np.float32) * np.float32(0.98) + np.float32(0.01)
        mod = ref_mod if backend == "reference" else oracle_mod
        with oracle_mod.plain_arithmetic():
            for w in range(6):
                cfg = synth.sampler_config("Original", 32)
                cfg.warping_type = w
                cfg.aabb_scale = 8
                out[f"warp{w}"] = mod.warp_position(cfg, pos)
                out[f"unwarp{w}"] = mod.warp_position(cfg, unit, inverse=True)
        return out
    if name == "calc_dt":
        t = np.exp(rng.uniform(np.log(0.05), np.log(2e6), 2000)).astype(np.float32)
        mod = ref_mod if backend == "reference" else oracle_mod
        with oracle_mod.plain_arithmetic():
            for st, nm in ((abi.SAMPLING_ORIGINAL, "original"), (abi.SAMPLING_DISPARITY, "disparity"), (abi.SAMPLING_LOG, "log")):
                cfg = synth.sampler_config("Disparity", 32)
                cfg.sampling_type = st
                cfg.cone_angle_constant = 0.004 if st == abi.SAMPLING_ORIGINAL else 0.0
                if st == abi.SAMPLING_LOG:
                    cfg.far_distance = 100.0
                out[nm] = mod.calc_dt(cfg, t)
        return out
    if name == "cells":
        pos = (rng.random((2000, 3)) * 3.8 - 1.4).astype(np.float32)      # inside the box of aabb_scale 4
        mod = ref_mod if backend == "reference" else oracle_mod
        with oracle_mod.plain_arithmetic():
            for w, casc, dist in ((abi.WARP_ERP, 1, abi.GRID_WARPED_EXP), (abi.WARP_NGP, 3, abi.GRID_WARPED_EXP),
                                  (abi.WARP_NGP, 3, abi.GRID_WARPED_RECIPROCAL), (abi.WARP_MIPNERF360, 2, abi.GRID_METRIC_EXP),
                                  (abi.WARP_SIGMOID, 2, abi.GRID_METRIC_RECIPROCAL)):
                cfg = synth.sampler_config("Original", 64)
                cfg.warping_type, cfg.num_cascades, cfg.grid_distribution_type, cfg.aabb_scale = w, casc, dist, 4
                level, idx = mod.grid_index(cfg, pos)
                out[f"level_{w}_{casc}_{dist}"] = level
                out[f"idx_{w}_{casc}_{dist}"] = idx
        return out
    if name == "output_stage":
        rgb = (rng.random((1000, 3)) * 4 - 0.5).astype(np.float32)
        x = (rng.random(1000) * 1.5 - 0.1).astype(np.float32)
        mod = ref_mod if backend == "reference" else oracle_mod
        with oracle_mod.plain_arithmetic():
            for curve in range(4):
                out[f"tonemap{curve}"] = mod.tonemap(rgb, curve)
            out["to_linear"] = mod.srgb(x, True)
            out["to_srgb"] = mod.srgb(x, False)
        return out
    if name == "losses":
        t = rng.random((1000, 3)).astype(np.float32)
        p = (rng.random((1000, 3)) * 1.4 - 0.2).astype(np.float32)
        mod = ref_mod if backend == "reference" else oracle_mod
        with oracle_mod.plain_arithmetic():
            for lt in range(7):
                l, g = mod.loss(t, p, lt)
                out[f"loss{lt}"] = l; out[f"grad{lt}"] = g
        return out
    raise KeyError(name)


TAPS = ["jitter", "warps", "calc_dt", "cells", "output_stage", "losses"]
MASKS = ["warped_exp", "warped_reciprocal", "metric_exp", "metric_reciprocal"]

# (group, case name, function)
ALL_CASES = ([("sampler", n, sampler_case) for n in SAMPLER_CASES] + [("frame", n, frame_case) for n in FRAME_CASES] +
             [("refresh", n, refresh_case) for n in REFRESH_CASES] + [("training", n, training_case) for n in TRAIN_CASES] +
             [("mask", n, mask_case) for n in MASKS] + [("taps", n, taps_case) for n in TAPS])


def compare(got: dict, want: dict, label: str):
    """Bit-for-bit equality of two result dictionaries; raises AssertionError naming the first difference."""
    assert sorted(got) == sorted(want), f"{label}: keys differ: {sorted(got)} vs {sorted(want)}"
    for k in sorted(want):
        a, b = np.ascontiguousarray(got[k]), np.ascontiguousarray(want[k])
        assert a.shape == b.shape and a.dtype == b.dtype, f"{label}/{k}: {a.dtype}{a.shape} vs {b.dtype}{b.shape}"
        if a.tobytes() != b.tobytes():
            if a.dtype.kind == "f":
                both_nan = np.isnan(a) & np.isnan(b)
                bad = ~both_nan & (a.view(f"u{a.itemsize}") != b.view(f"u{b.itemsize}"))
                if not bad.any():
                    continue
                diff = np.abs(a.astype(np.float64) - b.astype(np.float64))[bad]
                raise AssertionError(f"{label}/{k}: {int(bad.sum())} of {a.size} values differ, max |d| = {np.nanmax(diff):.3e}")
            raise AssertionError(f"{label}/{k}: {int((a != b).sum())} of {a.size} values differ")
