"""Seed-generated inputs that stand in for the datasets and trained snapshots the reference
is evaluated on (none of which ship with it): Gaussian-blob scenes, occupancy grids,
cameras on orbits, and random-initialised network parameters of the reference's shape.

Everything here produces INPUTS (arrays uploaded to the library and handed to the test
oracle alike); nothing here defines expected outputs.
"""
from __future__ import annotations

import math

import numpy as np

from . import abi

CENTER = np.array([0.5, 0.5, 0.5], dtype=np.float64)


# ---- Morton order (x -> bit 0, y -> bit 1, z -> bit 2), as the reference's grids use ---------
def _expand_bits(v):
    v = v.astype(np.uint64)
    v = (v * np.uint64(0x00010001)) & np.uint64(0xFF0000FF)
    v = (v * np.uint64(0x00000101)) & np.uint64(0x0F00F00F)
    v = (v * np.uint64(0x00000011)) & np.uint64(0xC30C30C3)
    v = (v * np.uint64(0x00000005)) & np.uint64(0x49249249)
    return v


def morton3d(x, y, z):
    return (_expand_bits(x) | (_expand_bits(y) << np.uint64(1)) | (_expand_bits(z) << np.uint64(2))).astype(np.uint32)


def morton3d_invert(m):
    x = m.astype(np.uint64) & np.uint64(0x49249249)
    x = (x | (x >> np.uint64(2))) & np.uint64(0xC30C30C3)
    x = (x | (x >> np.uint64(4))) & np.uint64(0x0F00F00F)
    x = (x | (x >> np.uint64(8))) & np.uint64(0xFF0000FF)
    x = (x | (x >> np.uint64(16))) & np.uint64(0x0000FFFF)
    return x.astype(np.uint32)


# ---- cameras ----------------------------------------------------------------------------------
def orbit_camera(radius, elevation_deg, azimuth_deg, scene_scale=1.0, scene_offset=(0.5, 0.5, 0.5)):
    """Camera-to-world 3x4 in the library's internal convention.

    Pose rule of the reference's trajectory generator (look at the centre, +z up:
    script/trajectory/generate_spherical_trajectory.py:22-51), then the conversion
    Testbed::set_nerf_camera_matrix applies (negate columns 1 and 2, scale and offset the
    position: internal/utils/common_device.h:123-141)."""
    el, az = math.radians(elevation_deg), math.radians(azimuth_deg)
    center = np.array([radius * math.cos(el) * math.cos(az), radius * math.cos(el) * math.sin(az),
                       radius * math.sin(el)], dtype=np.float32)
    up = np.array([0.0, 0.0, 1.0], dtype=np.float32)
    norm = lambda v: v / np.linalg.norm(v)
    lookat = norm(-center)
    right = norm(np.cross(lookat, up))
    up = norm(np.cross(right, lookat))
    c2w = np.stack([right, up, -lookat, center], axis=-1).astype(np.float32)   # 3x4, OpenGL style
    ocv = c2w.copy()
    ocv[:, 1] *= -1.0
    ocv[:, 2] *= -1.0
    ocv[:, 3] = ocv[:, 3] * np.float32(scene_scale) + np.asarray(scene_offset, dtype=np.float32)
    return ocv.astype(np.float32)


def relative_focal_length(fov_x_deg, width, height):
    """Testbed::set_fov_xy with fov_y = fov_x / aspect, as the reference's predict driver sets it
    (experiment/srf_mipnerf360/python/run.py:232-235; internal/utils/common_device.h:105-111)."""
    fx = math.radians(fov_x_deg)
    fy = fx / (float(width) / float(height))
    return (np.float32(0.5) / np.float32(math.tan(0.5 * fx)), np.float32(0.5) / np.float32(math.tan(0.5 * fy)))


# ---- blob scenes ------------------------------------------------------------------------------
def blob_scene(seed, n_blobs=32, peak=50.0, ball_radius=3.0, sigma_range=(0.05, 0.3)):
    """n blobs (cx, cy, cz, sigma, peak): centres uniform in a ball around the scene centre."""
    rng = np.random.Generator(np.random.PCG64(seed))
    d = rng.normal(size=(n_blobs, 3))
    d /= np.linalg.norm(d, axis=1, keepdims=True)
    r = ball_radius * rng.random(n_blobs) ** (1.0 / 3.0)
    c = CENTER[None, :] + d * r[:, None]
    sig = rng.uniform(sigma_range[0], sigma_range[1], size=n_blobs)
    out = np.zeros((n_blobs, 5), dtype=np.float32)
    out[:, :3] = c
    out[:, 3] = sig
    out[:, 4] = peak
    return out


def color_map(seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.uniform(-1.0, 1.0, size=(3, 3)).astype(np.float32)


def blob_density(blobs, x):
    """Density of the blob field at float64 points x (n,3)."""
    out = np.zeros(x.shape[0], dtype=np.float64)
    for b in blobs.astype(np.float64):
        d2 = ((x - b[None, :3]) ** 2).sum(axis=1)
        out += b[4] * np.exp(-0.5 * d2 / (b[3] * b[3]))
    return out


def unwarp_cell_centers(cfg: abi.Config):
    """Metric-space position of every grid cell centre, in Morton order (float64).

    Inverse of the reference's warps (internal/utils/common_device.h:455-526); "ERP" behaves as
    the sinusoidal projection there because its case lacks a break."""
    n = cfg.grid_size
    m = np.arange(n ** 3, dtype=np.uint32)
    gx, gy, gz = morton3d_invert(m), morton3d_invert(m >> np.uint32(1)), morton3d_invert(m >> np.uint32(2))
    w = (np.stack([gx, gy, gz], axis=1).astype(np.float64) + 0.5) / n
    wt = cfg.warping_type
    if wt in (abi.WARP_ERP, abi.WARP_SINUSOIDAL):
        phi = (w[:, 1] - 0.5) * math.pi
        theta = (w[:, 0] - 0.5) * 2.0 * math.pi / np.cos(phi)
        r = w[:, 2] * 2.0
        r = np.where(r <= 1.0, r, 1.0 / np.maximum(2.0 - r, 1e-12))
        x = np.stack([r * np.cos(phi) * np.cos(theta), r * np.cos(phi) * np.sin(theta), r * np.sin(phi)], axis=1) + 0.5
        reachable = np.abs(w[:, 0] - 0.5) <= 0.5 * np.cos(phi)
        return x, reachable
    if wt == abi.WARP_NGP:
        amount = 0.5 * cfg.aabb_scale
        return (0.5 - amount) + w * (2.0 * amount), np.ones(len(w), dtype=bool)
    if wt == abi.WARP_MIPNERF360:
        z = (w - 0.5) * 4.0
        mag = np.linalg.norm(z, axis=1, keepdims=True)
        x = np.where(mag <= 1.0, z, z / np.maximum(mag, 1e-12) / np.maximum(2.0 - mag, 1e-12))
        return x * 0.5 + 0.5, np.ones(len(w), dtype=bool)
    raise ValueError("unwarp_cell_centers: warp type not covered by the generators")


def density_grid_from_blobs(cfg: abi.Config, blobs, scale=1.0, chunk=1 << 18):
    """float32 density grid (Morton order): blob density at each unwarped cell centre x scale."""
    x, reachable = unwarp_cell_centers(cfg)
    out = np.empty(x.shape[0], dtype=np.float32)
    for s in range(0, x.shape[0], chunk):
        out[s:s + chunk] = (blob_density(blobs, x[s:s + chunk]) * scale).astype(np.float32)
    return out, reachable


def bitfield_from_grid(cfg: abi.Config, grid):
    """Host restatement of the thresholding rule for GENERATING inputs only (value > min(thr, mean),
    8 cells per byte). Tests take the bitfield from the oracle or the library, not from here."""
    mean = np.maximum(grid.astype(np.float64), 0.0).mean()
    thr = min(float(cfg.min_optical_thickness), mean)
    bits = (grid > np.float32(thr)).astype(np.uint8).reshape(-1, 8)
    return (bits << np.arange(8, dtype=np.uint8)[None, :]).sum(axis=1).astype(np.uint8)


# ---- network parameters -----------------------------------------------------------------------
def hashgrid_layout(cfg: abi.Config):
    """(offsets[L+1], resolutions[L], scales[L]); same rule as srf_hashgrid_layout."""
    pls = cfg.per_level_scale
    if pls <= 0 and cfg.n_levels > 1:
        pls = float(np.exp(np.log(np.float32(cfg.desired_resolution) / np.float32(cfg.base_resolution)) / np.float32(cfg.n_levels - 1)))
    pls = float(np.float32(pls))
    offsets, res, scales = [0], [], []
    T = 1 << cfg.log2_hashmap_size
    for l in range(cfg.n_levels):
        s = np.float32(float(cfg.base_resolution) * math.pow(pls, l) - 1.0)
        r = int(math.ceil(float(s))) + 1
        n = min(T, (r ** 3 + 7) // 8 * 8)
        offsets.append(offsets[-1] + n)
        res.append(r)
        scales.append(s)
    return np.array(offsets, dtype=np.uint32), np.array(res, dtype=np.uint32), np.array(scales, dtype=np.float32)


def network_params(cfg: abi.Config, seed_table, seed_mlp, table_range=1e-4):
    """Random-init parameters: hash table ~ U(-r, r), MLPs Xavier-uniform, all fp16.
    Returns (hash_table[n_entries*F], density_mlp[64*32+16*64], rgb_mlp[64*32+64*64+16*64])."""
    offsets, _, _ = hashgrid_layout(cfg)
    n = int(offsets[-1]) * cfg.n_features_per_level
    rng = np.random.Generator(np.random.PCG64(seed_table))
    table = rng.uniform(-table_range, table_range, size=n).astype(np.float16)
    rng = np.random.Generator(np.random.PCG64(seed_mlp))

    def xavier(n_out, n_in):
        a = math.sqrt(6.0 / (n_in + n_out))
        return rng.uniform(-a, a, size=(n_out, n_in)).astype(np.float16)

    density = np.concatenate([xavier(64, 32).ravel(), xavier(16, 64).ravel()])
    rgb = np.concatenate([xavier(64, 32).ravel(), xavier(64, 64).ravel(), xavier(16, 64).ravel()])
    return table, density, rgb


# ---- the benchmark configurations -------------------------------------------------------------
def sampler_config(sampling="Disparity", grid_size=128):
    """Sampler settings shared by the seed-generated configurations: the "ERP" warp of every
    shipped config, one cascade, and the reference's pairing of sampling type and box size
    (Original with a small box, Disparity with the 360-degree settings of srf_garden.json)."""
    c = abi.default_config()
    c.warping_type = abi.WARP_ERP
    c.grid_size = grid_size
    c.num_cascades = 1
    c.grid_distribution_type = abi.GRID_WARPED_EXP
    c.maximum_marching_steps = 1024
    if sampling == "Original":
        c.sampling_type = abi.SAMPLING_ORIGINAL
        c.aabb_scale = 16
        c.near_distance, c.far_distance = 0.2, 100.0
    else:
        c.sampling_type = abi.SAMPLING_DISPARITY
        c.aabb_scale = 2000000
        c.near_distance, c.far_distance = 0.1, 1e6
    return c


def scene_config0(variant="D", grid_size=128, width=800, height=800):
    """Sampler + compositing only, analytic blob field in fp32.  Variant "X" is variant "O" with the blob
    densities raised 80-fold after the grid is built: an opaque scene, as a trained one is, where every ray that
    meets a blob saturates inside it (same bitfield and march as "O", early termination everywhere)."""
    cfg = sampler_config("Disparity" if variant == "D" else "Original", grid_size)
    cfg.field_type = abi.FIELD_BLOBS
    cfg.density_activation = abi.ACT_NONE
    cfg.rgb_activation = abi.ACT_LOGISTIC
    blobs = blob_scene(1000, 32, 50.0)
    cmap = color_map(1001)
    grid, reachable = density_grid_from_blobs(cfg, blobs)
    if variant == "X":
        blobs = blobs.copy()
        blobs[:, 4] *= 80.0
    cam = orbit_camera(4.0, 20.0, 30.0)
    rfl = relative_focal_length(50.0, width, height)
    return dict(cfg=cfg, blobs=blobs, color_map=cmap, grid=grid, reachable=reachable,
                cameras=[cam], width=width, height=height, rfl=rfl)


def scene_config1(grid_size=128, width=1245, height=825, n_views=1, blob_seed=2000, n_blobs=32, peak=50.0,
                  radius=0.5, fov=60.0, sampling="Disparity"):
    """Full inference frame(s): random-init fp16 network, camera(s) on an orbit inside the sphere.
    n_views = 32 gives the 360-degree orbit with elevations alternating +-15 degrees."""
    cfg = sampler_config(sampling, grid_size)
    cfg.field_type = abi.FIELD_NETWORK
    cfg.per_level_scale = 1.447
    blobs = blob_scene(blob_seed, n_blobs, peak)
    grid, reachable = density_grid_from_blobs(cfg, blobs)
    table, dmlp, rmlp = network_params(cfg, 2001, 2002)
    if n_views == 1:
        cams = [orbit_camera(radius, 0.0, 0.0)]
    else:
        cams = [orbit_camera(radius, 15.0 if k % 2 == 0 else -15.0, 360.0 * k / n_views) for k in range(n_views)]
    rfl = relative_focal_length(fov, width, height)
    return dict(cfg=cfg, blobs=blobs, grid=grid, reachable=reachable, hash_table=table, density_mlp=dmlp,
                rgb_mlp=rmlp, cameras=cams, width=width, height=height, rfl=rfl)


def scene_config3(grid_size=128):
    """Density-grid refresh: config 1's network, a seeded prior grid in optical-thickness units."""
    sc = scene_config1(grid_size=grid_size, width=64, height=64)
    cfg = sc["cfg"]
    min_step = math.sqrt(3.0) / cfg.maximum_marching_steps
    rng = np.random.Generator(np.random.PCG64(3000))
    prior = (sc["grid"].astype(np.float64) * min_step * rng.uniform(0.5, 1.5, size=sc["grid"].shape[0])).astype(np.float32)
    sc["prior_grid"] = prior
    sc["rng_seed"] = 3001
    return sc


def scene_config4(grid_size=128, width=3840, height=2160):
    """High-resolution inward-facing stress scene: dense occupancy, Original sampling."""
    sc = scene_config1(grid_size=grid_size, width=width, height=height, blob_seed=4000, n_blobs=128, peak=200.0,
                       radius=3.0, fov=50.0, sampling="Original")
    sc["cameras"] = [orbit_camera(3.0, 0.0, 90.0 * k) for k in range(4)]
    sc["cfg"].max_samples_per_ray = 2048
    return sc


def training_views(seed, n_images=6, width=32, height=24, radius=3.0, fov_deg=50.0, zero_probability=0.2):
    """A seeded set of training views in the layout the training-side sampler reads: cameras on an orbit
    looking at the centre (3x4, column-major, internal convention), fp16 rgba images of uniform noise, and
    a per-pixel sampling probability with a fraction of zeros (pixels the sampler must never pick)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    xforms = np.stack([orbit_camera(radius, float(rng.uniform(-40, 40)), 360.0 * k / n_images).flatten(order="F")
                       for k in range(n_images)]).astype(np.float32)
    images = rng.random((n_images, height, width, 4)).astype(np.float16)
    prob = rng.random((n_images, height, width)).astype(np.float16)
    prob[rng.random((n_images, height, width)) < zero_probability] = 0
    focal = float(width) * 0.5 / math.tan(0.5 * math.radians(fov_deg))
    return dict(n_images=n_images, width=width, height=height, focal_length=(focal, focal), principal_point=(0.5, 0.5),
                xforms=xforms, images=images, sampling_probability=prob)
