"""Shared scene builders for the tests (small seeded cases the oracle finishes in seconds)."""
import numpy as np

from sphericalrf_b200 import abi, synth


def small_scene(kind="net", sampling="Disparity", warp=abi.WARP_ERP, grid_size=32, width=24, height=16, seed=7,
                n_blobs=12, radius=0.5, cascades=1, grid_dist=abi.GRID_WARPED_EXP, aabb_scale=None):
    """A small scene of the given field kind: dict(cfg, grid, arrays..., view)."""
    cfg = synth.sampler_config(sampling, grid_size)
    cfg.warping_type = warp
    cfg.num_cascades = cascades
    cfg.grid_distribution_type = grid_dist
    if aabb_scale is not None:
        cfg.aabb_scale = aabb_scale
    sc = dict(cfg=cfg)
    blobs = synth.blob_scene(seed, n_blobs, 50.0, ball_radius=1.5 if warp != abi.WARP_ERP else 3.0)
    sc["blobs"] = blobs
    rng = np.random.Generator(np.random.PCG64(seed + 1))
    n_cells = grid_size ** 3 * cascades
    if warp in (abi.WARP_ERP, abi.WARP_SINUSOIDAL, abi.WARP_NGP, abi.WARP_MIPNERF360) and cascades == 1:
        grid, _ = synth.density_grid_from_blobs(cfg, blobs)
    else:
        # any reproducible occupancy pattern will do for the other warps / cascades
        grid = (rng.random(n_cells) < 0.3).astype(np.float32) * rng.random(n_cells).astype(np.float32)
    sc["grid"] = grid.astype(np.float32)
    if kind == "net":
        cfg.field_type = abi.FIELD_NETWORK
        cfg.per_level_scale = 1.447
        t, d, c = synth.network_params(cfg, seed + 2, seed + 3, table_range=0.5)
        sc.update(hash_table=t, density_mlp=d, rgb_mlp=c)
    else:
        cfg.field_type = abi.FIELD_BLOBS
        cfg.density_activation = abi.ACT_NONE
        sc["color_map"] = synth.color_map(seed + 4)
    cam = synth.orbit_camera(radius, 10.0, 25.0)
    sc["view"] = abi.make_view(cam, width, height, synth.relative_focal_length(60.0, width, height))
    return sc


def make_oracle(oracle_mod, sc, bits):
    return oracle_mod.Oracle(sc["cfg"], bits, sc.get("hash_table"), sc.get("density_mlp"), sc.get("rgb_mlp"),
                             sc.get("blobs"), sc.get("color_map"))


def make_renderer(sc):
    from sphericalrf_b200.testbed import Renderer
    r = Renderer(sc["cfg"], 0)
    if sc["cfg"].field_type == abi.FIELD_NETWORK:
        r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    else:
        r.upload_blobs(sc["blobs"], sc["color_map"])
    r.upload_density_grid(sc["grid"])
    r.update_grid_bitfield()
    return r
