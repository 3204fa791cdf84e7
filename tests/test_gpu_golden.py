"""The CUDA path against the committed golden fixtures (tests/golden/*.npz, frozen answers of the oracle on tiny
seeded cases): the same inputs are rebuilt from their seeds and run through the C-ABI on the GPU."""
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import make_renderer, small_scene
from sphericalrf_b200 import abi, synth

GOLDEN = Path(__file__).parent / "golden"
pytestmark = pytest.mark.gpu


def _eq(a, b):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    return a.shape == b.shape and a.tobytes() == b.tobytes()


@pytest.mark.parametrize("name,kw,exact", [
    ("blobs_disparity", dict(kind="blobs", sampling="Disparity"), True),
    ("blobs_original", dict(kind="blobs", sampling="Original", radius=4.0), True),
    ("net_disparity", dict(kind="net", sampling="Disparity"), False),
])
def test_frames_match_fixture(built_lib, name, kw, exact):
    want = np.load(GOLDEN / f"{name}.npz")
    sc = small_scene(width=12, height=8, grid_size=16, **kw)
    r = make_renderer(sc)
    assert _eq(r.download_bitfield(), want["bits"]) and _eq(np.float32(r.grid_mean()), want["mean"])
    n = r.n_rays(sc["view"])
    counts, pos_dt, ordinal, cell = r.dump_samples(sc["view"], 0, n, 1 << 20)
    assert _eq(counts, want["counts"])
    assert _eq(pos_dt[:4096], want["pos_dt"]) and _eq(ordinal[:4096], want["ordinal"]) and _eq(cell[:4096], want["cell"])
    got = r.render_frame(sc["view"], abi.default_post(), want_raw=True)
    if exact:
        assert _eq(got["rgba_raw"], want["rgba_raw"]) and _eq(got["out"], want["out"])
    else:
        assert np.abs(got["rgba_raw"] - want["rgba_raw"]).max() <= 1e-3 and np.abs(got["out"] - want["out"]).max() <= 1e-3


def test_refresh_matches_fixture(built_lib):
    want = np.load(GOLDEN / "refresh.npz")
    sc = small_scene(kind="net", grid_size=16)
    rng = np.random.Generator(np.random.PCG64(1))
    grid = (rng.random(16 ** 3) * 0.02).astype(np.float32)
    grid[::7] = -1.0
    r = make_renderer(sc)
    r.upload_density_grid(grid)
    r.refresh_reset(3001)
    for k in range(3):
        r.refresh_grid(0 if k < 2 else 300)
        assert _eq(r.download_density_grid(), want[f"grid{k}"]), k
        assert _eq(r.download_bitfield(), want[f"bits{k}"]) and _eq(np.float32(r.grid_mean()), want[f"mean{k}"])


def test_normals_match_fixture(built_lib):
    want = np.load(GOLDEN / "normals.npz")
    sc = small_scene(kind="net", width=10, height=6, grid_size=16)
    sc["view"].render_mode = abi.MODE_NORMALS
    got = make_renderer(sc).render_frame(sc["view"], abi.default_post(), want_raw=True)
    assert _eq(got["rgba_raw"], want["rgba_raw"]) and _eq(got["out"], want["out"])


def test_training_side_matches_fixture(built_lib, oracle_mod):
    want = np.load(GOLDEN / "training.npz")
    sc = small_scene(kind="net", grid_size=16)
    sc["cfg"].maximum_marching_steps = 64
    sc["cfg"].train_in_linear_color = 0
    r = make_renderer(sc)
    views = synth.training_views(41, n_images=3, width=16, height=12, radius=0.4)
    rng = oracle_mod.rng_seed(77)             # only the PCG32 seeding rule is taken from the checker here
    ts = r.sample_training_rays(views, 48, 5, 2048, rng.state, rng.inc, True)
    used = int(want["numsteps"][:, 0].sum())
    assert ts["n_samples_total"] == int(want["n_total"])
    assert _eq(ts["rays"], want["rays"]) and _eq(ts["rgba"], want["rgba"]) and _eq(ts["numsteps"], want["numsteps"])
    assert _eq(ts["coords"][:used], want["coords"])
    net_want = want["net"].view(np.float16)
    net_got = r.network_inference(ts["coords"][:used])
    assert np.abs(net_got.astype(np.float32) - net_want.astype(np.float32)).max() <= 2e-3 * max(1.0, float(np.abs(net_want).max()))
    p = abi.LossParams()
    p.n_rays, p.n_max_compacted_coords, p.loss_type, p.loss_scale = 48, 1024, abi.LOSS_SMOOTH_L1, 128.0
    p.regularization_type = abi.REG_DISTORTION
    p.background_color[:] = [0.3, 0.6, 0.1]
    p.color_space, p.train_with_random_bg_color, p.padded_output_width = abi.COLOR_SRGB, 1, 4
    p.rng_state, p.rng_inc = rng.state, rng.inc
    coords = np.zeros((2048, 7), np.float32); coords[:used] = want["coords"]
    ls = r.volume_rendering_loss(p, ts["n_rays"], want["numsteps"], want["rgba"], coords, np.pad(net_want, ((0, 2048 - used), (0, 0))))
    assert ls["n_compacted"] == int(want["n_compacted"]) and _eq(ls["indices"], want["indices"])
    assert _eq(ls["dloss"].view(np.uint16), want["dloss"]) and _eq(ls["loss"], want["loss"]) and _eq(ls["reg"], want["reg"])
    mask_cfg = synth.sampler_config("Original", 16)
    mask_cfg.warping_type, mask_cfg.grid_distribution_type, mask_cfg.aabb_scale = abi.WARP_NGP, abi.GRID_METRIC_EXP, 4
    mask_cfg.field_type = abi.FIELD_BLOBS
    from sphericalrf_b200.testbed import Renderer
    rm = Renderer(mask_cfg, 0)
    rm.sampler_init(synth.training_views(3, n_images=2, width=16, height=16, radius=1.5, fov_deg=30.0), True, 0)
    assert _eq(np.packbits(rm.download_density_grid() == 0), want["mask"])
