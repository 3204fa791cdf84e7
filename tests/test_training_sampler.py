"""Training-side sampler: generate_training_samples_nerf and mark_untrained_density_grid
(internal/sampler/occupancy_sampler.cu:12-102,513-689).  CPU: properties of the oracle's serial execution.
GPU: the CUDA entry points against the oracle, bit for bit."""
import ctypes as C

import numpy as np
import pytest

from helpers import make_renderer, small_scene
from sphericalrf_b200 import abi, synth


def _rng(oracle_mod, seed):
    r = oracle_mod.Rng()
    oracle_mod.lib().srfo_rng_seed(C.byref(r), C.c_uint64(seed))
    return r


def _scene(warp=abi.WARP_ERP, sampling="Disparity", cascades=1, grid_dist=abi.GRID_WARPED_EXP, use_grid=True, radius=3.0):
    sc = small_scene(kind="blobs", sampling=sampling, warp=warp, cascades=cascades, grid_dist=grid_dist,
                     radius=0.5 if sampling == "Disparity" else 4.0)
    sc["cfg"].use_grid = 1 if use_grid else 0
    sc["cfg"].maximum_marching_steps = 128
    views = synth.training_views(31, n_images=5, width=28, height=20, radius=radius if sampling != "Disparity" else 0.4)
    return sc, views


def _bits(oracle_mod, sc):
    from helpers import make_oracle
    orc = make_oracle(oracle_mod, sc, None)
    return orc.update_grid_bitfield(sc["grid"])[0]


def test_serial_order_properties(oracle_mod):
    sc, views = _scene()
    bits = _bits(oracle_mod, sc)
    n_rays, n_coords = 300, 40000
    out = oracle_mod.sample_training_rays(sc["cfg"], views, bits, n_rays, 0, n_coords, _rng(oracle_mod, 5))
    k = out["n_rays"]
    assert 0 < k <= n_rays
    counts, bases = out["numsteps"][:, 0].astype(np.int64), out["numsteps"][:, 1].astype(np.int64)
    assert (counts > 0).all() and (counts <= 128).all()
    assert bases[0] == 0 and np.array_equal(bases[1:], np.cumsum(counts)[:-1])        # no ray dropped here: bases are contiguous
    assert out["n_samples_total"] == counts.sum() <= n_coords
    used = out["coords"][: counts.sum()]
    assert (used[:, 3] > 0).all()                                                     # dt
    assert ((used[:, :3] >= 0) & (used[:, :3] <= 1)).all()                            # warped positions
    for r in range(k):                                                                # one direction per ray, warped to [0,1]
        seg = used[bases[r]: bases[r] + counts[r], 4:7]
        assert (seg == seg[0]).all()
        assert np.allclose(seg[0], (out["rays"][r, 3:6] + 1) * 0.5, atol=1e-7)
    assert np.allclose(np.linalg.norm(out["rays"][:, 3:6], axis=1), 1.0, atol=1e-6)
    # a ray's colour is a pixel of the training images
    flat = views["images"].reshape(-1, 4).astype(np.float32)
    for r in range(min(k, 20)):
        assert (flat == out["rgba"][r]).all(axis=1).any()
    # same stream, same answer
    again = oracle_mod.sample_training_rays(sc["cfg"], views, bits, n_rays, 0, n_coords, _rng(oracle_mod, 5))
    assert again["coords"].tobytes() == out["coords"].tobytes() and again["numsteps"].tobytes() == out["numsteps"].tobytes()


def test_zero_probability_pixels_and_overflow(oracle_mod):
    sc, views = _scene()
    bits = _bits(oracle_mod, sc)
    full = oracle_mod.sample_training_rays(sc["cfg"], views, bits, 400, 7, 1 << 20, _rng(oracle_mod, 9))
    none = dict(views); none["sampling_probability"] = np.zeros_like(views["sampling_probability"])
    out = oracle_mod.sample_training_rays(sc["cfg"], none, bits, 400, 7, 1 << 20, _rng(oracle_mod, 9))
    assert out["n_rays"] == 0 and out["n_samples_total"] == 0
    allp = dict(views); allp["sampling_probability"] = None
    out = oracle_mod.sample_training_rays(sc["cfg"], allp, bits, 400, 7, 1 << 20, _rng(oracle_mod, 9))
    assert out["n_rays"] >= full["n_rays"]
    # a buffer that is too small: the kept rays are a prefix, the sample counter still counts every ray
    small = int(full["numsteps"][:, 0].sum() // 3)
    cut = oracle_mod.sample_training_rays(sc["cfg"], views, bits, 400, 7, small, _rng(oracle_mod, 9))
    assert cut["n_samples_total"] == full["n_samples_total"]
    assert 0 < cut["n_rays"] < full["n_rays"]
    assert np.array_equal(cut["numsteps"], full["numsteps"][: cut["n_rays"]])
    assert (cut["numsteps"][:, 0].astype(np.int64) + cut["numsteps"][:, 1] <= small).all()


def test_mark_untrained_masks_cells_no_view_sees(oracle_mod):
    cfg = synth.sampler_config("Original", 16)
    cfg.warping_type = abi.WARP_NGP
    cfg.grid_distribution_type = abi.GRID_METRIC_RECIPROCAL
    cfg.aabb_scale = 4
    views = synth.training_views(3, n_images=2, width=32, height=32, radius=1.5, fov_deg=30.0)
    grid = oracle_mod.mark_untrained(cfg, views)
    assert set(np.unique(grid)) == {-1.0, 0.0}
    seen = (grid == 0).mean()
    assert 0.02 < seen < 0.9
    # the cell that contains the point the cameras look at is seen
    from sphericalrf_b200.synth import morton3d
    centre = int(morton3d(np.array([8], np.uint32), np.array([8], np.uint32), np.array([8], np.uint32))[0])
    assert grid[centre] == 0.0
    # more views see more
    more = synth.training_views(3, n_images=6, width=32, height=32, radius=1.5, fov_deg=30.0)
    assert (oracle_mod.mark_untrained(cfg, more) == 0).mean() >= seen


TRAIN_CASES = [
    dict(warp=abi.WARP_ERP, sampling="Disparity"),
    dict(warp=abi.WARP_ERP, sampling="Original"),
    dict(warp=abi.WARP_NGP, sampling="Original"),
    dict(warp=abi.WARP_MIPNERF360, sampling="Original", cascades=2, grid_dist=abi.GRID_WARPED_RECIPROCAL),
    dict(warp=abi.WARP_ERP, sampling="Original", use_grid=False),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", TRAIN_CASES, ids=lambda c: f"warp{c['warp']}-{c['sampling']}-c{c.get('cascades', 1)}-g{int(c.get('use_grid', True))}")
def test_training_sampler_bit_exact(built_lib, oracle_mod, case):
    sc, views = _scene(**case)
    r = make_renderer(sc)
    bits = r.download_bitfield()
    rng = _rng(oracle_mod, 1234)
    for n_rays, shift, n_coords, snap in ((257, 0, 1 << 16, True), (257, 257, 1 << 16, False), (500, 1000, 3000, True)):
        want = oracle_mod.sample_training_rays(sc["cfg"], views, bits, n_rays, shift, n_coords, rng, snap)
        got = r.sample_training_rays(views, n_rays, shift, n_coords, rng.state, rng.inc, snap)
        assert got["n_rays"] == want["n_rays"] and got["n_samples_total"] == want["n_samples_total"]
        assert want["n_rays"] > 0
        assert np.array_equal(got["numsteps"], want["numsteps"])
        assert got["rays"].tobytes() == want["rays"].tobytes()
        assert got["rgba"].tobytes() == want["rgba"].tobytes()
        used = int((want["numsteps"][:, 0].astype(np.int64)).sum()) if n_coords >= want["n_samples_total"] else None
        if used is None:           # overflow: compare the slots of the kept rays
            for cnt, base in want["numsteps"]:
                assert got["coords"][base: base + cnt].tobytes() == want["coords"][base: base + cnt].tobytes()
        else:
            assert got["coords"][:used].tobytes() == want["coords"][:used].tobytes()


@pytest.mark.gpu
@pytest.mark.parametrize("grid_dist", [abi.GRID_WARPED_EXP, abi.GRID_WARPED_RECIPROCAL, abi.GRID_METRIC_EXP, abi.GRID_METRIC_RECIPROCAL])
@pytest.mark.parametrize("cascades", [1, 3])
def test_sampler_init_mask_bit_exact(built_lib, oracle_mod, grid_dist, cascades):
    from sphericalrf_b200.testbed import Renderer
    cfg = synth.sampler_config("Original", 32)
    cfg.warping_type = abi.WARP_NGP
    cfg.grid_distribution_type = grid_dist
    cfg.num_cascades = cascades
    cfg.aabb_scale = 4
    cfg.field_type = abi.FIELD_BLOBS
    views = synth.training_views(3, n_images=4, width=32, height=32, radius=1.5, fov_deg=35.0)
    r = Renderer(cfg, 0)
    r.upload_density_grid(np.full(32 ** 3 * cascades, 7.0, np.float32))
    r.sampler_init(views, init_grid_with_mask=True, rng_seed=3)
    want = oracle_mod.mark_untrained(cfg, views)
    got = r.download_density_grid()
    assert got.tobytes() == want.tobytes()
    assert 0 < (want == 0).sum() < want.size
    # without the mask (or with another warp) the grid is cleared, as OccupancySampler::init does
    r.upload_density_grid(np.full(32 ** 3 * cascades, 7.0, np.float32))
    r.sampler_init(None, init_grid_with_mask=False, rng_seed=3)
    assert not r.download_density_grid().any()


@pytest.mark.gpu
def test_training_sampler_large_batch(built_lib, oracle_mod):
    """32 768 rays (16 tiles of the exclusive scans), a sample buffer that overflows part of the way through:
    every output equals the oracle's serial execution."""
    sc, views = _scene(warp=abi.WARP_ERP, sampling="Disparity")
    views = synth.training_views(77, n_images=7, width=64, height=48, radius=0.4, zero_probability=0.1)
    r = make_renderer(sc)
    bits = r.download_bitfield()
    rng = _rng(oracle_mod, 99)
    n_rays = 32768
    probe = oracle_mod.sample_training_rays(sc["cfg"], views, bits, n_rays, 12345, 1 << 23, rng, True)
    total = probe["n_samples_total"]
    assert probe["n_rays"] > n_rays // 2 and total > 100000
    n_coords = int(total * 0.7)                                    # the last ~30 % of the rays find no room
    want = oracle_mod.sample_training_rays(sc["cfg"], views, bits, n_rays, 12345, n_coords, rng, True)
    got = r.sample_training_rays(views, n_rays, 12345, n_coords, rng.state, rng.inc, True)
    assert 0 < want["n_rays"] < probe["n_rays"]
    assert got["n_rays"] == want["n_rays"] and got["n_samples_total"] == want["n_samples_total"] == total
    assert np.array_equal(got["numsteps"], want["numsteps"])
    assert got["rays"].tobytes() == want["rays"].tobytes() and got["rgba"].tobytes() == want["rgba"].tobytes()
    used = int(want["numsteps"][-1, 0]) + int(want["numsteps"][-1, 1])
    assert got["coords"][:used].tobytes() == want["coords"][:used].tobytes()
    # every emitted position lies in an occupied cell of the bitfield (sinusoidal warp, one cascade: cell = floor(w * N))
    w = want["coords"][:used, :3]
    cell = np.clip((w * 32).astype(np.int64), 0, 31)
    idx = synth.morton3d(cell[:, 0].astype(np.uint32), cell[:, 1].astype(np.uint32), cell[:, 2].astype(np.uint32))
    assert ((bits[idx >> 3] >> (idx & 7)) & 1).all()
