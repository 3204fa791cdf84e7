"""Parity at BASELINE's full sizes through size-independent properties, plus oracle spot checks on
windows of rays (the oracle needs minutes for a full frame, seconds for a window)."""
import ctypes as C

import numpy as np
import pytest

from sphericalrf_b200 import abi, synth
from sphericalrf_b200.testbed import Renderer

pytestmark = pytest.mark.gpu


def _renderer(sc):
    r = Renderer(sc["cfg"], 0)
    if sc["cfg"].field_type == abi.FIELD_NETWORK:
        r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    else:
        r.upload_blobs(sc["blobs"], sc["color_map"])
    r.upload_density_grid(sc["grid"])
    r.update_grid_bitfield()
    return r


def _oracle(oracle_mod, sc, bits):
    return oracle_mod.Oracle(sc["cfg"], bits, sc.get("hash_table"), sc.get("density_mlp"), sc.get("rgb_mlp"),
                             sc.get("blobs"), sc.get("color_map"))


@pytest.mark.parametrize("variant", ["O", "D"])
def test_config0_full_frame(built_lib, oracle_mod, variant):
    """800x800 analytic-field frame: deterministic, shard-invariant, conserving, and bit-exact against the
    oracle on ray windows spread over the image."""
    sc = synth.scene_config0(variant)
    r = _renderer(sc)
    view = abi.make_view(sc["cameras"][0], 800, 800, sc["rfl"])
    post = abi.default_post()
    a = r.render_frame(view, post, want_raw=True, want_counts=True, want_stats=True)
    b = r.render_frame(view, post, want_raw=True)
    assert np.array_equal(a["out"].view(np.uint32), b["out"].view(np.uint32))                 # run-to-run identical
    st = a["stats"]
    assert st["n_rays"] == 640000 and st["n_samples"] == int(a["n_samples"].astype(np.int64).sum())
    assert st["n_samples_composited"] <= st["n_samples"]
    assert (a["rgba_raw"][:, 3] <= 1.0 + 1e-6).all() and (a["rgba_raw"][:, 3] >= 0).all()
    occ = np.unpackbits(r.download_bitfield()).mean()
    assert 0.02 < occ < 0.6
    # two shards assemble to the same image
    img = np.zeros((800, 800, 4), np.float32)
    for rank in range(2):
        v = abi.make_view(sc["cameras"][0], 800, 800, sc["rfl"], shard_rows=8, shard_count=2, shard_rank=rank)
        part = r.render_frame(v, post)["out"]
        rows = [y for y in range(800) if (y // 8) % 2 == rank]
        img[rows] = part.reshape(len(rows), 800, 4)
    assert np.array_equal(img.reshape(-1, 4).view(np.uint32), a["out"].view(np.uint32))
    # oracle windows
    orc = _oracle(oracle_mod, sc, r.download_bitfield())
    for first in (0, 800 * 400 + 300, 800 * 799):
        n = 256
        ref = orc.render_frame(view, post, first, n)
        sl = slice(first, first + n)
        assert np.array_equal(ref["rgba_raw"][sl].view(np.uint32), a["rgba_raw"][sl].view(np.uint32))
        assert np.array_equal(ref["out"][sl].view(np.uint32), a["out"][sl].view(np.uint32))
        counts, *_ = orc.march(view, first, n, 1 << 24)
        assert np.array_equal(counts, a["n_samples"][sl])


def test_config1_full_frame(built_lib, oracle_mod):
    """1245x825 network frame (the benchmark workload): determinism, conservation, oracle windows within 1e-3."""
    sc = synth.scene_config1()
    r = _renderer(sc)
    view = abi.make_view(sc["cameras"][0], 1245, 825, sc["rfl"])
    post = abi.default_post()
    a = r.render_frame(view, post, want_raw=True, want_counts=True, want_stats=True)
    b = r.render_frame(view, post)
    assert np.array_equal(a["out"].view(np.uint32), b["out"].view(np.uint32))
    st = a["stats"]
    assert st["n_rays"] == 1027125 and st["n_samples"] == int(a["n_samples"].astype(np.int64).sum())
    assert st["n_batches"] >= 1 and st["error_flags"] == 0
    orc = _oracle(oracle_mod, sc, r.download_bitfield())
    # 16 windows of 256 consecutive rays spread over the image (4 096 rays, ~6.6 M samples through the oracle)
    n = 256
    for k in range(16):
        first = (825 * k // 16 + 25) * 1245 + (k * 61) % (1245 - n)
        ref = orc.render_frame(view, post, first, n)
        sl = slice(first, first + n)
        assert np.abs(ref["rgba_raw"][sl] - a["rgba_raw"][sl]).max() <= 1e-3, f"window {k}"
        assert np.abs(ref["out"][sl] - a["out"][sl]).max() <= 1e-3, f"window {k}"
        assert np.array_equal(orc.march(view, first, n, 1 << 23)[0], a["n_samples"][sl]), f"window {k}: per-ray sample counts"


def test_config2_all_orbit_views_against_the_oracle(built_lib, oracle_mod):
    """All 32 views of the 360-degree orbit at the full 1245x825 through srf_render (host image): a window of 64 rays of
    every view against the oracle (counts exact, pixels within 1e-3), opaque background, distinct views."""
    sc = synth.scene_config1(n_views=32)
    r = _renderer(sc)
    orc = _oracle(oracle_mod, sc, r.download_bitfield())
    post = abi.default_post()
    prev = None
    for k in range(32):
        view = abi.make_view(sc["cameras"][k], 1245, 825, sc["rfl"])
        img = r.render(view, post, spp=1)
        assert img.shape == (825, 1245, 4) and np.isfinite(img).all()
        assert np.allclose(img[..., 3], 1.0, atol=1e-6)                  # opaque background
        first = ((37 * k) % 800 + 10) * 1245 + (101 * k) % 1100
        ref = orc.render_frame(view, post, first, 64)
        flat = img.reshape(-1, 4)
        assert np.abs(ref["out"][first:first + 64] - flat[first:first + 64]).max() <= 1e-3, f"view {k}"
        counts = r.dump_samples(view, first, 64, 1 << 20)[0]
        assert np.array_equal(counts, orc.march(view, first, 64, 1 << 21)[0]), f"view {k}: per-ray sample counts"
        if prev is not None:
            assert np.abs(img - prev).max() > 1e-3
        prev = img


def test_config3_full_grid_refresh(built_lib, oracle_mod):
    """128^3 grid, 16 refreshes: every float and bit against the oracle at steps 1, 2 and 16."""
    sc = synth.scene_config3()
    r = _renderer(sc)
    r.upload_density_grid(sc["prior_grid"])
    r.refresh_reset(sc["rng_seed"])
    orc = _oracle(oracle_mod, sc, None)
    grid = sc["prior_grid"].copy()
    rng = oracle_mod.rng_seed(sc["rng_seed"])
    step = 0
    for k in range(16):
        bits, mean, step = orc.refresh(grid, step, 0, rng)
        r.refresh_grid(0)
        if k in (0, 1, 15):
            assert np.array_equal(r.download_density_grid().view(np.uint32), grid.view(np.uint32)), f"refresh {k}"
            assert np.array_equal(r.download_bitfield(), bits), f"refresh {k}"
            assert np.float32(r.grid_mean()).tobytes() == np.float32(mean).tobytes()
    assert 0.0 < np.unpackbits(bits).mean() < 1.0


def test_config4_high_resolution_shard(built_lib, oracle_mod):
    """One of eight shards of a 3840x2160 view of the dense scene, with the opt-in 2048-sample cap."""
    sc = synth.scene_config4()
    r = _renderer(sc)
    view = abi.make_view(sc["cameras"][0], 3840, 2160, sc["rfl"], shard_rows=8, shard_count=8, shard_rank=3)
    a = r.render_frame(view, abi.default_post(), want_counts=True, want_stats=True)
    from sphericalrf_b200.sharding import shard_ray_count
    assert a["stats"]["n_rays"] == r.n_rays(view) == shard_ray_count(3840, 2160, 8, 8, 3)
    assert a["n_samples"].max() <= 2048
    assert np.isfinite(a["out"]).all()
    b = r.render_frame(view, abi.default_post())
    assert np.array_equal(a["out"].view(np.uint32), b["out"].view(np.uint32))
    # three windows of the shard against the oracle, with the cap in force
    orc = _oracle(oracle_mod, sc, r.download_bitfield())
    n_local = r.n_rays(view)
    a = r.render_frame(view, abi.default_post(), want_raw=True, want_counts=True)
    for first in (5 * 3840 + 100, n_local // 2 + 1700, n_local - 3840 - 500):
        ref = orc.render_frame(view, abi.default_post(), first, 48)
        sl = slice(first, first + 48)
        assert np.array_equal(orc.march(view, first, 48, 1 << 21)[0], a["n_samples"][sl])
        assert np.abs(ref["rgba_raw"][sl] - a["rgba_raw"][sl]).max() <= 1e-3
        assert np.abs(ref["out"][sl] - a["out"][sl]).max() <= 1e-3
