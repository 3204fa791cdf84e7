"""Edge cases through the C-ABI on the GPU: empty and ragged shards, one-pixel images, empty and full grids,
zero-capacity training buffers, a 256^3 grid, capacity errors.  Where the case has a meaningful answer it is
compared with the oracle."""
import numpy as np
import pytest

from helpers import make_oracle, make_renderer, small_scene
from sphericalrf_b200 import abi, synth

pytestmark = pytest.mark.gpu


def _bits_equal(a, b):
    a, b = np.ascontiguousarray(a, np.float32), np.ascontiguousarray(b, np.float32)
    return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_empty_shard_and_ragged_shards(built_lib, oracle_mod):
    sc = small_scene(kind="blobs", width=13, height=7)
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    post = abi.default_post()
    whole = r.render_frame(sc["view"], post)["out"]
    pieces = np.full_like(whole, np.nan)
    for rank in range(5):                                  # 7 rows in blocks of 2 over 5 ranks: rank 4 owns nothing
        v = abi.View.from_buffer_copy(sc["view"])
        v.shard_rows, v.shard_count, v.shard_rank = 2, 5, rank
        n = r.n_rays(v)
        rows = [y for y in range(7) if (y // 2) % 5 == rank]
        assert n == len(rows) * 13
        got = r.render_frame(v, post, want_stats=True)
        assert got["out"].shape == (n, 4) and got["stats"]["n_rays"] in (n, 0)
        if n:
            ref = orc.render_frame(v, post)
            assert _bits_equal(got["out"], ref["out"])
            idx = (np.array(rows)[:, None] * 13 + np.arange(13)[None, :]).reshape(-1)
            pieces[idx] = got["out"]
    assert _bits_equal(pieces, whole)


def test_one_pixel_image(built_lib, oracle_mod):
    sc = small_scene(kind="net", width=1, height=1)
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    got = r.render_frame(sc["view"], abi.default_post(), want_counts=True)
    ref = orc.render_frame(sc["view"], abi.default_post())
    assert got["n_samples"][0] == ref["n_samples"][0]
    assert np.abs(got["out"] - ref["out"]).max() <= 1e-3
    img = r.render(sc["view"], abi.default_post(), spp=2)
    assert img.shape == (1, 1, 4) and np.isfinite(img).all()


@pytest.mark.parametrize("fill", [0, 255])
def test_empty_and_full_bitfield(built_lib, oracle_mod, fill):
    sc = small_scene(kind="blobs", sampling="Original", radius=4.0, width=16, height=10)
    sc["cfg"].maximum_marching_steps = 128                # keeps the full grid's 8-unit march at ~1000 samples per ray
    r = make_renderer(sc)
    bits = np.full(32 ** 3 // 8, fill, np.uint8)
    r.upload_bitfield(bits)
    orc = make_oracle(oracle_mod, sc, bits)
    post = abi.default_post()
    post.background_color[:] = [0.25, 0.5, 0.75, 1.0]
    got = r.render_frame(sc["view"], post, want_raw=True, want_counts=True, want_stats=True)
    ref = orc.render_frame(sc["view"], post)
    counts, *_ = orc.march(sc["view"], 0, orc.n_rays(sc["view"]), 1 << 22)
    assert np.array_equal(got["n_samples"], counts)
    assert _bits_equal(got["rgba_raw"], ref["rgba_raw"]) and _bits_equal(got["out"], ref["out"])
    if fill == 0:
        assert got["stats"]["n_samples"] == 0 and got["stats"]["n_rays_hit"] == 0
        assert (got["out"] == got["out"][0]).all() and got["out"][0, 3] == 1.0    # the (linearised) background everywhere
    else:
        assert got["stats"]["n_samples"] == got["stats"]["n_march_steps"] - got["stats"]["n_rays_alive"]   # every step but the exit step


def test_training_buffers_of_zero_capacity(built_lib, oracle_mod):
    sc = small_scene(kind="blobs", sampling="Original", radius=4.0)
    sc["cfg"].maximum_marching_steps = 64
    r = make_renderer(sc)
    views = synth.training_views(5, n_images=2, width=8, height=8, radius=3.0)
    rng = oracle_mod.rng_seed(1)
    full = r.sample_training_rays(views, 64, 0, 1 << 14, rng.state, rng.inc, True)
    none = r.sample_training_rays(views, 64, 0, 1, rng.state, rng.inc, True)        # room for one sample only
    want = oracle_mod.sample_training_rays(sc["cfg"], views, r.download_bitfield(), 64, 0, 1, rng, True)
    assert none["n_rays"] == want["n_rays"] <= 1 and none["n_samples_total"] == full["n_samples_total"] > 0
    assert np.array_equal(none["numsteps"], want["numsteps"])
    # compositor with no kept rays: counters zero, nothing written
    p = abi.LossParams()
    p.n_rays, p.n_max_compacted_coords, p.loss_type, p.loss_scale, p.padded_output_width = 64, 128, abi.LOSS_L2, 1.0, 4
    out = r.volume_rendering_loss(p, 0, np.zeros((64, 2), np.uint32), np.zeros((64, 4), np.float32), np.zeros((1, 7), np.float32),
                                  np.zeros((1, 4), np.float16))
    assert out["n_compacted"] == 0 and not out["dloss"].any() and not out["loss"].any()
    # compacted capacity of one sample: the first ray is clipped to it, the others are emptied, the counter counts all
    used = int(full["numsteps"][:, 0].sum())
    p.n_max_compacted_coords = 1
    out = r.volume_rendering_loss(p, full["n_rays"], full["numsteps"], full["rgba"], full["coords"][:used], np.zeros((used, 4), np.float16))
    assert out["n_compacted"] == used and out["indices"][0, 0] == 1 and not out["indices"][1:, 0].any()


def test_grid_256(built_lib, oracle_mod):
    """The shipped configs use grid_size 256: bitfield rule, mean and a few rays at that size."""
    sc = small_scene(kind="blobs", grid_size=256, width=6, height=4)
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, None)
    bits, mean = orc.update_grid_bitfield(sc["grid"])
    assert np.array_equal(r.download_bitfield(), bits) and np.float32(r.grid_mean()).tobytes() == np.float32(mean).tobytes()
    orc.bitfield = bits
    got = r.render_frame(sc["view"], abi.default_post(), want_counts=True)
    ref = orc.render_frame(sc["view"], abi.default_post())
    counts, *_ = orc.march(sc["view"], 0, orc.n_rays(sc["view"]), 1 << 22)
    assert np.array_equal(got["n_samples"], counts) and _bits_equal(got["out"], ref["out"])
    assert (ref["n_composited"] < counts).any()            # some rays saturate before their march ends


def test_capacity_errors(built_lib):
    sc = small_scene(kind="blobs")
    r = make_renderer(sc)
    r.reserve(16)                                          # fewer sample slots than one ray may need
    with pytest.raises(abi.SrfError) as e:
        r.render_frame(sc["view"], abi.default_post())
    assert e.value.status == abi.ERR_CAPACITY
    r.reserve(0)
    r.render_frame(sc["view"], abi.default_post())
    with pytest.raises(abi.SrfError):
        r.set_wave_schedule([0])
    with pytest.raises(abi.SrfError):
        r.set_wave_schedule(list(range(1, 10)))
