"""Host-side logic above the C-ABI: the C++ host (include/srf_testbed.hpp) through the compiled `pyngp` module --
configuration parsing with the reference's keys, defaults and error messages, the Testbed surface, the JSON and
msgpack readers --; sharding; the generators."""
import math

import numpy as np
import pytest

from sphericalrf_b200 import abi, sharding, synth
from sphericalrf_b200 import pyngp as ngp
from sphericalrf_b200.testbed import config_from_json

NgpTestbed = ngp.Testbed

# The structure of experiment/srf_nerfsynthetic/config/srf_lego.json (keys as the reference spells them).
LEGO = {
    "samlper": {"warping_type": "ERP", "aabb_scale": 1, "use_grid": True, "init_grid_with_mask": False, "grid_size": 256,
                "num_cascades": 1, "ema_decay": 0.95, "grid_distribution_type": "WarpedSpace_Exp",
                "maximum_marching_steps": 1024, "cone_angle_constant": 0, "near_distance": 0.2, "far_distance": 2,
                "sampling_type": "Original", "snap_to_pixel_centers_in_rendering": True, "min_optical_thickness": 0.01},
    "network": {"encoding": {"otype": "HashGrid", "n_levels": 16, "n_features_per_level": 2, "log2_hashmap_size": 19, "base_resolution": 16},
                "network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 1},
                "dir_encoding": {"otype": "SphericalHarmonics", "degree": 4},
                "rgb_network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 2}},
    "render": {"train_with_random_bg_color": True, "train_in_linear_color": False, "transmittance_threshold": 0.0001},
    "loss": "SmoothL1",
}


def test_config_from_json_reads_the_reference_keys():
    c = config_from_json(LEGO)
    assert c.warping_type == abi.WARP_ERP and c.grid_size == 256 and c.sampling_type == abi.SAMPLING_ORIGINAL
    assert c.grid_distribution_type == abi.GRID_WARPED_EXP and c.aabb_scale == 1
    assert c.far_distance == 2.0 and abs(c.near_distance - 0.2) < 1e-7 and c.n_levels == 16 and c.log2_hashmap_size == 19
    assert c.per_level_scale == 0.0            # resolved later as exp(log(2048/16)/15)
    off, res, sc = synth.hashgrid_layout(c)
    assert abs(float(sc[-1]) + 1 - 2048.0) < 0.5


def test_config_errors_use_the_reference_messages():
    import copy
    bad = copy.deepcopy(LEGO); bad["samlper"]["warping_type"] = "Nope"
    with pytest.raises(RuntimeError, match="Unknown warping type."):
        config_from_json(bad)
    bad = copy.deepcopy(LEGO); bad["samlper"]["grid_distribution_type"] = "Exp"       # the light-field configs say this
    with pytest.raises(RuntimeError, match="Unknown grid distribution type."):
        config_from_json(bad)
    bad = copy.deepcopy(LEGO); del bad["samlper"]["grid_distribution_type"]           # the default "Exp" throws too
    with pytest.raises(RuntimeError, match="Unknown grid distribution type."):
        config_from_json(bad)
    bad = copy.deepcopy(LEGO); bad["samlper"]["sampling_type"] = "Linear"
    with pytest.raises(RuntimeError, match="Unknown sampling type."):
        config_from_json(bad)
    with pytest.raises(RuntimeError, match="samlper"):
        config_from_json({"sampler": {}})         # the section is spelled "samlper"
    t = NgpTestbed()
    with pytest.raises(RuntimeError, match="The model config must exist."):
        t.load_model_config("/nonexistent/config.json")


def test_fov_setters_take_radians_and_getters_return_degrees():
    t = NgpTestbed()
    t.fov = math.radians(50.0)
    assert abs(t.rendering_buffer.relative_focal_length[0] - 0.5 / math.tan(math.radians(25.0))) < 1e-6
    assert abs(t.fov - 50.0) < 1e-3
    t.fov_xy = [math.radians(60.0), math.radians(40.0)]
    fx, fy = t.fov_xy
    assert abs(fx - 60.0) < 1e-3 and abs(fy - 40.0) < 1e-3


def test_set_nerf_camera_matrix_convention():
    t = NgpTestbed()
    cam = np.array([[1, 0, 0, 0.1], [0, 1, 0, 0.2], [0, 0, 1, 0.3]], np.float32)
    t.set_nerf_camera_matrix(cam)
    want = np.array([[1, 0, 0, 0.6], [0, -1, 0, 0.7], [0, 0, -1, 0.8]], np.float32)
    assert np.allclose(t.camera_matrix, want)
    m = synth.orbit_camera(0.5, 15.0, 40.0)
    assert np.allclose(np.linalg.norm(m[:, 3] - 0.5), 0.5, atol=1e-6)
    fwd = m[:, 2]                                   # camera looks along +z of the converted matrix
    assert np.allclose(fwd, -(m[:, 3] - 0.5) / 0.5, atol=1e-6)


def test_shard_rows_cover_the_image_once():
    for h, rows, world in [(825, 8, 1), (825, 8, 2), (825, 8, 8), (21, 4, 3), (7, 8, 4)]:
        seen = []
        for r in range(world):
            idx = sharding.shard_row_indices(h, rows, world, r)
            assert idx == sorted(idx)
            seen += idx
            assert sharding.shard_ray_count(100, h, rows, world, r) == 100 * len(idx)
        assert sorted(seen) == list(range(h))


def test_shard_ray_order_matches_the_oracle(oracle_mod):
    cam = synth.orbit_camera(0.5, 0, 0)
    for world, rank in [(1, 0), (3, 1), (4, 3)]:
        v = abi.make_view(cam, 10, 21, (1.0, 1.0), shard_rows=4, shard_count=world, shard_rank=rank)
        cfg = synth.sampler_config("Original", 16)
        orc = oracle_mod.Oracle(cfg, np.zeros(16 ** 3 // 8, np.uint8))
        _, _, _, pixel = orc.generate_rays(v)
        rows = sharding.shard_row_indices(21, 4, world, rank)
        want = (np.array(rows)[:, None] * 10 + np.arange(10)[None, :]).reshape(-1)
        assert np.array_equal(pixel, want.astype(np.uint32))


def test_generators_are_deterministic_and_shaped():
    a = synth.blob_scene(1000); b = synth.blob_scene(1000)
    assert np.array_equal(a, b) and a.shape == (32, 5)
    assert (np.linalg.norm(a[:, :3] - 0.5, axis=1) <= 3.0 + 1e-5).all() and (a[:, 3] >= 0.05).all() and (a[:, 3] <= 0.3).all()
    cfg = synth.sampler_config("Disparity", 16)
    cfg.per_level_scale = 1.447
    t, d, c = synth.network_params(cfg, 1, 2)
    off, _, _ = synth.hashgrid_layout(cfg)
    assert t.dtype == np.float16 and t.size == int(off[-1]) * 2 and d.size == 64 * 32 + 16 * 64 and c.size == 64 * 32 + 64 * 64 + 16 * 64
    assert np.abs(t.astype(np.float32)).max() <= 1e-4 + 1e-7
    grid, reach = synth.density_grid_from_blobs(cfg, a)
    assert grid.shape == (16 ** 3,) and grid.dtype == np.float32 and 0.3 < reach.mean() < 0.9


def test_cpp_json_reader_accepts_what_the_reference_configs_contain(tmp_path):
    text = r"""
    // comment lines, as the shipped configs have them
    { "samlper": { "warping_type": "ERP", /* inline */ "aabb_scale": 2000000, "use_grid": true, "grid_size": 64,
                   "grid_distribution_type": "WarpedSpace_Exp", "near_distance": 1e-1, "far_distance": 1.0E6,
                   "sampling_type": "Disparity", "note": "unicode \u00e9 and escapes \"\\ \n" },
      "network": { "encoding": {"n_levels": 16, "n_features_per_level": 2, "log2_hashmap_size": 19, "base_resolution": 16},
                   "network": {"n_neurons": 64, "n_hidden_layers": 1}, "dir_encoding": {"degree": 4},
                   "rgb_network": {"n_neurons": 64, "n_hidden_layers": 2} },
      "render": {}, "loss": "SmoothL1", "envmap": null, "list": [1, -2, 3.5, false] }
    """
    doc = ngp.parse_json(text)
    assert doc["samlper"]["aabb_scale"] == 2000000 and doc["samlper"]["far_distance"] == 1e6 and doc["envmap"] is None
    assert doc["list"] == [1, -2, 3.5, False] and doc["samlper"]["note"] == 'unicode \u00e9 and escapes "\\ \n'
    c = config_from_json(doc)
    assert c.sampling_type == abi.SAMPLING_DISPARITY and c.grid_size == 64 and abs(c.near_distance - 0.1) < 1e-7
    p = tmp_path / "cfg.json"
    p.write_text(text)
    t = NgpTestbed()
    try:
        t.load_model_config(str(p))            # parses, then needs a GPU for the context
    except RuntimeError as e:
        assert "CUDA" in str(e) or "sm_100" in str(e)
    with pytest.raises(RuntimeError, match="JSON parse error"):
        ngp.parse_json('{"a": }')


def test_cpp_msgpack_round_trip():
    doc = {"a": 1, "b": -7, "c": 3.25, "d": "text", "e": b"\x00\x01\xff", "f": [True, None, {"g": 2 ** 40}], "h": {}}
    blob = ngp.write_msgpack(doc)
    assert ngp.parse_msgpack(blob) == doc
    try:
        import msgpack
    except ImportError:
        return
    assert msgpack.unpackb(blob, raw=False) == doc                           # what the C++ writer writes, a standard reader reads
    assert ngp.parse_msgpack(msgpack.packb(doc, use_bin_type=True)) == doc   # and the other way round (compact encodings)
