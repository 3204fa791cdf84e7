"""Snapshot files (.msgpack) and the compiled `pyngp` module: structure, round trip, error messages (CPU);
a snapshot rendered through `pyngp.Testbed` equals the same parameters rendered through the C-ABI (GPU)."""
import copy

import numpy as np
import pytest

from sphericalrf_b200 import abi, snapshot, synth
from sphericalrf_b200 import pyngp as ngp
from sphericalrf_b200.testbed import config_from_json

SMALL = {
    "samlper": {"warping_type": "ERP", "aabb_scale": 2000000, "use_grid": True, "grid_size": 32, "num_cascades": 1,
                "ema_decay": 0.95, "grid_distribution_type": "WarpedSpace_Exp", "maximum_marching_steps": 256,
                "cone_angle_constant": 0, "near_distance": 0.1, "far_distance": 1000000.0, "sampling_type": "Disparity",
                "snap_to_pixel_centers_in_rendering": True, "min_optical_thickness": 0.01},
    "network": {"encoding": {"otype": "HashGrid", "n_levels": 16, "n_features_per_level": 2, "log2_hashmap_size": 12,
                             "base_resolution": 4, "per_level_scale": 1.3},
                "network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 1},
                "dir_encoding": {"otype": "SphericalHarmonics", "degree": 4},
                "rgb_network": {"otype": "FullyFusedMLP", "activation": "ReLU", "output_activation": "None", "n_neurons": 64, "n_hidden_layers": 2}},
    "render": {"train_in_linear_color": False, "transmittance_threshold": 0.0001},
    "loss": "SmoothL1",
    "optimizer": {"otype": "Adam"},
}


def _scene():
    cfg = config_from_json(SMALL)
    cfg.field_type = abi.FIELD_NETWORK
    table, dmlp, rmlp = synth.network_params(cfg, 71, 72, table_range=0.5)
    blobs = synth.blob_scene(73, 12, 50.0)
    grid, _ = synth.density_grid_from_blobs(cfg, blobs)
    return cfg, table, dmlp, rmlp, grid


def test_snapshot_round_trip_and_structure(tmp_path):
    cfg, table, dmlp, rmlp, grid = _scene()
    for full in (False, True):
        path = tmp_path / f"s{int(full)}.msgpack"
        snapshot.write_snapshot(str(path), SMALL, grid, dmlp, rmlp, table, 0.33, (0.5, 0.25, 0.75), full_precision=full)
        doc = ngp.parse_msgpack(path.read_bytes())
        assert set(SMALL) <= set(doc) and doc["samlper"]["grid_size"] == 32
        s = doc["snapshot"]
        assert s["params_type"] == ("float" if full else "__half")
        assert s["n_params"] == 3072 + 7168 + table.size == 3072 + 7168 + snapshot.table_entries(cfg)
        assert isinstance(s["params_binary"], bytes) and len(s["params_binary"]) == s["n_params"] * (4 if full else 2)
        assert len(s["density_grid"]) == 32 ** 3 * 4 and s["scene_offset"] == [0.5, 0.25, 0.75]
        back = snapshot.read_snapshot(str(path))
        assert "snapshot" not in back["model_config"] and back["model_config"]["samlper"] == SMALL["samlper"]
        assert np.array_equal(back["density_grid"].view(np.uint32), grid.view(np.uint32))
        assert np.array_equal(back["density_mlp"].view(np.uint16), dmlp.view(np.uint16))      # fp16 -> fp32 -> fp16 is exact
        assert np.array_equal(back["rgb_mlp"].view(np.uint16), rmlp.view(np.uint16))
        assert np.array_equal(back["hash_table"].view(np.uint16), table.view(np.uint16))
        assert back["scene_scale"] == pytest.approx(0.33) and np.allclose(back["scene_offset"], [0.5, 0.25, 0.75])


def test_snapshot_errors(tmp_path):
    p = tmp_path / "plain.msgpack"
    p.write_bytes(ngp.write_msgpack(SMALL))
    with pytest.raises(RuntimeError, match="ERROR in loading snapshot."):
        snapshot.read_snapshot(str(p))
    bad = copy.deepcopy(SMALL)
    bad["snapshot"] = {"n_params": 4, "params_type": "__half", "params_binary": b"\0" * 8, "density_grid": b"",
                       "scene_scale": 1.0, "scene_offset": [0, 0, 0]}
    p.write_bytes(ngp.write_msgpack(bad))
    with pytest.raises(RuntimeError, match="shorter"):
        snapshot.read_snapshot(str(p))
    t = ngp.Testbed()
    with pytest.raises(RuntimeError, match="The model config must be a .json or .msgpack file."):
        q = tmp_path / "cfg.txt"; q.write_text("{}"); t.load_model_config(str(q))
    with pytest.raises(RuntimeError, match="training is not part"):
        t.train(16, 1 << 18)


def test_pyngp_names_match_the_reference_module():
    # internal/python_api.cu:46-82: enum members in the reference's order, exported at module level
    assert ngp.__file__.endswith(".so"), "pyngp is the compiled extension"
    names = lambda e: [k for k, _ in sorted(e.__members__.items(), key=lambda kv: int(kv[1]))]
    assert names(ngp.RenderMode) == ["AO", "Shade", "Normals", "Depth", "Distance", "Cost"]
    assert names(ngp.Activation) == ["None", "ReLU", "Logistic", "Exponential"]
    assert names(ngp.TonemapCurve) == ["Identity", "ACES", "Hable", "Reinhard"]
    assert names(ngp.ColorSpace) == ["Linear", "SRGB"]
    assert names(ngp.LossType) == ["L2", "L1", "Mape", "Smape", "SmoothL1", "LogL1", "RelativeL2"]
    assert ngp.Depth == ngp.RenderMode.Depth and ngp.SRGB == ngp.ColorSpace.SRGB and ngp.SmoothL1 == ngp.LossType.SmoothL1
    t = ngp.Testbed()
    for name in ("load_model_config", "load_snapshot", "save_snapshot", "load_training_data", "train", "render",
                 "set_nerf_camera_matrix", "fov", "fov_xy", "background_color", "color_space", "density_activation",
                 "rgb_activation", "loss_type", "rendering_buffer"):
        assert hasattr(type(t), name) or hasattr(t, name), name
    for name in ("render_mode", "tonemap_curve", "exposure", "fov_axis", "relative_focal_length", "principal_point",
                 "MIN_STEPS_INBETWEEN_COMPACTION", "MAX_STEPS_INBETWEEN_COMPACTION"):
        assert hasattr(t.rendering_buffer, name), name


@pytest.mark.gpu
def test_snapshot_renders_like_uploaded_parameters(built_lib, oracle_mod, tmp_path):
    """The reference's eval sequence (experiment/*/python/run.py:128-250) on a snapshot file, against the C-ABI
    path fed with the same arrays, and against the oracle."""
    from sphericalrf_b200.testbed import Renderer
    cfg, table, dmlp, rmlp, grid = _scene()
    path = tmp_path / "scene.msgpack"
    snapshot.write_snapshot(str(path), SMALL, grid, dmlp, rmlp, table, 1.0, (0.5, 0.5, 0.5))
    W, H = 40, 24
    testbed = ngp.Testbed()
    testbed.load_snapshot(str(path))
    testbed.background_color = [1.0, 1.0, 1.0, 1.0]
    testbed.fov_xy = [1.0, 1.0 * H / W]
    nerf_cam = np.array([[1, 0, 0, 0.1], [0, 0, -1, -0.3], [0, 1, 0, 0.05]], np.float32)
    testbed.set_nerf_camera_matrix(nerf_cam)
    img = testbed.render(W, H, 2, False)
    assert img.shape == (H, W, 4) and np.isfinite(img).all()
    testbed.rendering_buffer.render_mode = ngp.Depth
    depth = testbed.render(W, H, 1, False)
    assert depth.shape == (H, W, 4) and not np.array_equal(depth, img)

    cfg.density_activation, cfg.rgb_activation = abi.ACT_EXPONENTIAL, abi.ACT_LOGISTIC
    r = Renderer(cfg, 0)
    r.upload_network(table, dmlp, rmlp)
    r.upload_density_grid(grid)
    r.update_grid_bitfield()
    view = abi.make_view(testbed.camera_matrix, W, H, testbed.rendering_buffer.relative_focal_length, [0.5, 0.5], 0, abi.MODE_SHADE, 1.0)
    post = abi.default_post()
    post.background_color[:] = [1.0, 1.0, 1.0, 1.0]
    post.to_srgb = 0
    direct = r.render(view, post, 2)
    assert np.array_equal(direct.view(np.uint32), img.view(np.uint32))

    from helpers import make_oracle
    sc = dict(cfg=cfg, hash_table=table, density_mlp=dmlp, rgb_mlp=rmlp)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    n = orc.n_rays(view)
    acc = np.zeros((n, 4), np.float32)
    for spp in range(2):
        v = abi.View.from_buffer_copy(view); v.spp_index = spp
        res = orc.render_frame(v, post, 0, n, acc)
        acc = res["accum"]
    assert np.abs(res["out"].reshape(H, W, 4) - img).max() < 1e-3


@pytest.mark.gpu
def test_predict_driver_on_a_trajectory_file(built_lib, tmp_path):
    """The reference's predict loop (experiment/*/python/run.py:218-250) on a snapshot and a three-frame transforms file:
    colour + depth per frame, same pixels as calling the module by hand."""
    from sphericalrf_b200 import predict
    cfg, table, dmlp, rmlp, grid = _scene()
    path = tmp_path / "scene.msgpack"
    snapshot.write_snapshot(str(path), SMALL, grid, dmlp, rmlp, table, 1.0, (0.5, 0.5, 0.5))
    frames = []
    for k in range(3):
        c, s_ = np.cos(0.7 * k), np.sin(0.7 * k)
        frames.append({"file_path": f"./spherical/{k:03d}.png",
                       "transform_matrix": [[c, 0, s_, 0.2 * s_], [s_, 0, -c, -0.2 * c], [0, 1, 0, 0.05], [0, 0, 0, 1]]})
    W, H = 36, 24
    testbed = ngp.Testbed()
    testbed.load_snapshot(str(path))
    res = predict.predict(testbed, {"frames": frames}, W, H, angle_x_deg=60.0, spp=2, output_dir=str(tmp_path / "out"))
    assert len(res["images"]) == 3 and res["fps"] > 0 and all(d.shape == (H, W, 4) for d in res["depths"])
    assert (tmp_path / "out" / "image_predict" / "001.npy").exists() and (tmp_path / "out" / "depth_predict" / "002.npy").exists()
    again = ngp.Testbed()
    again.load_snapshot(str(path))
    again.background_color = [1.0, 1.0, 1.0, 1.0]
    again.fov_xy = [np.radians(60.0), np.radians(np.degrees(np.radians(30.0) / (W / H)) * 2.0)]
    again.set_nerf_camera_matrix(np.asarray(frames[1]["transform_matrix"], np.float32)[:-1, :])
    assert np.array_equal(again.render(W, H, 2, False), res["images"][1])
    assert not np.array_equal(res["images"][0], res["images"][1])
