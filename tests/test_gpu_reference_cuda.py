"""This library's frames against the REFERENCE's own CUDA kernels on the same GPU.

baseline/build_refgpu.py compiles the reference's ray generation, marching, compaction, compositing, shading,
accumulation and tonemapping kernels for sm_100a from its sources (where they are mounted; the shared object travels)
with nvcc's defaults, and runs them in the reference's host loop; the network is this library's stage entry in both
pipelines.  So the two sides differ in exactly what parity is about: the CUDA math library and nvcc's contraction in the
reference's kernels against this library's own elementary functions and kernels.  Sampling is a chain of float steps
tested against cell boundaries, so a last-bit difference moves a sample across a boundary now and then; the test bounds
how often and reports the measured numbers (written as reference_cuda_parity.json into the run's output directory when it exists).
"""
import json
from pathlib import Path

import numpy as np
import pytest

from sphericalrf_b200 import abi, synth

from helpers import make_renderer, small_scene

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
RESULTS = {}


@pytest.fixture(scope="module")
def refgpu():
    from baseline import refgpu as m
    if not m.available():
        pytest.skip("baseline/_ref/libsrf_refgpu.so is not available (reference not mounted and no earlier build)")
    return m


def _compare(name, ours, theirs, n_rays):
    ca, cb = ours["n_samples"].astype(np.int64), theirs["n_samples"].astype(np.int64)
    same = ca == cb
    d_raw = np.abs(ours["rgba_raw"] - theirs["rgba_raw"])
    d_out = np.abs(ours["out"] - theirs["out"])
    RESULTS[name] = {
        "rays": int(n_rays), "samples": int(ca.sum()), "samples_reference_cuda": int(cb.sum()),
        "rays_with_different_sample_count": int((~same).sum()), "largest_count_difference": int(np.abs(ca - cb).max()),
        "max_abs_rgba_difference_rays_with_equal_counts": float(d_raw[same].max()) if same.any() else None,
        "max_abs_output_difference_rays_with_equal_counts": float(d_out[same].max()) if same.any() else None,
        "max_abs_rgba_difference": float(d_raw.max()), "max_abs_output_difference": float(d_out.max()),
        "reference_rounds": theirs["rounds"], "reference_network_slots": theirs["network_samples"],
    }
    out_dir = ROOT / "gpurun_out"
    if out_dir.is_dir():
        (out_dir / "reference_cuda_parity.json").write_text(json.dumps(RESULTS, indent=1))
    print(name, json.dumps(RESULTS[name]))
    return same, d_raw, d_out


SMALL = {
    "disparity_erp": dict(sampling="Disparity", warp=abi.WARP_ERP),
    "original_erp": dict(sampling="Original", warp=abi.WARP_ERP, radius=4.0),
    "original_ngp_3cascades": dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=3, grid_dist=abi.GRID_WARPED_EXP),
    "original_mipnerf360": dict(sampling="Original", warp=abi.WARP_MIPNERF360, aabb_scale=8, radius=1.5),
}


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("mode", [abi.MODE_SHADE, abi.MODE_DEPTH])
def test_small_scenes_against_the_reference_kernels(built_lib, refgpu, name, mode):
    sc = small_scene(kind="net", width=48, height=32, **SMALL[name])
    sc["view"].render_mode = mode
    r = make_renderer(sc)
    ref = refgpu.RefGpu(r)
    post = abi.default_post()
    post.background_color[:] = [0.1, 0.2, 0.3, 1.0]
    ours = r.render_frame(sc["view"], post, want_raw=True, want_counts=True)
    theirs = ref.render_frame(sc["view"], post)
    n = sc["view"].width * sc["view"].height
    same, d_raw, d_out = _compare(f"{name}/mode{mode}", ours, theirs, n)
    assert ours["n_samples"].sum() > 0
    assert (~same).sum() <= max(2, n // 100), "sample counts differ on more than 1 % of the rays"
    assert d_raw[same].max() <= 1e-3 and d_out[same].max() <= 1e-3


def test_config1_frame_against_the_reference_kernels(built_lib, refgpu):
    """The benchmark scene at 320x208 (108 M samples): per-ray sample counts, composited RGBA and pixels."""
    W, H = 320, 208
    sc = synth.scene_config1(width=W, height=H)
    from sphericalrf_b200.testbed import Renderer
    r = Renderer(sc["cfg"], 0)
    r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    r.upload_density_grid(sc["grid"]); r.update_grid_bitfield()
    ref = refgpu.RefGpu(r)
    view = abi.make_view(sc["cameras"][0], W, H, sc["rfl"])
    post = abi.default_post()
    ours = r.render_frame(view, post, want_raw=True, want_counts=True)
    theirs = ref.render_frame(view, post)
    same, d_raw, d_out = _compare("config1 320x208", ours, theirs, W * H)
    assert (~same).sum() <= W * H // 1000, "sample counts differ on more than 0.1 % of the rays"
    assert d_raw[same].max() <= 1e-3 and d_out[same].max() <= 1e-3


def test_config1_full_frame_against_the_reference_kernels(built_lib, refgpu):
    """The benchmark frame itself, 1245x825, 1.67 G samples: per-ray sample counts, composited RGBA and pixels of all
    1 027 125 rays against the reference's CUDA kernels."""
    W, H = 1245, 825
    sc = synth.scene_config1(width=W, height=H)
    from sphericalrf_b200.testbed import Renderer
    r = Renderer(sc["cfg"], 0)
    r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    r.upload_density_grid(sc["grid"]); r.update_grid_bitfield()
    ref = refgpu.RefGpu(r)
    view = abi.make_view(sc["cameras"][0], W, H, sc["rfl"])
    post = abi.default_post()
    ours = r.render_frame(view, post, want_raw=True, want_counts=True)
    theirs = ref.render_frame(view, post)
    same, d_raw, d_out = _compare("config1 1245x825", ours, theirs, W * H)
    assert (~same).sum() <= W * H // 10000, "sample counts differ on more than 0.01 % of the rays"
    assert d_raw[same].max() <= 1e-3 and d_out[same].max() <= 1e-3


def test_dense_original_sampling_with_output_stage_against_the_reference_kernels(built_lib, refgpu):
    """The dense inward-facing scene of configuration 4 (Original sampling; the opt-in sample cap off, the reference has
    none) at 480x270, three jittered passes per pixel, ACES curve and sRGB output."""
    W, H = 480, 270
    sc = synth.scene_config4(width=W, height=H)
    sc["cfg"].max_samples_per_ray = 0
    sc["cfg"].snap_to_pixel_centers_in_rendering = 0
    from sphericalrf_b200.testbed import Renderer
    r = Renderer(sc["cfg"], 0)
    r.upload_network(sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"])
    r.upload_density_grid(sc["grid"]); r.update_grid_bitfield()
    ref = refgpu.RefGpu(r)
    post = abi.default_post()
    post.tonemap_curve, post.to_srgb, post.exposure = abi.TONEMAP_ACES, 1, 0.5
    post.background_color[:] = [1.0, 1.0, 1.0, 1.0]
    import torch
    dev = torch.device("cuda", 0)
    n = W * H
    ours_out = torch.zeros((n, 4), device=dev); ours_acc = torch.zeros((n, 4), device=dev)
    ref_out = torch.zeros((n, 4), device=dev); ref_acc = torch.zeros((n, 4), device=dev)
    for spp in range(3):
        view = abi.make_view(sc["cameras"][1], W, H, sc["rfl"], spp_index=spp)
        r.render_frame_device(view, post, ours_out, ours_acc)
        ref.render_frame_device(view, post, ref_out, ref_acc)
    torch.cuda.synchronize()
    d = (ours_out - ref_out).abs()
    worst = float(d.max())
    frac = float((d.max(dim=1).values > 1e-3).float().mean())
    RESULTS["config4 480x270 spp3 aces srgb"] = {"max_abs_output_difference": worst, "fraction_of_pixels_beyond_1e-3": frac}
    print(RESULTS["config4 480x270 spp3 aces srgb"])
    assert frac <= 1e-3
