"""GPU parity tests: the CUDA library, called through its C-ABI, against the CPU oracle on the same
seeded inputs.  Integers (sample counts, march-step ordinals, Morton cells, occupancy bits) and the
sampler's floats must be bit-exact; RGBA within 1e-3 for the fp16 network (tensor-core accumulation
order is unspecified) and bit-exact (checked as <= 1e-5) for the fp32 analytic field."""
import numpy as np
import pytest

from sphericalrf_b200 import abi, synth

from helpers import make_oracle, make_renderer, small_scene

pytestmark = pytest.mark.gpu


def _fp16_tolerance(ref, ulps=4):
    """`ulps` units in the last place of fp16 at the magnitude of the largest reference output: the bound for raw
    network outputs.  The kernels accumulate in fp32 like the oracle but in the tensor core's order, so a hidden
    activation now and then rounds to the neighbouring half; through at most three more layers of weights below 1
    that stays within a few fp16 ulps of the output scale."""
    scale = max(1.0, float(np.abs(ref).max()))
    return ulps * 2.0 ** (np.floor(np.log2(scale)) - 10)


def _bits_equal(a, b):
    return np.array_equal(np.ascontiguousarray(a).view(np.uint32), np.ascontiguousarray(b).view(np.uint32))


def test_device_math_matches_oracle_bit_for_bit(built_lib, oracle_mod):
    from sphericalrf_b200.testbed import eval_math
    rng = np.random.default_rng(3)
    n = 1 << 20
    cases = {
        0: (rng.normal(size=n), rng.normal(size=n)),
        1: (rng.random(n) * 2.002 - 1.001, None),
        2: ((rng.random(n) * 2 - 1) * 300, None),
        3: ((rng.random(n) * 2 - 1) * 300, None),
        4: ((rng.random(n) * 2 - 1) * 100, None),
        5: (np.exp((rng.random(n) * 2 - 1) * 80), None),
    }
    for op, (a, b) in cases.items():
        a = a.astype(np.float32)
        b = None if b is None else b.astype(np.float32)
        dev = eval_math(op, a, b)
        ref = oracle_mod.eval_math(op, a, b)
        assert _bits_equal(dev, ref), f"op {op}: {np.count_nonzero(dev.view(np.uint32) != ref.view(np.uint32))} mismatches"


SAMPLER_CASES = [
    dict(sampling="Disparity", warp=abi.WARP_ERP),
    dict(sampling="Original", warp=abi.WARP_ERP, radius=4.0),
    dict(sampling="Log", warp=abi.WARP_SINUSOIDAL, aabb_scale=64),
    dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.2),
    dict(sampling="Original", warp=abi.WARP_MIPNERF360, aabb_scale=8, radius=1.5),
    dict(sampling="Original", warp=abi.WARP_DONERF, aabb_scale=4, radius=1.5),
    dict(sampling="Original", warp=abi.WARP_SIGMOID, aabb_scale=8, radius=2.0),
    dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=3, grid_dist=abi.GRID_WARPED_EXP),
    dict(sampling="Original", warp=abi.WARP_NGP, aabb_scale=4, radius=1.5, cascades=2, grid_dist=abi.GRID_METRIC_RECIPROCAL),
]


@pytest.mark.parametrize("case", SAMPLER_CASES, ids=lambda c: f"{c['sampling']}-warp{c['warp']}-c{c.get('cascades', 1)}")
def test_sampler_bit_exact(built_lib, oracle_mod, case):
    kw = dict(case)
    sampling = kw.pop("sampling")
    sc = small_scene(kind="blobs", sampling="Disparity" if sampling == "Log" else sampling, **kw)
    if sampling == "Log":
        sc["cfg"].sampling_type = abi.SAMPLING_LOG
        sc["cfg"].far_distance = 100.0
    r = make_renderer(sc)
    bits = r.download_bitfield()
    orc = make_oracle(oracle_mod, sc, bits)
    b2, mean = orc.update_grid_bitfield(sc["grid"])
    assert np.array_equal(bits, b2)
    assert _bits_equal(np.float32(mean), np.float32(r.grid_mean()))
    view = sc["view"]
    n = orc.n_rays(view)
    cap = 1 << 22
    oc, opd, oo, ocell, _ = orc.march(view, 0, n, cap)
    gc, gpd, go, gcell = r.dump_samples(view, 0, n, cap)
    assert np.array_equal(oc, gc), "per-ray sample counts"
    assert np.array_equal(oo, go), "march-step ordinals"
    assert np.array_equal(ocell, gcell), "Morton cell indices"
    assert _bits_equal(opd, gpd), "warped positions and step widths"
    assert oc.sum() > 0
    # rays: direction, t at the first occupied step, alive flag
    import torch
    dev = torch.device("cuda", 0)
    d = torch.zeros((n, 3), device=dev); t = torch.zeros(n, device=dev)
    al = torch.zeros(n, dtype=torch.uint8, device=dev); px = torch.zeros(n, dtype=torch.int32, device=dev)
    st = built_lib.srf_generate_rays(r.ctx, view, d.data_ptr(), t.data_ptr(), al.data_ptr(), px.data_ptr(), None)
    assert st == 0
    torch.cuda.synchronize()
    od, ot, oal, opx = orc.generate_rays(view)
    assert np.array_equal(oal, al.cpu().numpy())
    assert np.array_equal(opx, px.cpu().numpy().astype(np.uint32))
    assert _bits_equal(od, d.cpu().numpy())
    assert _bits_equal(ot, t.cpu().numpy())


@pytest.mark.parametrize("sampling,radius", [("Disparity", 0.5), ("Original", 4.0)])
@pytest.mark.parametrize("mode", [abi.MODE_SHADE, abi.MODE_DEPTH, abi.MODE_DISTANCE, abi.MODE_AO, abi.MODE_COST])
def test_blob_field_frame_bit_exact(built_lib, oracle_mod, sampling, radius, mode):
    sc = small_scene(kind="blobs", sampling=sampling, radius=radius, width=32, height=24)
    sc["view"].render_mode = mode
    r = make_renderer(sc)
    bits = r.download_bitfield()
    orc = make_oracle(oracle_mod, sc, bits)
    post = abi.default_post()
    got = r.render_frame(sc["view"], post, want_raw=True, want_counts=True, want_stats=True)
    ref = orc.render_frame(sc["view"], post)
    counts, *_ = orc.march(sc["view"], 0, orc.n_rays(sc["view"]), 1 << 22)
    assert np.array_equal(counts, got["n_samples"])
    assert got["stats"]["n_samples_composited"] == ref["stats"]["n_samples_composited"]
    assert got["stats"]["n_rays_hit"] == ref["stats"]["n_rays_hit"]
    assert np.abs(got["rgba_raw"] - ref["rgba_raw"]).max() <= 1e-5
    assert np.abs(got["out"] - ref["out"]).max() <= 1e-5
    assert _bits_equal(got["rgba_raw"], ref["rgba_raw"]), "analytic field: premultiplied RGBA bit-exact"
    assert _bits_equal(got["out"], ref["out"]), "analytic field: output pixels bit-exact"
    assert ref["stats"]["n_rays_hit"] > 0


def test_early_termination_bit_exact(built_lib, oracle_mod):
    sc = small_scene(kind="blobs", sampling="Original", radius=4.0, width=32, height=24)
    sc["blobs"][:, 4] = 4000.0            # opaque blobs: rays stop inside them
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    got = r.render_frame(sc["view"], abi.default_post(), want_raw=True, want_stats=True)
    ref = orc.render_frame(sc["view"], abi.default_post())
    assert ref["stats"]["n_samples_composited"] < ref["stats"]["n_samples"] or ref["stats"]["n_samples_composited"] < got["stats"]["n_samples"]
    assert got["stats"]["n_samples_composited"] == ref["stats"]["n_samples_composited"]
    assert _bits_equal(got["rgba_raw"], ref["rgba_raw"])


@pytest.mark.parametrize("levels,features", [(16, 2), (8, 4)])
def test_normals_mode_bit_exact(built_lib, oracle_mod, levels, features):
    """Render mode Normals: density gradient through hash grid and density MLP in fp32, composited and shaded
    as testbed.cu:463-465 does.  The fp32 path has a fixed operation order, so the frame is the oracle's."""
    sc = small_scene(kind="net", width=20, height=12)
    cfg = sc["cfg"]
    cfg.n_levels, cfg.n_features_per_level = levels, features
    if features == 4:
        cfg.per_level_scale = 2.0
        from sphericalrf_b200 import synth
        sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"] = synth.network_params(cfg, 11, 12, table_range=0.5)
    sc["view"].render_mode = abi.MODE_NORMALS
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    post = abi.default_post()
    got = r.render_frame(sc["view"], post, want_raw=True)
    ref = orc.render_frame(sc["view"], post)
    assert _bits_equal(got["rgba_raw"], ref["rgba_raw"])
    assert _bits_equal(got["out"], ref["out"])
    hit = ref["rgba_raw"][:, 3] > 0.05
    assert hit.any()
    # shaded normals: 0.5 n + 0.5 scaled by the opacity, so every channel lies in [0, A]
    assert (ref["out"][hit, :3] >= 0).all() and (ref["out"][hit, :3] <= ref["out"][hit, 3:4] + 1e-6).all()
    assert np.ptp(ref["out"][hit, :3], axis=0).min() > 1e-3          # and they vary over the image


@pytest.fixture(params=["tcgen05", "mma_sync"])
def mlp_engine(request, monkeypatch):
    """Both MLP engines of the render path: tcgen05/TMEM (the default) and the mma.sync kernel."""
    monkeypatch.setenv("SRF_B200_MLP", request.param)
    return request.param


@pytest.mark.parametrize("levels,features", [(16, 2), (8, 4)])
def test_network_frame_within_tolerance(built_lib, oracle_mod, levels, features, mlp_engine):
    sc = small_scene(kind="net", width=24, height=16)
    cfg = sc["cfg"]
    cfg.n_levels, cfg.n_features_per_level = levels, features
    if features == 4:
        cfg.per_level_scale = 2.0
        from sphericalrf_b200 import synth
        sc["hash_table"], sc["density_mlp"], sc["rgb_mlp"] = synth.network_params(cfg, 11, 12, table_range=0.5)
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    post = abi.default_post()
    got = r.render_frame(sc["view"], post, want_raw=True, want_counts=True)
    ref = orc.render_frame(sc["view"], post)
    counts, *_ = orc.march(sc["view"], 0, orc.n_rays(sc["view"]), 1 << 22)
    assert np.array_equal(counts, got["n_samples"])
    assert np.abs(got["rgba_raw"] - ref["rgba_raw"]).max() <= 1e-3     # fp16 MLP tolerance
    assert np.abs(got["out"] - ref["out"]).max() <= 1e-3
    assert ref["rgba_raw"][:, 3].max() > 0.05


def test_network_stage_entry_points(built_lib, oracle_mod, mlp_engine):
    """srf_sample_count/offsets/emit -> srf_network_inference -> srf_volume_rendering, the reference's
    class-method sequence, against the oracle stage by stage."""
    import torch
    sc = small_scene(kind="net", width=16, height=12)
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    view = sc["view"]
    n = r.n_rays(view)
    dev = torch.device("cuda", 0)
    counts = torch.zeros(n, dtype=torch.int32, device=dev)
    offsets = torch.zeros(n + 1, dtype=torch.int64, device=dev)
    assert built_lib.srf_sample_count(r.ctx, view, counts.data_ptr(), None) == 0
    assert built_lib.srf_sample_offsets(r.ctx, counts.data_ptr(), n, offsets.data_ptr(), None) == 0
    total = int(offsets[-1].item())
    coords = torch.zeros((total, 7), device=dev)
    assert built_lib.srf_sample_emit(r.ctx, view, offsets.data_ptr(), total, coords.data_ptr(), None, None, None) == 0
    rgbs = torch.zeros((total, 4), dtype=torch.float16, device=dev)
    assert built_lib.srf_network_inference(r.ctx, coords.data_ptr(), total, rgbs.data_ptr(), None) == 0
    rgba = torch.zeros((n, 4), device=dev)
    ncomp = torch.zeros(n, dtype=torch.int32, device=dev)
    assert built_lib.srf_volume_rendering(r.ctx, view, offsets.data_ptr(), n, coords.data_ptr(), rgbs.data_ptr(),
                                          rgba.data_ptr(), ncomp.data_ptr(), None) == 0
    dens = torch.zeros((total, 16), dtype=torch.float16, device=dev)
    pos = coords[:, :3].contiguous()
    assert built_lib.srf_network_density(r.ctx, pos.data_ptr(), total, dens.data_ptr(), None) == 0
    torch.cuda.synchronize()
    oc, opd, _, _, _ = orc.march(view, 0, n, total + 1)
    assert np.array_equal(oc, counts.cpu().numpy().astype(np.uint32))
    c = coords.cpu().numpy()
    assert _bits_equal(c[:, :4], opd)
    ref = orc.network_inference(c).astype(np.float32)
    got = rgbs.cpu().numpy().astype(np.float32)
    assert np.abs(ref - got).max() <= _fp16_tolerance(ref)   # raw fp16 network outputs
    refd = orc.network_density(c[:, :3]).astype(np.float32)
    gotd = dens.cpu().numpy().astype(np.float32)
    assert np.abs(refd - gotd).max() <= _fp16_tolerance(refd)
    assert np.abs(got[:, 3] - gotd[:, 0]).max() == 0.0     # sigma is density output 0
    frame = orc.render_frame(view, abi.default_post())
    assert np.abs(frame["rgba_raw"] - rgba.cpu().numpy()).max() <= 1e-3


def test_mlp_engines_agree_on_raw_outputs(built_lib, oracle_mod, monkeypatch):
    """The tcgen05 kernel and the mma.sync kernel on the same 100k random coordinates (ragged tail included)."""
    import torch
    sc = small_scene(kind="net")
    rng = np.random.default_rng(9)
    n = 100_003
    coords = rng.random((n, 7)).astype(np.float32)
    dev = torch.device("cuda", 0)
    c = torch.from_numpy(coords).to(dev)
    outs = {}
    for engine in ("tcgen05", "mma_sync"):
        monkeypatch.setenv("SRF_B200_MLP", engine)
        r = make_renderer(sc)
        o = torch.zeros((n, 4), dtype=torch.float16, device=dev)
        assert built_lib.srf_network_inference(r.ctx, c.data_ptr(), n, o.data_ptr(), None) == 0
        torch.cuda.synchronize()
        outs[engine] = o.cpu().numpy().astype(np.float32)
    ref = make_oracle(oracle_mod, sc, None).network_inference(coords[:4096]).astype(np.float32)
    tol = _fp16_tolerance(ref)
    assert np.abs(outs["tcgen05"][:4096] - ref).max() <= tol
    assert np.abs(outs["mma_sync"][:4096] - ref).max() <= tol
    assert np.abs(outs["tcgen05"] - outs["mma_sync"]).max() <= tol
    assert np.isfinite(outs["tcgen05"]).all()


@pytest.mark.parametrize("path", ["masked_cells", "fused", "unfused"])
def test_grid_refresh_bit_exact(built_lib, oracle_mod, monkeypatch, path):
    """16 consecutive refreshes: every float of the grid and every bit after every step.  "masked_cells": a grid with
    never-seen cells (their samples are redirected: the multi-launch path with the atomic splat).  "fused": no masked
    cells and the two-launch refresh switched on, so the all-cells refreshes run as the fused kernel pair; "unfused": the
    default multi-launch path on the same grid.  The quarter/quarter refreshes at the end always take the multi-launch path."""
    monkeypatch.setenv("SRF_B200_FUSED_REFRESH", "1" if path == "fused" else "0")
    sc = small_scene(kind="net", grid_size=32)
    cfg = sc["cfg"]
    min_step = np.float32(np.sqrt(3.0) / cfg.maximum_marching_steps)
    rng = np.random.Generator(np.random.PCG64(3000))
    prior = (sc["grid"].astype(np.float64) * min_step * rng.uniform(0.5, 1.5, sc["grid"].shape[0])).astype(np.float32)
    if path == "masked_cells":
        prior[::97] = -1.0                   # masked cells stay negative
    sc["grid"] = prior
    r = make_renderer(sc)
    r.refresh_reset(3001)
    orc = make_oracle(oracle_mod, sc, None)
    grid = prior.copy()
    orng = oracle_mod.rng_seed(3001)
    step = 0
    for k in range(16):
        training_step = 0 if k < 12 else 256 + k       # the last refreshes use the quarter/quarter sampling
        obits, omean, step = orc.refresh(grid, step, training_step, orng)
        r.refresh_grid(training_step)
        g = r.download_density_grid()
        assert _bits_equal(g, grid), f"refresh {k}: grid floats"
        assert np.array_equal(r.download_bitfield(), obits), f"refresh {k}: bits"
        assert _bits_equal(np.float32(r.grid_mean()), np.float32(omean)), f"refresh {k}: mean"
    assert np.unpackbits(obits).mean() > 0.0
    r.check_errors()
    # the sampler's skip tables follow the bitfield on every path: a frame after the refreshes marches like the oracle
    orc2 = make_oracle(oracle_mod, sc, obits)
    n = orc2.n_rays(sc["view"])
    assert np.array_equal(orc2.march(sc["view"], 0, n, 1 << 22)[0], r.dump_samples(sc["view"], 0, n, 1 << 22)[0])


def test_sharded_frame_equals_whole_frame(built_lib):
    """Rays partitioned into row-block shards give byte-identical pixels to the single-shard frame."""
    sc = small_scene(kind="net", width=24, height=21)      # 21 rows: a partial last block
    r = make_renderer(sc)
    post = abi.default_post()
    whole = r.render_frame(sc["view"], post)["out"].reshape(21, 24, 4)
    for count in (2, 3):
        img = np.zeros_like(whole)
        for rank in range(count):
            v = abi.View.from_buffer_copy(sc["view"])
            v.shard_count, v.shard_rank, v.shard_rows = count, rank, 4
            part = r.render_frame(v, post)["out"]
            rows = [y for y in range(21) if (y // 4) % count == rank]
            img[rows] = part.reshape(len(rows), 24, 4)
        assert np.array_equal(img.view(np.uint32), whole.view(np.uint32))


def test_batched_frame_equals_single_batch(built_lib):
    sc = small_scene(kind="blobs", width=160, height=128, sampling="Original", radius=4.0)   # > 4096 rays: several groups
    r = make_renderer(sc)
    a = r.render_frame(sc["view"], abi.default_post(), want_stats=True)
    assert a["stats"]["n_batches"] == 1
    r.reserve(max(1, a["stats"]["n_samples"] // 3))
    b = r.render_frame(sc["view"], abi.default_post(), want_stats=True)
    assert b["stats"]["n_batches"] > 1
    assert np.array_equal(a["out"].view(np.uint32), b["out"].view(np.uint32))


OUTPUT_STAGES = {
    # tonemap curve, accumulation colour space, output sRGB, exposure, background
    "aces_srgb_out": (abi.TONEMAP_ACES, abi.COLOR_LINEAR, 1, 0.0, (1.0, 1.0, 1.0, 1.0)),
    "hable": (abi.TONEMAP_HABLE, abi.COLOR_LINEAR, 0, -0.4, (1.0, 1.0, 1.0, 0.5)),
    "reinhard_srgb_space": (abi.TONEMAP_REINHARD, abi.COLOR_SRGB, 1, 0.7, (0.3, 0.6, 0.1, 1.0)),
    "identity_visposneg": (abi.TONEMAP_IDENTITY, abi.COLOR_VISPOSNEG, 0, 0.0, (0.0, 0.0, 0.0, 1.0)),
    "hable_visposneg": (abi.TONEMAP_HABLE, abi.COLOR_VISPOSNEG, 1, 0.3, (0.2, 0.2, 0.2, 1.0)),
}


@pytest.mark.parametrize("stage", list(OUTPUT_STAGES))
def test_host_image_and_spp_accumulation(built_lib, oracle_mod, stage):
    """srf_render with three jittered passes: accumulate (all three colour spaces), exposure, background, the four
    tonemap curves and the output conversion (internal/utils/render_buffer.cu:46-181), bit for bit."""
    curve, space, to_srgb, exposure, bg = OUTPUT_STAGES[stage]
    sc = small_scene(kind="blobs", width=20, height=12)
    sc["cfg"].snap_to_pixel_centers_in_rendering = 0      # spp passes differ
    r = make_renderer(sc)
    orc = make_oracle(oracle_mod, sc, r.download_bitfield())
    post = abi.default_post()
    post.background_color[:] = list(bg)
    post.tonemap_curve, post.color_space, post.to_srgb, post.exposure = curve, space, to_srgb, exposure
    img = r.render(sc["view"], post, spp=3)
    accum = None
    for i in range(3):
        v = abi.View.from_buffer_copy(sc["view"])
        v.spp_index = i
        ref = orc.render_frame(v, post, accum=accum)
        accum = ref["accum"]
    assert np.abs(img.reshape(-1, 4) - ref["out"]).max() <= 1e-5
    assert _bits_equal(img.reshape(-1, 4), ref["out"])
    assert np.abs(ref["out"][:, :3]).max() > 0


def test_errors_are_reported_not_faked(built_lib):
    from sphericalrf_b200.testbed import Renderer
    cfg = abi.default_config()
    cfg.grid_size = 100
    with pytest.raises(abi.SrfError) as e:
        Renderer(cfg, 0)
    assert e.value.status == abi.ERR_ARG
    sc = small_scene(kind="net")
    r = Renderer(sc["cfg"], 0)
    with pytest.raises(abi.SrfError) as e:      # no weights uploaded
        r.render_frame(sc["view"], abi.default_post())
    assert e.value.status == abi.ERR_STATE
    sb = small_scene(kind="blobs")
    sb["view"].render_mode = abi.MODE_NORMALS                 # Normals is the density MLP's input gradient: network field only
    rb = make_renderer(sb)
    with pytest.raises(abi.SrfError) as e:
        rb.render_frame(sb["view"], abi.default_post())
    assert e.value.status == abi.ERR_ARG


def test_scatter_output_equals_compact_output(built_lib):
    """srf_render_frame_scatter: three shards write straight into one whole-image buffer; byte-equal to the
    single-shard frame, pixels of other shards untouched by each call."""
    import torch
    sc = small_scene(kind="net", width=24, height=21)
    r = make_renderer(sc)
    post = abi.default_post()
    whole = r.render_frame(sc["view"], post)["out"]
    dev = torch.device("cuda", 0)
    image = torch.full((21 * 24, 4), -7.0, dtype=torch.float32, device=dev)
    for rank in range(3):
        v = abi.View.from_buffer_copy(sc["view"])
        v.shard_count, v.shard_rank, v.shard_rows = 3, rank, 4
        accum = torch.zeros((r.n_rays(v), 4), dtype=torch.float32, device=dev)
        before = image.clone()
        r.render_frame_scatter_device(v, post, image, accum)
        torch.cuda.synchronize()
        rows = [y for y in range(21) if (y // 4) % 3 == rank]
        mask = torch.zeros(21, dtype=torch.bool)
        mask[rows] = True
        mask = mask.repeat_interleave(24).to(dev)
        assert torch.equal(image[~mask], before[~mask])
    assert np.array_equal(image.cpu().numpy().view(np.uint32), whole.view(np.uint32))


@pytest.mark.parametrize("sampling", ["Disparity", "Original"])
@pytest.mark.parametrize("fill", [0.002, 0.05])
def test_staged_empty_space_tests_change_nothing(built_lib, oracle_mod, monkeypatch, sampling, fill):
    """The sampler's 1-D / 2-D summaries of the bitfield only skip work: on a sparse random bitfield the sample
    list is the oracle's, and the one a context built without the summaries produces."""
    from sphericalrf_b200.testbed import Renderer
    sc = small_scene(kind="blobs", sampling=sampling, radius=0.5 if sampling == "Disparity" else 4.0, grid_size=64)
    rng = np.random.Generator(np.random.PCG64(11))
    n_cells = 64 ** 3
    bits = np.packbits(rng.random(n_cells) < fill, bitorder="little")
    view = sc["view"]
    outs = []
    for flag in ("1", "0"):
        monkeypatch.setenv("SRF_B200_SKIP_TABLES", flag)
        r = Renderer(sc["cfg"], 0)
        r.upload_blobs(sc["blobs"], sc["color_map"])
        r.upload_bitfield(bits)
        outs.append(r.dump_samples(view, 0, r.n_rays(view), 1 << 22))
        frame = r.render_frame(view, abi.default_post())["out"]
        outs[-1] = outs[-1] + (frame,)
    for a, b in zip(outs[0], outs[1]):
        assert np.array_equal(a.view(np.uint32) if a.dtype == np.float32 else a, b.view(np.uint32) if b.dtype == np.float32 else b)
    orc = make_oracle(oracle_mod, sc, bits)
    oc, opd, oo, ocell, _ = orc.march(view, 0, orc.n_rays(view), 1 << 22)
    gc, gpd, go, gcell, _ = outs[0]
    assert np.array_equal(oc, gc) and np.array_equal(oo, go) and np.array_equal(ocell, gcell)
    assert _bits_equal(opd, gpd)
    assert oc.sum() > 0


@pytest.mark.parametrize("kind,budgets", [("blobs", "1000,1000,1000"), ("blobs", "64,512"), ("net", "5,40,300"), ("blobs", "1")])
def test_waves_change_nothing_but_the_work(built_lib, monkeypatch, kind, budgets):
    """A frame rendered in waves (a budget of march steps per ray and wave, compositing in between, finished rays dropped) is
    byte-identical to the one-pass frame; on a scene with opaque blobs it generates and evaluates fewer samples."""
    sc = small_scene(kind=kind, sampling="Original", radius=4.0, width=32, height=24)
    if kind == "blobs":
        sc["blobs"][:, 4] = 4000.0            # opaque blobs: rays stop inside them
    post = abi.default_post()
    post.background_color[:] = [0.2, 0.4, 0.6, 1.0]
    res = {}
    for key, env in (("one", "0"), ("waves", budgets)):
        monkeypatch.setenv("SRF_B200_WAVES", "0" if key == "one" else "7")
        r = make_renderer(sc)
        if key == "waves":
            r.set_wave_schedule([int(x) for x in budgets.split(",")])      # replaces the environment's schedule
        a = r.render_frame(sc["view"], post, want_raw=True, want_stats=True)
        v2 = abi.View.from_buffer_copy(sc["view"]); v2.spp_index = 1
        b = r.render_frame(v2, post, accum=a["accum"], want_raw=True)
        v3 = abi.View.from_buffer_copy(sc["view"]); v3.render_mode = abi.MODE_DEPTH
        c = r.render_frame(v3, post, want_raw=True)
        res[key] = (a, b, c)
    for x, y in zip(res["one"], res["waves"]):
        for k in ("out", "accum", "rgba_raw"):
            assert _bits_equal(x[k], y[k]), k
    s1, s2 = res["one"][0]["stats"], res["waves"][0]["stats"]
    assert s1["n_samples_composited"] == s2["n_samples_composited"] and s1["n_rays_hit"] == s2["n_rays_hit"]
    assert s1["n_rays_alive"] == s2["n_rays_alive"]
    assert s2["n_samples"] <= s1["n_samples"] and s2["n_march_steps"] <= s1["n_march_steps"]
    if kind == "blobs":
        assert s1["n_samples_composited"] < s1["n_samples"]                 # rays do terminate early here
        if budgets == "1000,1000,1000":                                     # the blobs start ~1500 steps into the march
            assert s2["n_samples"] < s1["n_samples"]                        # and the waves skip what lies behind
    # per-ray sampler counts are those of the whole march, whatever the schedule
    counts_waves = make_renderer(sc).render_frame(sc["view"], post, want_counts=True)["n_samples"]
    monkeypatch.setenv("SRF_B200_WAVES", "0")
    counts_one = make_renderer(sc).render_frame(sc["view"], post, want_counts=True)["n_samples"]
    assert np.array_equal(counts_waves, counts_one) and int(counts_one.sum()) == s1["n_samples"]


@pytest.mark.parametrize("levels,features", [(16, 2), (8, 4)])
def test_table_copies_change_nothing(built_lib, monkeypatch, levels, features):
    """Cell-major copies of the leading hash-grid levels (dense and hashed ones) and the tabulated activations are
    memory layouts, not arithmetic: frames, raw network outputs (also for coordinates outside the unit cube, which take
    the scattered path) and the frame after a second srf_upload_network are byte-identical with and without them."""
    sc = small_scene(kind="net", width=24, height=16)
    cfg = sc["cfg"]
    cfg.n_levels = levels; cfg.n_features_per_level = features
    t, d, c = synth.network_params(cfg, 11, 12, table_range=0.5)
    sc.update(hash_table=t, density_mlp=d, rgb_mlp=c)
    t2, _, _ = synth.network_params(cfg, 21, 12, table_range=0.5)
    rng = np.random.Generator(np.random.PCG64(5))
    coords = rng.random((20000, 7), dtype=np.float32)
    coords[:4000, :3] = coords[:4000, :3] * 3.0 - 1.0          # outside [0,1]: cells outside the levels
    coords[4000:4100, :3] = np.array([1.0, 1.0, 1.0], np.float32)
    coords[4100:4200, :3] = 0.0
    post = abi.default_post()
    out = {}
    for key in ("plain", "copies"):
        monkeypatch.setenv("SRF_B200_ACT_LUT", "0" if key == "plain" else "1")
        r = make_renderer(sc)
        r.set_cell_table_budget(0 if key == "plain" else 96 << 20)
        a = r.render_frame(sc["view"], post, want_raw=True)
        v3 = abi.View.from_buffer_copy(sc["view"]); v3.render_mode = abi.MODE_AO
        b = r.render_frame(v3, post, want_raw=True)
        raw = r.network_inference(coords)
        r.upload_network(t2, sc["density_mlp"], sc["rgb_mlp"])
        a2 = r.render_frame(sc["view"], post, want_raw=True)
        out[key] = (a["out"], a["rgba_raw"], b["out"], raw.view(np.uint16), a2["out"], a2["rgba_raw"])
        r.check_errors()
    for x, y in zip(out["plain"], out["copies"]):
        assert _bits_equal(np.asarray(x), np.asarray(y))
    assert not _bits_equal(out["copies"][0], out["copies"][4])      # the second upload did change the picture
