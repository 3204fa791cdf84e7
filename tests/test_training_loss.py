"""Training compositor: volume rendering with loss and gradient (internal/render/ray_marcher.cu:9-202) and the
seven losses (internal/utils/loss.cu).  CPU: the oracle's gradient against finite differences of a float64
restatement of the forward pass.  GPU: the CUDA entry point against the oracle, bit for bit."""
import numpy as np
import pytest

from sphericalrf_b200 import abi, synth


def _batch(seed, n_rays=40, max_steps=24, early=False):
    """Random ragged batch: per-ray sample lists, raw fp16 network outputs, target pixels."""
    rng = np.random.Generator(np.random.PCG64(seed))
    counts = rng.integers(1, max_steps, n_rays).astype(np.uint32)
    bases = np.concatenate([[0], np.cumsum(counts)[:-1]]).astype(np.uint32)
    total = int(counts.sum())
    coords = rng.random((total, 7)).astype(np.float32)
    coords[:, 3] = rng.uniform(0.002, 0.05 if not early else 2.0, total).astype(np.float32)       # dt
    net = rng.normal(0, 1.0, (total, 4)).astype(np.float16)
    rgba = rng.random((n_rays, 4)).astype(np.float32)
    rgba[:, :3] *= rgba[:, 3:4]                                                                    # premultiplied, as the loader stores
    rgba[::7, 3] = 0.0; rgba[::7, :3] = 0.0
    return np.stack([counts, bases], 1).astype(np.uint32), coords, net, rgba


def _params(n_rays, cap, loss=abi.LOSS_L2, space=abi.COLOR_LINEAR, random_bg=False, reg=abi.REG_NONE, width=4):
    p = abi.LossParams()
    p.n_rays, p.n_max_compacted_coords, p.loss_type, p.loss_scale = n_rays, cap, loss, 128.0
    p.regularization_type = reg
    p.background_color[:] = [0.2, 0.5, 0.9]
    p.color_space = space
    p.train_with_random_bg_color = 1 if random_bg else 0
    p.rng_state, p.rng_inc = 0x853c49e6748fea9b, 0xda3e39cb94b95bdb
    p.padded_output_width = width
    return p


def _cfg(til=True, rgb_act=abi.ACT_LOGISTIC, thr=1e-4):
    cfg = synth.sampler_config("Original", 32)
    cfg.train_in_linear_color = 1 if til else 0
    cfg.rgb_activation, cfg.density_activation = rgb_act, abi.ACT_EXPONENTIAL
    cfg.transmittance_threshold = thr
    return cfg


def _total_loss64(idx, coords, net64, rgba, bg, loss_type):
    """Sum over rays and channels of the loss, float64, linear colour, no early stop."""
    out = 0.0
    for (cnt, base), tex in zip(idx, rgba.astype(np.float64)):
        T, ray = 1.0, np.zeros(3)
        for j in range(base, base + cnt):
            a = 1.0 - np.exp(-np.exp(net64[j, 3]) * float(coords[j, 3]))
            ray += a * T / (1.0 + np.exp(-net64[j, :3]))
            T *= 1.0 - a
        ray += T * bg
        d = ray - (tex[:3] + (1 - tex[3]) * bg)
        if loss_type == abi.LOSS_L2:
            out += (d * d).sum()
        elif loss_type == abi.LOSS_SMOOTH_L1:
            out += np.where(np.abs(d) > 0.1, np.abs(d) - 0.05, 5.0 * d * d).sum()
        elif loss_type == abi.LOSS_LOG_L1:
            out += np.log(np.abs(d) + 1).sum()
        elif loss_type == abi.LOSS_RELATIVE_L2:
            out += (d * d / (ray * ray + 1e-2)).sum()       # the reference treats the factor as a constant in its gradient
    return out


@pytest.mark.parametrize("loss_type", [abi.LOSS_L2, abi.LOSS_SMOOTH_L1, abi.LOSS_LOG_L1])
def test_gradient_matches_finite_differences(oracle_mod, loss_type):
    idx, coords, net, rgba = _batch(3, n_rays=6, max_steps=9)
    n = idx.shape[0]
    total = int(idx[:, 0].sum())
    cfg = _cfg(til=True, thr=0.0)
    p = _params(n, total, loss=loss_type)
    p.loss_scale = float(n)                              # makes dloss = d(total loss)/d(output)
    res = oracle_mod.volume_rendering_loss(cfg, p, n, idx, rgba, coords, net, mean_density=1.0)
    assert res["n_compacted"] == total and np.array_equal(res["indices"], idx)
    assert res["compacted_coords"].tobytes() == coords.tobytes()
    bg = np.array([synth_srgb_to_linear(c) for c in (0.2, 0.5, 0.9)])
    net64 = net.astype(np.float64)
    g = res["dloss"].astype(np.float64)
    h = 1e-5
    rng = np.random.Generator(np.random.PCG64(1))
    for _ in range(40):
        j, k = int(rng.integers(total)), int(rng.integers(4))
        up, dn = net64.copy(), net64.copy()
        up[j, k] += h; dn[j, k] -= h
        num = (_total_loss64(idx, coords, up, rgba, bg, loss_type) - _total_loss64(idx, coords, dn, rgba, bg, loss_type)) / (2 * h)
        assert abs(num - g[j, k]) <= 2e-3 + 2e-2 * abs(num), (j, k, num, g[j, k])
    # per-ray loss output: mean over channels / n_rays
    assert res["loss"].sum() * 3 * n == pytest.approx(_total_loss64(idx, coords, net64, rgba, bg, loss_type), rel=2e-3)


def synth_srgb_to_linear(s):
    return s / 12.92 if s <= 0.04045 else ((s + 0.055) / 1.055) ** 2.4


def test_compaction_rules(oracle_mod):
    idx, coords, net, rgba = _batch(5, n_rays=50, max_steps=30, early=True)
    n = idx.shape[0]
    cfg = _cfg(til=False, thr=1e-2)
    full = oracle_mod.volume_rendering_loss(cfg, _params(n, 1 << 16, space=abi.COLOR_SRGB), n, idx, rgba, coords, net, 1.0)
    consumed = full["indices"][:, 0].astype(np.int64)
    assert (consumed <= idx[:, 0]).all() and (consumed < idx[:, 0]).any()               # early termination shortens rays
    assert np.array_equal(full["indices"][:, 1], np.concatenate([[0], np.cumsum(consumed)[:-1]]))
    assert full["n_compacted"] == consumed.sum()
    for r in range(n):                                                                    # compacted coords are the consumed prefix
        b0, c0 = int(idx[r, 1]), int(full["indices"][r, 1])
        assert full["compacted_coords"][c0: c0 + consumed[r]].tobytes() == coords[b0: b0 + consumed[r]].tobytes()
    # a small capacity clips the ray that crosses it and empties the rest; the counter still counts everything
    cap = int(consumed.sum() // 2)
    cut = oracle_mod.volume_rendering_loss(cfg, _params(n, cap, space=abi.COLOR_SRGB), n, idx, rgba, coords, net, 1.0)
    assert cut["n_compacted"] == full["n_compacted"]
    kept = cut["indices"][:, 0].astype(np.int64)
    assert kept.sum() == cap and (kept <= consumed).all()
    assert cut["dloss"][:cap].tobytes() != np.zeros_like(cut["dloss"][:cap]).tobytes()
    # only the first n_rays_kept rays are processed
    part = oracle_mod.volume_rendering_loss(cfg, _params(n, 1 << 16, space=abi.COLOR_SRGB), 10, idx, rgba, coords, net, 1.0)
    assert np.array_equal(part["indices"][10:], idx[10:]) and part["n_compacted"] == consumed[:10].sum()


LOSS_CASES = [
    dict(loss=abi.LOSS_L2, space=abi.COLOR_LINEAR, til=True),
    dict(loss=abi.LOSS_L1, space=abi.COLOR_SRGB, til=False),
    dict(loss=abi.LOSS_MAPE, space=abi.COLOR_LINEAR, til=False, random_bg=True),
    dict(loss=abi.LOSS_SMAPE, space=abi.COLOR_SRGB, til=False, rgb_act=abi.ACT_EXPONENTIAL),
    dict(loss=abi.LOSS_SMOOTH_L1, space=abi.COLOR_SRGB, til=False, random_bg=True, reg=abi.REG_DISTORTION),
    dict(loss=abi.LOSS_LOG_L1, space=abi.COLOR_LINEAR, til=True, width=16),
    dict(loss=abi.LOSS_RELATIVE_L2, space=abi.COLOR_SRGB, til=True, reg=abi.REG_DISTORTION, rgb_act=abi.ACT_RELU),
]


@pytest.mark.gpu
@pytest.mark.parametrize("case", LOSS_CASES, ids=lambda c: f"loss{c['loss']}-cs{c['space']}-til{int(c['til'])}")
def test_training_compositor_bit_exact(built_lib, oracle_mod, case):
    from sphericalrf_b200.testbed import Renderer
    idx, coords, net, rgba = _batch(11 + case["loss"], n_rays=300, max_steps=40, early=True)
    n = idx.shape[0]
    cfg = _cfg(til=case["til"], rgb_act=case.get("rgb_act", abi.ACT_LOGISTIC), thr=1e-3)
    cfg.field_type = abi.FIELD_BLOBS
    r = Renderer(cfg, 0)
    for mean_density, grid_value in ((0.0, 0.0), (0.5, 0.5)):        # below / above min_optical_thickness: the density L1 term on / off
        r.upload_density_grid(np.full(32 ** 3, grid_value, np.float32))
        r.update_grid_bitfield()
        assert float(r.grid_mean()) == mean_density
        for cap, kept in ((1 << 15, n), (1500, n), (1 << 15, 100)):
            p = _params(n, cap, loss=case["loss"], space=case["space"], random_bg=case.get("random_bg", False),
                        reg=case.get("reg", abi.REG_NONE), width=case.get("width", 4))
            want = oracle_mod.volume_rendering_loss(cfg, p, kept, idx, rgba, coords, net, mean_density)
            got = r.volume_rendering_loss(p, kept, idx, rgba, coords, net)
            assert got["n_compacted"] == want["n_compacted"] > 0
            assert np.array_equal(got["indices"], want["indices"])
            used = int(want["indices"][:kept, 0].sum())
            assert used > 0
            assert got["compacted_coords"][:used].tobytes() == want["compacted_coords"][:used].tobytes()
            assert got["dloss"][:used].view(np.uint16).tobytes() == want["dloss"][:used].view(np.uint16).tobytes()
            assert np.isfinite(want["dloss"][:used].astype(np.float32)).all()
            assert got["loss"].tobytes() == want["loss"].tobytes()
            if p.regularization_type == abi.REG_DISTORTION:
                assert got["reg"][:used].tobytes() == want["reg"][:used].tobytes()


@pytest.mark.gpu
def test_training_compositor_large_batch(built_lib, oracle_mod):
    """6 000 rays (three tiles of the scan over consumed counts), capacity reached part of the way through."""
    from sphericalrf_b200.testbed import Renderer
    idx, coords, net, rgba = _batch(123, n_rays=6000, max_steps=60, early=True)
    n = idx.shape[0]
    cfg = _cfg(til=False, thr=1e-3)
    cfg.field_type = abi.FIELD_BLOBS
    r = Renderer(cfg, 0)
    r.upload_density_grid(np.full(32 ** 3, 0.5, np.float32))
    r.update_grid_bitfield()
    for cap in (1 << 18, 40000):
        p = _params(n, cap, loss=abi.LOSS_SMOOTH_L1, space=abi.COLOR_SRGB, random_bg=True, reg=abi.REG_DISTORTION)
        want = oracle_mod.volume_rendering_loss(cfg, p, n, idx, rgba, coords, net, 0.5)
        got = r.volume_rendering_loss(p, n, idx, rgba, coords, net)
        assert got["n_compacted"] == want["n_compacted"] and np.array_equal(got["indices"], want["indices"])
        used = int(want["indices"][:, 0].sum())
        assert used == min(cap, want["n_compacted"])
        assert got["compacted_coords"][:used].tobytes() == want["compacted_coords"][:used].tobytes()
        assert got["dloss"][:used].view(np.uint16).tobytes() == want["dloss"][:used].view(np.uint16).tobytes()
        assert got["loss"].tobytes() == want["loss"].tobytes() and got["reg"][:used].tobytes() == want["reg"][:used].tobytes()
