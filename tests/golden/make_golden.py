"""Generates the golden fixtures of tests/golden/ from the CPU oracle.

The reference has no tests, fixtures or golden outputs and cannot be run (GPU-only, unbuildable
here), so these vectors do not come from it: they freeze the oracle's own answers on tiny seeded
cases so that a later change to the oracle (or to a compiler flag) that alters a single bit is
caught.  Run from the repository root:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from sphericalrf_b200 import abi  # noqa: E402

from helpers import make_oracle, small_scene  # noqa: E402


def _frame(oracle_mod, **kw):
    sc = small_scene(width=12, height=8, grid_size=16, **kw)
    orc = make_oracle(oracle_mod, sc, None)
    bits, mean = orc.update_grid_bitfield(sc["grid"])
    orc.bitfield = bits
    n = orc.n_rays(sc["view"])
    counts, pos_dt, ordinal, cell, _ = orc.march(sc["view"], 0, n, 1 << 20)
    res = orc.render_frame(sc["view"], abi.default_post())
    keep = slice(0, 4096)
    return dict(bits=bits, mean=np.float32(mean), counts=counts, pos_dt=pos_dt[keep], ordinal=ordinal[keep], cell=cell[keep],
                rgba_raw=res["rgba_raw"], out=res["out"], n_composited=res["n_composited"])


def _refresh(oracle_mod):
    sc = small_scene(kind="net", grid_size=16)
    rng = np.random.Generator(np.random.PCG64(1))
    grid = (rng.random(16 ** 3) * 0.02).astype(np.float32)
    grid[::7] = -1.0
    orc = make_oracle(oracle_mod, sc, None)
    r = oracle_mod.rng_seed(3001)
    step, out = 0, {}
    for k in range(3):
        bits, mean, step = orc.refresh(grid, step, 0 if k < 2 else 300, r)
        out[f"grid{k}"] = grid.copy(); out[f"bits{k}"] = bits; out[f"mean{k}"] = np.float32(mean)
    return out


def _normals(oracle_mod):
    sc = small_scene(kind="net", width=10, height=6, grid_size=16)
    sc["view"].render_mode = abi.MODE_NORMALS
    orc = make_oracle(oracle_mod, sc, None)
    orc.bitfield = orc.update_grid_bitfield(sc["grid"])[0]
    res = orc.render_frame(sc["view"], abi.default_post())
    return dict(rgba_raw=res["rgba_raw"], out=res["out"])


def _training(oracle_mod):
    """Training rays -> network -> loss and gradient, on a 16^3 scene."""
    from sphericalrf_b200 import synth
    sc = small_scene(kind="net", grid_size=16)
    sc["cfg"].maximum_marching_steps = 64
    sc["cfg"].train_in_linear_color = 0
    orc = make_oracle(oracle_mod, sc, None)
    bits, mean = orc.update_grid_bitfield(sc["grid"])
    orc.bitfield = bits
    views = synth.training_views(41, n_images=3, width=16, height=12, radius=0.4)
    rng = oracle_mod.rng_seed(77)
    ts = oracle_mod.sample_training_rays(sc["cfg"], views, bits, 48, 5, 2048, rng, True)
    used = int(ts["numsteps"][:, 0].sum())
    net = orc.network_inference(ts["coords"][:used])
    p = abi.LossParams()
    p.n_rays, p.n_max_compacted_coords, p.loss_type, p.loss_scale = 48, 1024, abi.LOSS_SMOOTH_L1, 128.0
    p.regularization_type = abi.REG_DISTORTION
    p.background_color[:] = [0.3, 0.6, 0.1]
    p.color_space, p.train_with_random_bg_color, p.padded_output_width = abi.COLOR_SRGB, 1, 4
    p.rng_state, p.rng_inc = rng.state, rng.inc
    ls = oracle_mod.volume_rendering_loss(sc["cfg"], p, ts["n_rays"], ts["numsteps"], ts["rgba"], ts["coords"], net, float(mean))
    mask_cfg = synth.sampler_config("Original", 16)
    mask_cfg.warping_type, mask_cfg.grid_distribution_type, mask_cfg.aabb_scale = abi.WARP_NGP, abi.GRID_METRIC_EXP, 4
    mask = oracle_mod.mark_untrained(mask_cfg, synth.training_views(3, n_images=2, width=16, height=16, radius=1.5, fov_deg=30.0))
    return dict(rays=ts["rays"], rgba=ts["rgba"], numsteps=ts["numsteps"], coords=ts["coords"][:used],
                n_total=np.uint32(ts["n_samples_total"]), net=net.view(np.uint16), indices=ls["indices"],
                n_compacted=np.uint32(ls["n_compacted"]), dloss=ls["dloss"].view(np.uint16), loss=ls["loss"], reg=ls["reg"],
                mask=np.packbits(mask == 0))


CASES = {
    "blobs_disparity": lambda o: _frame(o, kind="blobs", sampling="Disparity"),
    "blobs_original": lambda o: _frame(o, kind="blobs", sampling="Original", radius=4.0),
    "net_disparity": lambda o: _frame(o, kind="net", sampling="Disparity"),
    "refresh": _refresh,
    "normals": _normals,
    "training": _training,
}

if __name__ == "__main__":
    from oracle import srf_oracle
    for name, fn in CASES.items():
        np.savez_compressed(HERE / f"{name}.npz", **fn(srf_oracle))
        print("wrote", name)
