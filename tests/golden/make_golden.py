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


CASES = {
    "blobs_disparity": lambda o: _frame(o, kind="blobs", sampling="Disparity"),
    "blobs_original": lambda o: _frame(o, kind="blobs", sampling="Original", radius=4.0),
    "net_disparity": lambda o: _frame(o, kind="net", sampling="Disparity"),
    "refresh": _refresh,
}

if __name__ == "__main__":
    from oracle import srf_oracle
    for name, fn in CASES.items():
        np.savez_compressed(HERE / f"{name}.npz", **fn(srf_oracle))
        print("wrote", name)
