"""Writes tests/golden/ref_pins.npz: what the reference's own kernels, compiled for the host
(oracle/build_ref.py), compute for every case of tests/refpin_cases.py.  Run where the reference is mounted:

    python tests/golden/make_ref_golden.py

The fixture lets tests/test_reference_pins.py check the oracle against the reference's source on machines that
do not have the reference.  Large arrays are stored as CRC-32 digests by the cases themselves.
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from oracle import srf_oracle, srf_ref  # noqa: E402
import refpin_cases  # noqa: E402


def main():
    if not srf_ref.available():
        raise SystemExit("the reference is not mounted here: cannot regenerate the fixture")
    store = {}
    for group, name, fn in refpin_cases.ALL_CASES:
        res = fn(name, "reference", srf_oracle, srf_ref)
        for key, arr in res.items():
            store[f"{group}/{name}/{key}"] = np.ascontiguousarray(arr)
        print(group, name, len(res), "arrays")
    out = Path(__file__).resolve().parent / "ref_pins.npz"
    np.savez_compressed(out, **store)
    print("wrote", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
