"""The oracle against the reference's own source.

The reference has no CPU path and cannot be built as it is, but its kernels are plain C++ once Eigen, tiny-cuda-nn and
the CUDA built-ins are stood in for (oracle/ref_stub/): oracle/build_ref.py compiles them for the host where the
reference is mounted.  The oracle, built with the same arithmetic (the C library's elementary functions, no fused
multiply-adds: SRF_CANON_PLAIN), must reproduce what those kernels compute bit for bit -- sample counts, positions,
step widths, cell indices, colours, grids, bitfields, gradients.  That pins the oracle's control flow, statement
order and association order to the reference; what stays unpinned is named in oracle/ref_harness.cpp.

Two sources of the reference side: the committed fixture tests/golden/ref_pins.npz (always), and a live run of
oracle/_ref/libsrf_ref.so where it exists or can be built.
"""
from pathlib import Path

import numpy as np
import pytest

import refpin_cases

GOLDEN = Path(__file__).resolve().parent / "golden" / "ref_pins.npz"
IDS = [f"{g}-{n}" for g, n, _ in refpin_cases.ALL_CASES]


@pytest.fixture(scope="module")
def fixture_store():
    assert GOLDEN.exists(), "tests/golden/ref_pins.npz is missing (tests/golden/make_ref_golden.py writes it)"
    return np.load(GOLDEN)


@pytest.fixture(scope="module")
def ref_mod():
    from oracle import srf_ref
    return srf_ref


@pytest.mark.parametrize("case", refpin_cases.ALL_CASES, ids=IDS)
def test_oracle_reproduces_the_reference_fixture(oracle_mod, fixture_store, case):
    group, name, fn = case
    got = fn(name, "oracle", oracle_mod, None)
    prefix = f"{group}/{name}/"
    want = {k[len(prefix):]: fixture_store[k] for k in fixture_store.files if k.startswith(prefix)}
    assert want, f"no fixture entries for {prefix}"
    refpin_cases.compare(got, want, prefix[:-1])


@pytest.mark.parametrize("case", refpin_cases.ALL_CASES, ids=IDS)
def test_fixture_is_what_the_reference_kernels_compute(oracle_mod, ref_mod, fixture_store, case):
    """Live: the fixture is not stale with respect to the reference sources (skipped where they cannot be had)."""
    if not ref_mod.available():
        pytest.skip("reference not mounted and no earlier build of oracle/_ref/libsrf_ref.so")
    group, name, fn = case
    live = fn(name, "reference", oracle_mod, ref_mod)
    prefix = f"{group}/{name}/"
    want = {k[len(prefix):]: fixture_store[k] for k in fixture_store.files if k.startswith(prefix)}
    refpin_cases.compare(live, want, prefix[:-1])


def test_canonical_build_differs_only_in_rounding(oracle_mod):
    """The shipping oracle (canonical elementary functions, fused multiply-adds where written) and the plain build
    answer the same scene with the same structure: equal ray liveness, sample counts within a few per ray."""
    from helpers import make_oracle
    sc = refpin_cases._scene(refpin_cases.SAMPLER_CASES["disparity_erp"])
    bits = refpin_cases._bitfield(oracle_mod, sc)
    view = sc["view"]
    n = view.width * view.height
    orc = make_oracle(oracle_mod, sc, bits)
    c_canon = orc.march(view, 0, n, 1 << 22)[0].astype(np.int64)
    with oracle_mod.plain_arithmetic():
        c_plain = make_oracle(oracle_mod, sc, bits).march(view, 0, n, 1 << 22)[0].astype(np.int64)
    assert ((c_canon > 0) == (c_plain > 0)).all()
    assert np.abs(c_canon - c_plain).max() <= 8 and np.abs(c_canon - c_plain).mean() < 1.0
