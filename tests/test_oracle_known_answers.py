"""Pins the oracle to what CAN be pinned without running the reference:
 - the constants the reference itself carries (its Sobol direction-number table rows 0 and 1,
   internal/utils/random_val.cuh:139-155);
 - published test vectors of the algorithms it takes from absent dependencies (PCG32);
 - independent restatements in Python integers / numpy float64 of its integer and warp code.
The reference ships no tests, fixtures or golden outputs, so beyond this parity is unpinned."""
import ctypes as C

import numpy as np

from sphericalrf_b200 import abi, synth

# internal/utils/random_val.cuh:139-146 (dimension 0) and :148-155 (dimension 1)
SOBOL_DIM0 = [0x80000000 >> k for k in range(32)]
SOBOL_DIM1 = [
    0x80000000, 0xc0000000, 0xa0000000, 0xf0000000, 0x88000000, 0xcc000000, 0xaa000000, 0xff000000,
    0x80800000, 0xc0c00000, 0xa0a00000, 0xf0f00000, 0x88880000, 0xcccc0000, 0xaaaa0000, 0xffff0000,
    0x80008000, 0xc000c000, 0xa000a000, 0xf000f000, 0x88008800, 0xcc00cc00, 0xaa00aa00, 0xff00ff00,
    0x80808080, 0xc0c0c0c0, 0xa0a0a0a0, 0xf0f0f0f0, 0x88888888, 0xcccccccc, 0xaaaaaaaa, 0xffffffff,
]


def _lib(oracle_mod):
    lib = oracle_mod.lib()
    lib.srfo_rng_next_uint.restype = C.c_uint32
    lib.srfo_rng_next_float.restype = C.c_float
    lib.srfo_ld_random_val.restype = C.c_float
    lib.srfo_morton3d.restype = C.c_uint32
    lib.srfo_sobol.restype = C.c_uint32
    return lib


def test_sobol_direction_numbers_match_the_reference_table(oracle_mod):
    lib = _lib(oracle_mod)
    for k in range(32):
        assert lib.srfo_sobol(C.c_uint32(1 << k), C.c_uint32(0)) == SOBOL_DIM0[k]
        assert lib.srfo_sobol(C.c_uint32(1 << k), C.c_uint32(1)) == SOBOL_DIM1[k]
    # linearity over GF(2)
    assert lib.srfo_sobol(C.c_uint32(0b1011), C.c_uint32(1)) == SOBOL_DIM1[0] ^ SOBOL_DIM1[1] ^ SOBOL_DIM1[3]


def _owen(x, seed):
    M = 0xFFFFFFFF
    rev = lambda v: int(f"{v:032b}"[::-1], 2)
    x = rev(x)
    x = (x + seed) & M
    for c in (0x6c50b47c, 0xb82f1e52, 0xc7afe638, 0x8d22f6e6):
        x ^= (x * c) & M
    return rev(x)


def test_low_discrepancy_value_against_python_integers(oracle_mod):
    """ld_random_val (random_val.cuh:204-266) restated with Python integers."""
    lib = _lib(oracle_mod)
    M = 0xFFFFFFFF
    for index, seed in [(0, 0xdeadbeef), (5, 0xdeadbeef), (0, 786433 * 1234 & M), (3, 786433 * 99991 & M)]:
        i = _owen(index, seed)
        s = int(f"{i:032b}"[::-1], 2)                    # Sobol dimension 0 = bit reversal
        hc = seed ^ ((0 + ((seed << 6) & M) + (seed >> 2)) & M)
        want = np.float32(np.float32(_owen(s, hc)) * np.float32(2.0 ** -32))
        got = lib.srfo_ld_random_val(C.c_uint32(index), C.c_uint32(seed), C.c_uint32(0))
        assert np.float32(got) == want


def test_pcg32_published_vector(oracle_mod):
    """PCG32 demo output for seed 42, sequence 54 (O'Neill's pcg32-demo)."""
    lib = _lib(oracle_mod)
    r = oracle_mod.Rng()
    lib.srfo_rng_seed_seq(C.byref(r), C.c_uint64(42), C.c_uint64(54))
    got = [lib.srfo_rng_next_uint(C.byref(r)) for _ in range(6)]
    assert got == [0xa15c02b7, 0x7b47f409, 0xba1d3330, 0x83d2f293, 0xbfa4784b, 0xcbed606e]
    # advance(n) equals n single steps; floats lie in [0, 1)
    a = oracle_mod.rng_seed(7); b = oracle_mod.rng_seed(7)
    for _ in range(1000):
        lib.srfo_rng_next_uint(C.byref(a))
    lib.srfo_rng_advance(C.byref(b), C.c_uint64(1000))
    assert (a.state, a.inc) == (b.state, b.inc)
    f = [lib.srfo_rng_next_float(C.byref(a)) for _ in range(1000)]
    assert 0.0 <= min(f) and max(f) < 1.0


def test_morton_code(oracle_mod):
    lib = _lib(oracle_mod)
    def ref(x, y, z):
        m = 0
        for b in range(10):
            m |= ((x >> b) & 1) << (3 * b) | ((y >> b) & 1) << (3 * b + 1) | ((z >> b) & 1) << (3 * b + 2)
        return m
    rng = np.random.default_rng(0)
    for x, y, z in rng.integers(0, 1024, size=(200, 3)):
        assert lib.srfo_morton3d(C.c_uint32(int(x)), C.c_uint32(int(y)), C.c_uint32(int(z))) == ref(int(x), int(y), int(z))
    m = np.arange(4096, dtype=np.uint32)
    x, y, z = synth.morton3d_invert(m), synth.morton3d_invert(m >> np.uint32(1)), synth.morton3d_invert(m >> np.uint32(2))
    assert np.array_equal(synth.morton3d(x, y, z), m)


def test_sinusoidal_warp_against_float64(oracle_mod):
    """warp_position with the "ERP" type is the sinusoidal projection (the case has no break,
    internal/utils/common_device.h:412-447); checked against the closed form in float64."""
    cfg = synth.sampler_config("Disparity", 32)
    rng = np.random.default_rng(5)
    d = rng.normal(size=(20000, 3)); d /= np.linalg.norm(d, axis=1, keepdims=True)
    r = np.concatenate([rng.random(10000), 1.0 + rng.random(10000) * 50])
    pos = (0.5 + d * r[:, None]).astype(np.float32)
    for wt in (abi.WARP_ERP, abi.WARP_SINUSOIDAL):
        cfg.warping_type = wt
        got = oracle_mod.warp_position(cfg, pos).astype(np.float64)
        p = pos.astype(np.float64) - 0.5
        mag = np.linalg.norm(p, axis=1)
        theta = np.arctan2(p[:, 1], p[:, 0]); phi = np.arcsin(p[:, 2] / mag)
        want = np.stack([theta * np.cos(phi) / (2 * np.pi) + 0.5, phi / np.pi + 0.5,
                         0.5 * np.where(mag <= 1, mag, 2 - 1 / mag)], axis=1)
        assert np.abs(got - want).max() < 4e-6      # float asin is ill-conditioned near the poles
        back = oracle_mod.warp_position(cfg, got.astype(np.float32), inverse=True).astype(np.float64)
        inner = mag < 0.9                       # the outer shell's inverse is ill-conditioned near z = 1
        assert np.abs(back[inner] - pos[inner]).max() < 2e-5
    cfg.warping_type = abi.WARP_NGP
    cfg.aabb_scale = 4
    got = oracle_mod.warp_position(cfg, pos[:10000])
    assert np.abs(got - (pos[:10000] + 1.5) / 4.0).max() < 1e-6


def test_hashgrid_layout_rule(oracle_mod):
    cfg = synth.sampler_config()
    cfg.per_level_scale = 1.447
    off, res, sc = oracle_mod.hashgrid_layout(cfg)
    off2, res2, sc2 = synth.hashgrid_layout(cfg)
    assert np.array_equal(off, off2) and np.array_equal(res, res2) and np.array_equal(sc.view(np.uint32), sc2.view(np.uint32))
    assert res[0] == 16 and (np.diff(off.astype(np.int64)) <= 1 << 19).all() and (np.diff(off.astype(np.int64)) % 8 == 0).all()
    dense = res.astype(np.int64) ** 3 <= np.diff(off.astype(np.int64))
    assert dense[:5].all() and not dense[5:].any()
