"""The canonical elementary functions (include/srf_canon_math.h, evaluated through the oracle)
against float64 libm: they must stay inside the error bounds the CUDA math library documents for
the functions they replace (atan2f, asinf, sinf, cosf: 2 ulp; expf, logf: 1-2 ulp)."""
import numpy as np


def _ulp_err(approx, exact):
    e32 = exact.astype(np.float32)
    ulp = np.maximum(np.spacing(np.abs(e32)).astype(np.float64), 1e-45)
    return np.abs(approx.astype(np.float64) - exact) / ulp


def test_atan2(oracle_mod):
    rng = np.random.default_rng(0)
    y = rng.normal(size=1_000_000).astype(np.float32); x = rng.normal(size=1_000_000).astype(np.float32)
    got = oracle_mod.eval_math(0, y, x)
    assert _ulp_err(got, np.arctan2(y.astype(np.float64), x.astype(np.float64))).max() <= 2.0
    # axes, quadrants, signed zero
    ys = np.array([0, 0, 1, -1, 1, -1, 0.0, 1e-30, 3.0], np.float32); xs = np.array([1, -1, 0, 0, 1, -1, 0.0, 1e30, -3.0], np.float32)
    exp = np.arctan2(ys.astype(np.float64), xs.astype(np.float64))
    assert np.abs(oracle_mod.eval_math(0, ys, xs) - exp).max() < 3e-7


def test_asin(oracle_mod):
    rng = np.random.default_rng(1)
    a = (rng.random(1_000_000) * 2 - 1).astype(np.float32)
    a[:5] = [0.0, 1.0, -1.0, 0.5, -0.5]
    got = oracle_mod.eval_math(1, a)
    assert _ulp_err(got, np.arcsin(a.astype(np.float64))).max() <= 2.0
    assert np.isnan(oracle_mod.eval_math(1, np.array([1.0000001, -1.5], np.float32))).all()   # as asinf does


def test_sincos(oracle_mod):
    rng = np.random.default_rng(2)
    a = ((rng.random(1_000_000) * 2 - 1) * 256).astype(np.float32)
    for op, f in ((2, np.cos), (3, np.sin)):
        got = oracle_mod.eval_math(op, a).astype(np.float64)
        assert (np.abs(got - f(a.astype(np.float64))) / 5.97e-8).max() <= 2.0    # in units of ulp(1)
    assert oracle_mod.eval_math(2, np.zeros(1, np.float32))[0] == 1.0
    assert oracle_mod.eval_math(3, np.zeros(1, np.float32))[0] == 0.0


def test_exp_log(oracle_mod):
    rng = np.random.default_rng(3)
    a = ((rng.random(1_000_000) * 2 - 1) * 87).astype(np.float32)
    assert _ulp_err(oracle_mod.eval_math(4, a), np.exp(a.astype(np.float64))).max() <= 1.5
    assert oracle_mod.eval_math(4, np.zeros(1, np.float32))[0] == 1.0
    assert oracle_mod.eval_math(4, np.array([-200.0], np.float32))[0] == 0.0
    assert np.isinf(oracle_mod.eval_math(4, np.array([100.0], np.float32))[0])
    b = np.exp((rng.random(1_000_000) * 2 - 1) * 80).astype(np.float32)
    assert _ulp_err(oracle_mod.eval_math(5, b), np.log(b.astype(np.float64))).max() <= 1.5
    assert oracle_mod.eval_math(5, np.ones(1, np.float32))[0] == 0.0
