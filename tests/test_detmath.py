"""Accuracy of include/mrl_detmath.h against double-precision libm."""
import numpy as np

from _util import fp, oracle


def _ulps(got, ref):
    ref32 = ref.astype(np.float32)
    ulp = np.spacing(np.abs(ref32)).astype(np.float64)
    return np.abs(got.astype(np.float64) - ref) / ulp


def _run(fn, x):
    y = np.empty_like(x)
    oracle().orc_detmath(fn, fp(x), fp(y), x.size)
    return y


def test_sin_cos():
    rng = np.random.default_rng(0)
    x = (rng.random(400000) * 200 - 100).astype(np.float32)
    s, c = _run(0, x), _run(1, x)
    rs, rc = np.sin(x.astype(np.float64)), np.cos(x.astype(np.float64))
    ok = np.abs(rs) > 1e-4
    assert _ulps(s, rs)[ok].max() <= 2.0 and np.abs(s - rs).max() < 2e-7
    ok = np.abs(rc) > 1e-4
    assert _ulps(c, rc)[ok].max() <= 2.0 and np.abs(c - rc).max() < 2e-7
    assert _run(0, np.zeros(1, np.float32))[0] == 0.0 and _run(1, np.zeros(1, np.float32))[0] == 1.0


def test_exp_log_tanh():
    rng = np.random.default_rng(1)
    x = (rng.random(400000) * 175 - 87).astype(np.float32)
    assert _ulps(_run(2, x), np.exp(x.astype(np.float64))).max() <= 2.0
    z = np.exp(rng.random(400000) * 170 - 85).astype(np.float32)
    rl = np.log(z.astype(np.float64))
    ok = np.abs(rl) > 1e-3
    assert _ulps(_run(3, z), rl)[ok].max() <= 2.5
    w = (rng.random(400000) * 24 - 12).astype(np.float32)
    w[::2] *= 0.03
    assert _ulps(_run(4, w), np.tanh(w.astype(np.float64))).max() <= 4.0
    edge = np.array([-200.0, 100.0, 0.0], np.float32)
    e = _run(2, edge)
    assert e[0] == 0.0 and np.isinf(e[1]) and e[2] == 1.0
    l = _run(3, np.array([1.0, 0.0, -1.0, np.inf], np.float32))
    assert l[0] == 0.0 and l[1] == -np.inf and np.isnan(l[2]) and l[3] == np.inf
