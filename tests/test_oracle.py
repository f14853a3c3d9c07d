"""Pins the CPU oracle (pocketfft in double precision) against the committed
long-double fixtures and against the O(N^2) long-double DFT, and checks the
layout walker and the accuracy bounds (CPU only)."""
import json
import os

import numpy as np
import pytest

from oracle import fft_oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))


def _fixtures():
    with open(os.path.join(HERE, "golden", "dft_golden.json")) as f:
        return json.load(f)["fixtures"]


def _c(lst):
    a = np.array(lst, dtype=np.float64)
    return a[:, 0] + 1j * a[:, 1]


@pytest.mark.parametrize("fx", _fixtures(), ids=lambda f: f["name"])
def test_oracle_matches_golden(fx):
    n = fx["n"]
    if fx["kind"] == "c2c":
        got = orc.c2c(_c(fx["input"])[None, :], fx["direction"])[0]
        ref = _c(fx["output"])
    elif fx["kind"] == "r2c":
        got = orc.r2c(np.array(fx["input"])[None, :])[0]
        ref = _c(fx["output"])
    else:
        got = orc.c2r(_c(fx["input"])[None, :], [n])[0]
        ref = np.array(fx["output"])
    scale = max(1.0, np.max(np.abs(ref)))
    assert np.max(np.abs(got - ref)) <= 64 * np.finfo(np.float64).eps * scale * max(1, np.log2(max(n, 2)))


@pytest.mark.parametrize("n", [6, 17, 36, 210, 256, 331])
def test_oracle_vs_longdouble_dft(n):
    x = orc.uniform_input((3, n), np.complex128, seed=n)
    for d in (-1, 1):
        a = orc.c2c(x, d)
        b = orc.dft_c2c_longdouble(x, d)
        assert np.max(np.abs(a - b)) < 1e-12 * np.sqrt(n)
    xr = orc.uniform_input((2, n), np.float64, seed=n + 1)
    assert np.max(np.abs(orc.r2c(xr) - orc.dft_r2c_longdouble(xr))) < 1e-12 * np.sqrt(n)
    X = orc.r2c(xr)
    assert np.max(np.abs(orc.c2r(X, [n]) - orc.dft_c2r_longdouble(X, n))) < 1e-11 * n


def test_multidim_is_separable():
    x = orc.uniform_input((2, 5, 6, 8), np.complex128, seed=3)
    y = orc.c2c(x, -1)
    z = x.copy()
    for ax in (1, 2, 3):
        z = np.fft.fft(z, axis=ax)
    assert np.allclose(y, z, atol=1e-12)
    # inverse is unnormalised
    back = orc.c2c(y, +1) / (5 * 6 * 8)
    assert np.allclose(back, x, atol=1e-12)


def test_real_layout_halves_fastest_dim():
    x = orc.uniform_input((2, 4, 10), np.float64, seed=5)
    X = orc.r2c(x)
    assert X.shape == (2, 4, 6)
    full = orc.c2c(x.astype(np.complex128), -1)
    assert np.allclose(X, full[..., :6], atol=1e-12)
    assert np.allclose(orc.c2r(X, [10, 4]) / 40, x, atol=1e-12)


def test_layout_walker():
    lay = orc.Layout(lengths=(4, 3), strides=(2, 10), dist=40, batch=2, offset=5)
    idx = lay.indices()
    assert idx.shape == (2, 3, 4)
    assert idx[0, 0, 0] == 5 and idx[0, 0, 1] == 7 and idx[0, 1, 0] == 15 and idx[1, 0, 0] == 45
    assert lay.extent() == 5 + 40 + 20 + 6 + 1
    buf = np.zeros(lay.extent())
    vals = np.arange(24.0).reshape(2, 3, 4)
    lay.scatter(buf, vals)
    assert np.array_equal(lay.gather(buf), vals)
    assert np.count_nonzero(buf) == 23


def test_accuracy_bounds():
    ref = orc.uniform_input((4, 64), np.complex128, seed=9)
    ok, _ = orc.check_accuracy(ref.astype(np.complex64), ref, "single", 64)
    assert ok
    bad = ref.copy()
    bad[0, 0] += 1e-2
    ok, _ = orc.check_accuracy(bad, ref, "single", 64)
    assert not ok
    ok, _ = orc.check_accuracy(ref * (1 + 1e-13), ref, "double", 64)
    assert not ok


def test_canary_check():
    lay = orc.Layout(lengths=(3,), strides=(2,), dist=8, batch=2)
    b = np.full(lay.extent() * 4, 0xCD, dtype=np.uint8)
    lay.scatter(b.view(np.float32), np.ones((2, 3), np.float32))
    assert orc.canary_untouched(b, lay, 4)
    b.view(np.float32)[1] = 0
    assert not orc.canary_untouched(b, lay, 4)
