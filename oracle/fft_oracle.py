"""TEST INFRASTRUCTURE ONLY — the CPU oracle for the FFT hot path.

Nothing in the shipped library imports this module.  Only ``tests/``,
``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py`` may use it, and only as the checker or as the timed CPU
baseline.

What it restates
----------------
rocFFT has no CPU implementation of its transforms; ``rocfft-test`` compares the
GPU against FFTW (``shared/rocfft_against_fftw.h:50-143``, planned through
``shared/fftw_transform.h``).  FFTW 3.3.9 is a third-party dependency that the
reference downloads at configure time (``clients/tests/CMakeLists.txt:101-132``)
and it is not installed here, so this module restates the same mathematical
definition with pocketfft (``scipy.fft``) in double precision:

* forward  X[k] = sum_n x[n] exp(-2 pi i n k / N), inverse with the opposite
  sign and **no** 1/N factor (``docs/design/bluestein.rst:20-31``; round-trip
  scaling is done by the test itself, ``shared/accuracy_test.h:804``);
* multi-dimensional transforms are separable products over all dimensions;
* real forward keeps the non-redundant half ``N0/2+1`` along the fastest
  dimension (``library/src/plan.cpp:2980-2987``); real inverse consumes it and
  ignores Im(DC) / Im(Nyquist) (``clients/tests/hermitian_test.cpp:35-168``);
* ``lengths[0]`` is the fastest-varying dimension (``rocfft.h:161-164``);
  strides, distances and offsets are counted in elements of the array's own
  type (``docs/how-to/working-with-rocfft.rst:241-266``), defaults as in
  ``rocfft_plan_description_t::init_defaults`` (``library/src/plan.cpp:87-197``);
* error norms and pass/fail bounds as ``shared/accuracy_test.h:1497-1498,
  1609-1619`` with the epsilons of ``clients/tests/gtest_main.cpp:555-557``;
* inputs iid uniform in [-0.5, 0.5) per component
  (``shared/data_gen_host.h:507-700``) from a seeded generator.

Parity status: **unpinned in the stored-answer sense** — the reference tree holds
no golden vectors or known-answer files for this path (all expectations come
from FFTW at test time) and its GPU code cannot run here.  The oracle is
instead pinned against an independent long-double O(N^2) DFT
(``oracle/dft_ref.c``) in ``tests/test_oracle.py`` and against the committed
fixtures in ``tests/golden/``.
"""
from __future__ import annotations

import ctypes
import math
import os
import subprocess
from dataclasses import dataclass
from typing import Sequence

import numpy as np
import scipy.fft as _sfft

# --------------------------------------------------------------------------
# accuracy bounds (shared/accuracy_test.h:1497-1498, 1609-1619;
# clients/tests/gtest_main.cpp:555-557)
# --------------------------------------------------------------------------
EPS_SINGLE = 3.75e-5
EPS_DOUBLE = 1e-15
EPS_HALF = 9.77e-4


def type_epsilon(precision: str) -> float:
    return {"single": EPS_SINGLE, "double": EPS_DOUBLE, "half": EPS_HALF}[precision]


@dataclass
class Norms:
    l_2: float
    l_inf: float


def _components(a: np.ndarray) -> np.ndarray:
    """View complex data as separate real/imag components, as
    shared/fft_params.h:2657-2745 does when it accumulates norms."""
    a = np.asarray(a)
    if np.iscomplexobj(a):
        a = np.ascontiguousarray(a)
        return a.view(a.real.dtype)
    return a


def norms(a: np.ndarray) -> Norms:
    c = _components(a).astype(np.float64, copy=False).ravel()
    if c.size == 0:
        return Norms(0.0, 0.0)
    return Norms(float(np.sqrt(np.dot(c, c))), float(np.max(np.abs(c))))


def distance(a: np.ndarray, b: np.ndarray) -> Norms:
    ca = _components(a).astype(np.float64, copy=False)
    cb = _components(b).astype(np.float64, copy=False)
    return norms(ca - cb)


def check_accuracy(got: np.ndarray, ref: np.ndarray, precision: str, total_length: int):
    """Return (ok, message) under rocfft-test's two bounds:
    Linf:  |got-ref|_inf <= eps * |ref|_inf * ln(N_total)
    L2:    |got-ref|_2 / |ref|_2 < eps * sqrt(log2(N_total))"""
    eps = type_epsilon(precision)
    rn = norms(ref)
    d = distance(got, ref)
    n = max(int(total_length), 2)
    linf_cut = eps * rn.l_inf * math.log(n)
    l2_cut = eps * math.sqrt(math.log2(n))
    l2_rel = d.l_2 / rn.l_2 if rn.l_2 > 0 else d.l_2
    ok = (d.l_inf <= linf_cut) and (l2_rel < l2_cut)
    if not np.all(np.isfinite(_components(got))):
        ok = False
    msg = (f"Linf {d.l_inf:.3e} (cut {linf_cut:.3e}), "
           f"L2rel {l2_rel:.3e} (cut {l2_cut:.3e})")
    return ok, msg


# --------------------------------------------------------------------------
# seeded inputs (shared/data_gen_host.h:507-700: uniform [-0.5, 0.5) per
# component).  The reference seeds std::mt19937 per element index; any
# documented seeded generator with the same distribution serves the purpose,
# so numpy's PCG64 is used here.
# --------------------------------------------------------------------------
def uniform_input(shape, dtype, seed: int) -> np.ndarray:
    rng = np.random.default_rng(seed)
    dt = np.dtype(dtype)
    if dt.kind == "c":
        rdt = np.float32 if dt == np.complex64 else np.float64
        re = rng.random(shape, dtype=np.float64) - 0.5
        im = rng.random(shape, dtype=np.float64) - 0.5
        return (re.astype(rdt) + 1j * im.astype(rdt)).astype(dt)
    return (rng.random(shape, dtype=np.float64) - 0.5).astype(dt)


def hermitian_input(real_lengths: Sequence[int], batch: int, dtype, seed: int) -> np.ndarray:
    """A valid Hermitian half-spectrum for a c2r transform, produced the
    simple way: forward-transform a random real array.  (The reference imposes
    symmetry in place, shared/data_gen_host.h:66-339; the result is the same
    kind of object.)  Shape: (batch, len[r-1], ..., len[0]//2+1)."""
    shp = (batch,) + tuple(reversed(real_lengths))
    x = uniform_input(shp, np.float64, seed)
    axes = tuple(range(1, len(shp)))
    X = _sfft.rfftn(x, axes=axes) / math.sqrt(np.prod(real_lengths))
    return X.astype(dtype)


# --------------------------------------------------------------------------
# transforms on contiguous "logical" arrays, shape (batch, len[r-1], ..., len[0])
# --------------------------------------------------------------------------
def _workers():
    return os.cpu_count() or 1


def c2c(x: np.ndarray, direction: int, workers: int | None = None) -> np.ndarray:
    """Unnormalised complex transform over all axes but the first (batch).
    direction -1 = forward, +1 = inverse."""
    x = np.asarray(x, dtype=np.complex128)
    axes = tuple(range(1, x.ndim))
    w = workers or _workers()
    if direction < 0:
        return _sfft.fftn(x, axes=axes, workers=w)
    return _sfft.ifftn(x, axes=axes, norm="forward", workers=w)


def r2c(x: np.ndarray, workers: int | None = None) -> np.ndarray:
    """Real forward; the last numpy axis (= rocFFT dimension 0) is halved."""
    x = np.asarray(x, dtype=np.float64)
    axes = tuple(range(1, x.ndim))
    return _sfft.rfftn(x, axes=axes, workers=workers or _workers())


def c2r(X: np.ndarray, real_lengths: Sequence[int], workers: int | None = None) -> np.ndarray:
    """Real inverse, unnormalised.  `real_lengths` in rocFFT order (fastest
    first).  Im(DC)/Im(Nyquist) are ignored as pocketfft's c2r does."""
    X = np.asarray(X, dtype=np.complex128)
    axes = tuple(range(1, X.ndim))
    s = tuple(reversed(real_lengths))
    return _sfft.irfftn(X, s=s, axes=axes, norm="forward", workers=workers or _workers())


# --------------------------------------------------------------------------
# layout walker: rocFFT strides / distance / offset  <->  logical arrays
# --------------------------------------------------------------------------
def default_strides(lengths: Sequence[int]) -> list[int]:
    s = [1]
    for i in range(1, len(lengths)):
        s.append(s[-1] * lengths[i - 1])
    return s


@dataclass
class Layout:
    """lengths/strides are in rocFFT order (index 0 = fastest dimension);
    all counts are in elements of the buffer's own type."""
    lengths: tuple
    strides: tuple
    dist: int
    batch: int
    offset: int = 0

    def indices(self) -> np.ndarray:
        """Flat buffer index of every logical element, shape
        (batch, len[r-1], ..., len[0])."""
        idx = np.arange(self.batch, dtype=np.int64) * self.dist + self.offset
        idx = idx.reshape((self.batch,) + (1,) * len(self.lengths))
        r = len(self.lengths)
        for d in range(r):
            ax = 1 + (r - 1 - d)
            shp = [1] * (r + 1)
            shp[ax] = self.lengths[d]
            idx = idx + (np.arange(self.lengths[d], dtype=np.int64) * self.strides[d]).reshape(shp)
        return idx

    def extent(self) -> int:
        """Smallest buffer length (elements) that holds the layout."""
        if self.batch == 0 or any(l == 0 for l in self.lengths):
            return self.offset
        m = self.offset + (self.batch - 1) * self.dist
        for l, s in zip(self.lengths, self.strides):
            m += (l - 1) * s
        return m + 1

    def gather(self, buf: np.ndarray) -> np.ndarray:
        return buf[self.indices()]

    def scatter(self, buf: np.ndarray, values: np.ndarray) -> None:
        buf[self.indices()] = values


def canary_untouched(buf_bytes: np.ndarray, layout: Layout, itemsize: int, canary: int = 0xCD) -> bool:
    """True when every byte of `buf_bytes` that lies outside `layout` still
    holds the canary byte — the output-stride guard of
    shared/accuracy_test.h:611-682."""
    mask = np.ones(buf_bytes.size // itemsize, dtype=bool)
    mask[layout.indices().ravel()] = False
    view = buf_bytes[: mask.size * itemsize].reshape(-1, itemsize)
    return bool(np.all(view[mask] == canary))


# --------------------------------------------------------------------------
# long-double DFT (oracle/dft_ref.c) used to pin pocketfft
# --------------------------------------------------------------------------
_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build_dft_ref() -> str:
    so = os.path.join(_HERE, "libdft_ref.so")
    src = os.path.join(_HERE, "dft_ref.c")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-o", so, src, "-lm"])
    return so


def _lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build_dft_ref())
        dp = ctypes.POINTER(ctypes.c_double)
        _LIB.dft_ref_c2c.argtypes = [dp, dp, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int]
        _LIB.dft_ref_r2c.argtypes = [dp, dp, ctypes.c_size_t, ctypes.c_size_t]
        _LIB.dft_ref_c2r.argtypes = [dp, dp, ctypes.c_size_t, ctypes.c_size_t]
    return _LIB


def _dp(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_double))


def dft_c2c_longdouble(x: np.ndarray, direction: int) -> np.ndarray:
    """1D transform of every row of a 2D complex128 array (rows, n)."""
    x = np.ascontiguousarray(x, dtype=np.complex128)
    out = np.empty_like(x)
    rc = _lib().dft_ref_c2c(_dp(x.view(np.float64)), _dp(out.view(np.float64)),
                            x.shape[1], x.shape[0], -1 if direction < 0 else 1)
    assert rc == 0
    return out


def dft_r2c_longdouble(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float64)
    n = x.shape[1]
    out = np.empty((x.shape[0], n // 2 + 1), dtype=np.complex128)
    _lib().dft_ref_r2c(_dp(x), _dp(out.view(np.float64)), n, x.shape[0])
    return out


def dft_c2r_longdouble(X: np.ndarray, n: int) -> np.ndarray:
    X = np.ascontiguousarray(X, dtype=np.complex128)
    assert X.shape[1] == n // 2 + 1
    out = np.empty((X.shape[0], n), dtype=np.float64)
    _lib().dft_ref_c2r(_dp(X.view(np.float64)), _dp(out), n, X.shape[0])
    return out
