"""CPU checks of the offline kernel generator: the emitted butterflies are
compiled as plain C++ and compared with a long-double DFT, and the function
pool it emits is consistent (factor products, required variants)."""
import ctypes
import os
import subprocess

import pytest

import rocfft_b200 as rf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "rocfft_b200", "csrc")


def test_generated_butterflies_match_dft(built_library, tmp_path):
    exe = str(tmp_path / "bfly_check")
    cmd = ["g++", "-O1", "-std=c++17", "-I", os.path.join(CSRC, "generated"), "-I", os.path.join(CSRC, "kernels"),
           os.path.join(ROOT, "tests", "butterfly_host_check.cpp"), "-o", exe, "-lm"]
    subprocess.check_call(cmd)
    r = subprocess.run([exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout


def test_function_pool_is_consistent(built_library):
    L = built_library
    L.b200fft_pool_query.argtypes = [ctypes.c_size_t, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                     ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                     ctypes.POINTER(ctypes.c_size_t)]
    cnt = ctypes.c_size_t()
    L.b200fft_pool_query(0, None, None, None, None, ctypes.byref(cnt))
    assert cnt.value > 0
    seen = {}
    for i in range(cnt.value):
        n, pr, va = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        f = (ctypes.c_int * 8)()
        assert L.b200fft_pool_query(i, ctypes.byref(n), ctypes.byref(pr), ctypes.byref(va), f, None) == 0
        prod = 1
        for v in f:
            if v:
                prod *= v
        assert prod == n.value
        seen.setdefault((n.value, pr.value), set()).add(va.value)
    for prec in (0, 1):
        for n in (4096, 1024, 1000, 500, 128, 160):
            assert (n, prec) in seen, (n, prec)
            # every length needs at least the unit-stride row kernel and the fully general one
            assert {0, 1} <= seen[(n, prec)]
