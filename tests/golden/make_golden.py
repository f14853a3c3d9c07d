"""Generates tests/golden/*.json: small input/output pairs that pin the CPU
oracle.  Outputs come from the long-double O(N^2) DFT of oracle/dft_ref.c, which
follows the transform definition of the reference's documentation
(docs/design/bluestein.rst:20-31), not from the fast oracle being pinned.

The reference's test tree stores no expected outputs; the only literal data it
holds for this path is the 8-point complex input of
clients/tests/unit_test.cpp:135-142, reproduced below as the first fixture's
input.  Run:  python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import fft_oracle as orc  # noqa: E402


def cplx_list(a):
    return [[float(v.real), float(v.imag)] for v in np.asarray(a).ravel()]


def main():
    fixtures = []
    unit8 = np.array([-0.100 + 0.380j, 0.0166 + 0.439j, -0.475 + 0.212j, 0.440 - 0.432j,
                      0.445 + 0.0589j, 0.296 + 0.164j, -0.084 + 0.077j, 0.320 + 0.087j])
    for direction in (-1, 1):
        out = orc.dft_c2c_longdouble(unit8[None, :], direction)[0]
        fixtures.append({"name": f"unit_test_8pt_dir{direction}", "kind": "c2c", "n": 8, "direction": direction,
                         "input": cplx_list(unit8), "output": cplx_list(out)})
    rng = np.random.default_rng(20240607)
    for n in (1, 2, 3, 4, 5, 7, 12, 16, 25, 31, 64, 100, 127):
        x = (rng.random(n) - 0.5) + 1j * (rng.random(n) - 0.5)
        for direction in (-1, 1):
            out = orc.dft_c2c_longdouble(x[None, :], direction)[0]
            fixtures.append({"name": f"c2c_{n}_dir{direction}", "kind": "c2c", "n": n, "direction": direction,
                             "input": cplx_list(x), "output": cplx_list(out)})
    for n in (2, 3, 8, 9, 10, 30, 100, 101):
        x = rng.random(n) - 0.5
        X = orc.dft_r2c_longdouble(x[None, :])[0]
        fixtures.append({"name": f"r2c_{n}", "kind": "r2c", "n": n, "input": [float(v) for v in x],
                         "output": cplx_list(X)})
        # inverse of a spectrum whose DC / Nyquist imaginary parts are junk: they must not matter
        Xj = X.copy()
        Xj[0] += 0.25j
        if n % 2 == 0:
            Xj[-1] -= 0.5j
        y = orc.dft_c2r_longdouble(Xj[None, :], n)[0]
        fixtures.append({"name": f"c2r_{n}", "kind": "c2r", "n": n, "input": cplx_list(Xj),
                         "output": [float(v) for v in y]})
    with open(os.path.join(HERE, "dft_golden.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "fixtures": fixtures}, f, indent=0)
    print(f"wrote {len(fixtures)} fixtures")


if __name__ == "__main__":
    main()
