"""The row-per-warp Bluestein kernel (bluestein_rc.cuh; padded lengths R x 1024, R = 6 ... 20 in single and 6 ... 12 in double precision) against the CPU oracle:
lengths across the range of the largest padded length, 8193 ... 10240 (primes, a composite outside the pool, the
largest length it takes), one or two lengths for each of the smaller padded lengths,
forward and inverse, in place and out of place, strided and planar layouts, scale factors, several
transforms per launch.  Bounds: rocfft-test's (shared/accuracy_test.h:1497-1498, 1609-1619)."""
import pytest

import rocfft_b200 as rf
from harness import C2C_FWD, C2C_INV, CI, CP, IP, OOP, Case, run_case

pytestmark = pytest.mark.gpu

CASES = [
    Case(C2C_FWD, "single", [10007], 5, OOP),
    Case(C2C_INV, "single", [10007], 3, IP, scale=1.0 / 10007),
    Case(C2C_FWD, "single", [8209], 4, IP),                      # just above half of the next smaller padded length
    Case(C2C_FWD, "single", [10223], 2, OOP),                    # prime close to the top of the range
    Case(C2C_FWD, "single", [10239], 3, OOP),                    # 3 x 3413: 2n - 1 = 20477 <= 20480
    Case(C2C_FWD, "single", [9973], 3, OOP, CP, CP),             # planar on both sides
    Case(C2C_INV, "single", [9973], 2, OOP, CI, CP),
    Case(C2C_FWD, "single", [10007], 4, OOP, in_strides=[3], in_dist=3 * 10007 + 5, out_strides=[2], out_dist=2 * 10007),
    Case(C2C_FWD, "single", [10007, 3], 2, OOP),                 # as the first dimension of a 2D transform
    Case(C2C_FWD, "single", [3001], 7, OOP),                     # 6 x 1024
    Case(C2C_INV, "single", [3067], 5, IP),
    Case(C2C_FWD, "single", [4093], 6, IP),                      # 8 x 1024
    Case(C2C_FWD, "single", [4099], 9, OOP),                     # 10 x 1024
    Case(C2C_INV, "single", [5119], 4, OOP, CP, CI),
    Case(C2C_FWD, "single", [6007], 5, OOP),                     # 12 x 1024
    Case(C2C_FWD, "single", [8191], 3, IP),                      # 16 x 1024
    Case(C2C_INV, "single", [7919], 4, OOP, scale=0.5),
    Case(C2C_FWD, "single", [2503], 6, OOP),                     # 6 x 1024 preferred over the three-pass kernel at 5120
    Case(C2C_INV, "double", [2557], 3, IP),
    # double precision: padded lengths 6 ... 12 x 1024
    Case(C2C_FWD, "double", [3001], 5, OOP),
    Case(C2C_INV, "double", [4093], 3, IP),
    Case(C2C_FWD, "double", [4099], 4, OOP, CP, CP),
    Case(C2C_FWD, "double", [5119], 3, IP),
    Case(C2C_INV, "double", [6143], 2, OOP, scale=0.25),
]


def _plan_text(case):
    p = rf.Plan(case.placement, case.ttype, 0 if case.precision == "single" else 1, list(case.lengths), case.batch, scale=case.scale,
                in_array_type=case.in_type, out_array_type=case.out_type, in_strides=case.in_strides, out_strides=case.out_strides,
                in_distance=case.in_dist, out_distance=case.out_dist)
    t = p.describe()
    p.destroy()
    return t


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.ident())
def test_bluestein_one_warp_per_row(gpu, case):
    assert "row_blue_rc" in _plan_text(case), "the row-per-warp Bluestein kernel should serve this length"
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"


def test_matches_the_three_pass_kernel(gpu, monkeypatch):
    """Same answer (within the bounds) from the kernel it replaced."""
    case = Case(C2C_FWD, "single", [10007], 3, OOP)
    monkeypatch.setenv("ROCFFT_B200_NO_BLUE_RC", "1")
    assert "row_blue_rc" not in _plan_text(case) and "row_blue" in _plan_text(case)
    ok, msg = run_case(case)
    assert ok, msg
