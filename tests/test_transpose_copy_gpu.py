"""Layout changes whose fastest dimension differs between input and output — here: in-place 2D transforms
whose output strides are the transpose of the input strides — go through a scratch array and a copy back;
that copy is a transpose and runs as 32 x 32 shared-memory tiles (launch/elementwise.cu; reference:
library/src/rtc_transpose_gen.cpp:77-326).  Checked against the CPU oracle with the placement canaries of the
harness, for sizes that are and are not multiples of the tile."""
import pytest

import rocfft_b200 as rf
from harness import C2C_FWD, C2C_INV, CI, IP, OOP, Case, run_case

pytestmark = pytest.mark.gpu

CASES = [
    Case(C2C_FWD, "single", [64, 128], 2, IP, CI, CI, [1, 64], [128, 1], 8192, 8192),
    Case(C2C_FWD, "double", [64, 128], 3, IP, CI, CI, [1, 64], [128, 1], 8192, 8192),
    Case(C2C_INV, "single", [100, 72], 2, IP, CI, CI, [1, 100], [72, 1], 7200, 7200),
    Case(C2C_FWD, "single", [1024, 512], 1, IP, CI, CI, [1, 1024], [512, 1], 1 << 19, 1 << 19),
    Case(C2C_FWD, "double", [48, 33], 4, IP, CI, CI, [1, 48], [33, 1], 1584, 1584),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.ident())
def test_in_place_with_transposed_output(gpu, case):
    prec = rf.rocfft_precision_single if case.precision == "single" else rf.rocfft_precision_double
    p = rf.Plan(case.placement, case.ttype, prec, list(case.lengths), case.batch, in_array_type=CI, out_array_type=CI,
                in_offsets=[0], out_offsets=[0], in_strides=list(case.in_strides), in_distance=case.in_dist,
                out_strides=list(case.out_strides), out_distance=case.out_dist)
    text = p.describe()
    p.destroy()
    assert "copy" in text, text  # the plan ends with the layout change under test
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"
