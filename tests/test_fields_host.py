"""Brick-layout validation of single-process multi-brick plans (no GPU needed: plans are
inspectable without one).  Reference: clients/tests/multi_device_test.cpp:189-280."""
import copy

import pytest

import rocfft_b200 as rf
from fields_util import describe, grid_bricks, plan_with_fields

FWD = rf.rocfft_transform_type_complex_forward
IP, OOP = rf.rocfft_placement_inplace, rf.rocfft_placement_notinplace


def _create(in_bricks, out_bricks, lengths=(8, 6, 4), batch=2, placement=OOP, ttype=FWD):
    st, plan, desc, _, _ = plan_with_fields(placement, ttype, rf.rocfft_precision_single, list(lengths), batch,
                                            in_bricks, out_bricks)
    text = None
    if st == 0:
        text = describe(plan)
    rf.rocfft_plan_destroy(plan)
    rf.rocfft_plan_description_destroy(desc)
    return st, text


@pytest.mark.parametrize("in_grid,out_grid", [((1, 1, 2, 1), (1, 1, 2, 1)), ((1, 1, 4, 1), (1, 1, 1, 1)),
                                              ((1, 1, 1, 1), (1, 1, 4, 1)), ((1, 1, 2, 1), (2, 1, 1, 1)),
                                              ((1, 2, 2, 1), (2, 2, 1, 1)), ((1, 1, 1, 2), (1, 3, 1, 1))])
def test_valid_layouts_are_accepted(in_grid, out_grid):
    rf.rocfft_setup()
    dims = [8, 6, 4, 2]
    st, text = _create(grid_bricks(dims, in_grid), grid_bricks(dims, out_grid))
    assert st == rf.rocfft_status_success
    assert text.startswith("gather/scatter plan")


@pytest.mark.parametrize("defect", ["missing", "lower_minus", "lower_plus", "upper_minus", "upper_plus", "duplicate",
                                    "short_dim"])
@pytest.mark.parametrize("side", ["in", "out"])
def test_invalid_layouts_are_refused(defect, side):
    rf.rocfft_setup()
    dims = [8, 6, 4, 2]
    good = grid_bricks(dims, (1, 2, 2, 1))
    bad = copy.deepcopy(good)
    lo, hi = bad[1]
    if defect == "missing":
        bad.pop(2)
    elif defect == "lower_minus":
        lo[1] -= 1  # overlaps its neighbour (or wraps below zero)
    elif defect == "lower_plus":
        lo[1] += 1  # leaves a gap
    elif defect == "upper_minus":
        hi[2] -= 1
    elif defect == "upper_plus":
        hi[2] += 1  # overlaps the next slab or leaves the field
    elif defect == "duplicate":
        bad.append(copy.deepcopy(bad[0]))
    elif defect == "short_dim":
        bad[0] = (bad[0][0][:3], bad[0][1][:3])
    if defect == "lower_minus" and lo[1] < 0:
        pytest.skip("negative index cannot be expressed in size_t")
    st, _ = _create(bad if side == "in" else good, good if side == "in" else bad)
    assert st != rf.rocfft_status_success


def test_inplace_needs_matching_brick_counts():
    rf.rocfft_setup()
    dims = [8, 6, 4, 2]
    st, _ = _create(grid_bricks(dims, (1, 1, 2, 1)), grid_bricks(dims, (1, 1, 4, 1)), placement=IP)
    assert st != rf.rocfft_status_success
    st, _ = _create(grid_bricks(dims, (1, 1, 2, 1)), grid_bricks(dims, (1, 2, 1, 1)), placement=IP)
    assert st == rf.rocfft_status_success


def test_real_fields_use_the_hermitian_lattice_on_the_complex_side():
    rf.rocfft_setup()
    r2c = rf.rocfft_transform_type_real_forward
    ok_in = grid_bricks([8, 6, 4, 2], (1, 1, 2, 1))
    ok_out = grid_bricks([5, 6, 4, 2], (1, 1, 2, 1))
    st, _ = _create(ok_in, ok_out, ttype=r2c)
    assert st == rf.rocfft_status_success
    st, _ = _create(ok_in, ok_in, ttype=r2c)  # output bricks on the real lattice: too large
    assert st != rf.rocfft_status_success
