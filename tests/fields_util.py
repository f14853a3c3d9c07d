"""Helpers for tests of fields and bricks: split a lattice into a grid of bricks and build
the plan description the way shared/fft_params.h:2075-2156 (distribute_field) does."""
import ctypes
import itertools

import numpy as np

import rocfft_b200 as rf


def grid_bricks(lengths_with_batch, grid):
    """lengths_with_batch / grid: fastest dimension first, batch last.  Returns (lower, upper)
    pairs that tile the lattice; dimension i is cut into grid[i] nearly equal parts."""
    cuts = []
    for n, g in zip(lengths_with_batch, grid):
        edges = [n * k // g for k in range(g + 1)]
        cuts.append([(edges[k], edges[k + 1]) for k in range(g)])
    out = []
    for combo in itertools.product(*reversed(cuts)):  # slowest dimension outermost
        combo = list(reversed(combo))
        out.append(([c[0] for c in combo], [c[1] for c in combo]))
    return out


def contiguous_strides(lower, upper):
    s, st = 1, []
    for lo, hi in zip(lower, upper):
        st.append(s)
        s *= hi - lo
    return st, s


def make_field(bricks, devices=None, strides=None):
    """bricks: list of (lower, upper); contiguous strides unless given.  Returns (field, sizes)."""
    st, field = rf.rocfft_field_create()
    assert st == 0
    sizes = []
    for i, (lo, hi) in enumerate(bricks):
        stv, count = contiguous_strides(lo, hi)
        if strides is not None:
            stv = strides[i]
        st, b = rf.rocfft_brick_create(lo, hi, stv, 0 if devices is None else devices[i])
        assert st == 0
        assert rf.rocfft_field_add_brick(field, b) == 0
        rf.rocfft_brick_destroy(b)
        sizes.append(count)
    return field, sizes


def plan_with_fields(placement, ttype, precision, lengths, batch, in_bricks, out_bricks, in_dev=None, out_dev=None,
                     scale=None):
    """Returns (status, plan, desc, in_sizes, out_sizes)."""
    st, desc = rf.rocfft_plan_description_create()
    assert st == 0
    fin, in_sizes = make_field(in_bricks, in_dev)
    fout, out_sizes = make_field(out_bricks, out_dev)
    assert rf.rocfft_plan_description_add_infield(desc, fin) == 0
    assert rf.rocfft_plan_description_add_outfield(desc, fout) == 0
    rf.rocfft_field_destroy(fin)
    rf.rocfft_field_destroy(fout)
    if scale is not None:
        assert rf.rocfft_plan_description_set_scale_factor(desc, scale) == 0
    st, plan = rf.rocfft_plan_create(placement, ttype, precision, lengths, batch, desc)
    return st, plan, desc, in_sizes, out_sizes


def cut(array_cm, lower, upper):
    """array_cm indexed [batch][..slow..][fast]; lower / upper fastest first, batch last."""
    sl = tuple(slice(lo, hi) for lo, hi in zip(reversed(lower), reversed(upper)))
    return np.ascontiguousarray(array_cm[sl])


def paste(array_cm, lower, upper, block):
    sl = tuple(slice(lo, hi) for lo, hi in zip(reversed(lower), reversed(upper)))
    array_cm[sl] = block.reshape(array_cm[sl].shape)


def describe(plan):
    L = rf.lib()
    L.b200fft_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    buf = ctypes.create_string_buffer(1 << 16)
    assert L.b200fft_plan_describe(plan, buf, len(buf)) == 0
    return buf.value.decode()
