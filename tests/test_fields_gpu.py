"""Single-process plans on fields of several bricks (gather -> transform -> scatter): the split
types of clients/tests/multi_device_test.cpp:38-187, with every brick on the GPU that is there
(bricks on distinct devices are covered by tests/test_multi_gpu.py)."""
import numpy as np
import pytest

import rocfft_b200 as rf
from fields_util import cut, grid_bricks, paste, plan_with_fields

pytestmark = pytest.mark.gpu

FWD, INV = rf.rocfft_transform_type_complex_forward, rf.rocfft_transform_type_complex_inverse
R2C, C2R = rf.rocfft_transform_type_real_forward, rf.rocfft_transform_type_real_inverse
IP, OOP = rf.rocfft_placement_inplace, rf.rocfft_placement_notinplace


def run_field_case(ttype, prec, lengths, batch, in_grid, out_grid, placement=OOP, devices=None, scale=None):
    """lengths fastest first.  Returns the relative l2 error against numpy in double precision."""
    import torch
    assert rf.rocfft_setup() == 0
    rank = len(lengths)
    rdt, cdt = (np.float32, np.complex64) if prec == 0 else (np.float64, np.complex128)
    rng = np.random.default_rng(42)
    shape = (batch,) + tuple(reversed(lengths))
    axes = tuple(range(1, rank + 1))
    herm = list(lengths)
    herm[0] = lengths[0] // 2 + 1
    if ttype in (FWD, INV):
        x = (rng.random(shape) - 0.5 + 1j * (rng.random(shape) - 0.5)).astype(cdt)
        ref = (np.fft.fftn if ttype == FWD else lambda a, axes: np.fft.ifftn(a, axes=axes) * np.prod(lengths))(
            x.astype(np.complex128), axes=axes)
        in_lat, out_lat, odt = list(lengths), list(lengths), cdt
    elif ttype == R2C:
        x = (rng.random(shape) - 0.5).astype(rdt)
        ref = np.fft.rfftn(x.astype(np.float64), axes=axes)
        in_lat, out_lat, odt = list(lengths), herm, cdt
    else:
        real = rng.random(shape) - 0.5
        x = np.fft.rfftn(real, axes=axes).astype(cdt)
        ref = np.fft.irfftn(x.astype(np.complex128), s=tuple(reversed(lengths)), axes=axes) * np.prod(lengths)
        in_lat, out_lat, odt = herm, list(lengths), rdt
    if scale is not None:
        ref = ref * scale
    in_bricks = grid_bricks(in_lat + [batch], in_grid)
    out_bricks = grid_bricks(out_lat + [batch], out_grid)
    in_dev = None if devices is None else [devices[i % len(devices)] for i in range(len(in_bricks))]
    out_dev = None if devices is None else [devices[i % len(devices)] for i in range(len(out_bricks))]
    st, plan, desc, in_sizes, out_sizes = plan_with_fields(placement, ttype, prec, lengths, batch, in_bricks, out_bricks,
                                                           in_dev, out_dev, scale)
    assert st == 0, f"plan creation failed: {st}"
    st, work_bytes = rf.rocfft_plan_get_work_buffer_size(plan)
    st, info = rf.rocfft_execution_info_create()
    work = None
    if work_bytes:
        work = torch.empty(work_bytes, dtype=torch.uint8, device="cuda:0")
        assert rf.rocfft_execution_info_set_work_buffer(info, work.data_ptr(), work_bytes) == 0
    tin = []
    for i, (lo, hi) in enumerate(in_bricks):
        dev = 0 if in_dev is None else in_dev[i]
        tin.append(torch.from_numpy(cut(x, lo, hi).reshape(-1)).to(f"cuda:{dev}"))
    if placement == IP:
        # the buffers must hold the larger of the input and the output brick
        for i, n in enumerate(out_sizes):
            need = n * np.dtype(odt).itemsize
            have = tin[i].numel() * tin[i].element_size()
            if need > have:
                big = torch.zeros(need, dtype=torch.uint8, device=tin[i].device)
                big[:have] = tin[i].view(torch.uint8)
                tin[i] = big
        tout = tin
        outs = None
    else:
        tout = []
        for j, n in enumerate(out_sizes):
            dev = 0 if out_dev is None else out_dev[j]
            tout.append(torch.zeros(n, dtype=torch.from_numpy(np.zeros(1, odt)).dtype, device=f"cuda:{dev}"))
        outs = [t.data_ptr() for t in tout]
    torch.cuda.synchronize()
    st = rf.rocfft_execute(plan, [t.data_ptr() for t in tin], outs, info)
    assert st == 0, f"execute failed: {st}"
    torch.cuda.synchronize()
    got = np.zeros(ref.shape, dtype=np.complex128 if odt == cdt else np.float64)
    for j, (lo, hi) in enumerate(out_bricks):
        raw = tout[j].view(torch.uint8).cpu().numpy()
        n = out_sizes[j]
        paste(got, lo, hi, raw[:n * np.dtype(odt).itemsize].view(odt))
    rf.rocfft_execution_info_destroy(info)
    rf.rocfft_plan_destroy(plan)
    rf.rocfft_plan_description_destroy(desc)
    return np.linalg.norm(got - ref) / np.linalg.norm(ref)


TOL = {0: 2e-5, 1: 1e-13}

SPLITS = {
    "slowest_both": ((1, 1, 2, 1), (1, 1, 2, 1)),
    "slowest_in_only": ((1, 1, 4, 1), (1, 1, 1, 1)),
    "slowest_out_only": ((1, 1, 1, 1), (1, 1, 3, 1)),
    "slow_in_fast_out": ((1, 1, 2, 1), (2, 1, 1, 1)),
    "pencils": ((1, 2, 2, 1), (2, 2, 1, 1)),
    "batch_split": ((1, 1, 1, 2), (1, 1, 1, 2)),
}


@pytest.mark.parametrize("split", list(SPLITS))
@pytest.mark.parametrize("prec", [0, 1])
def test_c2c_3d_splits(split, prec):
    gi, go = SPLITS[split]
    err = run_field_case(FWD, prec, [32, 20, 12], 2, gi, go)
    assert err < TOL[prec], err


@pytest.mark.parametrize("ttype", [FWD, INV])
def test_c2c_inplace_slabs(ttype):
    err = run_field_case(ttype, 0, [64, 16, 8], 1, (1, 1, 4, 1), (1, 1, 4, 1), placement=IP)
    assert err < TOL[0], err


@pytest.mark.parametrize("lengths,gi,go", [([64], (2, 1), (1, 2)), ([48, 40], (1, 2, 1), (2, 1, 1)),
                                           ([1000], (1, 4), (1, 4))])
def test_lower_ranks(lengths, gi, go):
    err = run_field_case(FWD, 0, lengths, 4, gi, go)
    assert err < TOL[0], err


@pytest.mark.parametrize("ttype", [R2C, C2R])
@pytest.mark.parametrize("placement", [OOP, IP])
def test_real_fields(ttype, placement):
    err = run_field_case(ttype, 0, [30, 16, 6], 2, (1, 1, 2, 1), (1, 2, 1, 1), placement=placement)
    assert err < TOL[0], err
    err = run_field_case(ttype, 1, [64, 10], 3, (1, 2, 1), (2, 1, 1), placement=placement)
    assert err < TOL[1], err


def test_scale_factor_reaches_the_gathered_plan():
    err = run_field_case(FWD, 0, [16, 16, 16], 1, (1, 1, 2, 1), (1, 2, 1, 1), scale=0.125)
    assert err < TOL[0], err
