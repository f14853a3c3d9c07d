"""Batches of 1024 x 1024 images through the persistent kernel that interleaves the row pass of one image
with the column pass of the previous one and keeps the intermediate array in L2 (stockham_fused2d.cuh),
against the CPU oracle under rocfft-test's bounds.  Covers both precisions, both tile widths, in place and out
of place, inverse transforms with a scale factor, padded image distances, XY planes of a 3D transform,
enough images that CTAs wait for one another's row tiles, and base pointers that are not 16-byte aligned
(the step then runs the two ordinary passes it replaces)."""
import numpy as np
import pytest

import rocfft_b200 as rf
from harness import C2C_FWD, C2C_INV, IP, OOP, Case, run_case
from oracle import fft_oracle as orc

pytestmark = pytest.mark.gpu


def _plan_text(case):
    prec = rf.rocfft_precision_single if case.precision == "single" else rf.rocfft_precision_double
    kw = {}
    if case.in_dist or case.out_dist:
        kw = dict(in_array_type=rf.rocfft_array_type_complex_interleaved, out_array_type=rf.rocfft_array_type_complex_interleaved,
                  in_offsets=[0], out_offsets=[0], in_strides=None, in_distance=case.in_dist, out_strides=None,
                  out_distance=case.out_dist)
    p = rf.Plan(case.placement, case.ttype, prec, list(case.lengths), case.batch, scale=case.scale, **kw)
    t = p.describe()
    p.destroy()
    return t


CASES = [
    Case(C2C_FWD, "single", [1024, 1024], 4, IP),
    Case(C2C_FWD, "single", [1024, 1024], 5, OOP),
    Case(C2C_INV, "single", [1024, 1024], 6, OOP, scale=1.0 / (1 << 20)),
    Case(C2C_FWD, "double", [1024, 1024], 4, OOP),
    Case(C2C_INV, "double", [1024, 1024], 5, IP, scale=0.5),
    Case(C2C_FWD, "single", [1024, 1024, 4], 1, IP),       # XY planes of a 3D transform, then Z
    Case(C2C_FWD, "single", [1024, 1024, 8], 2, OOP),      # planes and batch merge into one image index
    Case(C2C_FWD, "single", [1024, 1024], 4, OOP, in_dist=(1 << 20) + 64, out_dist=(1 << 20) + 16),
    Case(C2C_FWD, "single", [1024, 1024], 40, IP),         # more images than fit between two waits
]


@pytest.mark.parametrize("units", ["8", "4"])
@pytest.mark.parametrize("case", CASES, ids=lambda c: c.ident())
def test_image_batches_through_l2(gpu, case, units, monkeypatch):
    monkeypatch.setenv("ROCFFT_B200_2D_L2_UNITS", units)
    monkeypatch.setenv("ROCFFT_B200_2D_L2", "1")  # single precision uses the kernel on request only
    text = _plan_text(case)
    assert "fft2d_l2" in text and f"_w{int(units) * 16}" in text, text
    ok, msg = run_case(case)
    assert ok, f"{case.ident()} units={units}: {msg}"


def test_misaligned_bases_take_the_two_ordinary_passes(gpu, monkeypatch):
    torch = gpu
    monkeypatch.setenv("ROCFFT_B200_2D_L2", "1")
    n, batch = 1024, 4
    x = orc.uniform_input((batch, n, n), np.complex64, seed=21)
    buf = torch.zeros(batch * n * n + 1, dtype=torch.complex64, device="cuda")
    view = buf[1:]  # 8 bytes past a 16-byte boundary
    assert view.data_ptr() % 16 == 8
    view.copy_(torch.from_numpy(x.reshape(-1)))
    plan = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [n, n], batch)
    assert "fft2d_l2" in plan.describe()
    plan.set_stream(torch.cuda.current_stream().cuda_stream)
    assert plan.execute([view.data_ptr()]) == 0
    torch.cuda.synchronize()
    assert plan.device_error() is False
    ok, msg = orc.check_accuracy(view.cpu().numpy().reshape(batch, n, n), orc.c2c(x, -1), "single", n * n)
    assert ok, msg
    plan.destroy()


def test_repeated_execution_reuses_the_counters(gpu, monkeypatch):
    """The per-image counters are reset by every launch: three executes in a row, each checked."""
    torch = gpu
    monkeypatch.setenv("ROCFFT_B200_2D_L2", "1")
    n, batch = 1024, 6
    plan = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [n, n], batch)
    plan.set_stream(torch.cuda.current_stream().cuda_stream)
    for rep in range(3):
        x = orc.uniform_input((batch, n, n), np.complex64, seed=30 + rep)
        d_in = torch.from_numpy(x).cuda()
        d_out = torch.full_like(d_in, float("nan"))
        assert plan.execute([d_in.data_ptr()], [d_out.data_ptr()]) == 0
        torch.cuda.synchronize()
        assert plan.device_error() is False
        ok, msg = orc.check_accuracy(d_out.cpu().numpy(), orc.c2c(x, -1), "single", n * n)
        assert ok, f"execute {rep}: {msg}"
    plan.destroy()
