"""The persistent TMA-fed column kernel (stockham_colstream.cuh) against the CPU oracle: 1024-point
transforms along the strided dimensions of 2D / 3D arrays in both precisions (its default use), the
shorter lengths it exists for (forced through ROCFFT_B200_COLTMA), inverse transforms, scale factors,
in place and out of place, and many tiles per CTA (more tiles than resident CTAs, so every CTA reuses
its stage and flips its mbarrier phase several times).  Bounds: rocfft-test's
(shared/accuracy_test.h:1497-1498, 1609-1619); placement is checked through the canary bytes."""
import numpy as np
import pytest

import rocfft_b200 as rf
from harness import C2C_FWD, C2C_INV, IP, OOP, Case, run_case

pytestmark = pytest.mark.gpu


def _plan_text(case):
    prec = rf.rocfft_precision_single if case.precision == "single" else rf.rocfft_precision_double
    p = rf.Plan(case.placement, case.ttype, prec, list(case.lengths), case.batch, scale=case.scale)
    t = p.describe()
    p.destroy()
    return t


CASES_1024 = [
    Case(C2C_FWD, "single", [1024, 1024], 2, IP),
    Case(C2C_INV, "single", [1024, 1024], 1, OOP, scale=1.0 / 1024),
    Case(C2C_FWD, "double", [1024, 1024], 2, OOP),
    Case(C2C_INV, "double", [1024, 1024], 1, IP),
    Case(C2C_FWD, "single", [32, 1024, 4], 1, IP),      # few columns per row
    Case(C2C_FWD, "single", [64, 16, 1024], 1, OOP),    # Z transform, outer dimension below the transform's stride
    Case(C2C_FWD, "double", [16, 8, 1024], 2, IP),
    Case(C2C_FWD, "single", [4096, 1024], 1, IP),       # 256 tiles over 148 CTAs: stage reuse
    Case(C2C_FWD, "single", [256, 1024, 16], 1, IP),
]


@pytest.mark.parametrize("case", CASES_1024, ids=lambda c: c.ident())
def test_1024_point_columns(gpu, case):
    assert "col_tma" in _plan_text(case), "the TMA column kernel should serve 1024-point columns"
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"


CASES_FORCED = [
    Case(C2C_FWD, "single", [64, 512], 3, IP),
    Case(C2C_INV, "single", [128, 256], 2, OOP),
    Case(C2C_FWD, "double", [64, 512], 2, OOP),
    Case(C2C_FWD, "double", [32, 256, 3], 1, IP),
    Case(C2C_FWD, "single", [2048, 512, 2], 1, IP),
]


@pytest.mark.parametrize("case", CASES_FORCED, ids=lambda c: c.ident())
def test_shorter_lengths_forced(gpu, case, monkeypatch):
    monkeypatch.setenv("ROCFFT_B200_COLTMA", "1")
    assert "col_tma" in _plan_text(case)
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"


def test_device_error_flag_stays_clear(gpu):
    torch = gpu
    rng = np.random.default_rng(3)
    x = (rng.random((1024, 64)) - 0.5 + 1j * (rng.random((1024, 64)) - 0.5)).astype(np.complex64)
    d = torch.from_numpy(x).cuda()
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024], 64,
                in_strides=[64], in_distance=1, out_strides=[64], out_distance=1)
    assert "col_tma" in p.describe()
    assert p.execute([d.data_ptr()]) == 0
    torch.cuda.synchronize()
    assert p.device_error() is False
    ref = np.fft.fft(x.astype(np.complex128), axis=0)
    assert np.linalg.norm(d.cpu().numpy() - ref) / np.linalg.norm(ref) < 5e-6
    p.destroy()


# Volumes whose slowest dimension has a row pitch of 4 MB or more take the work-array plan: rows in the
# caller's array, the slowest dimension out of it into a work array, the middle dimension back.
CASES_LONG_PITCH = [
    Case(C2C_FWD, "single", [1024, 512, 256], 1, IP),
    Case(C2C_INV, "single", [1024, 512, 256], 1, OOP, scale=1.0 / 4096),
    Case(C2C_FWD, "single", [2048, 256, 256], 2, IP),
    Case(C2C_FWD, "double", [512, 512, 256], 1, OOP),
    Case(C2C_INV, "double", [1024, 256, 256], 1, IP),
    # padded rows and planes on both sides (in place), different layouts in and out (out of place), no caller work buffer
    Case(C2C_FWD, "single", [1024, 512, 256], 1, IP, in_strides=[1, 1040, 1040 * 514], out_strides=[1, 1040, 1040 * 514],
         in_dist=1040 * 514 * 256, out_dist=1040 * 514 * 256),
    Case(C2C_FWD, "single", [1024, 512, 256], 1, OOP, in_strides=[1, 1026, 1026 * 512], in_dist=1026 * 512 * 256,
         out_strides=[1, 1024, 1024 * 520], out_dist=1024 * 520 * 256),
    Case(C2C_FWD, "single", [1024, 512, 256], 1, IP, user_work_buffer=False),
]


@pytest.mark.parametrize("case", CASES_LONG_PITCH, ids=lambda c: c.ident())
def test_long_pitch_volumes_use_a_work_array(gpu, case, monkeypatch):
    text = _plan_text(case)
    assert text.count("col_tma") == 2 and "work" in text.lower(), text
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"
    # the plain three in-place passes give the same answer
    monkeypatch.setenv("ROCFFT_B200_NO_LONG_PITCH_PLAN", "1")
    ok, msg = run_case(case)
    assert ok, f"{case.ident()} (plain plan): {msg}"
