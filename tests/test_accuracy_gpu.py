"""Accuracy tests on the GPU: every case runs through the C API and is
compared with the double-precision CPU oracle under rocfft-test's bounds
(reference: clients/tests/accuracy_test_1D.cpp, _2D.cpp, _3D.cpp,
accuracy_test_checkstride.cpp; bounds in shared/accuracy_test.h:1497-1498,
1609-1619).  Data placement (strides, distances, offsets, planar/interleaved,
Hermitian layout) is checked bit-exactly through the canary bytes."""
import numpy as np
import pytest

from harness import (C2C_FWD, C2C_INV, C2R, CI, CP, HI, HP, IP, OOP, R2C, RE, Case, run_case)

pytestmark = pytest.mark.gpu

POW2 = [2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096]
MIXED = [3, 5, 6, 7, 9, 10, 11, 12, 13, 15, 20, 25, 27, 49, 50, 100, 125, 160, 200, 243, 500, 1000]
PRIMES_ETC = [17, 19, 23, 31, 37, 97, 127, 211, 509, 1021, 4099, 10007, 10243, 20011]  # Bluestein
LARGE = [8192, 16384, 65536, 20480, 40000, 1 << 20]  # two-kernel decompositions
UNPOOLED = [14, 18, 21, 22, 24, 26, 28, 30, 36, 77, 120, 143, 1001, 3000, 6000]


def _run(case):
    ok, msg = run_case(case)
    assert ok, f"{case.ident()}: {msg}"


def cases_1d():
    out = []
    for prec in ("single", "double"):
        for n in POW2 + MIXED:
            b = 3 if n >= 1024 else 7
            out.append(Case(C2C_FWD, prec, [n], b, IP))
            out.append(Case(C2C_INV, prec, [n], b, OOP))
        for n in PRIMES_ETC + UNPOOLED:
            out.append(Case(C2C_FWD, prec, [n], 3, OOP))
            out.append(Case(C2C_INV, prec, [n], 2, IP))
        for n in LARGE:
            out.append(Case(C2C_FWD, prec, [n], 2, IP))
            out.append(Case(C2C_INV, prec, [n], 2, OOP))
    return out


@pytest.mark.parametrize("case", cases_1d(), ids=lambda c: c.ident())
def test_c2c_1d(gpu, case):
    _run(case)


def cases_layout():
    out = []
    for prec in ("single", "double"):
        # strides, distances, offsets
        out.append(Case(C2C_FWD, prec, [64], 5, OOP, CI, CI, [2], [3], 130, 200))
        out.append(Case(C2C_FWD, prec, [100], 4, OOP, CI, CI, [1], [1], 128, 100, [7], [3]))
        out.append(Case(C2C_INV, prec, [128], 6, IP, CI, CI, [3], [3], 400, 400))
        # batch along the fast index (distance 1): column transforms
        out.append(Case(C2C_FWD, prec, [256], 40, OOP, CI, CI, [40], [40], 1, 1))
        out.append(Case(C2C_FWD, prec, [1024], 19, IP, CI, CI, [19], [19], 1, 1))
        out.append(Case(C2C_FWD, prec, [100], 33, OOP, CI, CI, [33], [1], 1, 100))  # transposing
        out.append(Case(C2C_FWD, prec, [128], 50, OOP, CI, CI, [1], [50], 128, 1))  # transposing
        # planar
        out.append(Case(C2C_FWD, prec, [512], 3, OOP, CP, CP))
        out.append(Case(C2C_FWD, prec, [200], 3, OOP, CI, CP))
        out.append(Case(C2C_INV, prec, [64], 3, OOP, CP, CI, None, None, 0, 0, [5, 9], [2]))
        out.append(Case(C2C_FWD, prec, [32], 9, IP, CP, CP))
        out.append(Case(C2C_FWD, prec, [31], 4, OOP, CP, CP))  # Bluestein + planar
        # scale factor
        out.append(Case(C2C_INV, prec, [1000], 2, OOP, scale=1e-3))
        out.append(Case(C2C_FWD, prec, [37], 2, OOP, scale=0.25))
        # in-place with differing layouts goes through scratch
        out.append(Case(C2C_FWD, prec, [16], 4, IP, CI, CI, [1], [2], 16, 40))
        # without a caller-supplied work buffer the library allocates its own
        out.append(Case(C2C_FWD, prec, [1 << 17], 2, IP, user_work_buffer=False))
        out.append(Case(C2C_FWD, prec, [1], 5, OOP))
    return out


@pytest.mark.parametrize("case", cases_layout(), ids=lambda c: c.ident())
def test_c2c_layouts(gpu, case):
    _run(case)


def cases_nd():
    out = []
    for prec in ("single", "double"):
        for lens in ([8, 8], [16, 32], [64, 64], [100, 50], [256, 128], [1024, 32], [5, 7], [31, 16], [12, 13],
                     [512, 512]):
            out.append(Case(C2C_FWD, prec, lens, 3, OOP))
            out.append(Case(C2C_INV, prec, lens, 2, IP))
        for lens in ([8, 8, 8], [16, 32, 8], [64, 64, 64], [5, 6, 7], [100, 20, 10], [128, 3, 128], [17, 8, 4]):
            out.append(Case(C2C_FWD, prec, lens, 2, IP))
            out.append(Case(C2C_INV, prec, lens, 1, OOP))
        # non-default strides in 2D/3D and planar
        out.append(Case(C2C_FWD, prec, [16, 8], 3, OOP, CI, CP, [1, 20], [1, 16], 200, 128))
        out.append(Case(C2C_FWD, prec, [8, 4, 6], 2, OOP, CI, CI, [2, 20, 100], [1, 8, 32], 700, 192))
        # dimensions given slowest-first get re-sorted
        out.append(Case(C2C_FWD, prec, [8, 16], 2, OOP, CI, CI, [16, 1], [16, 1], 128, 128))
        out.append(Case(C2C_FWD, prec, [16, 1, 8], 2, OOP))
    return out


@pytest.mark.parametrize("case", cases_nd(), ids=lambda c: c.ident())
def test_c2c_nd(gpu, case):
    _run(case)


def cases_2d_single():
    """Pairs of lengths that the pool holds as one fused 2D kernel (reference scheme CS_KERNEL_2D_SINGLE),
    in every layout flavour; pairs outside the pool fall back to two passes and must agree as well."""
    out = []
    for prec in ("single", "double"):
        for lens in ([16, 16], [32, 8], [8, 128], [64, 64], [128, 64], [64, 128], [32, 128], [27, 9], [9, 81], [81, 81],
                     [27, 81]):
            out.append(Case(C2C_FWD, prec, lens, 5, OOP))
            out.append(Case(C2C_INV, prec, lens, 3, IP))
        out.append(Case(C2C_FWD, prec, [64, 32], 3, OOP, CP, CP))
        out.append(Case(C2C_INV, prec, [32, 64], 3, OOP, CI, CP))
        out.append(Case(C2C_FWD, prec, [16, 64], 2, IP, CP, CP))
        out.append(Case(C2C_FWD, prec, [64, 16], 3, OOP, CI, CI, [1, 70], [2, 130], 70 * 16 + 3, 130 * 16 + 7))
        out.append(Case(C2C_FWD, prec, [32, 32], 2, OOP, CI, CI, [32, 1], [32, 1], 1024, 1024))  # slowest-first
        out.append(Case(C2C_FWD, prec, [64, 64], 4, OOP, scale=1.0 / 64))
        out.append(Case(C2C_INV, prec, [64, 64, 6], 2, IP, scale=0.5))
        out.append(Case(C2C_FWD, prec, [32, 16, 100], 1, OOP))
        out.append(Case(C2C_FWD, prec, [27, 27, 27], 2, IP))
    return out


def cases_big():
    """A few transforms of 2^24 points and more: three-kernel 1D decompositions, long column pitches,
    grids beyond 65535 tiles."""
    return [Case(C2C_FWD, "single", [1 << 24], 1, IP), Case(C2C_INV, "single", [1 << 22], 3, OOP),
            Case(C2C_FWD, "single", [4096, 4096], 1, IP), Case(C2C_FWD, "double", [2048, 2048], 2, OOP),
            Case(C2C_FWD, "single", [256, 256, 256], 1, IP), Case(C2C_INV, "single", [243, 243, 243], 1, OOP),
            Case(R2C, "single", [1 << 22], 2, OOP), Case(C2R, "single", [4096, 2048], 1, OOP),
            Case(C2C_FWD, "single", [64], 300000, IP), Case(C2C_FWD, "single", [512, 512, 64], 1, IP)]


def test_unfused_large_twiddle_path_agrees(gpu, monkeypatch):
    """The separate twiddle pass (kept for second stages that are not a single kernel) stays correct."""
    monkeypatch.setenv("ROCFFT_B200_NO_FUSED_LARGE_TWIDDLE", "1")
    for case in (Case(C2C_FWD, "single", [65536], 2, IP), Case(C2C_INV, "double", [40000], 2, OOP)):
        _run(case)


@pytest.mark.parametrize("case", cases_big(), ids=lambda c: c.ident())
def test_big_transforms(gpu, case):
    _run(case)


@pytest.mark.parametrize("case", cases_2d_single(), ids=lambda c: c.ident())
def test_c2c_2d_single_kernel(gpu, case):
    _run(case)


def cases_real():
    out = []
    for prec in ("single", "double"):
        for n in [2, 4, 6, 8, 10, 16, 30, 64, 100, 128, 200, 256, 1000, 1024, 2000, 4096, 8192, 3, 5, 9, 15, 27, 31,
                  101, 125, 243, 1001]:
            out.append(Case(R2C, prec, [n], 5, OOP))
            out.append(Case(C2R, prec, [n], 5, OOP))
            out.append(Case(R2C, prec, [n], 3, IP))
            out.append(Case(C2R, prec, [n], 3, IP))
        for lens in ([8, 8], [16, 10], [100, 30], [9, 6], [64, 64], [8, 4, 6], [32, 16, 8], [10, 5, 3], [7, 8, 9]):
            out.append(Case(R2C, prec, lens, 2, OOP))
            out.append(Case(C2R, prec, lens, 2, OOP))
            out.append(Case(R2C, prec, lens, 2, IP))
            out.append(Case(C2R, prec, lens, 2, IP))
        out.append(Case(R2C, prec, [64], 3, OOP, RE, HP))
        out.append(Case(C2R, prec, [64], 3, OOP, HP, RE))
        out.append(Case(R2C, prec, [30], 3, OOP, RE, HI, [2], [3], 70, 50))
        out.append(Case(C2R, prec, [30], 3, OOP, HI, RE, [2], [3], 40, 100))
        out.append(Case(R2C, prec, [64], 3, OOP, RE, HI, [1], [1], 66, 33, [2], [1]))
        out.append(Case(R2C, prec, [64], 3, OOP, RE, HI, [1], [1], 65, 33, [1], [1]))  # odd distance: general path
        # odd lengths: one full-length complex kernel each way, in every layout flavour
        out.append(Case(R2C, prec, [125], 3, OOP, RE, HP))
        out.append(Case(C2R, prec, [125], 3, OOP, HP, RE))
        out.append(Case(R2C, prec, [27], 3, OOP, RE, HI, [2], [3], 60, 50))
        out.append(Case(C2R, prec, [27], 3, OOP, HI, RE, [3], [2], 50, 60))
        out.append(Case(R2C, prec, [243], 700, OOP, scale=0.5))
        out.append(Case(C2R, prec, [3125], 5, IP, scale=1.0 / 3125))
        out.append(Case(R2C, prec, [81, 27], 3, IP))
        out.append(Case(C2R, prec, [15, 15, 15], 2, OOP))
        out.append(Case(C2R, prec, [1000], 4, OOP, scale=1e-3))
        out.append(Case(R2C, prec, [1000], 4, OOP, scale=2.0))
    return out


@pytest.mark.parametrize("case", cases_real(), ids=lambda c: c.ident())
def test_real(gpu, case):
    _run(case)


def test_hermitian_dc_nyquist_imag_ignored(gpu):
    """c2r output must be bit-identical whether or not Im(DC)/Im(Nyquist) are
    zero (reference: clients/tests/hermitian_test.cpp:35-168)."""
    import torch
    import rocfft_b200 as rf
    from oracle import fft_oracle as orc
    for n in (16, 30, 1000, 15):
        X = orc.hermitian_input([n], 4, np.complex64, seed=n)
        X[:, 0].imag = 0
        if n % 2 == 0:
            X[:, -1].imag = 0
        outs = []
        for junk in (False, True):
            Y = X.copy()
            if junk:
                Y[:, 0] += 0.37j
                if n % 2 == 0:
                    Y[:, -1] -= 0.21j
            d_in = torch.from_numpy(Y).cuda()
            d_out = torch.zeros((4, n), dtype=torch.float32, device="cuda")
            p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_inverse, 0, [n], 4)
            w = torch.empty(max(p.work_bytes, 1), dtype=torch.uint8, device="cuda")
            if p.work_bytes:
                p.set_work_buffer(w.data_ptr(), p.work_bytes)
            assert p.execute([d_in.data_ptr()], [d_out.data_ptr()]) == 0
            torch.cuda.synchronize()
            outs.append(d_out.cpu().numpy())
            p.destroy()
        assert np.array_equal(outs[0], outs[1]), n


def test_work_buffer_contract(gpu):
    """Too-small work buffer -> invalid_work_buffer at execute
    (reference: clients/tests/unit_test.cpp:256-345)."""
    import torch
    import rocfft_b200 as rf
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1 << 17], 2)
    assert p.work_bytes > 0
    x = torch.zeros(2 << 17, dtype=torch.complex64, device="cuda")
    small = torch.empty(16, dtype=torch.uint8, device="cuda")
    assert p.set_work_buffer(small.data_ptr(), 16) == rf.rocfft_status_success
    assert p.execute([x.data_ptr()]) == rf.rocfft_status_invalid_work_buffer
    p.destroy()


def test_description_is_copied_and_reusable(gpu):
    """A description may be reused for several plans and destroyed right after
    plan creation (reference: clients/tests/unit_test.cpp:104-193)."""
    import torch
    import rocfft_b200 as rf
    from oracle import fft_oracle as orc
    st, d = rf.rocfft_plan_description_create()
    x = orc.uniform_input((8,), np.complex64, seed=8)
    ref = orc.c2c(x[None, :], -1)[0]
    plans = []
    for stride in (1, 2, 3):
        rf.rocfft_plan_description_set_data_layout(d, rf.rocfft_array_type_complex_interleaved,
                                                   rf.rocfft_array_type_complex_interleaved, None, None, [stride],
                                                   8 * stride, [stride], 8 * stride)
        st, p = rf.rocfft_plan_create(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [8],
                                      1, d)
        assert st == 0
        plans.append((stride, p))
    rf.rocfft_plan_description_destroy(d)
    for stride, p in plans:
        host = np.zeros(8 * stride, np.complex64)
        host[::stride] = x
        dev = torch.from_numpy(host).cuda()
        assert rf.rocfft_execute(p, [dev.data_ptr()], None, None) == 0
        torch.cuda.synchronize()
        got = dev.cpu().numpy()
        ok, msg = orc.check_accuracy(got[::stride], ref, "single", 8)
        assert ok, msg
        if stride > 1:
            assert np.all(got.reshape(8, stride)[:, 1:] == 0)
        rf.rocfft_plan_destroy(p)


def test_run_to_run_bitwise_reproducible(gpu):
    """Same plan, same input -> identical bits (reference:
    clients/tests/bitwise_repro, docs/how-to/working-with-rocfft.rst:372-385)."""
    import torch
    import rocfft_b200 as rf
    from oracle import fft_oracle as orc
    for lens, b in (([4096], 8), ([1000], 9), ([64, 64], 3), ([10007], 2)):
        n = int(np.prod(lens))
        x = torch.from_numpy(orc.uniform_input((b, n), np.complex64, seed=3)).cuda()
        p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, lens, b)
        w = torch.empty(max(p.work_bytes, 1), dtype=torch.uint8, device="cuda")
        if p.work_bytes:
            p.set_work_buffer(w.data_ptr(), p.work_bytes)
        outs = []
        for _ in range(2):
            y = torch.zeros_like(x)
            assert p.execute([x.data_ptr()], [y.data_ptr()]) == 0
            torch.cuda.synchronize()
            outs.append(y.cpu().numpy())
        assert np.array_equal(outs[0].view(np.uint8), outs[1].view(np.uint8))
        p.destroy()
