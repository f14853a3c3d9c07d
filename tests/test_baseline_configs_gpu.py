"""The five benchmark configurations at their FULL sizes through the C API, each checked against the
double-precision CPU oracle under rocfft-test's bounds (shared/accuracy_test.h:1497-1498, 1609-1619;
round trip as :757-861).  Small-batch cases elsewhere do not reach the steady state of the persistent
kernels (dozens of tiles per CTA, every pipeline stage reused, mbarrier phases flipping) nor the row
pitches of the large 2D/3D arrays; these do.

  1. c2c 1D 4096 x 16384, fp32, in place
  2. r2c 1D 1000 x 65536 fp32 out of place, then c2r with scale 1/1000 back to the input
  3. c2c 2D 1024 x 1024 x 64, fp64, out of place
  4. c2c 1D 10007 x 4096 (prime length), fp32, out of place
  5. c2c 3D 1024^3 fp32 in place on one GPU: sampled output planes and lines recomputed in complex128
     from the seeded input (the whole volume in double precision would need 16 GiB of host memory per copy),
     plus Parseval's identity over the full volume.
"""
import math

import numpy as np
import pytest

import rocfft_b200 as rf
from oracle import fft_oracle as orc

pytestmark = pytest.mark.gpu


def _execute(torch, plan, d_in, d_out):
    work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
    if plan.work_bytes:
        assert plan.set_work_buffer(work.data_ptr(), plan.work_bytes) == 0
    plan.set_stream(torch.cuda.current_stream().cuda_stream)
    st = plan.execute([d_in.data_ptr()], None if d_out is None else [d_out.data_ptr()])
    torch.cuda.synchronize()
    assert st == rf.rocfft_status_success, st
    assert plan.device_error() is False
    del work


def test_config1_c2c_1d_4096x16384_fp32_inplace(gpu):
    torch = gpu
    n, batch = 4096, 16384
    x = orc.uniform_input((batch, n), np.complex64, seed=1)
    d = torch.from_numpy(x).cuda()
    plan = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [n], batch)
    _execute(torch, plan, d, None)
    got = d.cpu().numpy()
    ref = orc.c2c(x, -1)
    ok, msg = orc.check_accuracy(got, ref, "single", n)
    assert ok, msg
    plan.destroy()


def test_config2_real_1d_1000x65536_fp32_forward_and_back(gpu):
    torch = gpu
    n, batch = 1000, 65536
    x = orc.uniform_input((batch, n), np.float32, seed=2)
    d_x = torch.from_numpy(x).cuda()
    d_h = torch.full((batch, n // 2 + 1), float("nan"), dtype=torch.complex64, device="cuda")
    fwd = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_forward, 0, [n], batch)
    assert "tma" in fwd.describe()  # the persistent bulk-copy kernel is the one under test
    _execute(torch, fwd, d_x, d_h)
    got = d_h.cpu().numpy()
    ref = orc.r2c(x)
    ok, msg = orc.check_accuracy(got, ref, "single", n)
    assert ok, "forward: " + msg
    # Hermitian layout: DC and Nyquist come out purely real
    assert np.all(got[:, 0].imag == 0) and np.all(got[:, -1].imag == 0)
    # inverse, normalised by 1/N, must return the input (rocfft-test's round trip)
    inv = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_inverse, 0, [n], batch, scale=1.0 / n)
    d_back = torch.full((batch, n), float("nan"), dtype=torch.float32, device="cuda")
    _execute(torch, inv, d_h, d_back)
    back = d_back.cpu().numpy()
    ok, msg = orc.check_accuracy(back, x.astype(np.float64), "single", n)
    assert ok, "round trip: " + msg
    # and the inverse on its own against the oracle's c2r of the same Hermitian rows
    ref_inv = orc.c2r(got.astype(np.complex128), [n]) / n
    ok, msg = orc.check_accuracy(back, ref_inv, "single", n)
    assert ok, "inverse: " + msg
    fwd.destroy()
    inv.destroy()


def test_config3_c2c_2d_1024x1024x64_fp64(gpu):
    torch = gpu
    n, batch = 1024, 64
    x = orc.uniform_input((batch, n, n), np.complex128, seed=3)
    d_in = torch.from_numpy(x).cuda()
    d_out = torch.full_like(d_in, float("nan"))
    plan = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [n, n], batch)
    _execute(torch, plan, d_in, d_out)
    assert torch.equal(d_in.cpu(), torch.from_numpy(x)), "out-of-place c2c must leave its input alone"
    got = d_out.cpu().numpy()
    del d_in, d_out
    ref = orc.c2c(x, -1)
    ok, msg = orc.check_accuracy(got, ref, "double", n * n)
    assert ok, msg
    plan.destroy()


def test_config4_c2c_1d_prime_10007x4096_fp32(gpu):
    torch = gpu
    n, batch = 10007, 4096
    x = orc.uniform_input((batch, n), np.complex64, seed=4)
    d_in = torch.from_numpy(x).cuda()
    d_out = torch.full_like(d_in, float("nan"))
    plan = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [n], batch)
    _execute(torch, plan, d_in, d_out)
    got = d_out.cpu().numpy()
    ref = orc.c2c(x, -1)
    ok, msg = orc.check_accuracy(got, ref, "single", n)
    assert ok, msg
    plan.destroy()


def test_config5_c2c_3d_1024cubed_fp32_inplace_sampled(gpu):
    torch = gpu
    import bench
    n = 1024
    total = n ** 3
    scale = 1.0 / math.sqrt(total)
    chk = bench.SampledCheck3D((n, n, n), 0, n)
    d = torch.empty(total, dtype=torch.complex64, device="cuda")
    rng = np.random.default_rng(5)
    planes = 16
    energy_in = 0.0
    for z in range(0, n, planes):
        a = np.empty((planes, n, n), dtype=np.complex64)
        a.real = rng.random((planes, n, n), dtype=np.float32) - 0.5
        a.imag = rng.random((planes, n, n), dtype=np.float32) - 0.5
        d[z * n * n:(z + planes) * n * n].copy_(torch.from_numpy(a.reshape(-1)))
        chk.feed(z, a)
        energy_in += float(np.vdot(a.astype(np.complex128).ravel(), a.astype(np.complex128).ravel()).real)
    plan = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [n, n, n], 1, scale=scale)
    _execute(torch, plan, d, None)
    res = chk.finish(d, scale)
    assert res["ok"], res
    # the sampled values also pass the oracle's own statement of the bounds
    assert res["linf"] <= res["cut_linf"] and res["l2rel"] < orc.type_epsilon("single") * math.sqrt(math.log2(total))
    # Parseval over every output value: sum |X|^2 = N * scale^2 * sum |x|^2 = sum |x|^2
    energy_out = 0.0
    v = torch.view_as_real(d)
    for s in range(0, total, 1 << 26):
        energy_out += float((v[s:s + (1 << 26)].double() ** 2).sum().item())
    assert abs(energy_out / energy_in - 1.0) < 1e-5, (energy_out, energy_in)
    plan.destroy()
