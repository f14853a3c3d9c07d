"""The allocation-free entry point b200fft_c2c_1d_static_scratch.

Some callers cannot allocate device memory at the point where they need a
transform (a real-time loop, a frozen memory pool); for them the library offers
one entry point whose intermediate array and tables live in a static device
array.  These tests call it through the C ABI twice in a row — the second call
with different data, so a result that leaked from the shared scratch array
would show — and compare each result with the regular plan-based path and with
the CPU oracle under the accuracy bounds the other tests use.  The file is
collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _entry():
    import rocfft_b200 as rf
    fn = rf.lib().b200fft_c2c_1d_static_scratch
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def test_static_scratch_entry_matches_planned_transform(gpu):
    torch = gpu
    import rocfft_b200 as rf
    from oracle import fft_oracle as orc

    fn = _entry()
    # sizes beyond the static array are refused, not truncated
    dummy = torch.zeros(16, dtype=torch.complex64, device="cuda")
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 1 << 20, 2, 0, None) == rf.rocfft_status_invalid_arg_value
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 1 << 20, 1, 0, None) == rf.rocfft_status_invalid_arg_value
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 1 << 19, 2, 0, None) == rf.rocfft_status_invalid_arg_value
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 3000, 1, 0, None) == rf.rocfft_status_invalid_arg_value
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 128, 1, 0, None) == rf.rocfft_status_invalid_arg_value

    # balanced and unbalanced splits, the shortest and the longest accepted length
    for length, batch, inverse in ((16384, 4, 0), (16384, 4, 1), (65536, 8, 0), (1024, 64, 0),
                                   (256, 5, 0), (512, 9, 1), (1 << 19, 1, 0)):
        plan = rf.Plan(rf.rocfft_placement_notinplace,
                       rf.rocfft_transform_type_complex_inverse if inverse else rf.rocfft_transform_type_complex_forward,
                       rf.rocfft_precision_single, [length], batch)
        work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
        if plan.work_bytes:
            plan.set_work_buffer(work.data_ptr(), plan.work_bytes)
        stream = torch.cuda.current_stream().cuda_stream
        plan.set_stream(stream)
        for call in range(2):
            xh = orc.uniform_input((batch, length), np.complex64, seed=100 + call + length)
            x = torch.from_numpy(xh).cuda()
            y_ref = torch.empty_like(x)
            y_new = torch.full_like(x, float("nan"))
            assert plan.execute([x.data_ptr()], [y_ref.data_ptr()]) == 0
            assert fn(x.data_ptr(), y_new.data_ptr(), length, batch, inverse, ctypes.c_void_p(stream)) == 0
            torch.cuda.synchronize()
            got = y_new.cpu().numpy()
            ok, msg = orc.check_accuracy(got, y_ref.cpu().numpy().astype(np.complex128), "single", length)
            assert ok, f"vs planned path: length {length} batch {batch} inverse {inverse} call {call}: {msg}"
            ok, msg = orc.check_accuracy(got, orc.c2c(xh, +1 if inverse else -1), "single", length)
            assert ok, f"vs oracle: length {length} batch {batch} inverse {inverse} call {call}: {msg}"
        plan.destroy()


def test_static_scratch_in_place(gpu):
    torch = gpu
    from oracle import fft_oracle as orc
    fn = _entry()
    length, batch = 4096, 16
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        xh = orc.uniform_input((batch, length), np.complex64, seed=500 + call)
        x = torch.from_numpy(xh).cuda()
        assert fn(x.data_ptr(), x.data_ptr(), length, batch, 0, ctypes.c_void_p(stream)) == 0
        torch.cuda.synchronize()
        ok, msg = orc.check_accuracy(x.cpu().numpy(), orc.c2c(xh, -1), "single", length)
        assert ok, f"in place, call {call}: {msg}"


def test_static_scratch_length_changes_on_a_non_blocking_stream(gpu):
    """Two lengths alternate on one non-blocking stream with no host synchronisation between the calls:
    the table rewrite of each length change must wait for the kernels still queued with the old tables."""
    torch = gpu
    from oracle import fft_oracle as orc
    fn = _entry()
    side = torch.cuda.Stream()  # torch side streams are created non-blocking
    cases = [(8192, 16), (2048, 32), (8192, 16), (2048, 32), (1 << 17, 2)]
    hosts = [orc.uniform_input((b, n), np.complex64, seed=700 + i) for i, (n, b) in enumerate(cases)]
    torch.cuda.synchronize()
    with torch.cuda.stream(side):
        ins = [torch.from_numpy(h).cuda() for h in hosts]
        outs = [torch.full_like(t, float("nan")) for t in ins]
        side.synchronize()
        for (n, b), x, y in zip(cases, ins, outs):
            assert fn(x.data_ptr(), y.data_ptr(), n, b, 0, ctypes.c_void_p(side.cuda_stream)) == 0
    side.synchronize()
    for i, ((n, b), h, y) in enumerate(zip(cases, hosts, outs)):
        ok, msg = orc.check_accuracy(y.cpu().numpy(), orc.c2c(h, -1), "single", n)
        assert ok, f"call {i} (length {n}): {msg}"
