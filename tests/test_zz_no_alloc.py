"""The allocation-free entry point b200fft_c2c_1d_static_scratch against the
regular plan-based path.

Some callers cannot allocate device memory at the point where they need a
transform (a real-time loop, a frozen memory pool); for them the library offers
one entry point whose intermediate array and tables live in a static device
array.  This test calls it through the C ABI twice in a row — the second call
with different data, so a result that leaked from the shared scratch array
would show — and compares each result with rocfft_execute on the same input
under the accuracy bounds the other tests use.  It is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_planned_transform(gpu):
    torch = gpu
    import rocfft_b200 as rf
    from oracle import fft_oracle as orc

    L = rf.lib()
    fn = L.b200fft_c2c_1d_static_scratch
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p]
    fn.restype = ctypes.c_int

    # sizes beyond the static array are refused, not truncated
    dummy = torch.zeros(16, dtype=torch.complex64, device="cuda")
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 1 << 20, 2, 0, None) == rf.rocfft_status_invalid_arg_value
    assert fn(dummy.data_ptr(), dummy.data_ptr(), 3000, 1, 0, None) == rf.rocfft_status_invalid_arg_value

    for length, batch, inverse in ((16384, 4, 0), (16384, 4, 1), (65536, 8, 0), (1024, 64, 0)):
        plan = rf.Plan(rf.rocfft_placement_notinplace,
                       rf.rocfft_transform_type_complex_inverse if inverse else rf.rocfft_transform_type_complex_forward,
                       rf.rocfft_precision_single, [length], batch)
        work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
        if plan.work_bytes:
            plan.set_work_buffer(work.data_ptr(), plan.work_bytes)
        stream = torch.cuda.current_stream().cuda_stream
        plan.set_stream(stream)
        for call in range(2):
            x = torch.from_numpy(orc.uniform_input((batch, length), np.complex64, seed=100 + call + length)).cuda()
            y_ref = torch.empty_like(x)
            y_new = torch.full_like(x, float("nan"))
            assert plan.execute([x.data_ptr()], [y_ref.data_ptr()]) == 0
            assert fn(x.data_ptr(), y_new.data_ptr(), length, batch, inverse, ctypes.c_void_p(stream)) == 0
            torch.cuda.synchronize()
            ok, msg = orc.check_accuracy(y_new.cpu().numpy(), y_ref.cpu().numpy().astype(np.complex128), "single", length)
            assert ok, f"length {length} batch {batch} inverse {inverse} call {call}: {msg}"
        plan.destroy()
