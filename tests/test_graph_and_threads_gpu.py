"""rocfft_execute under stream capture, from several host threads and on several streams
(reference: clients/tests/hipGraph_test.cpp:272-392, clients/tests/multithread_test.cpp:323-351)."""
import threading

import numpy as np
import pytest

import rocfft_b200 as rf

pytestmark = pytest.mark.gpu

FWD = rf.rocfft_transform_type_complex_forward
INV = rf.rocfft_transform_type_complex_inverse
IP = rf.rocfft_placement_inplace
OOP = rf.rocfft_placement_notinplace


def _rand(shape, seed):
    rng = np.random.default_rng(seed)
    return (rng.random(shape) - 0.5 + 1j * (rng.random(shape) - 0.5)).astype(np.complex64)


def _rel(a, b):
    return np.linalg.norm(a - b) / np.linalg.norm(b)


@pytest.mark.parametrize("lengths,batch", [([256], 1), ([1024], 64), ([64, 64, 64], 1), ([1 << 17], 2), ([64, 1024], 2),
                                           ([1024, 1024], 4)],
                         ids=["256", "1024x64_rows", "64cubed", "131072_two_kernels", "1024_columns_tensor_copy",
                              "1024x1024x4_rows_and_columns_in_one_kernel"])
def test_execute_is_capturable_and_replayable(lengths, batch, monkeypatch):
    """Forward out of place, inverse in place and element-wise work on the same stream are captured
    into one graph; nothing runs before the graph is launched; ten launches give the input back and
    count to ten."""
    import torch
    assert rf.rocfft_setup() == 0
    if lengths == [1024, 1024]:
        # the one-kernel path (cooperative launch, counters reset by a memset node); opt-in in single precision
        monkeypatch.setenv("ROCFFT_B200_2D_L2", "1")
    n = int(np.prod(lengths))
    shape = (batch,) + tuple(reversed(lengths))
    host = _rand(shape, 100)
    x = torch.from_numpy(host).cuda()
    y = torch.zeros_like(x)
    counter = torch.zeros(16, dtype=torch.int64, device="cuda")
    fwd = rf.Plan(OOP, FWD, 0, lengths, batch)
    inv = rf.Plan(IP, INV, 0, lengths, batch)
    if lengths == [1024, 1024]:
        assert "fft2d_l2" in fwd.describe()
    if lengths == [64, 1024]:
        assert "col_tma" in fwd.describe()
    works = []
    for p in (fwd, inv):
        if p.work_bytes:  # capture-friendly: the caller owns the work buffer
            w = torch.empty(p.work_bytes, dtype=torch.uint8, device="cuda")
            assert p.set_work_buffer(w.data_ptr(), p.work_bytes) == 0
            works.append(w)
    torch.cuda.synchronize()
    s = torch.cuda.Stream()
    for p in (fwd, inv):
        assert p.set_stream(s.cuda_stream) == 0
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(10):
            x.add_(0.1 + 0.1j)
        for _ in range(10):
            x.sub_(0.1 + 0.1j)
        x.mul_(2.2)
        x.mul_(1.0 / 2.2)
        assert fwd.execute([x.data_ptr()], [y.data_ptr()]) == 0
        y.mul_(2.2)
        y.mul_(1.0 / 2.2)
        assert inv.execute([y.data_ptr()]) == 0
        y.mul_(1.0 / n)
        counter.add_(1)
    torch.cuda.synchronize()
    # capture enqueued nothing
    assert not y.cpu().numpy().any()
    assert int(counter[0]) == 0
    for _ in range(10):
        g.replay()
    torch.cuda.synchronize()
    assert _rel(y.cpu().numpy(), host) < 2e-5
    assert counter.cpu().tolist() == [10] * 16
    assert not fwd.device_error() and not inv.device_error()
    fwd.destroy()
    inv.destroy()


def _worker(idx, lengths, batch, results):
    import torch
    try:
        torch.cuda.set_device(0)
        shape = (batch,) + tuple(reversed(lengths))
        host = _rand(shape, 7 + idx)
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            x = torch.from_numpy(host).cuda()
        s.synchronize()
        p = rf.Plan(IP, FWD, 0, lengths, batch)
        w = None
        if p.work_bytes:
            w = torch.empty(p.work_bytes, dtype=torch.uint8, device="cuda")
            p.set_work_buffer(w.data_ptr(), p.work_bytes)
        p.set_stream(s.cuda_stream)
        for _ in range(3):  # forward three times on fresh data each time
            with torch.cuda.stream(s):
                x.copy_(torch.from_numpy(host), non_blocking=False)
            assert p.execute([x.data_ptr()]) == 0
        s.synchronize()
        ref = np.fft.fftn(host.astype(np.complex128), axes=tuple(range(1, len(shape))))
        results[idx] = _rel(x.cpu().numpy(), ref)
        p.destroy()
    except Exception as e:  # surfaced by the parent
        results[idx] = e


@pytest.mark.parametrize("dims", [1, 2, 3])
def test_plans_in_concurrent_host_threads(dims):
    """Each thread creates, executes and destroys its own plan on its own stream."""
    assert rf.rocfft_setup() == 0
    shapes = {1: [[4096], [1000], [10007], [1 << 16]], 2: [[64, 64], [100, 30], [256, 128], [17, 33]],
              3: [[32, 32, 32], [16, 10, 12], [64, 8, 4], [7, 9, 11]]}[dims]
    results = [None] * len(shapes)
    threads = [threading.Thread(target=_worker, args=(i, shp, 4, results)) for i, shp in enumerate(shapes)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    for shp, r in zip(shapes, results):
        assert not isinstance(r, Exception), f"{shp}: {r!r}"
        assert r is not None and r < 5e-6 * max(1.0, np.log2(np.prod(shp))), f"{shp}: {r}"


def test_one_thread_many_streams():
    """Several plans enqueued back to back on different streams from one thread."""
    import torch
    assert rf.rocfft_setup() == 0
    jobs = []
    for i, shp in enumerate([[2048], [512, 512], [48, 48, 48], [1000]]):
        batch = 8
        host = _rand((batch,) + tuple(reversed(shp)), 50 + i)
        s = torch.cuda.Stream()
        x = torch.from_numpy(host).cuda()
        p = rf.Plan(IP, FWD, 0, shp, batch)
        assert p.work_bytes == 0
        p.set_stream(s.cuda_stream)
        jobs.append((shp, host, s, x, p))
    torch.cuda.synchronize()
    for _, _, _, x, p in jobs:
        assert p.execute([x.data_ptr()]) == 0
    torch.cuda.synchronize()
    for shp, host, s, x, p in jobs:
        ref = np.fft.fftn(host.astype(np.complex128), axes=tuple(range(1, host.ndim)))
        assert _rel(x.cpu().numpy(), ref) < 1e-5, shp
        p.destroy()
