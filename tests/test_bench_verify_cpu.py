"""The sampled 3D check that bench.py runs before its timed region, tested on the CPU: it must accept the
true transform and reject a corrupted one, for one slab and for several slabs whose partial sums are merged
the way the ranks merge them."""
import numpy as np
import torch

import bench


def _volume(n, seed=3):
    rng = np.random.default_rng(seed)
    nz, ny, nx = n
    a = np.empty((nz, ny, nx), dtype=np.complex64)
    a.real = rng.random((nz, ny, nx), dtype=np.float32) - 0.5
    a.imag = rng.random((nz, ny, nx), dtype=np.float32) - 0.5
    return a


def test_single_slab_accepts_truth_and_rejects_corruption():
    n = (64, 16, 32)
    x = _volume(n)
    chk = bench.SampledCheck3D(n, 0, n[0])
    for z in range(0, n[0], 8):
        chk.feed(z, x[z:z + 8])
    scale = 1.0 / np.sqrt(np.prod(n))
    X = (np.fft.fftn(x.astype(np.complex128)) * scale).astype(np.complex64)
    res = chk.finish(torch.from_numpy(X.copy()), scale)
    assert res["ok"], res
    bad = X.copy()
    kz = chk.kz[0]
    bad[kz, 3, 5] += 0.01
    chk2 = bench.SampledCheck3D(n, 0, n[0])
    chk2.feed(0, x)
    assert not chk2.finish(torch.from_numpy(bad), scale)["ok"]


def test_slabs_merge_like_ranks():
    n = (64, 16, 32)
    world = 4
    lz = n[0] // world
    x = _volume(n, seed=9)
    chks = [bench.SampledCheck3D(n, r * lz, lz, world=world, rank=r) for r in range(world)]
    for r, c in enumerate(chks):
        c.feed(r * lz, x[r * lz:(r + 1) * lz])
    # merge on the host what all_reduce / all_gather merge across ranks
    planes = sum(c.planes for c in chks)
    s_all = np.concatenate([c.s for c in chks], axis=0)
    X = np.fft.fftn(x.astype(np.complex128))
    for r, c in enumerate(chks):
        kz = c.kz[r]
        assert r * lz <= kz < (r + 1) * lz
        got = np.fft.fft2(planes[r].reshape(n[1], n[2]))
        assert np.allclose(got, X[kz], rtol=1e-10, atol=1e-9)
    lines = np.fft.fft(s_all, axis=0)
    for p, (ky, kx) in enumerate(chks[0].lines):
        assert np.allclose(lines[:, p], X[:, ky, kx], rtol=1e-10, atol=1e-9)


def test_bounds_follow_rocfft_test():
    r = bench.accuracy_bounds(1e-6, 1e-12, 1.0, 1.0, 3.75e-5, 1 << 30)
    assert r["ok"] and abs(r["cut_l2"] - 3.75e-5 * np.sqrt(30)) < 1e-12
    assert not bench.accuracy_bounds(1.0, 1.0, 1.0, 1.0, 3.75e-5, 1 << 30)["ok"]
