"""Rank program of tests/test_bench_verify_gloo_cpu.py: every rank feeds its Z-slab of a seeded volume to the
sampled check that bench.py runs at every GPU count, hands it its slab of the true transform (one rank can be told
to corrupt a value) and the ranks merge their partial sums over gloo exactly as the GPU ranks do over NCCL."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import bench

    corrupt = int(sys.argv[1])
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    n = (32, 16, 64)
    lz = n[0] // world
    rng = np.random.default_rng(17)
    full = np.empty(n, dtype=np.complex64)
    full.real = rng.random(n, dtype=np.float32) - 0.5
    full.imag = rng.random(n, dtype=np.float32) - 0.5
    scale = 1.0 / np.sqrt(np.prod(n))
    X = (np.fft.fftn(full.astype(np.complex128)) * scale).astype(np.complex64)
    chk = bench.SampledCheck3D(n, rank * lz, lz, world=world, rank=rank)
    for z in range(rank * lz, (rank + 1) * lz, 4):
        chk.feed(z, full[z:z + 4])
    mine = X[rank * lz:(rank + 1) * lz].copy()
    if corrupt == rank:
        mine[chk.kz[rank] - rank * lz, 2, 3] += 0.05  # inside this rank's sampled plane
    res = chk.finish(torch.from_numpy(mine), scale, dist=dist, torch=torch)
    expect_ok = corrupt < 0
    ok = res["ok"] == expect_ok
    print(f"rank {rank}: verify ok={res['ok']} (expected {expect_ok}) linf={res['linf']:.3e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
