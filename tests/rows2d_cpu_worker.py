"""Rank program of tests/test_slab_schedule_cpu.py (rank-2 case): emulates the row-slab
2D transform on CPU ranks (gloo) with the buffer layouts and the store offsets of the
library's own plan builder (b200fft_rows2d_exchange_offsets):

  phase 1  copy: the x-range of rank q of my rows -> rank q's T[y][x_local] at rows y = rank*ly ...
  phase 2  FFT along Y on T; output rows y in rank q's range -> rank q's row buffer [y_local][x]
           at columns x = rank*lx ...
  phase 3  FFT along X on the row buffer -> result slab [y_local][x]
"""
import ctypes
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    import torch
    import torch.distributed as dist
    import rocfft_b200 as rf

    nx, ny, batch = (int(v) for v in sys.argv[1:4])
    dist.init_process_group("gloo")
    rank, P = dist.get_rank(), dist.get_world_size()
    L = rf.lib()
    fn = L.b200fft_rows2d_exchange_offsets
    szp = ctypes.POINTER(ctypes.c_size_t)
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, szp, szp]
    esz = 16
    o1, o2 = ctypes.c_size_t(), ctypes.c_size_t()
    assert fn(P, rank, nx, ny, esz, ctypes.byref(o1), ctypes.byref(o2)) == 0
    assert fn(P, P, nx, ny, esz, ctypes.byref(o1), ctypes.byref(o2)) != 0  # rank out of range
    assert fn(P, rank, nx, ny, esz, ctypes.byref(o1), ctypes.byref(o2)) == 0
    first_off, second_off = o1.value // esz, o2.value // esz

    lx, ly = nx // P, ny // P
    rng = np.random.default_rng(7)
    full = (rng.random((batch, ny, nx)) - 0.5) + 1j * (rng.random((batch, ny, nx)) - 0.5)
    slab = full[:, rank * ly:(rank + 1) * ly].copy()            # [b][ly][nx]

    def all_to_all(per_dest, nelem):
        """per_dest[q] = (flat element offsets in q's buffer, values).  Returns this rank's filled buffer."""
        buf = np.zeros(nelem, dtype=np.complex128)
        for q in range(P):
            for src in range(P):
                if src == rank and q == rank:
                    o, v = per_dest[q]
                    buf[o] = v
                elif src == rank:
                    o, v = per_dest[q]
                    dist.send(torch.from_numpy(np.ascontiguousarray(o).astype(np.int64)), q)
                    dist.send(torch.view_as_real(torch.from_numpy(np.ascontiguousarray(v))), q)
                elif q == rank:
                    n = per_dest[src][0].size  # blocks have the same size in both directions
                    o = torch.empty(n, dtype=torch.int64)
                    v = torch.empty((n, 2), dtype=torch.float64)
                    dist.recv(o, src)
                    dist.recv(v, src)
                    buf[o.numpy()] = torch.view_as_complex(v).numpy()
        return buf

    # phase 1: T of rank q is [b][ny][lx]; my block starts first_off elements into every image of it
    per_dest = []
    for q in range(P):
        blk = slab[:, :, q * lx:(q + 1) * lx]                     # [b][ly][lx]
        b_i, y_i, x_i = np.meshgrid(np.arange(batch), np.arange(ly), np.arange(lx), indexing="ij")
        offs = b_i * (ny * lx) + first_off + y_i * lx + x_i
        per_dest.append((offs.ravel(), blk.ravel()))
    T = all_to_all(per_dest, batch * ny * lx).reshape(batch, ny, lx)
    # phase 2: FFT along Y; rows of rank q's range go to its row buffer [b][ly][nx] at columns second_off ...
    Y = np.fft.fft(T, axis=1)
    per_dest = []
    for q in range(P):
        blk = Y[:, q * ly:(q + 1) * ly, :]                        # [b][ly][lx]
        b_i, y_i, x_i = np.meshgrid(np.arange(batch), np.arange(ly), np.arange(lx), indexing="ij")
        offs = b_i * (ly * nx) + y_i * nx + second_off + x_i
        per_dest.append((offs.ravel(), blk.ravel()))
    rows = all_to_all(per_dest, batch * ly * nx).reshape(batch, ly, nx)
    # phase 3
    out = np.fft.fft(rows, axis=2)
    ref = np.fft.fft2(full)[:, rank * ly:(rank + 1) * ly]
    err = np.max(np.abs(out - ref)) / np.max(np.abs(ref))
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: rel err {err:.2e}")
    sys.exit(0 if err < 1e-12 else 1)


if __name__ == "__main__":
    main()
