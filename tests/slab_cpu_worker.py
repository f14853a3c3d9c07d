"""Rank program of tests/test_slab_schedule_cpu.py: emulates the slab-decomposed
3D transform on CPU ranks (gloo), following the library's own exchange schedule
(b200fft_slab_exchange_offsets) and the packed layouts its FFT passes write:

  pass A  FFT along Y          slab[z][y][x] -> S_c[q][zc][yq][x]
  a2a #1                       -> T[z][y_local][x]
  pass B  FFT along Z          T -> S_c[q][zq][yc][x]
  a2a #2                       -> R2_c[r][z_local][yc][x]
  pass C  FFT along X          R2 -> slab[z_local][y][x]
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

    nx, ny, nz, chunks = (int(v) for v in sys.argv[1:5])
    dist.init_process_group("gloo")
    rank, P = dist.get_rank(), dist.get_world_size()
    L = rf.lib()
    fn = L.b200fft_slab_exchange_offsets
    szp = ctypes.POINTER(ctypes.c_size_t)
    fn.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_size_t, ctypes.c_int, ctypes.c_int, szp, szp, szp]

    lz, ly = nz // P, ny // P
    cz, cy = lz // chunks, ly // chunks
    rng = np.random.default_rng(42)
    full = (rng.random((nz, ny, nx)) - 0.5) + 1j * (rng.random((nz, ny, nx)) - 0.5)
    slab = full[rank * lz:(rank + 1) * lz].copy()
    esz = 16
    slab_bytes = slab.size * esz
    S = np.zeros(slab.size, dtype=np.complex128)
    R = np.zeros(slab.size, dtype=np.complex128)
    R2 = np.zeros(slab.size, dtype=np.complex128)
    chunk_elems = slab.size // chunks

    def exchange(send, recv, first, c):
        so, ro, blk = (ctypes.c_size_t * P)(), (ctypes.c_size_t * P)(), ctypes.c_size_t()
        assert fn(P, chunks, slab_bytes, first, c, so, ro, ctypes.byref(blk)) == 0
        n = blk.value // esz
        reqs, bufs = [], []
        for q in range(P):
            s_t = torch.from_numpy(send[so[q] // esz: so[q] // esz + n].copy())
            r_t = torch.empty(n, dtype=torch.complex128)
            if q == rank:
                r_t.copy_(s_t)
            else:
                reqs.append(dist.isend(torch.view_as_real(s_t), q, tag=first * 100 + c))
                reqs.append(dist.irecv(torch.view_as_real(r_t), q, tag=first * 100 + c))
            bufs.append((q, r_t))
        for r in reqs:
            r.wait()
        for q, r_t in bufs:
            recv[ro[q] // esz: ro[q] // esz + n] = r_t.numpy()

    # pass A + exchange 1, chunk by chunk over z_local
    for c in range(chunks):
        a = np.fft.fft(slab[c * cz:(c + 1) * cz], axis=1)          # [zc][y][x]
        packed = a.reshape(cz, P, ly, nx).transpose(1, 0, 2, 3)      # [q][zc][yq][x]
        S[c * chunk_elems:(c + 1) * chunk_elems] = packed.ravel()
        exchange(S, R, 1, c)
    T = R.reshape(nz, ly, nx)
    # pass B + exchange 2, chunk by chunk over y_local
    for c in range(chunks):
        b = np.fft.fft(T[:, c * cy:(c + 1) * cy, :], axis=0)        # [z][yc][x]
        packed = b.reshape(P, lz, cy, nx)                            # [q][zq][yc][x]
        S[c * chunk_elems:(c + 1) * chunk_elems] = packed.ravel()
        exchange(S, R2, 0, c)
    # pass C
    out = np.empty((lz, ny, nx), dtype=np.complex128)
    for c in range(chunks):
        st = R2[c * chunk_elems:(c + 1) * chunk_elems].reshape(P, lz, cy, nx)  # [r][z_local][yc][x]
        for r in range(P):
            out[:, r * ly + c * cy: r * ly + (c + 1) * cy, :] = np.fft.fft(st[r], axis=2)
    ref = np.fft.fftn(full)[rank * lz:(rank + 1) * lz]
    err = np.max(np.abs(out - ref)) / np.max(np.abs(ref))
    dist.barrier()
    dist.destroy_process_group()
    print(f"rank {rank}: rel err {err:.2e}")
    sys.exit(0 if err < 1e-12 else 1)


if __name__ == "__main__":
    main()
