"""Worker for the multi-GPU tests: one rank per GPU under torch.distributed.run.
Runs a slab-decomposed 3D (or, with two lengths, row-slab 2D) transform through the field/brick API and compares
the gathered result with the CPU oracle on rank 0 (the reference's MPI worker,
clients/tests/rocfft_mpi_worker.cpp, does the same against FFTW)."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def fft_describe(fft):
    import ctypes
    import rocfft_b200 as rf
    L = rf.lib()
    L.b200fft_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    buf = ctypes.create_string_buffer(1 << 16)
    L.b200fft_plan_describe(fft.plan, buf, len(buf))
    return buf.value.decode()


def main():
    import torch
    import rocfft_b200 as rf
    from rocfft_b200 import distributed as D
    from oracle import fft_oracle as orc

    lengths = [int(v) for v in sys.argv[1].split("x")]
    prec = sys.argv[2]
    inverse = sys.argv[3] == "inv"
    inplace = sys.argv[4] == "ip"
    batch = int(sys.argv[5]) if len(sys.argv) > 5 else 1
    out_split = sys.argv[6] if len(sys.argv) > 6 else "z"
    dist = D.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert rf.rocfft_setup() == 0
    comm = D.create_nccl_comm(dist)
    rows2d = len(lengths) == 2  # rank-2 transform on row slabs: the slab dimension is Y
    if rows2d:
        (nx, nz), ny = lengths, 1
    else:
        nx, ny, nz = lengths
    lz = nz // world
    cdt = np.complex64 if prec == "single" else np.complex128
    full = orc.uniform_input((batch, nz, ny, nx), cdt, seed=11)
    mine = torch.from_numpy(full[:, rank * lz:(rank + 1) * lz].copy()).cuda()  # [batch][lz][ny][nx]
    out = mine if inplace else torch.empty_like(mine)
    lx = nx // world
    fft = D.SlabFFT3D(comm, rank, world, lengths,
                      precision=rf.rocfft_precision_single if prec == "single" else rf.rocfft_precision_double,
                      inverse=inverse, inplace=inplace, scale=0.5, batch=batch, out_split=out_split)
    if world > 1 or batch > 1:
        assert "slab plan" in fft_describe(fft), "the optimised slab plan should serve this layout"
    if rows2d:
        assert "row slabs of a rank-2 transform" in fft_describe(fft)
    stream = torch.cuda.Stream()
    fft.attach(torch, stream.cuda_stream)
    for rep in range(2):  # twice: the second run exercises buffer reuse across calls
        if rep == 1:
            mine.copy_(torch.from_numpy(full[:, rank * lz:(rank + 1) * lz].copy()))
            torch.cuda.synchronize()
        st = fft.execute(mine.data_ptr(), None if inplace else out.data_ptr())
        assert st == 0, st
        torch.cuda.synchronize()
    if out_split == "x":
        out = out.reshape(-1)[: batch * nz * ny * lx].reshape(batch, nz, ny, lx)  # the X-split brick, same element count
        assert "one global transpose" in fft_describe(fft)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out.contiguous())
    ok = True
    if rank == 0:
        got = torch.cat(gathered, dim=3 if out_split == "x" else 1).cpu().numpy()
        ref = orc.c2c(full.reshape(batch, nz, nx) if rows2d else full, +1 if inverse else -1).reshape(full.shape) * 0.5
        ok, msg = orc.check_accuracy(got, ref, prec, nx * ny * nz)
        print(f"mgpu {lengths} batch {batch} {prec} inverse={inverse} inplace={inplace} world={world}: {msg} -> {'ok' if ok else 'FAIL'}",
              flush=True)
    fft.destroy()
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if ok else 1)


if __name__ == "__main__":
    main()
