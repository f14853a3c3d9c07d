"""Worker for multi-process plans on brick layouts the slab plan does not take (one rank per GPU
under torch.distributed.run): every rank adds its own bricks, as the ranks of the reference's MPI
sample do (clients/samples/mpi/rocfft_mpi_example.cpp:129-260), and checks its own output bricks
against numpy.

argv: case name.  Cases:
  slabs2d_uneven   2D c2c 30 x 17, rows of the slow dimension dealt out unevenly, out of place
  real3d           3D real forward 16 x 12 x 10, input split on z, output split on y
  pencils          3D c2c 12 x 8 x 6 batch 2, two bricks per rank on the input, z-slabs on the output, in place counts equal
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def split(n, parts, k):
    lo = k * (n // parts) + min(k, n % parts)
    return lo, lo + n // parts + (1 if k < n % parts else 0)


def main():
    import ctypes
    import torch
    import rocfft_b200 as rf
    from rocfft_b200 import distributed as D
    from fields_util import cut, make_field

    case = sys.argv[1]
    dist = D.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    assert rf.rocfft_setup() == 0
    comm = D.create_nccl_comm(dist)
    box = ctypes.c_void_p(comm.value)
    rng = np.random.default_rng(5)  # same data on every rank
    prec, tol = 0, 2e-5
    if case == "slabs2d_uneven":
        lengths, batch, ttype = [30, 17], 1, rf.rocfft_transform_type_complex_forward
        x = (rng.random((1, 17, 30)) - 0.5 + 1j * (rng.random((1, 17, 30)) - 0.5)).astype(np.complex64)
        ref = np.fft.fftn(x.astype(np.complex128), axes=(1, 2))
        lo, hi = split(17, world, rank)
        in_bricks = out_bricks = [([0, lo, 0], [30, hi, 1])]
        odt = np.complex64
    elif case == "real3d":
        lengths, batch, ttype = [16, 12, 10], 1, rf.rocfft_transform_type_real_forward
        prec, tol = 1, 1e-13
        x = rng.random((1, 10, 12, 16)) - 0.5
        ref = np.fft.rfftn(x, axes=(1, 2, 3))
        zlo, zhi = split(10, world, rank)
        ylo, yhi = split(12, world, rank)
        in_bricks = [([0, 0, zlo, 0], [16, 12, zhi, 1])]
        out_bricks = [([0, ylo, 0, 0], [9, yhi, 10, 1])]
        odt = np.complex128
    elif case == "pencils":
        lengths, batch, ttype = [12, 8, 6], 2, rf.rocfft_transform_type_complex_inverse
        x = (rng.random((2, 6, 8, 12)) - 0.5 + 1j * (rng.random((2, 6, 8, 12)) - 0.5)).astype(np.complex64)
        ref = np.fft.ifftn(x.astype(np.complex128), axes=(1, 2, 3)) * (12 * 8 * 6)
        zlo, zhi = split(6, world, rank)
        in_bricks = [([0, 0, zlo, 0], [12, 4, zhi, 2]), ([0, 4, zlo, 0], [12, 8, zhi, 2])]
        ylo, yhi = split(8, world, rank)
        out_bricks = [([0, ylo, 0, 0], [12, yhi, 6, 1]), ([0, ylo, 0, 1], [12, yhi, 6, 2])]
        odt = np.complex64
    else:
        raise SystemExit(f"unknown case {case}")

    st, desc = rf.rocfft_plan_description_create()
    assert rf.rocfft_plan_description_set_comm(desc, rf.rocfft_comm_nccl, ctypes.byref(box)) == 0
    dev = torch.cuda.current_device()
    fin, in_sizes = make_field(in_bricks, [dev] * len(in_bricks))
    fout, out_sizes = make_field(out_bricks, [dev] * len(out_bricks))
    assert rf.rocfft_plan_description_add_infield(desc, fin) == 0
    assert rf.rocfft_plan_description_add_outfield(desc, fout) == 0
    st, plan = rf.rocfft_plan_create(rf.rocfft_placement_notinplace, ttype, prec, lengths, batch, desc)
    assert st == 0, f"plan creation failed on rank {rank}: {st}"
    st, wb = rf.rocfft_plan_get_work_buffer_size(plan)
    st, info = rf.rocfft_execution_info_create()
    work = None
    if wb:
        work = torch.empty(wb, dtype=torch.uint8, device="cuda")
        assert rf.rocfft_execution_info_set_work_buffer(info, work.data_ptr(), wb) == 0
    tin = [torch.from_numpy(cut(x, lo, hi).reshape(-1)).cuda() for lo, hi in in_bricks]
    tout = [torch.zeros(n, dtype=torch.from_numpy(np.zeros(1, odt)).dtype, device="cuda") for n in out_sizes]
    ok = True
    for rep in range(2):
        for t in tout:
            t.zero_()
        torch.cuda.synchronize()
        st = rf.rocfft_execute(plan, [t.data_ptr() for t in tin], [t.data_ptr() for t in tout], info)
        assert st == 0, f"execute failed on rank {rank}: {st}"
        torch.cuda.synchronize()
        for (lo, hi), t in zip(out_bricks, tout):
            want = cut(ref, lo, hi).reshape(-1)
            err = np.linalg.norm(t.cpu().numpy() - want) / np.linalg.norm(want)
            ok = ok and err < tol
            if err >= tol:
                print(f"rank {rank} case {case} brick {lo}-{hi}: relative error {err}", flush=True)
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print(f"mgpu fields {case} world={world}: {'ok' if int(flag) else 'FAIL'}", flush=True)
    rf.rocfft_execution_info_destroy(info)
    rf.rocfft_plan_destroy(plan)
    rf.rocfft_plan_description_destroy(desc)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if int(flag) else 1)


if __name__ == "__main__":
    main()
