"""One-process-per-GPU driver for slab-decomposed 3D transforms.

torch.distributed is used only as plumbing: to ship the NCCL unique id between
ranks and for barriers / max-over-ranks reductions of timings.  The transform
itself — local FFT passes whose stores land directly in the peer GPUs' buffers
over NVLink (or, as an option, a chunked NCCL send/recv exchange) — lives in
librocfft.so behind the field / brick API of rocfft.h (reference call
sequence: clients/samples/mpi/rocfft_mpi_example.cpp).
"""
from __future__ import annotations

import ctypes
import json
import math
import os
import time

import numpy as np

import rocfft_b200 as rf


def init_process_group(backend="nccl"):
    import torch
    import torch.distributed as dist
    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        rank = int(os.environ.get("RANK", "0"))
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group(backend=backend, rank=rank, world_size=world)
    return dist


def create_nccl_comm(dist):
    """Collective: returns a ctypes c_void_p holding an ncclComm_t that spans
    the default process group."""
    import torch
    L = rf.lib()
    L.b200fft_nccl_unique_id.argtypes = [ctypes.c_void_p]
    L.b200fft_nccl_comm_create.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p)]
    L.b200fft_nccl_comm_destroy.argtypes = [ctypes.c_void_p]
    rank, world = dist.get_rank(), dist.get_world_size()
    idbuf = (ctypes.c_char * 128)()
    if rank == 0:
        assert L.b200fft_nccl_unique_id(idbuf) == 0, "ncclGetUniqueId failed"
    t = torch.tensor(list(bytes(idbuf)), dtype=torch.uint8)
    if dist.get_backend() == "nccl":
        t = t.cuda()
    dist.broadcast(t, src=0)
    raw = bytes(t.cpu().tolist())
    idbuf2 = (ctypes.c_char * 128).from_buffer_copy(raw)
    comm = ctypes.c_void_p()
    st = L.b200fft_nccl_comm_create(world, rank, idbuf2, ctypes.byref(comm))
    assert st == 0, "ncclCommInitRank failed"
    return comm


class SlabFFT3D:
    """3D complex transform of lengths (nx, ny, nz) [nx fastest] whose data is
    split into contiguous Z-slabs, one per rank, in place or out of place (two
    lengths (nx, ny): a 2D transform split into row slabs, rank q holding rows
    ``[q*ny/world, (q+1)*ny/world)`` of every image on both sides).  With
    ``out_split="x"`` the result is left split along X instead (rank q holds
    ``[batch][nz][ny][nx/world]``): one global transpose instead of two, the
    reference's "slow in, fast out" layout (clients/tests/multi_device_test.cpp:117-123)."""

    def __init__(self, comm, rank, world, lengths, precision=rf.rocfft_precision_single, inverse=False,
                 inplace=True, scale=None, batch=1, out_split="z"):
        lengths = list(lengths)
        self.comm = comm
        self._comm_box = ctypes.c_void_p(comm.value)
        st, self.desc = rf.rocfft_plan_description_create()
        assert st == 0
        st = rf.rocfft_plan_description_set_comm(self.desc, rf.rocfft_comm_nccl, ctypes.byref(self._comm_box))
        assert st == 0, st
        if len(lengths) == 2:
            # rank-2 transform: rank q holds the rows y in [q*ly, (q+1)*ly) of every image, in and out
            nx, ny = lengths
            assert ny % world == 0 and nx % world == 0 and out_split == "z"
            ly = ny // world
            bricks = [([0, rank * ly, 0], [nx, (rank + 1) * ly, batch], [1, nx, nx * ly])] * 2
        else:
            nx, ny, nz = lengths
            assert nz % world == 0 and ny % world == 0
            assert out_split in ("z", "x") and (out_split == "z" or nx % world == 0)
            self.lz = nz // world
            lx = nx // world
            zslab = ([0, 0, rank * self.lz, 0], [nx, ny, (rank + 1) * self.lz, batch], [1, nx, nx * ny, nx * ny * self.lz])
            xsplit = ([rank * lx, 0, 0, 0], [(rank + 1) * lx, ny, nz, batch], [1, lx, lx * ny, lx * ny * nz])
            bricks = [zslab, xsplit if out_split == "x" else zslab]
        for adder, (lower, upper, stride) in zip((rf.rocfft_plan_description_add_infield,
                                                  rf.rocfft_plan_description_add_outfield), bricks):
            st, field = rf.rocfft_field_create()
            st, brick = rf.rocfft_brick_create(lower, upper, stride, 0 if world == 1 else _current_device())
            assert st == 0
            assert rf.rocfft_field_add_brick(field, brick) == 0
            assert adder(self.desc, field) == 0
            rf.rocfft_brick_destroy(brick)
            rf.rocfft_field_destroy(field)
        if scale is not None:
            rf.rocfft_plan_description_set_scale_factor(self.desc, scale)
        tt = rf.rocfft_transform_type_complex_inverse if inverse else rf.rocfft_transform_type_complex_forward
        st, self.plan = rf.rocfft_plan_create(rf.rocfft_placement_inplace if inplace else rf.rocfft_placement_notinplace,
                                              tt, precision, lengths, batch, self.desc)
        if st != 0:
            raise RuntimeError(f"multi-device rocfft_plan_create failed: {st}")
        st, self.work_bytes = rf.rocfft_plan_get_work_buffer_size(self.plan)
        st, self.info = rf.rocfft_execution_info_create()
        self._work = None

    def attach(self, torch, stream):
        if self.work_bytes:
            self._work = torch.empty(self.work_bytes, dtype=torch.uint8, device="cuda")
            assert rf.rocfft_execution_info_set_work_buffer(self.info, self._work.data_ptr(), self.work_bytes) == 0
        assert rf.rocfft_execution_info_set_stream(self.info, stream) == 0

    def execute(self, in_ptr, out_ptr=None):
        return rf.rocfft_execute(self.plan, [in_ptr], None if out_ptr is None else [out_ptr], self.info)

    def destroy(self):
        rf.rocfft_execution_info_destroy(self.info)
        rf.rocfft_plan_destroy(self.plan)
        rf.rocfft_plan_description_destroy(self.desc)


def _current_device():
    import torch
    return torch.cuda.current_device()


def bench_main(args, METRIC, UNIT, HEADLINE, peak, peak_src):
    """`bench.py --gpus N` under torchrun: N ranks, slab-decomposed 1024^3."""
    import torch
    dist = init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    comm = create_nccl_comm(dist)
    nx = ny = nz = 1024
    ntot = nx * ny * nz
    scale = 1.0 / math.sqrt(ntot)
    fft = SlabFFT3D(comm, rank, world, [nx, ny, nz], scale=scale, inplace=True)
    stream = torch.cuda.Stream()
    fft.attach(torch, stream.cuda_stream)
    lz = nz // world
    from bench import ClockSampler, SampledCheck3D, headline_config
    verify = not getattr(args, "no_verify", False)
    chk = SampledCheck3D((nz, ny, nx), rank * lz, lz, world=world, rank=rank) if verify else None
    rng = np.random.default_rng(5 + rank)
    x = torch.empty(lz * ny * nx, dtype=torch.complex64, device="cuda")
    chunk = 1 << 24  # 16 XY planes
    for s in range(0, x.numel(), chunk):
        n = min(chunk, x.numel() - s)
        a = np.empty(n, dtype=np.complex64)
        a.real = rng.random(n, dtype=np.float32) - 0.5
        a.imag = rng.random(n, dtype=np.float32) - 0.5
        x[s:s + n].copy_(torch.from_numpy(a))
        if chk is not None:
            chk.feed(rank * lz + s // (ny * nx), a.reshape(-1, ny, nx))
    L = rf.lib()
    L.b200fft_launch_count.restype = ctypes.c_ulonglong

    def step():
        st = fft.execute(x.data_ptr())
        if st != 0:
            raise RuntimeError(f"rocfft_execute failed: {st}")

    # the first transform runs on the freshly seeded slabs and is checked before anything is timed
    verdict = None
    if chk is not None:
        with torch.cuda.stream(stream):
            step()
        torch.cuda.synchronize()
        verdict = chk.finish(x, scale, dist=dist, torch=torch)
        if not verdict["ok"]:
            if rank == 0:
                print(json.dumps({"verify": verdict, "n_gpus": world}), flush=True)
            raise SystemExit(f"verification FAILED on {world} GPUs: {verdict}")

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        l0 = L.b200fft_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(torch.cuda.current_device()) as cs:
            # a stream-ordered collective right before the first event lines the GPUs up, so the
            # timed region does not start with ranks waiting for the slowest host to enqueue
            align = torch.zeros(1, device="cuda")
            dist.all_reduce(align)
            e0.record(stream)
            h0 = time.perf_counter()
            for _ in range(args.steps):
                step()
            host_ms = (time.perf_counter() - h0) * 1e3 / args.steps  # host time to enqueue one step
            e1.record(stream)
            torch.cuda.synchronize()
        dist.barrier()
        ms = e0.elapsed_time(e1) / args.steps
        launches = int(L.b200fft_launch_count() - l0)
    t = torch.tensor([ms], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max = float(t.item())

    # end to end: host slab -> device, transform, device -> host, every step; steps are pipelined over two
    # device slabs and three streams (H2D of step i+1 overlaps the transform of step i and the D2H of step i-1)
    e2e = None
    if not args.no_e2e:
        nbytes = x.numel() * 8
        hin = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        hout = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        hin.copy_(x.view(torch.uint8))
        x2 = torch.empty_like(x)
        bufs = [x, x2]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        free_ev = [None, None]
        k = max(4, min(args.steps, 10))

        def e2e_step(i):
            xi = bufs[i % 2]
            if free_ev[i % 2] is not None:
                s_in.wait_event(free_ev[i % 2])
            with torch.cuda.stream(s_in):
                xi.view(torch.uint8).copy_(hin, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            stream.wait_event(ev_in)
            with torch.cuda.stream(stream):
                st = fft.execute(xi.data_ptr())
                if st != 0:
                    raise RuntimeError(f"rocfft_execute failed: {st}")
                ev_c = torch.cuda.Event()
                ev_c.record(stream)
            s_out.wait_event(ev_c)
            with torch.cuda.stream(s_out):
                hout.copy_(xi.view(torch.uint8), non_blocking=True)
                ev_o = torch.cuda.Event()
                ev_o.record(s_out)
            free_ev[i % 2] = ev_o

        for i in range(2):
            e2e_step(i)
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(s_in):
            dist.all_reduce(align)
            e0.record(s_in)
        for i in range(k):
            e2e_step(i)
        e1.record(s_out)
        torch.cuda.synchronize()
        dist.barrier()
        ems = e0.elapsed_time(e1) / k
        t = torch.tensor([ems], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ems = float(t.item())
        flops = 5 * 2 ** 30 * 30
        e2e = {"value": flops / ems / 1e6, "unit": UNIT, "ms_per_step": ems, "h2d_bytes_per_step": nbytes * world,
               "d2h_bytes_per_step": nbytes * world,
               "pipeline": "2 device slabs per rank, 3 streams: H2D of step i+1 overlaps the transform of step i and D2H of step i-1"}
        del hin, hout, x2

    if rank == 0:
        flops = 5 * 2 ** 30 * 30
        per_gpu_bytes = 2 * 3 * lz * ny * nx * 8  # three local passes, each reads and writes the slab
        a2a_bytes = 2 * lz * ny * nx * 8 * (world - 1) // world  # sent per GPU over NVLink, both exchanges
        line = {"metric": METRIC, "value": flops / ms_max / 1e6, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_max, "higher_is_better": True, "scaling": "strong",
                "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": headline_config(world),
                "exchange": ("NCCL grouped send/recv, 2 global transposes" if os.environ.get("ROCFFT_B200_MGPU_NCCL")
                             else "peer stores over NVLink fused into FFT passes A and B, 2 global transposes"),
                "roofline": {"bound": "nvlink", "achieved": a2a_bytes / ms_max / 1e6, "peak": 770.0,
                             "peak_source": "measured peer copy per direction", "unit": "GB/s",
                             "frac": a2a_bytes / ms_max / 1e6 / 770.0, "traffic": None,
                             "note": "bytes each GPU must send over NVLink per transform / step time",
                             "local_hbm_bytes_per_gpu": per_gpu_bytes},
                "clocks": cs.summary(), "gpu_launches": launches, "host_enqueue_ms_per_step": host_ms}
        if verdict is not None:
            line["verify"] = verdict
        if e2e:
            line["e2e"] = e2e
        print(json.dumps(line), flush=True)
    fft.destroy()
    dist.barrier()
    dist.destroy_process_group()
    return 0
