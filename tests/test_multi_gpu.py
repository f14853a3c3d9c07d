"""Slab-decomposed 3D transforms through the field/brick API, one rank per GPU
(reference: clients/tests/multi_device_test.cpp:30-187 and the MPI worker).
With one GPU the same code path runs with a single-rank communicator; with two
or more the exchange crosses NVLink."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(nproc, lengths, prec, direction, placement, port, batch=1, out_split="z"):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    if out_split == "x":
        env["ROCFFT_B200_MGPU_PREFER_XSPLIT"] = "1"  # a single rank fits both layouts: take the one under test
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mgpu_worker.py"),
           lengths, prec, direction, placement, str(batch), out_split]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("lengths,prec,direction,placement", [
    ("64x64x64", "single", "fwd", "ip"),
    ("32x64x16", "double", "inv", "op"),
    ("100x20x8", "single", "fwd", "op"),
])
def test_single_rank_slab_plan(gpu, lengths, prec, direction, placement):
    _launch(1, lengths, prec, direction, placement, 29631)


@pytest.mark.parametrize("lengths,prec,direction,placement", [
    ("64x64x64", "single", "fwd", "ip"),
    ("128x64x32", "double", "inv", "op"),
    ("256x256x256", "single", "fwd", "ip"),
])
def test_two_rank_slab_plan(gpu, lengths, prec, direction, placement):
    if gpu.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _launch(2, lengths, prec, direction, placement, 29632)


@pytest.mark.parametrize("lengths,prec,direction,placement,batch", [
    ("64x32x16", "single", "fwd", "ip", 4),     # the reference's multi-device tests use batch 4 and 1
    ("32x64x32", "double", "inv", "op", 3),
])
def test_batched_slab_plan(gpu, lengths, prec, direction, placement, batch):
    """Batches through the optimised slab plan (reference: clients/tests/multi_device_test.cpp:55-63, batch {4, 1});
    one rank when a single GPU is present, two across NVLink otherwise."""
    _launch(min(2, gpu.cuda.device_count()), lengths, prec, direction, placement, 29633, batch)


@pytest.mark.parametrize("split", ["slowest_both", "slow_in_fast_out", "pencils"])
def test_single_process_bricks_on_two_devices(gpu, split):
    """One process, bricks alternating between two GPUs: the gather / scatter plan reaches the
    other device through peer access (reference: multi_device_test.cpp with fft_mp_lib_none)."""
    if gpu.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import rocfft_b200 as rf
    from test_fields_gpu import SPLITS, TOL, run_field_case
    gi, go = SPLITS[split]
    gpu.cuda.set_device(0)
    err = run_field_case(rf.rocfft_transform_type_complex_forward, 0, [64, 32, 16], 2, gi, go, devices=[0, 1])
    assert err < TOL[0], err


def _launch_fields(nproc, case, port):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mgpu_fields_worker.py"),
           case]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("case", ["slabs2d_uneven", "real3d", "pencils"])
def test_multi_process_general_layouts(gpu, case):
    """Layouts outside the optimised slab plan run as gather -> transform on rank 0 -> scatter over NCCL;
    with one GPU the same path runs with a single-rank communicator."""
    _launch_fields(min(2, gpu.cuda.device_count()), case, 29641)


@pytest.mark.parametrize("lengths,prec,direction,placement,batch", [
    ("64x32x16", "single", "fwd", "op", 1),
    ("64x64x64", "single", "fwd", "ip", 1),
    ("32x32x64", "double", "inv", "op", 4),
])
def test_slab_in_x_split_out_single_transpose(gpu, lengths, prec, direction, placement, batch):
    """Input split along the slowest dimension, output along the fastest (the reference's SLOW_IN_FAST_OUT,
    clients/tests/multi_device_test.cpp:117-123): the optimised plan then needs one global transpose, not two."""
    _launch(min(2, gpu.cuda.device_count()), lengths, prec, direction, placement, 29634, batch, "x")


@pytest.mark.parametrize("lengths,prec,direction,placement,batch", [
    ("256x256", "single", "fwd", "ip", 4),
    ("64x128", "double", "inv", "op", 1),
    ("1024x1024", "single", "fwd", "op", 2),
])
def test_row_slab_2d_plan(gpu, lengths, prec, direction, placement, batch):
    """Rank-2 transforms split into row slabs on both sides (the 2D cases of the reference's multi-device tests,
    clients/tests/multi_device_test.cpp:100-136, split on the slowest dimension) run through the fused peer-store
    plan, not gather / scatter: copy into the owners' column blocks, Y transform with the store split over the
    ranks' row buffers, X transform."""
    _launch(min(2, gpu.cuda.device_count()), lengths, prec, direction, placement, 29635, batch)
