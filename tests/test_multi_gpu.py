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


def _launch(nproc, lengths, prec, direction, placement, port):
    env = dict(os.environ)
    env["NCCL_NVLS_ENABLE"] = "0"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "mgpu_worker.py"),
           lengths, prec, direction, placement]
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
