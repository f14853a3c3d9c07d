"""The multi-rank path of bench.py's verification on CPU ranks: two gloo processes merge their partial plane sums
(all-reduce), their line sums (all-gather) and their error norms the way the GPU ranks do over NCCL.  Every rank must
accept the true transform, and every rank must learn of a corrupted value in one rank's slab."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("corrupt,port", [(-1, 29711), (1, 29712)])
def test_sampled_check_across_two_gloo_ranks(corrupt, port):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", "verify_cpu_worker.py"), str(corrupt)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("verify ok=") == 2
