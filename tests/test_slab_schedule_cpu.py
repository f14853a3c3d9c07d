"""World-size-2 (and 4) CPU test of the multi-GPU decomposition: gloo ranks run
the slab plan's three passes in numpy and exchange blocks at the offsets the
library's own schedule function returns; the result must equal numpy's fftn.
Covers the host-side logic of the N > 1 path without GPUs."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,shape,chunks", [(2, (8, 8, 8), 1), (2, (4, 8, 16), 2), (4, (6, 16, 8), 2)])
def test_slab_decomposition_over_gloo(built_library, world, shape, chunks):
    env = dict(os.environ)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29740 + world + chunks),
           os.path.join(ROOT, "tests", "slab_cpu_worker.py")] + [str(v) for v in shape] + [str(chunks)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]


@pytest.mark.parametrize("world,nx,ny,batch", [(2, 8, 12, 1), (2, 16, 8, 3), (4, 8, 16, 2)])
def test_row_slab_2d_decomposition_over_gloo(built_library, world, nx, ny, batch):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29760 + world + batch),
           os.path.join(ROOT, "tests", "rows2d_cpu_worker.py"), str(nx), str(ny), str(batch)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=dict(os.environ))
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
