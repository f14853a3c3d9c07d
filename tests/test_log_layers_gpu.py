"""The kernelio and graph log layers (ROCFFT_LAYER bits 16 and 128; reference: library/src/include/logging.h:139-150,
library/src/powX.cpp:743-780, library/src/transform.cpp:178-254).  kernelio writes one checksum per kernel of what that
kernel left in its output buffer: two runs on the same input must write identical lines, a run on different input must not."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r'''
import sys, numpy as np, torch
sys.path.insert(0, %r)
import rocfft_b200 as rf
assert rf.rocfft_setup() == 0
seed = int(sys.argv[1])
rng = np.random.default_rng(seed)
x = (rng.random((8, 64, 128)) - 0.5 + 1j * (rng.random((8, 64, 128)) - 0.5)).astype(np.complex64)
d = torch.from_numpy(x).cuda()
p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [128, 64], 8)
assert p.execute([d.data_ptr()]) == 0
torch.cuda.synchronize()
ref = np.fft.fft2(x.astype(np.complex128))
assert np.linalg.norm(d.cpu().numpy() - ref) / np.linalg.norm(ref) < 1e-5
'''


def _run(seed, path):
    env = dict(os.environ, ROCFFT_LAYER="16", ROCFFT_LOG_KERNELIO_PATH=str(path))
    r = subprocess.run([sys.executable, "-c", SCRIPT % ROOT, str(seed)], capture_output=True, text=True, env=env, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    return open(path).read().strip().splitlines()


def test_kernelio_hashes_repeat_and_discriminate(gpu, tmp_path):
    a = _run(1, tmp_path / "a.log")
    b = _run(1, tmp_path / "b.log")
    c = _run(2, tmp_path / "c.log")
    assert len(a) >= 2 and all(re.match(r"--- --- kernel \d+ \(.+\) output: \d+ bytes, hash [0-9a-f]+", ln) for ln in a), a
    assert a == b, "same input, same plan: the per-kernel checksums must repeat"
    assert a != c and len(a) == len(c), "different input must change the checksums"


def test_graph_layer_prints_the_multi_device_plan(gpu, tmp_path):
    path = tmp_path / "graph.log"
    env = dict(os.environ, ROCFFT_LAYER="128", ROCFFT_LOG_GRAPH_PATH=str(path), NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=1", "--master-addr", "127.0.0.1",
           "--master-port", "29651", os.path.join(ROOT, "tests", "mgpu_worker.py"), "64x32x16", "single", "fwd", "ip"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    text = open(path).read()
    assert text.startswith("digraph plan {") and "bar0" in text and "-> bar1" in text and "FFT along X" in text, text
