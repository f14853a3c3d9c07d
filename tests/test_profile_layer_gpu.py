"""ROCFFT_LAYER bit 4 (profile): every kernel of an execute is timed and reported with bytes, GB/s
and the share of the device's peak bandwidth (reference: library/src/powX.cpp:817-883)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_profile_layer_reports_every_kernel(tmp_path):
    log = tmp_path / "profile.log"
    env = dict(os.environ, ROCFFT_LAYER="4", ROCFFT_LOG_PROFILE_PATH=str(log))
    code = ("import torch, rocfft_b200 as rf; rf.rocfft_setup();"
            "x = torch.zeros(512 * 512 * 8, dtype=torch.complex64, device='cuda');"
            "p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [512, 512], 8);"
            "assert p.execute([x.data_ptr()]) == 0; torch.cuda.synchronize(); p.destroy()")
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in log.read_text().splitlines() if ln.startswith("rocfft_execute,scheme,")]
    assert len(lines) == 2, lines  # one row pass, one column pass
    for i, ln in enumerate(lines):
        f = ln.split(",")
        kv = dict(zip(f[1::2], f[2::2]))
        assert int(kv["kernel_index"]) == i
        assert float(kv["duration_ms"]) > 0
        assert int(kv["total_size_bytes"]) == 2 * 512 * 512 * 8 * 8
        assert float(kv["max_mem_GB_s"]) > 1000
        assert 0 < float(kv["bw_efficiency_pct"]) < 120
