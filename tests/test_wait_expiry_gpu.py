"""A bounded device-side wait that runs out must end the kernel with the error flag set — no hang, no
fault.  The probe is built from the library's own kernel sources with a short spin limit and with every
expected transaction count raised by 16 bytes: all copies land, no load phase ever completes, each wait
gives up after a few thousand polls, the CTA raises the flag, waits (bounded) for what is still in
flight and returns.  Covers the bulk-copy row kernel and the tensor-copy column kernel."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "rocfft_b200", "csrc")


def test_bounded_waits_give_up_and_report(gpu, tmp_path):
    exe = str(tmp_path / "wait_expiry_probe")
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17",
           "-DB200FFT_MBAR_SPIN=4096u", "-DB200FFT_TEST_EXTRA_TX=16u",
           "-I", os.path.join(CSRC, "generated"), "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "launch"),
           "-I", CSRC, "-I", os.path.join(ROOT, "include"),
           "-o", exe, os.path.join(ROOT, "tests", "wait_expiry_probe.cu"), os.path.join(CSRC, "plan", "twiddles.cpp")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    lines = dict(ln.split(" ", 1) for ln in r.stdout.strip().splitlines())
    for name in ("rows_tma", "col_tma"):
        assert lines.get(name) == "flag=1 status=no error", (name, r.stdout)
