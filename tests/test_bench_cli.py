"""rocfft-bench-compatible client: token grammar (shared/fft_params.h:726-1010 in the reference),
defaults, and one timed run on the GPU."""
import os
import subprocess
import sys

import pytest

from rocfft_b200.bench_cli import Params, build_parser, params_from_args

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

TOKENS = [
    "complex_forward_len_4096_single_ip_batch_16384_istride_1_CI_ostride_1_CI_idist_4096_odist_4096_ioffset_0_0_ooffset_0_0",
    "real_forward_len_30_1000_single_op_batch_16_istride_1000_1_R_ostride_501_1_HI_idist_30000_odist_15030_ioffset_0_0_ooffset_0_0",
    "complex_inverse_len_8_8_8_double_op_batch_2_istride_64_8_1_CP_ostride_64_8_1_CI_idist_512_odist_512_ioffset_0_0_ooffset_0_0_scale",
]


@pytest.mark.parametrize("tok", TOKENS)
def test_token_round_trip(tok):
    assert Params.from_token(tok).token() == tok


def test_token_rejects_garbage():
    for bad in ["complex_sideways_len_8_single_ip_batch_1", "complex_forward_8_single", "real_forward_len_8_single_ip_batch_1_what_3"]:
        with pytest.raises((ValueError, KeyError, IndexError)):
            Params.from_token(bad)


def test_defaults_match_the_library_defaults():
    # the bench log layer's own line parses, and omitted strides default like rocfft_plan_create's
    line = ("--length 30 1000 -b 16 -o -t 2 --precision single --itype 2 --otype 3 --istride 1000 1 --ostride 501 1 "
            "--idist 30000 --odist 15030 --ioffset 0 0 --ooffset 0 0").split()
    explicit = params_from_args(build_parser().parse_args(line)).complete()
    implicit = params_from_args(build_parser().parse_args("--length 30 1000 -b 16 -o -t 2".split())).complete()
    assert explicit.token() == implicit.token() == TOKENS[1]
    ip = params_from_args(build_parser().parse_args("--length 1000 -b 4 -t 2".split())).complete()
    assert ip.istride == [1] and ip.idist == 1002 and ip.odist == 501  # in-place real rows are padded


@pytest.mark.gpu
def test_cli_runs_and_reports_like_rocfft_bench():
    r = subprocess.run([sys.executable, "-m", "rocfft_b200.bench_cli", "--length", "256", "256", "-b", "8", "-N", "3"],
                       cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    times = [ln for ln in r.stdout.splitlines() if ln.startswith("Execution gpu time:")]
    flops = [ln for ln in r.stdout.splitlines() if ln.startswith("Execution gflops:")]
    assert len(times) == 1 and len(flops) == 1
    assert len(times[0].split()) == 3 + 3 + 1 and times[0].endswith(" ms")
    assert all(float(v) > 0 for v in flops[0].split()[2:])
    r = subprocess.run([sys.executable, "-m", "rocfft_b200.bench_cli", "--token", TOKENS[1]], cwd=ROOT,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "Execution gflops:" in r.stdout
