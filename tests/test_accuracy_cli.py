"""The token-driven accuracy driver (tests/accuracy_cli.py): token -> case mapping on the CPU, and a few
tokens end to end on the GPU."""
import pytest

import accuracy_cli
import harness as H
from rocfft_b200 import bench_cli

TOKENS = [
    "complex_forward_len_4096_single_ip_batch_8_istride_1_CI_ostride_1_CI_idist_4096_odist_4096_ioffset_0_0_ooffset_0_0",
    "real_forward_len_1000_single_op_batch_16_istride_1_R_ostride_1_HI_idist_1000_odist_501_ioffset_0_0_ooffset_0_0",
    "complex_inverse_len_64_128_double_op_batch_3_istride_128_1_CP_ostride_128_1_CI_idist_8192_odist_8192_ioffset_0_0_ooffset_0_0",
    "complex_forward_len_16_32_64_single_ip_batch_2_istride_2048_64_1_CI_ostride_2048_64_1_CI_idist_32768_odist_32768_ioffset_0_0_ooffset_0_0",
    "real_inverse_len_36_50_double_op_batch_2_istride_26_1_HI_ostride_50_1_R_idist_936_odist_1800_ioffset_0_0_ooffset_0_0",
]


def test_token_to_case_mapping():
    p = bench_cli.Params.from_token(TOKENS[2])
    c = accuracy_cli.case_from_params(p)
    assert c.ttype == H.C2C_INV and c.precision == "double" and list(c.lengths) == [128, 64] and c.batch == 3
    assert c.placement == H.OOP and c.in_type == H.CP and c.out_type == H.CI
    assert list(c.in_strides) == [1, 128] and c.in_dist == 8192
    # a token made from options round-trips through the parser
    a = bench_cli.build_parser().parse_args(["--length", "8", "16", "-b", "5", "-t", "2", "-o"])
    tok = bench_cli.params_from_args(a).complete().token()
    q = bench_cli.Params.from_token(tok)
    assert q.length == [8, 16] and q.nbatch == 5 and q.transform_type == 2 and not q.inplace and q.ostride == [9, 1]


@pytest.mark.gpu
@pytest.mark.parametrize("token", TOKENS)
def test_tokens_pass_on_gpu(gpu, token):
    ok, msg = accuracy_cli.run_token(token)
    assert ok, f"{token}: {msg}"
