"""Accuracy driver by token, in the manner of rocfft-test's TEST_P(accuracy_test, vs_fftw)
(reference: clients/tests/rocfft_accuracy_test.cpp:57-128; token grammar shared/fft_params.h:726-899):

    python tests/accuracy_cli.py complex_forward_len_1024_1024_double_op_batch_4_istride_1024_1_CI_ostride_1024_1_CI_idist_1048576_odist_1048576_ioffset_0_0_ooffset_0_0
    python tests/accuracy_cli.py --length 1000 -b 64 -t 2 -o

Every token (or one rocfft-bench style argument list) is planned and executed through the C API on seeded
input, compared with the double-precision CPU oracle under rocfft-test's Linf / L2 bounds, and the bytes
around the output layout are checked for stray writes.  One line per token: PASS / FAIL with both norms.
This is test infrastructure: it imports the oracle, which the library itself never does.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from rocfft_b200 import bench_cli  # noqa: E402


def case_from_params(p):
    """bench_cli.Params (row-major, as tokens and rocfft-bench options are) -> harness.Case (fastest first)."""
    import harness as H
    placement = H.IP if p.inplace else H.OOP
    kw = {}
    if p.istride:
        kw["in_strides"] = list(reversed(p.istride))
    if p.ostride:
        kw["out_strides"] = list(reversed(p.ostride))
    planar_i, planar_o = p.itype in (1, 4), p.otype in (1, 4)
    return H.Case(p.transform_type, p.precision, list(reversed(p.length)), p.nbatch, placement,
                  in_type=None if p.itype == 5 else p.itype, out_type=None if p.otype == 5 else p.otype,
                  in_dist=p.idist, out_dist=p.odist,
                  in_offsets=list(p.ioffset)[: 2 if planar_i else 1] if any(p.ioffset) else None,
                  out_offsets=list(p.ooffset)[: 2 if planar_o else 1] if any(p.ooffset) else None,
                  scale=None if p.scale_factor == 1.0 else p.scale_factor, **kw)


def run_token(token):
    import harness as H
    p = bench_cli.Params.from_token(token)
    if p.precision == "half":
        return False, "half precision is not supported"
    return H.run_case(case_from_params(p))


def main(argv=None):
    argv = list(sys.argv[1:] if argv is None else argv)
    import rocfft_b200 as rf
    assert rf.rocfft_setup() == 0
    failed = 0
    if argv and not argv[0].startswith("-"):
        tokens = argv
    else:
        a = bench_cli.build_parser().parse_args(argv)
        tokens = [a.token] if a.token else [bench_cli.params_from_args(a).complete().token()]
    for tok in tokens:
        try:
            ok, msg = run_token(tok)
        except Exception as e:  # a token the library refuses is a failure of that token, not of the run
            ok, msg = False, f"{type(e).__name__}: {e}"
        print(("PASS " if ok else "FAIL ") + tok + "  " + msg, flush=True)
        failed += 0 if ok else 1
    rf.rocfft_cleanup()
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
