"""Host-side checks that need no GPU: the C-ABI library loads and exports every
symbol the headers declare, argument validation returns the reference's status
codes (library/src/plan.cpp:729-779, 2959-3074; transform.cpp:35-103), and the
planner picks the intended kernels for the benchmark configurations."""
import ctypes
import os
import re

import numpy as np
import pytest

import rocfft_b200 as rf

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L(built_library):
    L = built_library
    L.b200fft_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
    rf.rocfft_setup()
    return L


def describe(L, plan):
    buf = ctypes.create_string_buffer(1 << 16)
    assert L.b200fft_plan_describe(plan.plan, buf, len(buf)) == 0
    return buf.value.decode()


def test_every_declared_symbol_is_exported(L):
    declared = set()
    for hdr in ("include/rocfft/rocfft.h", "include/rocfft_b200_ext.h"):
        text = open(os.path.join(ROOT, hdr)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        declared |= set(re.findall(r"\b((?:rocfft|b200fft)_[a-z0-9_]+)\s*\(", text))
    assert set(rf.EXPORTED_SYMBOLS) <= declared
    for name in sorted(declared):
        assert hasattr(L, name), f"{name} is declared but not exported"


def test_version_string(L):
    st, v = rf.rocfft_get_version_string(64)
    assert st == rf.rocfft_status_success and v.startswith("1.0.32")
    st, _ = rf.rocfft_get_version_string(4)
    assert st == rf.rocfft_status_invalid_arg_value
    assert L.rocfft_get_version_string(None, 10) == rf.rocfft_status_failure


def test_dimension_limits(L):
    st, p = rf.rocfft_plan_create(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward,
                                  rf.rocfft_precision_single, [4, 4, 4, 4], 1)
    assert st == rf.rocfft_status_invalid_dimensions
    rf.rocfft_plan_destroy(p)


def _layout_status(ttype, placement, it, ot):
    st, d = rf.rocfft_plan_description_create()
    rf.rocfft_plan_description_set_data_layout(d, it, ot, None, None, None, 0, None, 0)
    st, p = rf.rocfft_plan_create(placement, ttype, rf.rocfft_precision_single, [16], 1, d)
    rf.rocfft_plan_destroy(p)
    rf.rocfft_plan_description_destroy(d)
    return st


def test_array_type_rules(L):
    CI, CP, RE, HI, HP = (rf.rocfft_array_type_complex_interleaved, rf.rocfft_array_type_complex_planar,
                          rf.rocfft_array_type_real, rf.rocfft_array_type_hermitian_interleaved,
                          rf.rocfft_array_type_hermitian_planar)
    F, I, RF, RI = (rf.rocfft_transform_type_complex_forward, rf.rocfft_transform_type_complex_inverse,
                    rf.rocfft_transform_type_real_forward, rf.rocfft_transform_type_real_inverse)
    ip, op = rf.rocfft_placement_inplace, rf.rocfft_placement_notinplace
    bad = rf.rocfft_status_invalid_array_type
    ok = rf.rocfft_status_success
    assert _layout_status(F, op, CI, CP) == ok
    assert _layout_status(F, ip, CI, CP) == bad  # in place needs identical formats
    assert _layout_status(F, op, RE, CI) == bad
    assert _layout_status(I, op, CI, HI) == bad
    assert _layout_status(RF, op, RE, HP) == ok
    assert _layout_status(RF, ip, RE, HP) == bad  # in place real forward must be interleaved
    assert _layout_status(RF, op, CI, HI) == bad
    assert _layout_status(RI, op, HP, RE) == ok
    assert _layout_status(RI, ip, HP, RE) == bad
    assert _layout_status(RI, op, HI, CI) == bad


def test_scale_factor_must_be_finite(L):
    st, d = rf.rocfft_plan_description_create()
    assert rf.rocfft_plan_description_set_scale_factor(d, float("nan")) == rf.rocfft_status_invalid_arg_value
    assert rf.rocfft_plan_description_set_scale_factor(d, float("inf")) == rf.rocfft_status_invalid_arg_value
    assert rf.rocfft_plan_description_set_scale_factor(d, 0.5) == rf.rocfft_status_success
    rf.rocfft_plan_description_destroy(d)


def test_stride_count_must_match_rank(L):
    st, d = rf.rocfft_plan_description_create()
    rf.rocfft_plan_description_set_data_layout(d, rf.rocfft_array_type_complex_interleaved,
                                               rf.rocfft_array_type_complex_interleaved, None, None, [1, 8, 64], 0,
                                               None, 0)
    st, p = rf.rocfft_plan_create(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward,
                                  rf.rocfft_precision_single, [8, 8], 1, d)
    assert st == rf.rocfft_status_invalid_strides
    rf.rocfft_plan_destroy(p)
    rf.rocfft_plan_description_destroy(d)


def test_execution_info_contract(L):
    st, info = rf.rocfft_execution_info_create()
    assert st == rf.rocfft_status_success
    assert rf.rocfft_execution_info_set_work_buffer(info, 0, 128) == rf.rocfft_status_invalid_work_buffer
    one = ctypes.c_void_p(0)
    arr = (ctypes.c_void_p * 1)(one)
    assert L.rocfft_execution_info_set_load_callback(info, arr, arr, 16) == rf.rocfft_status_invalid_arg_value
    assert L.rocfft_execution_info_set_store_callback(info, arr, arr, 0) == rf.rocfft_status_success
    assert rf.rocfft_execution_info_destroy(info) == rf.rocfft_status_success
    assert rf.rocfft_execution_info_destroy(None) == rf.rocfft_status_success
    assert rf.rocfft_plan_description_destroy(None) == rf.rocfft_status_success
    assert L.rocfft_execute(None, None, None, None) == rf.rocfft_status_failure


def test_cache_exports_are_inert(L):
    buf = ctypes.c_void_p()
    n = ctypes.c_size_t(123)
    assert L.rocfft_cache_serialize(ctypes.byref(buf), ctypes.byref(n)) == rf.rocfft_status_success
    assert n.value == 0
    assert L.rocfft_cache_deserialize(buf, 0) == rf.rocfft_status_success
    assert L.rocfft_cache_buffer_free(buf) == rf.rocfft_status_success


def test_planner_choices_for_benchmark_configs(L, monkeypatch):
    # config 1: one row kernel, no work buffer
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [4096], 16384)
    text = describe(L, p)
    assert "steps: 1" in text and "len4096" in text and p.work_bytes == 0
    # config 3: rows and columns of every image in one kernel that keeps the intermediate in L2; no work buffer
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [1024, 1024], 64)
    text = describe(L, p)
    assert "steps: 1" in text and "fft2d_l2_dp_1024x1024" in text and p.work_bytes == 0
    # config 5: three passes (rows in place, then the TMA-fed column kernel twice), no transposes; the slowest
    # dimension (rows 8 MB apart) goes out of the caller's array into one volume of work space and the middle
    # dimension comes back from there; in single precision the fused kernel is opt-in (measured: no gain)
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1024], 1)
    text = describe(L, p)
    assert "steps: 3" in text and text.count("col_tma") == 2 and p.work_bytes == 8 * 1024 ** 3
    assert "in+0 -> temp+0" in text and "temp+0 -> in+0" in text
    # with the work-array plan switched off: three in-place passes, no work buffer
    monkeypatch.setenv("ROCFFT_B200_NO_LONG_PITCH_PLAN", "1")
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1024], 1)
    text = describe(L, p)
    assert "steps: 3" in text and text.count("col_tma") == 2 and p.work_bytes == 0
    monkeypatch.delenv("ROCFFT_B200_NO_LONG_PITCH_PLAN")
    # the work-array plan is for rows 4 MB or more apart along the slowest dimension of interleaved 3D volumes only
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 1, [512, 512, 512], 1)
    assert p.work_bytes == 512 ** 3 * 16 and "temp+0" in describe(L, p)          # double precision: 4 MB pitch
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [512, 512, 512], 1)
    assert p.work_bytes == 0                                                       # single precision: 2 MB pitch
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1024], 1,
                in_array_type=rf.rocfft_array_type_complex_planar, out_array_type=rf.rocfft_array_type_complex_planar)
    assert "temp+0" not in describe(L, p)                                          # planar: column kernels of the general kind
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1000], 1)
    assert "temp+0" not in describe(L, p)                                          # 1000 has no TMA-fed column kernel
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 512, 256], 3)
    assert p.work_bytes == 3 * 1024 * 512 * 256 * 8                                # batches: one work volume per transform
    monkeypatch.setenv("ROCFFT_B200_2D_L2", "1")
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1024], 1)
    text = describe(L, p)
    assert "steps: 2" in text and "fft2d_l2_sp_1024x1024" in text and "col_tma" in text and p.work_bytes == 0
    monkeypatch.delenv("ROCFFT_B200_2D_L2")
    # without the fused kernel: a row pass and in-place column passes
    monkeypatch.setenv("ROCFFT_B200_NO_2D_L2", "1")
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [1024, 1024], 64)
    text = describe(L, p)
    assert "steps: 2" in text and "col" in text and p.work_bytes == 0
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024, 1024, 1024], 1)
    assert "steps: 3" in describe(L, p) and p.work_bytes == 8 * 1024 ** 3
    monkeypatch.delenv("ROCFFT_B200_NO_2D_L2")
    # a single image is not worth the interleaved schedule
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 1, [1024, 1024], 1)
    assert "steps: 2" in describe(L, p)
    # config 4: prime length goes through the single-kernel Bluestein with M = 20480 = 20 x 1024, one warp per row
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [10007], 4096)
    text = describe(L, p)
    assert "steps: 1" in text and "len20480_row_blue_rc" in text and p.work_bytes == 0
    # ... other lengths pick the smallest padded length of whole 1024-point rows the same way (double precision up to
    # 12 rows: primes up to 6144 in one kernel, longer ones through the multi-kernel path); short lengths and
    # switched-off plans keep the three-pass kernel
    for n, m in ((3001, 6144), (4099, 10240), (6007, 12288), (8191, 16384)):
        p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [n], 8)
        assert f"fft_sp_len{m}_row_blue_rc" in describe(L, p), (n, describe(L, p))
    for n, m in ((3001, 6144), (4099, 10240), (6143, 12288)):
        p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [n], 8)
        assert f"fft_dp_len{m}_row_blue_rc" in describe(L, p) and p.work_bytes == 0, (n, describe(L, p))
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [6151], 8)
    assert "bluestein_pad_mul" in describe(L, p)
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 1, [1021], 8)
    assert "row_blue" in describe(L, p) and "row_blue_rc" not in describe(L, p)
    monkeypatch.setenv("ROCFFT_B200_NO_BLUE_RC", "1")
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [10007], 4096)
    assert "len20480_row_blue " in describe(L, p) + " " and "row_blue_rc" not in describe(L, p)
    monkeypatch.delenv("ROCFFT_B200_NO_BLUE_RC")
    # a prime too long for one CTA's shared memory takes the multi-kernel Bluestein path
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_complex_forward, 0, [100003], 4)
    assert "bluestein_pad_mul" in describe(L, p) and p.work_bytes > 0
    # config 2: even-length real transforms are one fused kernel each way
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_forward, 0, [1000], 65536)
    text = describe(L, p)
    assert "steps: 1" in text and "len500_row_r2c" in text and p.work_bytes == 0
    p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_inverse, 0, [1000], 65536)
    assert "len500_row_c2r" in describe(L, p)


def test_stacked_twiddle_table_matches_pass_model(L):
    """Runs the Stockham pass structure the kernels implement (see
    stockham_engine.cuh) in numpy with the library's own twiddle table and
    compares with the oracle: validates table layout and index arithmetic."""
    from oracle import fft_oracle as orc
    L.b200fft_stacked_twiddles.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int,
                                           ctypes.c_void_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]
    for n, factors in [(4096, [16, 16, 16]), (1000, [10, 10, 10]), (500, [10, 10, 5]), (60, [5, 4, 3]), (16, [16])]:
        fa = (ctypes.c_int * len(factors))(*factors)
        need = ctypes.c_size_t()
        L.b200fft_stacked_twiddles(n, fa, len(factors), 1, None, 0, ctypes.byref(need))
        tab = np.empty(need.value // 16, dtype=np.complex128)
        L.b200fft_stacked_twiddles(n, fa, len(factors), 1, tab.ctypes.data, need.value, ctypes.byref(need))
        x = orc.uniform_input((n,), np.complex128, seed=n)
        cur = x.copy()
        ch, off = 1, 0
        for p, w in enumerate(factors):
            nb = n // w
            nxt = np.empty_like(cur)
            for b in range(nb):
                v = cur[b + np.arange(w) * nb].copy()
                k = b % ch
                if p > 0:
                    for j in range(1, w):
                        v[j] *= tab[off + (j - 1) * ch + k]
                V = np.fft.fft(v)
                base = (b // ch) * w * ch + k
                nxt[base + np.arange(w) * ch] = V
            if p > 0:
                off += (w - 1) * ch
            ch *= w
            cur = nxt
        ref = orc.c2c(x[None, :], -1)[0]
        assert np.max(np.abs(cur - ref)) < 1e-11 * np.max(np.abs(ref)), (n, factors)


def test_log_layers_write_trace_bench_and_plan_files(tmp_path):
    """ROCFFT_LAYER bits 1 (trace), 2 (bench: an equivalent rocfft-bench command line) and 8 (plan)
    write to the files named by ROCFFT_LOG_*_PATH (reference: library/src/auxiliary.cpp:83-137,
    library/src/plan.cpp:698-726)."""
    import subprocess
    import sys
    env = dict(os.environ, ROCFFT_LAYER="11", ROCFFT_LOG_TRACE_PATH=str(tmp_path / "trace.log"),
               ROCFFT_LOG_BENCH_PATH=str(tmp_path / "bench.log"), ROCFFT_LOG_PLAN_PATH=str(tmp_path / "plan.log"))
    code = ("import rocfft_b200 as rf; rf.rocfft_setup();"
            "p = rf.Plan(rf.rocfft_placement_notinplace, rf.rocfft_transform_type_real_forward, 0, [1000, 30], 16);"
            "p.destroy(); rf.rocfft_cleanup()")
    r = subprocess.run([sys.executable, "-c", code], env=env, cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    bench = (tmp_path / "bench.log").read_text().strip()
    assert bench == ("rocfft-bench --length 30 1000 -b 16 -o -t 2 --precision single --itype 2 --otype 3 "
                     "--istride 1000 1 --ostride 501 1 --idist 30000 --odist 15030 --ioffset 0 0 --ooffset 0 0")
    trace = (tmp_path / "trace.log").read_text()
    assert "rocfft_plan_create" in trace and "rocfft_plan_destroy" in trace
    assert "len500_row_r2c" in (tmp_path / "plan.log").read_text()


def test_small_2d_transforms_use_one_fused_kernel(L):
    """64 x 64 (and 64 x 64 x n: the two fastest dimensions) plan as one fused 2D kernel; a pair outside
    the pool plans as two passes."""
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [64, 64], 10)
    text = p.describe()
    assert "fft2d_sp_64x64" in text and text.count("  [") == 1, text
    p.destroy()
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 1, [27, 27, 5], 2)
    text = p.describe()
    assert "fft2d_dp_27x27" in text and text.count("  [") == 2, text
    p.destroy()
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [64, 100], 10)
    assert "fft2d" not in p.describe()
    p.destroy()


def test_long_1d_transform_is_two_kernels_with_the_twiddles_fused(L, monkeypatch):
    """n = n1 * n2 beyond the single-kernel lengths: column FFTs, then row FFTs that multiply by W_n^(k1 i2)
    on load and store transposed; the multiply is a pass of its own only on request."""
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [65536], 4)
    text = p.describe()
    assert "steps: 2" in text and "large_twiddle_mul" not in text and "row_tout" in text, text
    p.destroy()
    monkeypatch.setenv("ROCFFT_B200_NO_FUSED_LARGE_TWIDDLE", "1")
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [65536], 4)
    assert "steps: 3" in p.describe() and "large_twiddle_mul" in p.describe()
    p.destroy()
