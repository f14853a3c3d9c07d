"""The plan's device error flag stays clear on healthy runs of the kernels that wait on
hardware barriers (bulk-copy row kernel, cluster column kernel)."""
import numpy as np
import pytest

import rocfft_b200 as rf

pytestmark = pytest.mark.gpu


def test_flag_clear_after_tma_rows_and_cluster_columns(monkeypatch):
    import torch
    assert rf.rocfft_setup() == 0
    rng = np.random.default_rng(11)
    # rows: 1024-point transforms stored back to back -> bulk-copy pipelined kernel
    x = (rng.random((64, 1024)) - 0.5 + 1j * (rng.random((64, 1024)) - 0.5)).astype(np.complex64)
    d = torch.from_numpy(x).cuda()
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024], 64)
    assert "row_tma" in p.describe()
    assert p.execute([d.data_ptr()]) == 0
    assert p.device_error() is False
    ref = np.fft.fft(x.astype(np.complex128), axis=1)
    assert np.linalg.norm(d.cpu().numpy() - ref) / np.linalg.norm(ref) < 5e-6
    p.destroy()
    # columns: 1024-point transforms along the slow dimension of a [1024][64] array -> cluster kernel (opt-in here)
    monkeypatch.setenv("ROCFFT_B200_COLCLUSTER", "1")
    y = (rng.random((1024, 64)) - 0.5 + 1j * (rng.random((1024, 64)) - 0.5)).astype(np.complex64)
    d = torch.from_numpy(y).cuda()
    p = rf.Plan(rf.rocfft_placement_inplace, rf.rocfft_transform_type_complex_forward, 0, [1024], 64,
                in_strides=[64], in_distance=1, out_strides=[64], out_distance=1)
    assert "col_cl" in p.describe()
    assert p.execute([d.data_ptr()]) == 0
    assert p.device_error() is False
    ref = np.fft.fft(y.astype(np.complex128), axis=0)
    assert np.linalg.norm(d.cpu().numpy() - ref) / np.linalg.norm(ref) < 5e-6
    p.destroy()
