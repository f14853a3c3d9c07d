"""Runs one transform a few times through the C API: the command to put under
`ncu` (or to time by hand) when a kernel is profiled on a case smaller than
the benchmark's.

    python -m rocfft_b200.profile_cases --lengths 1024,1024,128 --precision single --type c2c --placement ip --reps 3

Lengths are given fastest first, as in rocfft_plan_create.
"""
from __future__ import annotations

import argparse
import sys

import numpy as np


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--lengths", required=True)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--precision", default="single", choices=["single", "double"])
    ap.add_argument("--type", default="c2c", choices=["c2c", "c2c_inv", "r2c", "c2r"])
    ap.add_argument("--placement", default="ip", choices=["ip", "op"])
    ap.add_argument("--reps", type=int, default=3)
    a = ap.parse_args()

    import torch
    import rocfft_b200 as rf
    assert rf.rocfft_setup() == 0
    lens = [int(v) for v in a.lengths.split(",")]
    prec = 0 if a.precision == "single" else 1
    rdt = torch.float32 if prec == 0 else torch.float64
    cdt = torch.complex64 if prec == 0 else torch.complex128
    tt = {"c2c": rf.rocfft_transform_type_complex_forward, "c2c_inv": rf.rocfft_transform_type_complex_inverse,
          "r2c": rf.rocfft_transform_type_real_forward, "c2r": rf.rocfft_transform_type_real_inverse}[a.type]
    pl = rf.rocfft_placement_inplace if a.placement == "ip" else rf.rocfft_placement_notinplace
    n_real = int(np.prod(lens)) * a.batch
    n_herm = (lens[0] // 2 + 1) * int(np.prod(lens[1:])) * a.batch
    gen = torch.Generator(device="cuda").manual_seed(1)
    if a.type in ("c2c", "c2c_inv"):
        x = torch.view_as_complex(torch.rand((n_real, 2), dtype=rdt, device="cuda", generator=gen) - 0.5)
        y = x if pl == rf.rocfft_placement_inplace else torch.empty_like(x)
    elif a.type == "r2c":
        pad = 2 * n_herm if pl == rf.rocfft_placement_inplace else n_real
        x = torch.rand(pad, dtype=rdt, device="cuda", generator=gen) - 0.5
        y = x if pl == rf.rocfft_placement_inplace else torch.empty(n_herm, dtype=cdt, device="cuda")
    else:
        x = torch.view_as_complex(torch.rand((n_herm, 2), dtype=rdt, device="cuda", generator=gen) - 0.5)
        y = x if pl == rf.rocfft_placement_inplace else torch.empty(n_real, dtype=rdt, device="cuda")
    plan = rf.Plan(pl, tt, prec, lens, a.batch, scale=1.0 / np.sqrt(np.prod(lens)))
    work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
    if plan.work_bytes:
        plan.set_work_buffer(work.data_ptr(), plan.work_bytes)
    plan.set_stream(torch.cuda.current_stream().cuda_stream)
    outs = None if pl == rf.rocfft_placement_inplace else [y.data_ptr()]
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(a.reps + 1)]
    ev[0].record()
    for i in range(a.reps):
        st = plan.execute([x.data_ptr()], outs)
        assert st == 0, st
        ev[i + 1].record()
    torch.cuda.synchronize()
    print("ms per execute:", [round(ev[i].elapsed_time(ev[i + 1]), 4) for i in range(a.reps)])
    plan.destroy()
    return 0


if __name__ == "__main__":
    sys.exit(main())
