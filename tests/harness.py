"""Accuracy-test harness: drives the library through its C API the way
rocfft-test drives rocFFT (reference: shared/accuracy_test.h:881-1631,
shared/rocfft_params.h:341-503), and compares against the CPU oracle.

For one `Case` it
  1. works out default strides / distances like the library must
     (reference rule: library/src/plan.cpp:87-197),
  2. builds seeded input in a logical array, scatters it into strided device
     buffers whose every other byte holds a canary,
  3. creates description -> plan -> info, supplies a work buffer, executes,
  4. gathers the output layout and checks it against the oracle with
     rocfft-test's Linf / L2 bounds, and checks that no byte outside the output
     layout changed (reference: shared/accuracy_test.h:611-682).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

import rocfft_b200 as rf
from oracle import fft_oracle as orc

C2C_FWD = rf.rocfft_transform_type_complex_forward
C2C_INV = rf.rocfft_transform_type_complex_inverse
R2C = rf.rocfft_transform_type_real_forward
C2R = rf.rocfft_transform_type_real_inverse
IP = rf.rocfft_placement_inplace
OOP = rf.rocfft_placement_notinplace
CI = rf.rocfft_array_type_complex_interleaved
CP = rf.rocfft_array_type_complex_planar
RE = rf.rocfft_array_type_real
HI = rf.rocfft_array_type_hermitian_interleaved
HP = rf.rocfft_array_type_hermitian_planar

CANARY = 0xCD


@dataclass
class Case:
    ttype: int
    precision: str  # "single" | "double"
    lengths: Sequence[int]  # rocFFT order, fastest first; real lengths for real transforms
    batch: int = 1
    placement: int = OOP
    in_type: Optional[int] = None
    out_type: Optional[int] = None
    in_strides: Optional[Sequence[int]] = None
    out_strides: Optional[Sequence[int]] = None
    in_dist: int = 0
    out_dist: int = 0
    in_offsets: Optional[Sequence[int]] = None
    out_offsets: Optional[Sequence[int]] = None
    scale: Optional[float] = None
    seed: int = 1
    user_work_buffer: bool = True

    def ident(self) -> str:
        t = {C2C_FWD: "c2cf", C2C_INV: "c2ci", R2C: "r2c", C2R: "c2r"}[self.ttype]
        s = f"{t}_{self.precision[0]}p_len{'x'.join(map(str, self.lengths))}_b{self.batch}_{'ip' if self.placement == IP else 'op'}"
        if self.in_type is not None or self.out_type is not None:
            s += f"_t{self.in_type}{self.out_type}"
        if self.in_strides is not None:
            s += "_is" + "x".join(map(str, self.in_strides))
        if self.out_strides is not None:
            s += "_os" + "x".join(map(str, self.out_strides))
        if self.in_dist or self.out_dist:
            s += f"_d{self.in_dist}x{self.out_dist}"
        if self.in_offsets or self.out_offsets:
            s += "_off"
        if self.scale is not None:
            s += "_sc"
        return s


def _is_planar(t):
    return t in (CP, HP)


def resolve_layout(case: Case):
    """Returns (in_type, out_type, in_len, out_len, in_layout, out_layout) with
    every default filled in."""
    real = case.ttype in (R2C, C2R)
    L = list(case.lengths)
    herm = list(L)
    if real:
        herm[0] = L[0] // 2 + 1
    if case.ttype == R2C:
        ilen, olen = L, herm
        dit, dot = RE, HI
    elif case.ttype == C2R:
        ilen, olen = herm, L
        dit, dot = HI, RE
    else:
        ilen, olen = L, L
        dit, dot = CI, CI
    it = dit if case.in_type is None else case.in_type
    ot = dot if case.out_type is None else case.out_type
    rank = len(L)
    ip = case.placement == IP

    if case.in_strides is not None:
        istr = list(case.in_strides)
    else:
        istr = [1]
        if case.ttype == R2C and ip:
            d = 2 * olen[0]
            for i in range(1, rank):
                istr.append(d)
                d *= ilen[i]
        else:
            for i in range(1, rank):
                istr.append(ilen[i - 1] * istr[i - 1])
    if case.out_strides is not None:
        ostr = list(case.out_strides)
    else:
        ostr = [1]
        if case.ttype == C2R and ip:
            d = 2 * ilen[0]
            for i in range(1, rank):
                ostr.append(d)
                d *= ilen[i]
        else:
            for i in range(1, rank):
                ostr.append(olen[i - 1] * ostr[i - 1])
    idist = case.in_dist
    if idist == 0:
        if case.ttype == R2C and rank == 1 and ip:
            idist = 2 * (ilen[0] // 2 + 1) * istr[0]
        else:
            idist = ilen[rank - 1] * istr[rank - 1]
    odist = case.out_dist
    if odist == 0:
        if case.ttype == C2R and rank == 1 and ip:
            odist = 2 * ilen[0] * ostr[0]
        else:
            odist = olen[rank - 1] * ostr[rank - 1]
    ioff = list(case.in_offsets) if case.in_offsets else [0, 0]
    ooff = list(case.out_offsets) if case.out_offsets else [0, 0]
    if len(ioff) == 1:
        ioff.append(0)
    if len(ooff) == 1:
        ooff.append(0)
    ilay = [orc.Layout(tuple(ilen), tuple(istr), idist, case.batch, ioff[k]) for k in range(2)]
    olay = [orc.Layout(tuple(olen), tuple(ostr), odist, case.batch, ooff[k]) for k in range(2)]
    return it, ot, ilen, olen, ilay, olay


def make_input(case: Case, ilen):
    """Logical input array, shape (batch, len[r-1], ..., len[0])."""
    rdt = np.float32 if case.precision == "single" else np.float64
    cdt = np.complex64 if case.precision == "single" else np.complex128
    shp = (case.batch,) + tuple(reversed(ilen))
    if case.ttype == R2C:
        return orc.uniform_input(shp, rdt, case.seed)
    if case.ttype == C2R:
        return orc.hermitian_input(case.lengths, case.batch, cdt, case.seed)
    return orc.uniform_input(shp, cdt, case.seed)


def reference_output(case: Case, x: np.ndarray) -> np.ndarray:
    if case.ttype == C2C_FWD:
        y = orc.c2c(x, -1)
    elif case.ttype == C2C_INV:
        y = orc.c2c(x, +1)
    elif case.ttype == R2C:
        y = orc.r2c(x)
    else:
        y = orc.c2r(x, case.lengths)
    if case.scale is not None:
        y = y * case.scale
    return y


def _to_device_bytes(torch, host_bytes: np.ndarray):
    t = torch.from_numpy(host_bytes.copy()).cuda()
    return t


def run_case(case: Case, check_canary: bool = True):
    """Executes `case` on the GPU; returns (ok, message)."""
    import torch

    it, ot, ilen, olen, ilay, olay = resolve_layout(case)
    rdt = np.float32 if case.precision == "single" else np.float64
    cdt = np.complex64 if case.precision == "single" else np.complex128
    rsz = np.dtype(rdt).itemsize
    x = make_input(case, ilen)
    ref = reference_output(case, x)

    def host_buffers(atype, lays, values):
        """-> list of (bytes array, elem dtype, layout) per pointer"""
        out = []
        if atype == RE:
            n = lays[0].extent()
            b = np.full(n * rsz, CANARY, dtype=np.uint8)
            if values is not None:
                lays[0].scatter(b.view(rdt), values.astype(rdt))
            out.append((b, rdt, lays[0]))
        elif _is_planar(atype):
            for k in range(2):
                n = lays[k].extent()
                b = np.full(n * rsz, CANARY, dtype=np.uint8)
                if values is not None:
                    part = values.real if k == 0 else values.imag
                    lays[k].scatter(b.view(rdt), part.astype(rdt))
                out.append((b, rdt, lays[k]))
        else:
            n = lays[0].extent()
            b = np.full(n * 2 * rsz, CANARY, dtype=np.uint8)
            if values is not None:
                lays[0].scatter(b.view(cdt), values.astype(cdt))
            out.append((b, cdt, lays[0]))
        return out

    ip = case.placement == IP
    in_host = host_buffers(it, ilay, x)
    if ip:
        # one allocation serves both layouts: make it large enough for either
        out_shape = host_buffers(ot, olay, None)
        merged = []
        for k in range(max(len(in_host), len(out_shape))):
            a = in_host[k][0] if k < len(in_host) else np.zeros(0, np.uint8)
            need = out_shape[k][0].size if k < len(out_shape) else 0
            if a.size < need:
                a = np.concatenate([a, np.full(need - a.size, CANARY, np.uint8)])
            merged.append(a)
        dev_in = [_to_device_bytes(torch, a) for a in merged]
        dev_out = dev_in
        out_meta = out_shape
        before_out = [a.copy() for a in merged]
    else:
        dev_in = [_to_device_bytes(torch, b) for b, _, _ in in_host]
        out_meta = host_buffers(ot, olay, None)
        dev_out = [_to_device_bytes(torch, b) for b, _, _ in out_meta]
        before_out = [b.copy() for b, _, _ in out_meta]

    prec = rf.rocfft_precision_single if case.precision == "single" else rf.rocfft_precision_double
    need_layout = any(v is not None for v in (case.in_type, case.out_type, case.in_strides, case.out_strides,
                                              case.in_offsets, case.out_offsets)) or case.in_dist or case.out_dist
    kw = {}
    if need_layout:
        kw = dict(in_array_type=it, out_array_type=ot,
                  in_offsets=[l.offset for l in ilay][: 2 if _is_planar(it) else 1],
                  out_offsets=[l.offset for l in olay][: 2 if _is_planar(ot) else 1],
                  in_strides=case.in_strides, in_distance=case.in_dist,
                  out_strides=case.out_strides, out_distance=case.out_dist)
    plan = rf.Plan(case.placement, case.ttype, prec, list(case.lengths), case.batch, scale=case.scale, **kw)
    work = None
    if plan.work_bytes and case.user_work_buffer:
        work = torch.empty(plan.work_bytes, dtype=torch.uint8, device="cuda")
        assert plan.set_work_buffer(work.data_ptr(), plan.work_bytes) == rf.rocfft_status_success
    stream = torch.cuda.current_stream().cuda_stream
    plan.set_stream(stream)
    st = plan.execute([t.data_ptr() for t in dev_in], None if ip else [t.data_ptr() for t in dev_out])
    torch.cuda.synchronize()
    if st != rf.rocfft_status_success:
        plan.destroy()
        return False, f"rocfft_execute returned {st}"

    # gather the output
    out_bytes = [t.cpu().numpy() for t in dev_out]
    if ot == RE:
        got = olay[0].gather(out_bytes[0][: (out_bytes[0].size // rsz) * rsz].view(rdt))
    elif _is_planar(ot):
        re = olay[0].gather(out_bytes[0][: (out_bytes[0].size // rsz) * rsz].view(rdt))
        im = olay[1].gather(out_bytes[1][: (out_bytes[1].size // rsz) * rsz].view(rdt))
        got = re + 1j * im
    else:
        csz = 2 * rsz
        got = olay[0].gather(out_bytes[0][: (out_bytes[0].size // csz) * csz].view(cdt))

    total = int(np.prod(case.lengths))
    ok, msg = orc.check_accuracy(got, ref, case.precision, total)

    if ok and check_canary:
        # bytes outside the output layout (and, in place, outside the input layout) must be unchanged
        for k, ob in enumerate(out_bytes):
            isz = rsz if (ot == RE or _is_planar(ot)) else 2 * rsz
            n_el = ob.size // isz
            mask = np.ones(n_el, dtype=bool)
            mask[olay[k].indices().ravel()] = False
            changed = (ob[: n_el * isz].reshape(n_el, isz) != before_out[k][: n_el * isz].reshape(n_el, isz)).any(axis=1)
            if ip:
                # in place: elements of the input layout may legitimately be overwritten
                # only where they coincide with output elements; real transforms reuse
                # padding, so restrict the check to bytes outside both layouts
                isz_in = rsz if (it == RE or _is_planar(it)) else 2 * rsz
                cover = np.zeros(ob.size, dtype=bool)
                idx_in = ilay[k if k < len(ilay) else 0].indices().ravel()
                for j in range(isz_in):
                    cover[idx_in * isz_in + j] = True
                cover_el = cover[: n_el * isz].reshape(n_el, isz).any(axis=1)
                mask &= ~cover_el
            if (changed & mask).any():
                bad = int(np.nonzero(changed & mask)[0][0])
                ok, msg = False, msg + f"; wrote outside the output layout at element {bad} of pointer {k}"
                break
    plan.destroy()
    return ok, msg
