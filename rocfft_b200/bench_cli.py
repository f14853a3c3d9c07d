"""Command-line benchmark with the argument and token conventions of rocfft-bench.

    python -m rocfft_b200.bench_cli --length 1024 1024 -b 64 --precision double -o -N 10
    python -m rocfft_b200.bench_cli --token complex_forward_len_4096_single_ip_batch_16384_istride_1_CI_ostride_1_CI_idist_4096_odist_4096_ioffset_0_0_ooffset_0_0

Reference: clients/bench/bench.cpp:60-150 (options), :383-481 (one warm-up, then N trials timed
with events around rocfft_execute, input regenerated before every trial, GFLOP/s =
batch * k * N * log2(N) / t with k = 5 complex / 2.5 real) and shared/fft_params.h:726-1010
(token grammar).  Lengths, strides and offsets on the command line and in tokens are row-major
(slowest dimension first), as in the reference; the C API takes them fastest first.  The line
written by the bench log layer (ROCFFT_LAYER=2) is a valid argument list for this program.
"""
from __future__ import annotations

import argparse
import math
import sys
from dataclasses import dataclass, field

TRANSFORMS = ["complex_forward", "complex_inverse", "real_forward", "real_inverse"]
ARRAY_TOKENS = {"CI": 0, "CP": 1, "R": 2, "HI": 3, "HP": 4, "UN": 5}
ARRAY_NAMES = {v: k for k, v in ARRAY_TOKENS.items()}
PRECISIONS = {"single": 0, "double": 1, "half": 2}


@dataclass
class Params:
    transform_type: int = 0
    length: list = field(default_factory=list)  # row-major
    precision: str = "single"
    inplace: bool = True
    nbatch: int = 1
    itype: int = 5
    otype: int = 5
    istride: list = field(default_factory=list)
    ostride: list = field(default_factory=list)
    idist: int = 0
    odist: int = 0
    ioffset: list = field(default_factory=lambda: [0, 0])
    ooffset: list = field(default_factory=lambda: [0, 0])
    scale_factor: float = 1.0

    # ---- defaults the reference's client fills in (shared/fft_params.h validate / set_iotypes) ----
    def complete(self):
        real_fwd, real_inv = self.transform_type == 2, self.transform_type == 3
        if self.itype == 5:
            self.itype = 2 if real_fwd else 3 if real_inv else 0
        if self.otype == 5:
            self.otype = 3 if real_fwd else 2 if real_inv else 0
        ilen, olen = list(self.length), list(self.length)
        if real_fwd:
            olen[-1] = olen[-1] // 2 + 1
        if real_inv:
            ilen[-1] = ilen[-1] // 2 + 1

        def contiguous(lens, pad_to=None):
            st, s = [0] * len(lens), 1
            for i in range(len(lens) - 1, -1, -1):
                st[i] = s
                s *= pad_to if (pad_to and i == len(lens) - 1) else lens[i]
            return st, s
        # in-place real transforms share one buffer: real rows are padded to 2 * (n/2 + 1)
        ipad = 2 * olen[-1] if (real_fwd and self.inplace) else None
        opad = 2 * ilen[-1] if (real_inv and self.inplace) else None
        if not self.istride:
            self.istride, d = contiguous(ilen, ipad)
            self.idist = self.idist or d
        if not self.ostride:
            self.ostride, d = contiguous(olen, opad)
            self.odist = self.odist or d
        if not self.idist:
            self.idist = max(s * n for s, n in zip(self.istride, ilen))
        if not self.odist:
            self.odist = max(s * n for s, n in zip(self.ostride, olen))
        self.ilength, self.olength = ilen, olen
        return self

    def token(self):
        t = TRANSFORMS[self.transform_type] + "_len" + "".join(f"_{v}" for v in self.length)
        t += f"_{self.precision}_" + ("ip_" if self.inplace else "op_") + f"batch_{self.nbatch}"
        t += "_istride" + "".join(f"_{v}" for v in self.istride) + "_" + ARRAY_NAMES[self.itype]
        t += "_ostride" + "".join(f"_{v}" for v in self.ostride) + "_" + ARRAY_NAMES[self.otype]
        t += f"_idist_{self.idist}_odist_{self.odist}"
        t += "_ioffset" + "".join(f"_{v}" for v in self.ioffset)
        t += "_ooffset" + "".join(f"_{v}" for v in self.ooffset)
        if self.scale_factor != 1.0:
            t += "_scale"
        return t

    @staticmethod
    def from_token(token):
        w = token.split("_")
        p = Params(ioffset=[], ooffset=[])
        name = "_".join(w[:2])
        if name not in TRANSFORMS:
            raise ValueError(f"bad transform type in token: {name}")
        p.transform_type = TRANSFORMS.index(name)
        i = 2

        def ints(i):
            out = []
            while i < len(w) and w[i].isdigit():
                out.append(int(w[i]))
                i += 1
            return out, i
        if w[i] != "len":
            raise ValueError("token: expected len")
        p.length, i = ints(i + 1)
        if w[i] not in PRECISIONS:
            raise ValueError("token: expected precision")
        p.precision = w[i]
        p.inplace = {"ip": True, "op": False}[w[i + 1]]
        if w[i + 2] != "batch":
            raise ValueError("token: expected batch")
        p.nbatch = int(w[i + 3])
        i += 4
        while i < len(w):
            key = w[i]
            if key in ("istride", "ostride"):
                v, i = ints(i + 1)
                setattr(p, key, v)
                setattr(p, "itype" if key == "istride" else "otype", ARRAY_TOKENS[w[i]])
                i += 1
            elif key in ("idist", "odist"):
                setattr(p, key, int(w[i + 1]))
                i += 2
            elif key in ("ioffset", "ooffset"):
                v, i = ints(i + 1)
                setattr(p, key, v)
            elif key == "scale":
                p.scale_factor = 2.0  # the token only records that a factor is set
                i += 1
            elif key in ("ifield", "ofield", "CB", "multigpu"):
                raise ValueError(f"token feature not supported by this client: {key}")
            else:
                raise ValueError(f"token: unexpected word {key}")
        p.ioffset = p.ioffset or [0, 0]
        p.ooffset = p.ooffset or [0, 0]
        return p


def build_parser():
    ap = argparse.ArgumentParser(prog="rocfft-bench", description="rocfft-bench-compatible client of librocfft (B200)")
    ap.add_argument("--version", action="store_true")
    ap.add_argument("--token", default="")
    ap.add_argument("--double", action="store_true")
    ap.add_argument("-t", "--transformType", type=int, default=0)
    ap.add_argument("--precision", default=None, choices=list(PRECISIONS))
    ap.add_argument("-o", "--notInPlace", action="store_true")
    ap.add_argument("--itype", type=int, default=5)
    ap.add_argument("--otype", type=int, default=5)
    ap.add_argument("--length", type=int, nargs="+")
    ap.add_argument("-b", "--batchSize", type=int, default=1)
    ap.add_argument("--istride", type=int, nargs="*", default=[])
    ap.add_argument("--ostride", type=int, nargs="*", default=[])
    ap.add_argument("--idist", type=int, default=0)
    ap.add_argument("--odist", type=int, default=0)
    ap.add_argument("--ioffset", type=int, nargs="*", default=[0, 0])
    ap.add_argument("--ooffset", type=int, nargs="*", default=[0, 0])
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--verbose", type=int, default=0)
    ap.add_argument("-N", "--ntrial", type=int, default=1)
    ap.add_argument("--scalefactor", type=float, default=1.0)
    return ap


def params_from_args(a):
    if a.token:
        return Params.from_token(a.token)
    if not a.length or not 1 <= len(a.length) <= 3:
        raise ValueError("--length takes one to three values")
    return Params(transform_type=a.transformType, length=list(a.length),
                  precision="double" if a.double else (a.precision or "single"), inplace=not a.notInPlace,
                  nbatch=a.batchSize, itype=a.itype, otype=a.otype, istride=list(a.istride), ostride=list(a.ostride),
                  idist=a.idist, odist=a.odist, ioffset=list(a.ioffset) or [0, 0], ooffset=list(a.ooffset) or [0, 0],
                  scale_factor=a.scalefactor)


def buffer_elems(lens, strides, dist, nbatch, offset):
    return offset + dist * (nbatch - 1) + sum(s * (n - 1) for s, n in zip(strides, lens)) + 1


def main(argv=None):
    a = build_parser().parse_args(argv)
    import rocfft_b200 as rf
    if a.version:
        print("version", rf.rocfft_get_version_string(256)[1])
        return 0
    p = params_from_args(a).complete()
    if p.precision == "half":
        print("half precision is not supported", file=sys.stderr)
        return 1
    print("Token:", p.token())
    import torch
    torch.cuda.set_device(a.device)
    assert rf.rocfft_setup() == 0
    prec = PRECISIONS[p.precision]
    rdt = torch.float32 if prec == 0 else torch.float64
    planar_i, planar_o = p.itype in (1, 4), p.otype in (1, 4)
    placement = rf.rocfft_placement_inplace if p.inplace else rf.rocfft_placement_notinplace
    plan = rf.Plan(placement, p.transform_type, prec, list(reversed(p.length)), p.nbatch, in_array_type=p.itype,
                   out_array_type=p.otype, in_offsets=p.ioffset, out_offsets=p.ooffset,
                   in_strides=list(reversed(p.istride)), in_distance=p.idist, out_strides=list(reversed(p.ostride)),
                   out_distance=p.odist, scale=None if p.scale_factor == 1.0 else p.scale_factor)
    work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
    if plan.work_bytes:
        plan.set_work_buffer(work.data_ptr(), plan.work_bytes)
    # buffers in units of real scalars: complex interleaved elements take two
    ielems = buffer_elems(p.ilength, p.istride, p.idist, p.nbatch, max(p.ioffset))
    oelems = buffer_elems(p.olength, p.ostride, p.odist, p.nbatch, max(p.ooffset))
    iscal = 1 if (p.itype == 2 or planar_i) else 2
    oscal = 1 if (p.otype == 2 or planar_o) else 2
    ibytes, obytes = ielems * iscal * rdt.itemsize, oelems * oscal * rdt.itemsize
    if p.inplace:
        ibytes = obytes = max(ibytes, obytes)
    gen = torch.Generator(device="cuda").manual_seed(1)
    ibuf = [torch.empty(ibytes // rdt.itemsize, dtype=rdt, device="cuda") for _ in range(2 if planar_i else 1)]
    obuf = ibuf if p.inplace else [torch.empty(obytes // rdt.itemsize, dtype=rdt, device="cuda")
                                   for _ in range(2 if planar_o else 1)]
    ins = [t.data_ptr() for t in ibuf]
    outs = None if p.inplace else [t.data_ptr() for t in obuf]

    def fill():
        for t in ibuf:
            t.uniform_(-0.5, 0.5, generator=gen)
    fill()
    st = plan.execute(ins, outs)  # warm-up
    if st != 0:
        print(f"rocfft_execute failed: {st}", file=sys.stderr)
        return 1
    times = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    stream = torch.cuda.current_stream()
    plan.set_stream(stream.cuda_stream)
    for _ in range(max(a.ntrial, 1)):
        fill()  # fresh input every trial, as the reference does, so in-place runs cannot overflow
        e0.record(stream)
        st = plan.execute(ins, outs)
        e1.record(stream)
        e1.synchronize()
        if st != 0:
            print(f"rocfft_execute failed: {st}", file=sys.stderr)
            return 1
        times.append(e0.elapsed_time(e1))
    print("\nExecution gpu time:" + "".join(f" {t:.6g}" for t in times) + " ms")
    tot = math.prod(p.length)
    k = 2.5 if (p.itype == 2 or p.otype == 2) else 5.0
    ops = p.nbatch * k * tot * math.log2(tot)
    print("Execution gflops:  " + "".join(f" {ops / (1e6 * t):.6g}" for t in times))
    plan.destroy()
    rf.rocfft_cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
