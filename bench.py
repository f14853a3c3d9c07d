#!/usr/bin/env python
"""Benchmark of the FFT hot path through the rocFFT-compatible C API.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...   # CPU baseline arm

Headline workload (every N): the 3D complex-to-complex forward FFT
1024 x 1024 x 1024, fp32 interleaved, in place (8 GiB) — the configuration that
scales over 1/2/4/8 GPUs.  Metric: GFLOP/s = 5 * N * log2(N) / t with
N = 2^30 (the definition rocfft-bench uses, clients/bench/bench.cpp:470-480).
At N = 1 the line also carries, under "configs", the four single-GPU
configurations (batched 1D c2c 4096, real 1000 forward/inverse, 2D fp64
1024x1024, prime-length 10007) with their own GFLOP/s and HBM-roofline
fractions.

One JSON line is printed by rank 0.  Inputs are synthetic: iid uniform
[-0.5, 0.5) per component from a seeded generator.  A scale factor 1/sqrt(N) is
set on the plans so that repeated in-place steps stay finite; it is fused into
the last kernel and removes no work.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import math
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "GFLOP/s (5*N*log2(N)/t), 3D c2c 1024^3 fp32 in-place"
UNIT = "GFLOP/s"


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# --------------------------------------------------------------------------
# clock sampling during the timed region (read-only NVML queries)
# --------------------------------------------------------------------------
class ClockSampler:
    def __init__(self, index=0, period=0.004):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        self.index, self.period = index, period
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4)}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for k, bit in names.items():
                    if r & bit:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._run, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# --------------------------------------------------------------------------
# workloads
# --------------------------------------------------------------------------
def workloads():
    import rocfft_b200 as rf
    F, RF, RI = (rf.rocfft_transform_type_complex_forward, rf.rocfft_transform_type_real_forward,
                 rf.rocfft_transform_type_real_inverse)
    IP, OP = rf.rocfft_placement_inplace, rf.rocfft_placement_notinplace
    lg = math.log2
    return {
        # name: (ttype, placement, precision, lengths, batch, in dtype, in elems, out dtype, out elems, flops)
        "c2c_1d_4096x16384_fp32_ip": dict(tt=F, pl=IP, prec=0, lens=[4096], batch=16384, idt="complex64",
                                          inel=4096 * 16384, odt="complex64", outel=4096 * 16384,
                                          flops=5 * 4096 * 12 * 16384),
        "r2c_1d_1000x65536_fp32": dict(tt=RF, pl=OP, prec=0, lens=[1000], batch=65536, idt="float32",
                                       inel=1000 * 65536, odt="complex64", outel=501 * 65536,
                                       flops=2.5 * 1000 * lg(1000) * 65536),
        "c2r_1d_1000x65536_fp32": dict(tt=RI, pl=OP, prec=0, lens=[1000], batch=65536, idt="complex64",
                                       inel=501 * 65536, odt="float32", outel=1000 * 65536,
                                       flops=2.5 * 1000 * lg(1000) * 65536, hermitian=True),
        "c2c_2d_1024x1024x64_fp64": dict(tt=F, pl=OP, prec=1, lens=[1024, 1024], batch=64, idt="complex128",
                                         inel=64 << 20, odt="complex128", outel=64 << 20,
                                         flops=5 * 2 ** 20 * 20 * 64),
        "c2c_1d_10007x4096_fp32_bluestein": dict(tt=F, pl=OP, prec=0, lens=[10007], batch=4096, idt="complex64",
                                                 inel=10007 * 4096, odt="complex64", outel=10007 * 4096,
                                                 flops=5 * 10007 * lg(10007) * 4096),
        "c2c_3d_1024x1024x1024_fp32_ip": dict(tt=F, pl=IP, prec=0, lens=[1024, 1024, 1024], batch=1,
                                              idt="complex64", inel=1 << 30, odt="complex64", outel=1 << 30,
                                              flops=5 * 2 ** 30 * 30),
    }


HEADLINE = "c2c_3d_1024x1024x1024_fp32_ip"


def _np_dtype(name):
    return np.dtype(name)


def _fill_device(torch, dt, nelem, seed, hermitian_rows=None, on_chunk=None):
    """Seeded uniform [-0.5, 0.5) input generated on the host in chunks (the
    device only receives copies), returned as a flat device tensor.  `on_chunk(first_element, array)`
    sees every chunk (the verification accumulates its sums there)."""
    tdt = {"complex64": torch.complex64, "complex128": torch.complex128, "float32": torch.float32}[dt]
    out = torch.empty(nelem, dtype=tdt, device="cuda")
    rng = np.random.default_rng(seed)
    chunk = 1 << 24
    ndt = _np_dtype(dt)
    for s in range(0, nelem, chunk):
        n = min(chunk, nelem - s)
        if ndt.kind == "c":
            rdt = np.float32 if ndt == np.complex64 else np.float64
            a = np.empty(n, dtype=ndt)
            a.real = rng.random(n, dtype=np.float32 if rdt == np.float32 else np.float64) - 0.5
            a.imag = rng.random(n, dtype=np.float32 if rdt == np.float32 else np.float64) - 0.5
        else:
            a = (rng.random(n, dtype=np.float32) - 0.5).astype(ndt)
        out[s:s + n].copy_(torch.from_numpy(a))
        if on_chunk is not None:
            on_chunk(s, a)
    if hermitian_rows:
        # Hermitian rows need real DC and Nyquist bins to be a valid spectrum
        v = out.view(-1, hermitian_rows)
        v[:, 0] = v[:, 0].real.to(tdt)
        v[:, -1] = v[:, -1].real.to(tdt)
    return out


def run_single_gpu(name, w, steps, warmup, peak, do_e2e=True, e2e_steps=None, sampler=None, verify=True):
    """Runs one workload on the current device; returns a result dict.  With `verify`, the first execute (before
    warm-up) runs on the freshly seeded input and sampled outputs are compared with a double-precision host FFT."""
    import torch
    import rocfft_b200 as rf

    L = rf.lib()
    L.b200fft_launch_count.restype = ctypes.c_ulonglong
    L.b200fft_execute_profiled.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_void_p),
                                           ctypes.POINTER(ctypes.c_void_p), ctypes.c_void_p,
                                           ctypes.POINTER(ctypes.c_float), ctypes.c_size_t,
                                           ctypes.POINTER(ctypes.c_size_t)]
    L.b200fft_plan_describe.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]

    ntot = int(np.prod(w["lens"]))
    ip = w["pl"] == rf.rocfft_placement_inplace
    # unitary scaling keeps repeated steps finite; fused into the last kernel
    scale = 1.0 / math.sqrt(ntot)
    plan = rf.Plan(w["pl"], w["tt"], w["prec"], w["lens"], w["batch"], scale=scale)
    chk3d = None
    if verify and name == HEADLINE:
        nz, ny, nx = w["lens"][2], w["lens"][1], w["lens"][0]
        chk3d = SampledCheck3D((nz, ny, nx), 0, nz)
    x = _fill_device(torch, w["idt"], w["inel"], seed=1, hermitian_rows=(w["lens"][0] // 2 + 1) if w.get("hermitian") else None,
                     on_chunk=(lambda s0, a: chk3d.feed(s0 // (ny * nx), a.reshape(-1, ny, nx))) if chk3d else None)
    y = x if ip else torch.empty(w["outel"], dtype={"complex64": torch.complex64, "complex128": torch.complex128,
                                                    "float32": torch.float32}[w["odt"]], device="cuda")
    work = torch.empty(max(plan.work_bytes, 1), dtype=torch.uint8, device="cuda")
    if plan.work_bytes:
        assert plan.set_work_buffer(work.data_ptr(), plan.work_bytes) == 0
    stream = torch.cuda.Stream()
    plan.set_stream(stream.cuda_stream)
    ins, outs = [x.data_ptr()], (None if ip else [y.data_ptr()])
    in_bytes = w["inel"] * _np_dtype(w["idt"]).itemsize
    out_bytes = w["outel"] * _np_dtype(w["odt"]).itemsize

    def step():
        st = plan.execute(ins, outs)
        if st != 0:
            raise RuntimeError(f"rocfft_execute failed: {st}")

    verdict = None
    if verify:
        per_in, per_out = w["inel"] // w["batch"], w["outel"] // w["batch"]
        if chk3d is None:
            nb = w["batch"]
            want = 3 if len(w["lens"]) > 1 else 520
            idx = sorted(set(np.linspace(0, nb - 1, min(want, nb)).astype(int).tolist() + list(range(max(0, nb - 8), nb))))
            xin = x.view(nb, per_in)[idx].cpu().numpy()  # before the (possibly in-place) execute
        with torch.cuda.stream(stream):
            step()
        stream.synchronize()
        if chk3d is not None:
            verdict = chk3d.finish(y, scale)
        else:
            got = y.view(nb, per_out)[idx].cpu().numpy()
            shp = tuple(reversed(w["lens"]))
            if len(shp) > 1:
                xin, got = xin.reshape((len(idx),) + shp), got.reshape((len(idx),) + shp)
            verdict = verify_batched(w, xin, got, scale)
        if not verdict["ok"]:
            raise SystemExit(f"verification FAILED for {name}: {json.dumps(verdict)}")

    with torch.cuda.stream(stream):
        for _ in range(warmup):
            step()
        stream.synchronize()
        launches0 = L.b200fft_launch_count()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record(stream)
        for _ in range(steps):
            step()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        launches = int(L.b200fft_launch_count() - launches0)

        # per-kernel times for the roofline of the dominant kernel
        ins_a = (ctypes.c_void_p * 1)(ctypes.c_void_p(ins[0]))
        outs_a = (ctypes.c_void_p * 1)(ctypes.c_void_p(outs[0])) if outs else None
        step_ms = (ctypes.c_float * 64)()
        nst = ctypes.c_size_t()
        prof = np.zeros(64)
        reps = 3
        for _ in range(reps):
            st = L.b200fft_execute_profiled(plan.plan, ins_a, outs_a, plan.info, step_ms, 64, ctypes.byref(nst))
            assert st == 0
            prof[:nst.value] += np.array(step_ms[:nst.value])
        prof = prof[:nst.value] / reps
    buf = ctypes.create_string_buffer(1 << 14)
    L.b200fft_plan_describe(plan.plan, buf, len(buf))
    kernel_names = [ln.split("]")[1].split()[0] for ln in buf.value.decode().splitlines() if ln.startswith("  [")]

    res = {
        "workload": name,
        "ms_per_step": ms,
        "gflops": w["flops"] / ms / 1e6,
        "algorithmic_bytes": in_bytes + out_bytes,
        "hbm_gbs": (in_bytes + out_bytes) / ms / 1e6,
        "hbm_frac": (in_bytes + out_bytes) / ms / 1e6 / peak,
        "kernels": [{"name": n, "ms": float(t)} for n, t in zip(kernel_names, prof)],
        "launches_per_step": launches // max(steps, 1),
        "gpu_launches": launches,
        "work_buffer_bytes": plan.work_bytes,
    }
    if verdict is not None:
        res["verify"] = verdict

    if do_e2e:
        # host buffers through the public API: H2D of the input, execute, D2H of the result, every step.
        # Steps are pipelined over two device buffers and three streams: the H2D copy of step i+1 runs while
        # step i executes and step i-1's result travels back (PCIe is full duplex), as a caller with a queue
        # of independent transforms would drive the library.
        k = e2e_steps or steps
        hin = torch.empty(in_bytes, dtype=torch.uint8).pin_memory()
        hin.copy_(x.view(torch.uint8))
        hout = torch.empty(out_bytes, dtype=torch.uint8).pin_memory()
        x2 = torch.empty_like(x)
        y2 = x2 if ip else torch.empty_like(y)
        bufs = [(x, y), (x2, y2)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        free_ev = [None, None]

        def e2e_step(i):
            xi, yi = bufs[i % 2]
            if free_ev[i % 2] is not None:
                s_in.wait_event(free_ev[i % 2])  # the buffer's previous result has left the device
            with torch.cuda.stream(s_in):
                xi.view(torch.uint8).copy_(hin, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(s_in)
            stream.wait_event(ev_in)
            with torch.cuda.stream(stream):
                st = plan.execute([xi.data_ptr()], None if ip else [yi.data_ptr()])
                if st != 0:
                    raise RuntimeError(f"rocfft_execute failed: {st}")
                ev_c = torch.cuda.Event()
                ev_c.record(stream)
            s_out.wait_event(ev_c)
            with torch.cuda.stream(s_out):
                hout.copy_(yi.view(torch.uint8), non_blocking=True)
                ev_o = torch.cuda.Event()
                ev_o.record(s_out)
            free_ev[i % 2] = ev_o

        for i in range(2):
            e2e_step(i)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        e0.record(s_in)
        for i in range(k):
            e2e_step(i)
        e1.record(s_out)
        torch.cuda.synchronize()
        wall = (time.perf_counter() - t0) * 1e3 / k
        ems = e0.elapsed_time(e1) / k
        res["e2e"] = {"value": w["flops"] / ems / 1e6, "unit": UNIT, "ms_per_step": ems, "wall_ms_per_step": wall,
                      "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                      "pipeline": "2 device buffers, 3 streams: H2D of step i+1 overlaps execute of step i and D2H of step i-1"}
        del hin, hout, x2, y2, bufs
    plan.destroy()
    del x, y, work
    torch.cuda.empty_cache()
    return res


# --------------------------------------------------------------------------
# verification (checker only; numpy / scipy in double precision on the host)
# --------------------------------------------------------------------------
EPS = {"f32": 3.75e-5, "f64": 1e-15}  # rocfft-test's type epsilons (clients/tests/gtest_main.cpp:555-557)


def accuracy_bounds(linf_diff, l2_diff_sq, linf_ref, l2_ref_sq, eps, total_length):
    """rocfft-test's two bounds (shared/accuracy_test.h:1497-1498, 1609-1619) on accumulated norms."""
    n = max(int(total_length), 2)
    cut_linf = eps * linf_ref * math.log(n)
    cut_l2 = eps * math.sqrt(math.log2(n))
    l2rel = math.sqrt(l2_diff_sq / l2_ref_sq) if l2_ref_sq > 0 else math.sqrt(l2_diff_sq)
    ok = bool(np.isfinite(linf_diff) and np.isfinite(l2rel) and linf_diff <= cut_linf and l2rel < cut_l2)
    return {"ok": ok, "linf": float(linf_diff), "l2rel": float(l2rel), "cut_linf": float(cut_linf),
            "cut_l2": float(cut_l2)}


class _Norms:
    def __init__(self):
        self.linf_d = self.linf_r = self.l2_d = self.l2_r = 0.0

    def add(self, got, ref):
        g = np.ascontiguousarray(got).astype(np.complex128).view(np.float64)
        r = np.ascontiguousarray(ref).astype(np.complex128).view(np.float64)
        if not np.all(np.isfinite(g)):
            self.linf_d = float("inf")
            return
        d = g - r
        self.linf_d = max(self.linf_d, float(np.max(np.abs(d))))
        self.linf_r = max(self.linf_r, float(np.max(np.abs(r))))
        self.l2_d += float(np.dot(d.ravel(), d.ravel()))
        self.l2_r += float(np.dot(r.ravel(), r.ravel()))

    def vector(self):
        return [self.linf_d, self.linf_r, self.l2_d, self.l2_r]


class SampledCheck3D:
    """Double-precision spot check of a forward 3D c2c transform whose input is split into Z-slabs.

    The whole output is never recomputed on the host.  While the seeded input is
    generated (chunks of whole XY planes), every rank accumulates in complex128
      * for each sampled output plane kz:  P_kz[y,x] += x[z,y,x] exp(-2 pi i z kz / nz)   (partial over its own z),
      * for each sampled output line (ky,kx):  s[z] = sum_{y,x} x[z,y,x] exp(-2 pi i (y ky/ny + x kx/nx)).
    After a sum of the partial planes over the ranks, a 2D FFT of P_kz is the output plane X[kz,:,:]; after a
    gather of s over the ranks, a 1D FFT of s is the output line X[:,ky,kx].  Both are compared with the
    device result under rocfft-test's Linf / L2 bounds, evaluated over the sampled values (every rank owns
    one sampled plane and a segment of every sampled line)."""

    def __init__(self, n, z0, lz, world=1, rank=0):
        self.nz, self.ny, self.nx = n
        self.z0, self.lz, self.world, self.rank = z0, lz, world, rank
        slab = self.nz // world
        self.kz = [r * slab + (37 * r + 5) % slab for r in range(world)]
        if world == 1:
            self.kz.append((self.nz * 2) // 3 + 1)
        self.lines = [(3, 1000 % self.nx), (self.ny // 2, self.nx // 2 + 1), (self.ny - 1, 0), (0, 7 % self.nx)]
        self.planes = np.zeros((len(self.kz), self.ny * self.nx), dtype=np.complex128)
        self.s = np.zeros((lz, len(self.lines)), dtype=np.complex128)
        ky = np.array([p[0] for p in self.lines])
        kx = np.array([p[1] for p in self.lines])
        self.wy = np.exp(-2j * np.pi * (np.outer(np.arange(self.ny), ky) % self.ny) / self.ny)  # [y, p]
        self.wx = np.exp(-2j * np.pi * (np.outer(np.arange(self.nx), kx) % self.nx) / self.nx)  # [x, p]

    def feed(self, zstart, chunk):
        """chunk: complex64 numpy array of whole planes, shape (nzc, ny, nx); zstart = global z of its first plane."""
        nzc = chunk.shape[0]
        c = chunk.reshape(nzc, -1).astype(np.complex128)
        z = np.arange(zstart, zstart + nzc)
        w = np.exp(-2j * np.pi * (np.outer(np.array(self.kz), z) % self.nz) / self.nz)  # [k, z]
        self.planes += w @ c
        v = (c.reshape(nzc * self.ny, self.nx) @ self.wx).reshape(nzc, self.ny, -1)
        self.s[zstart - self.z0: zstart - self.z0 + nzc] = (v * self.wy[None]).sum(axis=1)

    def finish(self, out_slab, scale, dist=None, torch=None):
        """out_slab: this rank's output, device tensor viewable as (lz, ny, nx) complex64.  Collective when dist is given."""
        import scipy.fft as sfft
        planes, s_all = self.planes, self.s
        # collectives run where the process group's backend wants its tensors (NCCL: the GPU; gloo: the host)
        dev = "cuda" if (dist is not None and dist.get_backend() == "nccl") else "cpu"
        if dist is not None and self.world > 1:
            t = torch.from_numpy(planes.view(np.float64).copy()).to(dev)
            dist.all_reduce(t)
            planes = t.cpu().numpy().view(np.complex128)
            parts = [torch.empty(self.s.size * 2, dtype=torch.float64, device=dev) for _ in range(self.world)]
            dist.all_gather(parts, torch.from_numpy(self.s.view(np.float64).ravel().copy()).to(dev))
            s_all = np.concatenate([p.cpu().numpy().view(np.complex128).reshape(self.lz, -1) for p in parts], axis=0)
        out = out_slab.view(self.lz, self.ny, self.nx)
        nr = _Norms()
        nsampled = 0
        for i, kz in enumerate(self.kz):
            if self.z0 <= kz < self.z0 + self.lz:
                ref = sfft.fft2(planes[i].reshape(self.ny, self.nx)) * scale
                nr.add(out[kz - self.z0].cpu().numpy(), ref)
                nsampled += ref.size
        ref_lines = sfft.fft(s_all, axis=0) * scale  # [kz, p]
        for p, (ky, kx) in enumerate(self.lines):
            nr.add(out[:, ky, kx].cpu().numpy(), ref_lines[self.z0:self.z0 + self.lz, p])
            nsampled += self.lz
        vec = nr.vector()
        if dist is not None and self.world > 1:
            mx = torch.tensor([vec[0], vec[1]], dtype=torch.float64, device=dev)
            sm = torch.tensor([vec[2], vec[3], float(nsampled)], dtype=torch.float64, device=dev)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
            dist.all_reduce(sm)
            vec = [float(mx[0]), float(mx[1]), float(sm[0]), float(sm[1])]
            nsampled = int(sm[2].item())
        res = accuracy_bounds(vec[0], vec[2], vec[1], vec[3], EPS["f32"], self.nz * self.ny * self.nx)
        res["sampled"] = (f"{len(self.kz)} output XY planes (kz={self.kz}) and {len(self.lines)} output Z lines "
                          f"(ky,kx={self.lines}) recomputed in complex128 from the seeded input; {nsampled} values")
        return res


def verify_batched(w, x_host_rows, got_rows, scale):
    """Sampled transforms of a batched 1D/2D workload against scipy.fft in double precision.
    x_host_rows / got_rows: arrays shaped (nsample, ...) holding the sampled transforms' input and device output."""
    import scipy.fft as sfft
    nd = len(w["lens"])
    axes = tuple(range(1, 1 + nd))
    if w["tt"] == 2:  # real forward
        ref = sfft.rfft(x_host_rows.astype(np.float64), axis=1)
    elif w["tt"] == 3:  # real inverse, unnormalised
        ref = sfft.irfft(x_host_rows.astype(np.complex128), n=w["lens"][0], axis=1, norm="forward")
    else:
        ref = sfft.fftn(x_host_rows.astype(np.complex128), axes=axes)
    ref = ref * scale
    nr = _Norms()
    nr.add(np.asarray(got_rows).astype(np.complex128), ref.astype(np.complex128))
    v = nr.vector()
    res = accuracy_bounds(v[0], v[2], v[1], v[3], EPS["f32" if w["prec"] == 0 else "f64"], int(np.prod(w["lens"])))
    res["sampled"] = f"{x_host_rows.shape[0]} of {w['batch']} transforms, scipy.fft in double precision"
    return res


# --------------------------------------------------------------------------
# CPU arm: pocketfft (scipy.fft) on the host cores
# --------------------------------------------------------------------------
def _mem_available_gib():
    try:
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable:"):
                return int(ln.split()[1]) / (1 << 20)
    except OSError:
        pass
    return 0.0


def cpu_leg_main(reps, warmup):
    """Child process: times scipy.fft.fftn on the FULL 1024^3 complex64 volume (in place where pocketfft allows),
    all host cores, `reps` real repetitions after `warmup`; prints one JSON object."""
    import scipy.fft as sfft
    try:
        os.sched_setaffinity(0, range(os.cpu_count() or 1))
    except (AttributeError, OSError):
        pass
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    flops = 5 * 2 ** 30 * 30
    rng = np.random.default_rng(5)
    # parallel speed-up on a small case, so that a silently single-threaded run cannot pass as `cores` threads
    small = (rng.random((32, 1024, 1024), dtype=np.float32) - 0.5).astype(np.complex64)
    sfft.fft2(small[:2], workers=cores)
    t0 = time.perf_counter(); sfft.fft2(small, workers=1); t1 = time.perf_counter() - t0
    t0 = time.perf_counter(); sfft.fft2(small, workers=cores); tn = time.perf_counter() - t0
    speedup = t1 / tn
    out = {"cores": cores, "parallel_speedup_small": speedup, "mem_available_gib": _mem_available_gib()}
    if out["mem_available_gib"] >= 22.0:
        a = np.empty((1024, 1024, 1024), dtype=np.complex64)
        for z in range(0, 1024, 32):
            a[z:z + 32].real = rng.random((32, 1024, 1024), dtype=np.float32) - 0.5
            a[z:z + 32].imag = rng.random((32, 1024, 1024), dtype=np.float32) - 0.5
        sc = np.float32(1.0 / math.sqrt(2.0 ** 30))
        times = []
        began = time.perf_counter()
        for i in range(warmup + reps):
            t0 = time.perf_counter()
            a = sfft.fftn(a, workers=cores, overwrite_x=True)
            dt = time.perf_counter() - t0
            a *= sc  # keeps repeated transforms finite; outside the timed call
            if i >= warmup:
                times.append(dt)
                if len(times) >= 3 and time.perf_counter() - began > 150.0:
                    break  # bounded run: report the repetitions that really ran
        reps = len(times)
        out.update({"sampled": False, "times_s": times, "ran_steps": reps, "ran_warmup": warmup,
                    "sample": f"full 1024^3 complex64 volume, scipy.fft.fftn(workers={cores}, overwrite_x=True), "
                              f"{reps} timed repetitions after {warmup} warm-up"})
    else:
        planes, cols = 32, 1 << 14
        z = (rng.random((cols, 1024), dtype=np.float32) - 0.5).astype(np.complex64)
        times = []
        for i in range(warmup + reps):
            t0 = time.perf_counter(); sfft.fft2(small, workers=cores); t_xy = (time.perf_counter() - t0) * (1024 / planes)
            t0 = time.perf_counter(); sfft.fft(z, axis=1, workers=cores); t_z = (time.perf_counter() - t0) * ((1 << 20) / cols)
            if i >= warmup:
                times.append(t_xy + t_z)
        out.update({"sampled": True, "times_s": times, "ran_steps": reps, "ran_warmup": warmup,
                    "sample": f"host RAM short ({out['mem_available_gib']:.0f} GiB available): {planes}/1024 XY planes (fft2) + "
                              f"{cols}/1048576 Z lines (fft) in complex64, scaled to the full volume; workers={cores}"})
    med = float(np.median(times))
    out.update({"seconds_median": med, "seconds_best": float(min(times)), "value": flops / med / 1e9,
                "value_best": flops / min(times) / 1e9})
    print("CPU_LEG " + json.dumps(out), flush=True)
    return 0


def cpu_reference_3d(reps, warmup):
    """Runs the CPU leg in a child process whose environment carries no thread limits inherited from a
    launcher (torch.distributed.run exports OMP_NUM_THREADS=1) and whose affinity mask spans every core."""
    import subprocess
    env = {k: v for k, v in os.environ.items()
           if not (k.endswith("_NUM_THREADS") or k in ("OMP_PROC_BIND", "OMP_PLACES", "GOMP_CPU_AFFINITY", "KMP_AFFINITY"))}
    r = subprocess.run([sys.executable, os.path.abspath(__file__), "--cpu-leg", "--steps", str(reps), "--warmup", str(warmup)],
                       capture_output=True, text=True, env=env)
    for ln in r.stdout.splitlines():
        if ln.startswith("CPU_LEG "):
            d = json.loads(ln[8:])
            return {"value": d["value"], "unit": UNIT, "cores": d["cores"], "kind": "port", "sample": d["sample"],
                    "sampled": d["sampled"], "seconds_median": d["seconds_median"], "seconds_best": d["seconds_best"],
                    "value_best": d["value_best"], "ran_steps": d["ran_steps"], "ran_warmup": d["ran_warmup"],
                    "parallel_speedup_small": d["parallel_speedup_small"], "mem_available_gib": d["mem_available_gib"]}
    raise RuntimeError("CPU leg failed: " + r.stderr[-2000:])


def headline_config(world):
    """`config` of the JSON line; both arms print the same object."""
    return {"workload": HEADLINE, "lengths": [1024, 1024, 1024], "batch": 1, "placement": "inplace",
            "decomposition": "single GPU" if world == 1 else f"z-slabs x{world}",
            "scale_factor": "1/sqrt(N) (fused, keeps repeated steps finite)",
            "l2": "input 8 GiB >> 126 MB L2, no flush needed"}


def traffic_ratios():
    """DRAM bytes per algorithmic byte of each kernel, taken from the ncu captures summarised under profiles/."""
    try:
        return json.load(open(os.path.join(ROOT, "profiles", "dram_traffic_ratios.json")))["kernels"]
    except (OSError, KeyError, ValueError):
        return {}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-detail", action="store_true", help="skip the four single-GPU configurations")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-verify", action="store_true")
    ap.add_argument("--cpu-leg", action="store_true", help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.cpu_leg:
        return cpu_leg_main(args.steps, args.warmup)
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    peak, peak_src = measured_peak_gbs()

    if args.impl == "reference":
        # the CPU arm: rank 0 alone transforms the full volume on the host cores; the other ranks leave at once
        if rank != 0:
            return 0
        t0 = time.perf_counter()
        cb = cpu_reference_3d(args.steps, args.warmup)
        line = {"impl": "reference", "metric": METRIC, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": cb["ran_steps"], "warmup": cb["ran_warmup"], "ms_per_step": cb["seconds_median"] * 1e3,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": headline_config(max(world, args.gpus)),
                "cpu_baseline": cb,
                "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0, "wall_s": time.perf_counter() - t0}
        print(json.dumps(line))
        return 0

    import torch
    import rocfft_b200 as rf
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: there is no CPU fallback")
    if not os.path.exists(rf.LIB_PATH):
        raise SystemExit(f"{rf.LIB_PATH} missing: run `python -m rocfft_b200.build` first")
    assert rf.rocfft_setup() == 0

    if world > 1 or args.gpus > 1:
        from rocfft_b200 import distributed as dist_fft
        return dist_fft.bench_main(args, METRIC, UNIT, HEADLINE, peak, peak_src)

    torch.cuda.set_device(0)
    W = workloads()
    with ClockSampler(0) as cs:
        head = run_single_gpu(HEADLINE, W[HEADLINE], args.steps, args.warmup, peak, do_e2e=False,
                              verify=not args.no_verify)
    clocks = cs.summary()
    if not args.no_e2e:
        e2e = run_single_gpu(HEADLINE, W[HEADLINE], 2, 1, peak, do_e2e=True, e2e_steps=max(4, min(args.steps, 10)),
                             verify=False)["e2e"]
    else:
        e2e = None
    detail = []
    if not args.no_detail:
        for name in W:
            if name == HEADLINE:
                continue
            r = run_single_gpu(name, W[name], max(args.steps, 10), args.warmup, peak, do_e2e=not args.no_e2e,
                               e2e_steps=10, verify=not args.no_verify)
            detail.append(r)

    dom = max(head["kernels"], key=lambda k: k["ms"])
    per_launch_bytes = 2 * (1 << 30) * 8  # each pass reads and writes the whole 8 GiB array
    tr = traffic_ratios().get(dom["name"])
    traffic = tr["dram_bytes"] / tr["algorithmic_bytes"] * per_launch_bytes if tr else None
    roof = {"bound": "hbm", "kernel": dom["name"], "achieved": per_launch_bytes / dom["ms"] / 1e6, "peak": peak,
            "peak_source": peak_src, "unit": "GB/s", "frac": per_launch_bytes / dom["ms"] / 1e6 / peak,
            "traffic": traffic,
            "traffic_source": (f"ncu dram bytes of a smaller launch of this kernel ({tr['source']}), scaled by volume"
                               if tr else None),
            "kernel_ms": dom["ms"],
            "whole_transform": {"algorithmic_bytes": head["algorithmic_bytes"], "achieved": head["hbm_gbs"],
                                "frac": head["hbm_frac"]}}
    # the four single-GPU configurations, with the bound that applies to each
    cfgs = []
    for r in detail:
        c = {"workload": r["workload"], "ms": r["ms_per_step"], "gflops": r["gflops"], "hbm_gbs": r["hbm_gbs"],
             "hbm_frac": r["hbm_frac"], "kernels": r["kernels"], "bound": "hbm",
             "verify_ok": r.get("verify", {}).get("ok")}
        if "bluestein" in r["workload"]:
            # two 20480-point FFTs per 10007-point row: ~ 2 * 5 * M * log2(M) flop with M = 20480 per row
            m = 20480
            flop = 2 * 5 * m * math.log2(m) * 4096
            c["bound"] = "fp32 issue"
            c["arithmetic_ms_at_fma_peak"] = flop / 74e12 * 1e3
            c["note"] = ("Bluestein with M = 20480 does ~4.4x the conventional flop count; the arithmetic alone exceeds the "
                         "HBM time of the algorithmic bytes, so the HBM fraction is reported for context only")
        cfgs.append(c)
    if cfgs:
        roof["configs"] = cfgs
    line = {"metric": METRIC, "value": head["gflops"], "unit": UNIT, "n_gpus": 1, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": headline_config(1),
            "roofline": roof, "clocks": clocks, "gpu_launches": head["gpu_launches"],
            "kernels": head["kernels"]}
    if "verify" in head:
        line["verify"] = head["verify"]
    if e2e:
        line["e2e"] = e2e
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_reference_3d(3, 1)
    if detail:
        line["configs"] = detail
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
