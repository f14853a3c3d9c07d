"""Builds librocfft.so in-tree: runs the offline kernel generator, compiles the
generated CUDA for sm_100a with nvcc, compiles the C++ host library and links.

Usage:  python -m rocfft_b200.build [--small] [--jobs N] [--force]

Nothing here needs a GPU (nvcc cross-compiles).  Objects are cached under
rocfft_b200/_obj keyed by a hash of the source text and flags.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import subprocess
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
GEN = os.path.join(CSRC, "generated")
OBJ = os.path.join(HERE, "_obj")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "librocfft.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA, "bin", "nvcc")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v",
              # the pool holds thousands of kernels: compressed fatbins keep the library near 100 MB
              "-Xfatbin", "-compress-all",
              "-I", os.path.join(CSRC, "kernels"), "-I", os.path.join(CSRC, "launch"), "-I", GEN,
              "-I", INCLUDE]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-I", INCLUDE, "-I", os.path.join(CUDA, "include"),
             "-I", os.path.join(CSRC, "launch"), "-I", os.path.join(CSRC, "kernels"), "-Wall"]

HOST_SOURCES = ["api/api.cpp", "plan/planner.cpp", "plan/twiddles.cpp", "plan/execute.cpp", "mgpu/mgpu.cpp", "mgpu/gather_scatter.cpp"]
CUDA_SOURCES = ["launch/elementwise.cu", "launch/noalloc.cu", "launch/brick_copy.cu"]


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    for p in paths:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _deps_text(device_only=False):
    """Headers an object depends on; CUDA sources include nothing from the planner / API / multi-GPU layers."""
    hs = []
    for root, _, files in os.walk(CSRC):
        if os.path.abspath(root).startswith(GEN):
            continue
        if device_only and os.path.basename(root) in ("api", "mgpu", "gen"):
            continue
        for f in files:
            if f.endswith((".h", ".cuh")) and not (device_only and f == "planner_impl.h"):
                hs.append(os.path.join(root, f))
    hs.append(os.path.join(INCLUDE, "rocfft", "rocfft.h"))
    hs.append(os.path.join(INCLUDE, "rocfft_b200_ext.h"))
    return sorted(hs)


def _compile(cmd, src, obj, stamp, log):
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stderr[-4000:]}")
    with open(obj + ".stamp", "w") as f:
        f.write(stamp)
    return src, time.time() - t0


def build(small: bool = False, jobs: int | None = None, force: bool = False, verbose: bool = True) -> str:
    os.makedirs(GEN, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    jobs = jobs or os.cpu_count() or 4
    nfiles = 8 if small else 48

    # 1. generator
    gen_src = [os.path.join(CSRC, "gen", "stockham_gen.cpp"), os.path.join(CSRC, "gen", "butterfly_emit.h")]
    gen_bin = os.path.join(OBJ, "stockham_gen")
    gstamp = _digest(gen_src, f"small={small} nfiles={nfiles}")
    gstamp_file = os.path.join(GEN, ".stamp")
    regen = force or not os.path.exists(gstamp_file) or open(gstamp_file).read() != gstamp
    if regen:
        subprocess.check_call(["g++", "-O1", "-std=c++17", "-o", gen_bin, gen_src[0]])
        for f in os.listdir(GEN):
            if f.startswith("gen_"):
                os.remove(os.path.join(GEN, f))
        cmd = [gen_bin, GEN, "--files", str(nfiles)] + (["--small"] if small else [])
        subprocess.check_call(cmd)
        with open(gstamp_file, "w") as f:
            f.write(gstamp)

    dep_hash_host = _digest(_deps_text())
    dep_hash_dev = _digest(_deps_text(device_only=True))
    tasks = []
    objs = []

    def add(src, cmd_prefix, flags, dep_hash):
        name = os.path.relpath(src, CSRC).replace(os.sep, "_")
        obj = os.path.join(OBJ, name + ".o")
        objs.append(obj)
        stamp = _digest([src], dep_hash + " ".join(flags))
        if not force and os.path.exists(obj) and os.path.exists(obj + ".stamp") \
                and open(obj + ".stamp").read() == stamp:
            return
        cmd = cmd_prefix + flags + ["-c", src, "-o", obj]
        tasks.append((cmd, src, obj, stamp, obj + ".log"))

    gen_cu = sorted(os.path.join(GEN, f) for f in os.listdir(GEN) if f.endswith(".cu"))
    for src in gen_cu + [os.path.join(CSRC, s) for s in CUDA_SOURCES]:
        add(src, [NVCC], NVCC_FLAGS, dep_hash_dev)
    for src in [os.path.join(CSRC, s) for s in HOST_SOURCES] + [os.path.join(GEN, "gen_pool.cpp")]:
        add(src, ["g++"], CXX_FLAGS, dep_hash_host)

    t0 = time.time()
    if tasks:
        with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
            futs = [ex.submit(_compile, *t) for t in tasks]
            for fu in cf.as_completed(futs):
                src, dt = fu.result()
                if verbose:
                    print(f"  compiled {os.path.basename(src)} in {dt:.1f}s", flush=True)
    need_link = bool(tasks) or not os.path.exists(LIB)
    if need_link:
        cmd = [NVCC, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a",
                                                      "-Xlinker", "--no-undefined", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stderr[-4000:])
    if verbose:
        print(f"build: {len(tasks)} objects compiled in {time.time() - t0:.1f}s -> {LIB}", flush=True)
    return LIB


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--small", action="store_true", help="short list of lengths (quick bring-up)")
    ap.add_argument("--jobs", type=int, default=None)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    build(small=a.small, jobs=a.jobs, force=a.force)


if __name__ == "__main__":
    main()
