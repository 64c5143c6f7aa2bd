"""Builds libnsa_sm100.so (the C-ABI kernel library) in-tree with nvcc for sm_100a.

    python build.py            # incremental: recompiles sources newer than their objects
    python build.py --force

Objects go to csrc/build/ (csrc/build/f16/ for the IEEE-half build), the libraries to csrc/libnsa_sm100.so and
csrc/libnsa_sm100_f16.so; all are git-ignored build products.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OUT = os.path.join(CSRC, "libnsa_sm100.so")
OUT_F16 = os.path.join(CSRC, "libnsa_sm100_f16.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
         "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _newer(a, b):
    return (not os.path.exists(b)) or os.path.getmtime(a) > os.path.getmtime(b)


def _build_one(out, obj_dir, extra_flags, force, verbose):
    os.makedirs(obj_dir, exist_ok=True)
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    hdr_time = max(os.path.getmtime(h) for h in hdrs)
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max([hdr_time] + [os.path.getmtime(s) for s in srcs]):
        return out  # library is newer than every source: nothing to do (also the case on a box that got a prebuilt .so)
    jobs = []
    objs = []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o")
        objs.append(o)
        if force or _newer(s, o) or hdr_time > os.path.getmtime(o):
            jobs.append((s, o))

    def run(job):
        s, o = job
        r = subprocess.run([NVCC, *FLAGS, *extra_flags, "-c", s, "-o", o], capture_output=True, text=True)
        log = r.stdout + r.stderr
        with open(o[:-2] + ".log", "w") as f:
            f.write(log)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {s}:\n{log}")
        if verbose:
            print(log)
        return s

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for s in ex.map(run, jobs):
                print("compiled", os.path.basename(s), *extra_flags)
    if jobs or not os.path.exists(out):
        r = subprocess.run([NVCC, "-shared", "-o", out, *objs, "-lcudart"], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed:\n" + r.stdout + r.stderr)
        print("linked", out)
    return out


def build(force=False, verbose=False):
    """Both builds of the library: bf16 elements (libnsa_sm100.so) and IEEE half (libnsa_sm100_f16.so, -DNSA_F16)."""
    _build_one(OUT, os.path.join(CSRC, "build"), [], force, verbose)
    _build_one(OUT_F16, os.path.join(CSRC, "build", "f16"), ["-DNSA_F16"], force, verbose)
    return OUT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose="-v" in sys.argv)
