"""Builds libmytorch_b200.so for sm_100a with nvcc (no torch, no cmake).

    python mytorch_b200/csrc/build.py [--force] [--verbose]

One object per .cu file (compiled in parallel, rebuilt only when the source or
a header is newer), linked into mytorch_b200/libmytorch_b200.so with the CUDA
runtime linked statically, so the library loads on a machine without a GPU or
driver. NCCL and the driver's tensor-map encoder are looked up at run time.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OUT = os.path.join(PKG, "libmytorch_b200.so")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
         "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def sources():
    return sorted(f for f in os.listdir(HERE) if f.endswith(".cu"))


def build(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    hdrs = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(os.path.dirname(PKG), "include", "mytorch_b200.h"))
    newest_hdr = max(os.path.getmtime(h) for h in hdrs)
    jobs = []
    for src in sources():
        s = os.path.join(HERE, src)
        o = os.path.join(OBJ, src[:-3] + ".o")
        if force or not os.path.exists(o) or os.path.getmtime(o) < max(os.path.getmtime(s), newest_hdr):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([NVCC, *FLAGS, "-c", s, "-o", o], capture_output=True, text=True)
        with open(o + ".log", "w") as fh:
            fh.write(r.stdout + r.stderr)
        return s, r.returncode, r.stdout + r.stderr

    failed = False
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        for s, rc, log in ex.map(compile_one, jobs):
            if rc != 0:
                failed = True
                sys.stderr.write(f"--- {s} failed ---\n{log}\n")
            elif verbose:
                sys.stderr.write(f"--- {s} ---\n{log}\n")
    if failed:
        raise RuntimeError("nvcc failed")
    objs = [os.path.join(OBJ, src[:-3] + ".o") for src in sources()]
    if jobs or not os.path.exists(OUT):
        subprocess.run([NVCC, "-shared", "-o", OUT, *objs, "-cudart", "static", "-ldl", "-lpthread"], check=True)
    return OUT


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
