"""Builds lib/libbitsqz_llm.so from csrc/*.cu for sm_100a with nvcc (no GPU needed).

    python bitsqueeze-llm_b200/build.py [--force] [--verbose]

Objects go to build/, the shared library to lib/; both stay out of version control.  The
CUDA runtime is linked statically (nvcc's default), cuRAND dynamically.
"""
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "build")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libbitsqz_llm.so")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
CFLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include")]


def _nvcc():
    return os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force=False, verbose=False):
    os.makedirs(BUILD, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    sources = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".hpp"))]
    headers += [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    headers.append(os.path.abspath(__file__))
    jobs = []
    objs = []
    for src in sources:
        obj = os.path.join(BUILD, src[:-3] + ".o")
        objs.append(obj)
        if force or not _newer(obj, [os.path.join(CSRC, src)] + headers):
            cmd = [_nvcc()] + ARCH + CFLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", os.path.join(CSRC, src), "-o", obj]
            jobs.append(cmd)

    def run(cmd):
        p = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, p.returncode, p.stdout + p.stderr

    with cf.ThreadPoolExecutor(max_workers=max(1, min(8, os.cpu_count() or 1))) as ex:
        for cmd, code, out in ex.map(run, jobs):
            if verbose or code != 0:
                sys.stderr.write(" ".join(cmd) + "\n" + out)
            if code != 0:
                raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or force or not _newer(LIB, objs):
        cmd = [_nvcc()] + ARCH + ["-shared", "-o", LIB] + objs + ["-lcurand", "-lcusolver", "-ldl"]
        code = subprocess.run(cmd, capture_output=True, text=True)
        if code.returncode != 0:
            raise RuntimeError("link failed:\n" + code.stdout + code.stderr)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
