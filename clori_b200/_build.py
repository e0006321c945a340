"""Builds libyvex_b200.so in-tree: CUDA kernels for sm_100a + the C11 host layer.

Run as `python -m clori_b200._build` or through `__graft_entry__.build()`.
nvcc cross-compiles without a GPU. Objects land in clori_b200/csrc/_obj/ and
are rebuilt only when a source or header is newer.

`python -m clori_b200._build --checked` builds libyvex_b200_checked.so beside it: the same
sources with -DYVX_CHECKED, which compiles index checks in front of the kernels' global
stores (a failing check records status 4 and skips the store). Setting the environment
variable YVEX_B200_LIBRARY=checked makes the Python mirror (and so the tests) load it.
"""
import os
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(CSRC, "_obj")
LIB = os.path.join(PKG, "libyvex_b200.so")
INCLUDE = os.path.join(ROOT, "include")

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CC = os.environ.get("CC", "gcc")
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math" if os.environ.get("YVX_FAST_MATH") else "-DYVX_PRECISE_MATH",
    "-Xcompiler", "-fPIC", "-I", INCLUDE, "-I", os.path.join(CSRC, "cuda"),
]
CC_FLAGS = ["-std=c11", "-O2", "-fPIC", "-Wall", "-Wextra", "-D_GNU_SOURCE", "-I", INCLUDE,
            "-I", os.path.join(CSRC, "host")]


def _sources():
    cuda = sorted(f for f in os.listdir(os.path.join(CSRC, "cuda")) if f.endswith(".cu"))
    host = sorted(f for f in os.listdir(os.path.join(CSRC, "host")) if f.endswith(".c"))
    return [os.path.join(CSRC, "cuda", f) for f in cuda], [os.path.join(CSRC, "host", f) for f in host]


def _headers():
    out = []
    for base in (INCLUDE, CSRC):
        for dirpath, _, files in os.walk(base):
            out += [os.path.join(dirpath, f) for f in files if f.endswith((".h", ".cuh"))]
    return out


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(verbose=False, ptxas_info=False, checked=False):
    obj_dir = OBJ + ("_checked" if checked else "")
    lib = LIB.replace(".so", "_checked.so") if checked else LIB
    define = ["-DYVX_CHECKED"] if checked else []
    os.makedirs(obj_dir, exist_ok=True)
    cuda, host = _sources()
    headers = _headers()
    objects = []
    jobs = []
    for src in cuda:
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objects.append(obj)
        if _stale(obj, [src] + headers):
            cmd = [NVCC] + NVCC_FLAGS + define + (["-Xptxas", "-v"] if ptxas_info else []) + ["-c", src, "-o", obj]
            jobs.append((src, cmd))
    for src in host:
        obj = os.path.join(obj_dir, os.path.basename(src) + ".o")
        objects.append(obj)
        if _stale(obj, [src] + headers):
            jobs.append((src, [CC] + CC_FLAGS + define + ["-c", src, "-o", obj]))
    procs = [(src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
             for src, cmd in jobs]
    failed = False
    for src, proc in procs:
        out, _ = proc.communicate()
        if proc.returncode != 0:
            failed = True
            sys.stderr.write(f"--- {src}\n{out}\n")
        elif verbose or ptxas_info:
            sys.stderr.write(out)
    if failed:
        raise RuntimeError("libyvex_b200 build failed")
    if jobs or _stale(lib, objects):
        subprocess.run([NVCC, "-shared", "-o", lib] + objects + ["-lm"], check=True)
    return lib


if __name__ == "__main__":
    print(build(verbose=True, ptxas_info="--ptxas" in sys.argv, checked="--checked" in sys.argv))
