"""Build libosmos_b200.so: the sm_100a kernels and the C host code behind the C ABI of include/osmos_b200/.

    python -m libosmos_b200.build            # build if sources are newer than the library
    python -m libosmos_b200.build --force

nvcc cross-compiles without a GPU. The codebook tables are generated from the installed gguf package first
(csrc/gen_grids.py); the generated header and every built file are kept out of version control.
"""
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
GEN = os.path.join(CSRC, "_gen")
OBJ = os.path.join(HERE, "_obj")
LIB = os.path.join(HERE, "libosmos_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "--fmad=false", "-std=c++17",
              "--extended-lambda", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-I" + GEN]
CC_FLAGS = ["-O2", "-ffp-contract=off", "-fPIC", "-Wall", "-Wextra", "-I" + os.path.join(ROOT, "include")]


def _newer(src_list, target):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in src_list)


def sources():
    cu = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    c = sorted(os.path.join(HOST, f) for f in os.listdir(HOST) if f.endswith(".c"))
    return cu, c


def headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h", ".py"))]
    inc = os.path.join(ROOT, "include", "osmos_b200")
    hs += [os.path.join(inc, f) for f in os.listdir(inc)]
    return hs


def build(force=False, verbose=False, jobs=8):
    os.makedirs(GEN, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    grids = os.path.join(GEN, "osmos_grids.h")
    if force or _newer([os.path.join(CSRC, "gen_grids.py")], grids):
        subprocess.check_call([sys.executable, os.path.join(CSRC, "gen_grids.py"), grids])
    cu, c = sources()
    deps = headers() + [grids]
    objs, procs = [], []
    for src in cu + c:
        obj = os.path.join(OBJ, os.path.basename(src) + ".o")
        objs.append(obj)
        if not (force or _newer([src] + deps, obj)):
            continue
        if src.endswith(".cu"):
            cmd = ["nvcc"] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        else:
            cmd = ["gcc"] + CC_FLAGS + ["-c", src, "-o", obj]
        log = tempfile.TemporaryFile(mode="w+")  # (a file, not a pipe: a compiler that prints much never blocks on us)
        procs.append((src, subprocess.Popen(cmd, stdout=log, stderr=subprocess.STDOUT, text=True), log))
        while len([p for _, p, _ in procs if p.poll() is None]) >= jobs:
            [p.wait() for _, p, _ in procs if p.poll() is None][:1]
    failed = False
    for src, p, log in procs:
        p.wait()
        log.seek(0)
        out = log.read()
        log.close()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (src, out))
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("libosmos_b200: compilation failed")
    if force or procs or _newer(objs, LIB):
        subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", LIB] + objs)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
