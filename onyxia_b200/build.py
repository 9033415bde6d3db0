"""Build step: compiles the three shared libraries in-tree.

* ``onyxia_b200/libonyxia_ir.so``   host-only IR (g++)
* ``onyxia_b200/libonyxia_cuda.so`` the backend: host runtime + CUDA kernels for
  sm_100a (nvcc ``-gencode arch=compute_100a,code=sm_100a``)
* ``oracle/libonyxia_ref.so``       the CPU oracle (test infrastructure)

A library is rebuilt when the hash of its sources differs from the stamp
written next to it, so a prebuilt tree copied to another machine is used as is.

Run ``python -m onyxia_b200.build [--force] [--verbose]``.
"""
from __future__ import annotations

import concurrent.futures
import glob
import hashlib
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(ROOT, "build", "obj")

NVCC = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
CXX = "g++"  # the environment's CXX may point at a compiler without OpenMP support files
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
# fast-math stays off: parity with the f64 interpreter needs IEEE division, sqrt and exp.
NVCC_FLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
              "--expt-relaxed-constexpr", "-diag-suppress", "20012"]
NVCC_FLAGS += os.environ.get("ONYXIA_EXTRA_NVCC_FLAGS", "").split()  # developer builds, e.g. -DOX_TRACE
CXX_FLAGS = ["-std=c++17", "-O2", "-fPIC", "-Wall", "-Wextra"]


def _hash(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(os.path.relpath(p, ROOT).encode())
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(target: str, sources) -> bool:
    stamp = target + ".stamp"
    if not os.path.exists(target) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != _hash(sources)


def _stamp(target: str, sources) -> None:
    with open(target + ".stamp", "w") as f:
        f.write(_hash(sources))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: %s\n%s" % (" ".join(cmd), r.stdout))
    if verbose and r.stdout.strip():
        print(r.stdout)
    return r.stdout


def ir_sources():
    return sorted(glob.glob(os.path.join(CSRC, "ir", "*.cpp")) + glob.glob(os.path.join(CSRC, "ir", "*.hpp")) +
                  [os.path.join(ROOT, "include", "onyxia_cuda.h")])


def cuda_sources():
    pats = ["backend/*.cpp", "backend/*.hpp", "backend/*.cu", "backend/*.cuh", "kernels/*.cu", "kernels/*.cuh", "kernels/*.hpp"]
    out = []
    for p in pats:
        out += glob.glob(os.path.join(CSRC, p))
    return sorted(out) + ir_sources()


def oracle_sources():
    d = os.path.join(ROOT, "oracle")
    return sorted(glob.glob(os.path.join(d, "*.cpp")) + glob.glob(os.path.join(d, "*.hpp"))) + ir_sources()


def build_ir(force=False, verbose=False) -> str:
    target = os.path.join(PKG, "libonyxia_ir.so")
    src = ir_sources()
    if force or _stale(target, src):
        cpp = [s for s in src if s.endswith(".cpp")]
        _run([CXX] + CXX_FLAGS + ["-shared", "-o", target] + cpp, verbose)
        _stamp(target, src)
    return target


def build_oracle(force=False, verbose=False) -> str:
    target = os.path.join(ROOT, "oracle", "libonyxia_ref.so")
    src = oracle_sources()
    if force or _stale(target, src):
        cpp = [s for s in src if s.endswith(".cpp") and os.sep + "oracle" + os.sep in s]
        _run([CXX, "-std=c++17", "-O3", "-fPIC", "-fopenmp", "-mf16c", "-Wall", "-shared", "-o", target] + cpp +
             ["-L" + PKG, "-lonyxia_ir", "-Wl,-rpath,$ORIGIN/../onyxia_b200"], verbose)
        _stamp(target, src)
    return target


def build_cuda(force=False, verbose=False) -> str:
    target = os.path.join(PKG, "libonyxia_cuda.so")
    src = cuda_sources()
    if not (force or _stale(target, src)):
        return target
    os.makedirs(OBJ, exist_ok=True)
    units = [s for s in src if s.endswith((".cu", ".cpp")) and os.sep + "ir" + os.sep not in s]
    headers = [s for s in src if s.endswith((".hpp", ".cuh", ".h"))]
    hdr_hash = _hash(headers)

    def compile_one(path):
        obj = os.path.join(OBJ, os.path.relpath(path, CSRC).replace(os.sep, "_") + ".o")
        key = hdr_hash + _hash([path]) + " ".join(NVCC_FLAGS)
        stamp = obj + ".stamp"
        if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == key:
            return obj
        cmd = [NVCC] + ARCH + NVCC_FLAGS + ["-Xptxas", "-v"] * (1 if verbose else 0) + ["-c", path, "-o", obj]
        if path.endswith(".cpp"):
            cmd = [NVCC] + ARCH + NVCC_FLAGS + ["-x", "cu", "-c", path, "-o", obj]
        _run(cmd, verbose)
        with open(stamp, "w") as f:
            f.write(key)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, units))
    _run([NVCC] + ARCH + ["-shared", "-o", target] + objs +
         ["-L" + PKG, "-lonyxia_ir", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"], verbose)
    _stamp(target, src)
    return target


def ensure_built(force=False, verbose=False, cuda=True, oracle=True) -> None:
    build_ir(force, verbose)
    if oracle:
        build_oracle(force, verbose)
    if cuda:
        build_cuda(force, verbose)


if __name__ == "__main__":
    ensure_built(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print("built:", os.path.join(PKG, "libonyxia_ir.so"), os.path.join(PKG, "libonyxia_cuda.so"),
          os.path.join(ROOT, "oracle", "libonyxia_ref.so"))
