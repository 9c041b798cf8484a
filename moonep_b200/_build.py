"""In-tree build of the native library ``moonep_b200/_lib/libmoonep_b200.so``.

Every native source of the package (CPU oracle, host-side symmetric heap, and all
sm_100a kernels) is compiled by ``nvcc`` into ONE shared object with a plain C ABI that
:mod:`moonep_b200._native` loads through ``ctypes``.  There is no JIT and no dependency on
the torch headers, so a cold build takes well under a minute and cross-compiles on a
machine without a GPU.  The library links cudart statically and resolves the few driver
API entry points it needs at run time through ``cudaGetDriverEntryPoint``, so it can be
loaded (for the CPU oracle) on a host that has no ``libcuda``.

The reference builds its only native code with a torch ``CUDAExtension`` without any arch
flag (setup.py:24-41); here the arch is fixed to sm_100a.
"""
from __future__ import annotations

import concurrent.futures as _fut
import hashlib
import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "_lib")
OBJ_DIR = os.path.join(LIB_DIR, "obj")
LIB_PATH = os.path.join(LIB_DIR, "libmoonep_b200.so")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fno-strict-aliasing",
    "-Xcompiler", "-Wno-psabi", "-DNDEBUG",
]
# extra nvcc flags for one-off builds (e.g. -DMEP_GEMM_EXPERIMENTS, which compiles the timing
# experiment switches of the GEMM in; a normal build has none of those branches)
NVCC_FLAGS += os.environ.get("MOONEP_B200_NVCC_FLAGS", "").split()


def _nvcc() -> str:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")
    return cand


def sources() -> list[str]:
    out = []
    for root, _dirs, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".cu", ".cc")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _headers() -> list[str]:
    out = []
    for root, _dirs, files in os.walk(CSRC):
        for f in sorted(files):
            if f.endswith((".h", ".cuh")):
                out.append(os.path.join(root, f))
    return sorted(out)


def _digest(paths: list[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in paths:
        h.update(p.encode())
        with open(p, "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()


def _compile_one(nvcc: str, src: str, obj: str, verbose: bool) -> str:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", CSRC, "-x", "cu", "-c", src, "-o", obj]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return res.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every source under ``csrc/`` for sm_100a and link the shared object.

    Objects are cached by a content hash of the source plus all headers, so an unchanged
    tree is a no-op.  Returns the path of the library.
    """
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    hdrs = _headers()
    flags_key = " ".join(ARCH_FLAGS + NVCC_FLAGS)
    jobs = []
    objs = []
    for src in sources():
        rel = os.path.relpath(src, CSRC).replace(os.sep, "__")
        obj = os.path.join(OBJ_DIR, rel + ".o")
        stamp = obj + ".sha"
        dig = _digest([src] + hdrs, flags_key)
        objs.append(obj)
        fresh = (not force and os.path.exists(obj) and os.path.exists(stamp)
                 and open(stamp).read() == dig)
        if not fresh:
            jobs.append((src, obj, stamp, dig))
    log = []
    if jobs:
        with _fut.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {ex.submit(_compile_one, nvcc, s, o, verbose): (s, o, st, d)
                    for (s, o, st, d) in jobs}
            for f in _fut.as_completed(futs):
                s, o, st, d = futs[f]
                log.append((s, f.result()))
                with open(st, "w") as fh:
                    fh.write(d)
    if jobs or not os.path.exists(LIB_PATH):
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", LIB_PATH, *objs, "-Xcompiler", "-fPIC",
               "-cudart", "static", "-ldl", "-lpthread", "-lrt"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    if verbose:
        for s, txt in log:
            print(f"==== {os.path.relpath(s, CSRC)}\n{txt}")
    return LIB_PATH


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
