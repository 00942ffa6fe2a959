"""Build the native kernel library in-tree: ``python -m speech_b200.ops.build``.

Every ``.cu`` under ``speech_b200/ops/csrc`` is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a -lineinfo``) into an object file and linked into
``speech_b200/ops/libspeech_b200.so``.  Files are compiled in parallel; an up-to-date object is reused.
nvcc cross-compiles without a GPU, so this also runs on build machines that have none.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "_build")
LIB = os.path.join(HERE, "libspeech_b200.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
              "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found")
    return cand


def _variant():
    """Optional diagnostic variant: ``SPEECH_B200_BUILD_DEFS="-DSB_GEMM_DIAG"`` builds ``libspeech_b200_diag.so`` in its own
    object directory, next to the product library (which never carries diagnostic code)."""
    defs = os.environ.get("SPEECH_B200_BUILD_DEFS", "").split()
    if not defs:
        return [], BUILD, LIB
    return defs, BUILD + "_diag", os.path.join(HERE, "libspeech_b200_diag.so")


def _digest(path: str) -> str:
    h = hashlib.sha1()
    for p in [path] + sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))):
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS + _variant()[0]).encode())
    return h.hexdigest()


def _compile(src: str, verbose: bool) -> str:
    name = os.path.splitext(os.path.basename(src))[0]
    defs, bdir, _ = _variant()
    obj = os.path.join(bdir, name + ".o")
    stamp = obj + ".sha1"
    dg = _digest(src)
    if os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dg:
        return obj
    cmd = [_nvcc()] + NVCC_FLAGS + defs + ["-I", CSRC, "-c", src, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    log = os.path.join(bdir, name + ".log")
    with open(log, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{r.stderr[-4000:]}")
    if verbose:
        for line in r.stderr.splitlines():
            if "registers" in line or "spill" in line and "0 bytes spill" not in line:
                print(f"[{name}] {line.strip()}")
    with open(stamp, "w") as f:
        f.write(dg)
    return obj


def build(verbose: bool = False, force: bool = False) -> str:
    _, bdir, lib = _variant()
    os.makedirs(bdir, exist_ok=True)
    if force:
        for f in os.listdir(bdir):
            os.remove(os.path.join(bdir, f))
    srcs: List[str] = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    newest = max(os.path.getmtime(o) for o in objs)
    if not os.path.exists(lib) or os.path.getmtime(lib) < newest:
        cmd = [_nvcc(), "-shared", "-o", lib] + objs + ["-lcudart", "-Xlinker", "-z,noexecstack"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stderr[-4000:]}")
    return lib


if __name__ == "__main__":
    path = build(verbose="-q" not in sys.argv, force="--force" in sys.argv)
    print(path)
