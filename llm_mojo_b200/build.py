"""Builds the sm_100a kernel library in-tree with nvcc (no torch headers, no JIT cache).

``python -m llm_mojo_b200.build`` compiles every ``csrc/*.cu`` to an object file and links
``csrc/libllmb200.so``.  Only files whose sources changed are recompiled.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
LIB_PATH = os.path.join(CSRC, "libllmb200.so")
CHECK_LIB_PATH = os.path.join(CSRC, "libllmb200_check.so")     # -DLLMB_BOUNDS_CHECK: data-dependent indices tested before use
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]
# Every kernel here is free of cluster-multicast TMA loads, so one library serves 1-GPU and multi-GPU runs.


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _digest(path: str, extra: str = "") -> str:
    h = hashlib.sha256()
    h.update(extra.encode())
    for name in sorted(os.listdir(CSRC)):
        if name.endswith((".cuh", ".h")) or name == os.path.basename(path):
            with open(os.path.join(CSRC, name), "rb") as f:
                h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(verbose: bool = True, force: bool = False, check: bool = False) -> str:
    """Compile and link the library; ``check=True`` builds the bounds-checked variant beside it."""
    nvcc = _nvcc()
    objs, jobs = [], []
    flags = NVCC_FLAGS + (["-DLLMB_BOUNDS_CHECK"] if check else [])
    lib_path = CHECK_LIB_PATH if check else LIB_PATH
    for src in sources():
        sp = os.path.join(CSRC, src)
        obj = sp[:-3] + (".check.o" if check else ".o")
        stamp = obj + ".sha"
        dig = _digest(sp, "check" if check else "")
        objs.append(obj)
        if not force and os.path.exists(obj) and os.path.exists(stamp) and open(stamp).read() == dig:
            continue
        jobs.append((sp, obj, stamp, dig))

    def compile_one(job):
        sp, obj, stamp, dig = job
        cmd = [nvcc, *flags, "-c", sp, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {sp}:\n{r.stdout}\n{r.stderr}")
        with open(stamp, "w") as f:
            f.write(dig)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not os.path.exists(lib_path):
        cmd = [nvcc, "-shared", "-o", lib_path, *objs, "-lcudart"]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return lib_path


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, check="--check" in sys.argv))
