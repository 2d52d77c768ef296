"""Build the native sm_100a library in-tree.

``python -m kohakuwullm_b200.build`` compiles every ``csrc/*.cu`` with nvcc for
``compute_100a/sm_100a`` and links ``kohakuwullm_b200/_kwu_native.so``. nvcc cross-compiles,
so this runs on a machine without a GPU. Objects are rebuilt only when their source (or a
header) is newer. The C++ CPU oracles under ``csrc/cpu`` are built with the host compiler into
``kohakuwullm_b200/_kwu_cpu.so``.
"""

from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = PKG / "csrc" / "build"
LIB = PKG / "_kwu_native.so"
CPU_SRC = CSRC / "cpu"
CPU_LIB = PKG / "_kwu_cpu.so"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or put /usr/local/cuda/bin on PATH")


def _stale(target: Path, deps: list[Path]) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def _compile(nvcc: str, src: Path, obj: Path, verbose: bool) -> str:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    return r.stderr


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile what is stale and link. Safe to call from several processes at once (the ranks of a job that start on
    a machine where the library has not been built yet): one holds an exclusive file lock and builds, the others wait
    for it and then find everything up to date."""
    import fcntl

    OBJ.mkdir(parents=True, exist_ok=True)
    with open(OBJ / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            return _build_locked(force, verbose)
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def _build_locked(force: bool, verbose: bool) -> Path:
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            jobs.append((src, obj))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = {ex.submit(_compile, nvcc, s, o, verbose): s for s, o in jobs}
            for f in cf.as_completed(futs):
                out = f.result()
                if verbose and out:
                    print(f"--- {futs[f].name}\n{out}")
    objs = [OBJ / (s.stem + ".o") for s in sources]
    if force or jobs or _stale(LIB, objs):
        # link next to the target and rename: a process that loads the library meanwhile sees the old or the new file
        tmp = LIB.with_suffix(".so.tmp")
        cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart_static", "-lpthread", "-ldl", "-lrt"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, LIB)
    return LIB


def build_cpu(force: bool = False) -> Path:
    """C++ CPU oracles (``csrc/cpu/*.cpp``) -> ``_kwu_cpu.so`` with the host compiler."""
    import fcntl

    sources = sorted(CPU_SRC.glob("*.cpp"))
    OBJ.mkdir(parents=True, exist_ok=True)
    with open(OBJ / ".lock_cpu", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)        # as for the device library: one builder at a time, atomic publish
        if force or _stale(CPU_LIB, sources):
            cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
            tmp = CPU_LIB.with_suffix(".so.tmp")
            cmd = [cxx, "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden", "-o", str(tmp), *map(str, sources)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"host compile failed:\n{r.stdout}\n{r.stderr}")
            os.replace(tmp, CPU_LIB)
    return CPU_LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    print(build_cpu(force="--force" in sys.argv))
