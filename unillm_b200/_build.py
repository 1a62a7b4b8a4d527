"""In-tree build of the native libraries.

Two shared objects are produced next to this file's package, so that they travel with the source
tree and are visible to whatever inspects the process's loaded libraries:

* ``unillm_b200/_native/libunillm_b200_cuda.so``  -- every CUDA kernel (``csrc/**/*.cu``), compiled
  with ``nvcc -gencode arch=compute_100a,code=sm_100a`` (Blackwell only; no other arch is built).
* ``unillm_b200/_native/libunillm_b200_host.so``  -- host-side C++ runtime (``csrc/**/*.cpp``): KV block
  pool, radix tree, GGUF block (de)quantisation oracle, scheduler core.

Objects are rebuilt only when a source or header is newer than the object.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
OUT = Path(__file__).resolve().parent / "_native"
OBJ = OUT / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _newest_header_mtime() -> float:
    m = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for h in CSRC.rglob(pat):
            m = max(m, h.stat().st_mtime)
    return m


def _stale(src: Path, obj: Path, hdr_m: float) -> bool:
    if not obj.exists():
        return True
    om = obj.stat().st_mtime
    return src.stat().st_mtime > om or hdr_m > om


def _run(cmd, log: Path | None = None) -> None:
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(r.stdout)
    if r.returncode != 0:
        sys.stderr.write(r.stdout)
        raise RuntimeError(f"build step failed: {' '.join(map(str, cmd))}")


def nvcc_path() -> str:
    p = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(p):
        raise RuntimeError("nvcc not found")
    return p


def build_cuda(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = nvcc_path()
    srcs = sorted(CSRC.rglob("*.cu"))
    hdr_m = _newest_header_mtime()
    lib = OUT / "libunillm_b200_cuda.so"
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(o)
        if force or _stale(s, o, hdr_m):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        _run([nvcc, *NVCC_FLAGS, "-c", str(s), "-o", str(o)], log=o.with_suffix(".log"))
        if verbose:
            print(f"[build] nvcc {s.relative_to(ROOT)}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if jobs or not lib.exists():
        # link beside the target and rename: a reader (another process, a snapshot) never sees a half-written library
        tmp = lib.with_suffix(".so.tmp")
        _run([nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-cudart", "static"])
        os.replace(tmp, lib)
    return lib


def build_host(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.rglob("*.cpp"))
    hdr_m = _newest_header_mtime()
    lib = OUT / "libunillm_b200_host.so"
    objs = []
    jobs = []
    for s in srcs:
        o = OBJ / (s.relative_to(CSRC).as_posix().replace("/", "__") + ".o")
        objs.append(o)
        if force or _stale(s, o, hdr_m):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        _run(["g++", *CXX_FLAGS, "-c", str(s), "-o", str(o)])
        if verbose:
            print(f"[build] g++ {s.relative_to(ROOT)}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(compile_one, jobs))
    if srcs and (jobs or not lib.exists()):
        tmp = lib.with_suffix(".so.tmp")
        _run(["g++", "-shared", "-o", str(tmp), *map(str, objs), "-pthread"])
        os.replace(tmp, lib)
    return lib


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_cuda(force, verbose)
    build_host(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
