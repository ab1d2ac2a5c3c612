"""In-tree native build: CUDA kernels (nvcc, sm_100a) and the C++ host core (g++, pybind11).

Both libraries are written next to the package (``skein_b200/_native``) so that a snapshot of the
source tree carries them along; nothing is installed into site-packages and nothing depends on a
JIT cache in the home directory.

    python -m skein_b200._build            # build whatever is out of date
    python -m skein_b200._build --force    # rebuild everything
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
NATIVE = Path(__file__).resolve().parent / "_native"
OBJ = ROOT / "build" / "obj"

KERNEL_LIB = NATIVE / "libskein_kernels.so"
CORE_LIB_STEM = "_skein_core"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=default",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-sign-compare", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC or put /usr/local/cuda/bin on PATH)")


def _newer(src: Path, dst: Path, extra_deps=()) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in (src, *extra_deps))


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("command failed: %s\n%s\n%s" % (" ".join(map(str, cmd)), r.stdout, r.stderr))
    return r.stdout + r.stderr


def core_lib_path() -> Path:
    return NATIVE / (CORE_LIB_STEM + sysconfig.get_config_var("EXT_SUFFIX"))


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    """Compile every csrc/kernels/*.cu for sm_100a and link libskein_kernels.so."""
    NATIVE.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    kdir = CSRC / "kernels"
    headers = sorted(kdir.glob("*.cuh")) + sorted(kdir.glob("*.h"))
    srcs = sorted(kdir.glob("*.cu"))
    nvcc = _nvcc()
    jobs = []
    objs = []
    for s in srcs:
        o = OBJ / (s.stem + ".o")
        objs.append(o)
        if force or _newer(s, o, headers):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(kdir), "-c", str(s), "-o", str(o)]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for out in ex.map(_run, jobs):
                if verbose and out.strip():
                    print(out)
    if force or jobs or not KERNEL_LIB.exists():
        _run([nvcc, "-shared", "-o", str(KERNEL_LIB), *map(str, objs), "-lcudart"])
    return KERNEL_LIB


def build_core(force: bool = False) -> Path:
    """Compile the C++ host core (planner, cost model, KV manager, batcher, ...) as a pybind11 module."""
    import pybind11

    NATIVE.mkdir(parents=True, exist_ok=True)
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted((CSRC / "core").glob("*.cpp")) + sorted((CSRC / "runtime").glob("*.cpp"))
    headers = sorted((CSRC / "core").glob("*.hpp")) + sorted((CSRC / "runtime").glob("*.hpp"))
    if not srcs:
        return core_lib_path()
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], "-I", str(CSRC / "core"),
           "-I", str(CSRC / "runtime")]
    jobs, objs = [], []
    for s in srcs:
        o = OBJ / ("core_" + s.stem + ".o")
        objs.append(o)
        if force or _newer(s, o, headers):
            jobs.append(["g++", *CXX_FLAGS, *inc, "-c", str(s), "-o", str(o)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_run, jobs))
    out = core_lib_path()
    if force or jobs or not out.exists():
        _run(["g++", "-shared", "-o", str(out), *map(str, objs), "-pthread"])
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_core(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", KERNEL_LIB, core_lib_path())
