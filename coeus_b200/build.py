"""In-tree builder for the native libraries.

Two shared objects are produced under ``coeus_b200/lib/``:

* ``libcoeus_kernels.so`` – every ``.cu`` file of ``coeus_b200/csrc`` compiled by ``nvcc`` for
  ``sm_100a`` only (``-gencode arch=compute_100a,code=sm_100a``); plain ``extern "C"`` entry
  points that take raw device pointers and a stream, loaded through ``ctypes``.
* ``_coeus_host*.so`` – the host-side C++ components of ``csrc/host`` (``tokenizers.cpp``,
  ``io.cpp`` checkpoint formats, ``pipeline.cpp`` data loader / suffix array / bloom filter /
  arena, ``oracle.cpp`` CPU oracle) as a pybind11 module.

``python -m coeus_b200.build`` builds both; ``build_all(force=True)`` rebuilds from scratch.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
HOST = ROOT / "csrc" / "host"
LIB = ROOT / "lib"
OBJ = ROOT / "lib" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA kernels cannot be built")


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def kernels_lib_path() -> Path:
    return LIB / "libcoeus_kernels.so"


def host_lib_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB / f"_coeus_host{suffix}"


def build_kernels(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    OBJ.mkdir(exist_ok=True)
    out = kernels_lib_path()
    cus = sorted(CSRC.glob("*.cu"))
    hdrs = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))
    stamp = LIB / "kernels.sha256"
    digest = _digest(cus + hdrs)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    nvcc = _nvcc()

    def compile_one(cu: Path) -> Path:
        o = OBJ / (cu.stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(cu), "-o", str(o)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {cu.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return o

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(cus)))) as ex:
        objs = list(ex.map(compile_one, cus))
    cmd = [nvcc, "-shared", "-o", str(out), *[str(o) for o in objs], "-gencode",
           "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    return out


def build_host(force: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = host_lib_path()
    # selftest.cpp is a stand-alone program (sanitizer builds), not part of the module
    srcs = sorted(p for p in HOST.glob("*.cpp") if p.name != "selftest.cpp")
    hdrs = sorted(HOST.glob("*.hpp"))
    if not srcs:
        return out
    stamp = LIB / "host.sha256"
    digest = _digest(srcs + hdrs)
    if not force and out.exists() and stamp.exists() and stamp.read_text() == digest:
        return out
    import pybind11

    inc = [pybind11.get_include(), sysconfig.get_paths()["include"], str(HOST)]
    OBJ.mkdir(exist_ok=True)

    def compile_one(src: Path) -> Path:
        o = OBJ / ("host_" + src.stem + ".o")
        cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread",
               *[f"-I{i}" for i in inc], "-c", str(src), "-o", str(o)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"g++ failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        return o

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    cmd = ["g++", "-shared", "-pthread", "-o", str(out), *[str(o) for o in objs]]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host link failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(digest)
    return out


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_kernels(force=force, verbose=verbose)
    build_host(force=force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", kernels_lib_path(), host_lib_path())
