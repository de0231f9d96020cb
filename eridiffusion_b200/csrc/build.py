"""In-tree build of the native libraries.

Two shared objects are produced under ``eridiffusion_b200/lib``:

* ``liberi_b200_kernels.so`` — every ``.cu`` file of this directory, compiled for sm_100a only
  (``-gencode arch=compute_100a,code=sm_100a``), exporting plain C entry points that take raw
  device pointers and a stream. Python binds them with ``ctypes`` (see ``ops/_native.py``).
* ``liberi_b200_host.so`` — the C++ host runtime (safetensors mmap reader / writer, pinned staging
  pool, manifest loader worker), no CUDA device code.

``ERI_B200_DEBUG_BOUNDS=1`` (or ``build_kernels(debug_bounds=True)``) builds a second library,
``liberi_b200_kernels_debug.so``, from the same sources with ``-DERI_DEBUG_BOUNDS``: every guarded
global / peer access range-checks itself against the extent the host passed and records a
violation instead of performing the access (see ``ptx.cuh``). ``ops/_native.py`` loads that library
when the variable is set. It is the stand-in for a memory checker on the small test shapes.

The sources are compiled in parallel with one ``nvcc -c`` per file and relinked only when an
object changed, so a rebuild after touching one kernel takes seconds. Nothing is written outside
the package directory.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_DIR = CSRC.parent / "lib"
OBJ_DIR = CSRC / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
    "--expt-relaxed-constexpr",
]
HOST_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-shared", "-pthread"]


def _nvcc() -> str:
    cand = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/bin/nvcc"
    if os.path.exists(cand):
        return cand
    found = shutil.which("nvcc")
    if not found:
        raise RuntimeError("nvcc not found; set CUDA_HOME")
    return found


def _digest(path: Path, extra: str) -> str:
    h = hashlib.sha256()
    h.update(path.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")):
        h.update(hdr.read_bytes())
    h.update(extra.encode())
    return h.hexdigest()


def _compile_one(src: Path, verbose: bool, ptxas_v: bool, debug_bounds: bool = False) -> tuple[Path, bool, str]:
    suffix = ".dbg" if debug_bounds else ""
    obj = OBJ_DIR / (src.stem + suffix + ".o")
    stamp = OBJ_DIR / (src.stem + suffix + ".sha")
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_v else []) + (["-DERI_DEBUG_BOUNDS=1"] if debug_bounds else [])
    dig = _digest(src, " ".join(flags))
    if obj.exists() and stamp.exists() and stamp.read_text() == dig:
        return obj, False, ""
    cmd = [_nvcc(), *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(dig)
    return obj, True, r.stderr if (verbose or ptxas_v) else ""


def build_kernels(verbose: bool = False, ptxas_v: bool = False, debug_bounds: bool = False) -> Path:
    OBJ_DIR.mkdir(exist_ok=True)
    LIB_DIR.mkdir(exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    out = LIB_DIR / ("liberi_b200_kernels_debug.so" if debug_bounds else "liberi_b200_kernels.so")
    changed = False
    objs = []
    with cf.ThreadPoolExecutor(max_workers=min(8, len(srcs) or 1)) as ex:
        for obj, ch, log in ex.map(lambda s: _compile_one(s, verbose, ptxas_v, debug_bounds), srcs):
            objs.append(obj)
            changed |= ch
            if log:
                print(log, file=sys.stderr)
    if changed or not out.exists():
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-Xcompiler", "-fPIC", "-o", str(out), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return out


def build_host(verbose: bool = False) -> Path:
    LIB_DIR.mkdir(exist_ok=True)
    OBJ_DIR.mkdir(exist_ok=True)
    srcs = sorted((CSRC / "host").glob("*.cpp"))
    out = LIB_DIR / "liberi_b200_host.so"
    if not srcs:
        return out
    h = hashlib.sha256()
    for s in srcs + sorted((CSRC / "host").glob("*.h")):
        h.update(s.read_bytes())
    stamp = OBJ_DIR / "host.sha"
    if out.exists() and stamp.exists() and stamp.read_text() == h.hexdigest():
        return out
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", *HOST_FLAGS, "-I", f"{cuda_home}/include", "-o", str(out), *map(str, srcs),
           f"-L{cuda_home}/lib64", "-lcudart", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"host build failed:\n{r.stdout}\n{r.stderr}")
    stamp.write_text(h.hexdigest())
    return out


def build_all(verbose: bool = False, ptxas_v: bool = False, debug_bounds: bool | None = None) -> list[Path]:
    """Kernel library, host library and — with ``debug_bounds`` (default: ``ERI_B200_DEBUG_BOUNDS=1``
    in the environment) — the bounds-checked debug variant of the kernel library."""
    if debug_bounds is None:
        debug_bounds = os.environ.get("ERI_B200_DEBUG_BOUNDS") == "1"
    out = [build_kernels(verbose, ptxas_v), build_host(verbose)]
    if debug_bounds:
        out.append(build_kernels(verbose, False, debug_bounds=True))
    return out


if __name__ == "__main__":
    v = "-v" in sys.argv
    for p in build_all(verbose=v, ptxas_v="--ptxas" in sys.argv, debug_bounds=True if "--debug-bounds" in sys.argv else None):
        print(p)
