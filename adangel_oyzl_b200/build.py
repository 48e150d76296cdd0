"""Build the native library ``libadangel_b200.so`` in-tree with nvcc for sm_100a.

    python -m adangel_oyzl_b200.build [--force] [--verbose]

Each ``csrc/*.cu`` is compiled to an object file (in parallel) and linked into one shared library
with a static CUDA runtime, so the library loads on machines without a GPU driver (the tensor-map
encoder is looked up through the runtime at first use).  Objects are rebuilt only when a source or
header is newer than the object; ``build/<name>.ptxas.log`` keeps ptxas' register / shared-memory report.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
INCLUDE = PKG.parent / "include"
BUILD = PKG / "build"
LIB = PKG / "lib" / "libadangel_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v"]
# gemm_o1_bf16.cu: the O1 recurrence rounds after the multiply AND after the add; no contraction into fma
PER_FILE = {"gemm_o1_bf16.cu": ["-fmad=false"]}


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, force: bool, verbose: bool) -> Path:
    build_dir = BUILD
    obj = build_dir / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest_header()):
        return obj
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON, *PER_FILE.get(src.name, []), "-I", str(INCLUDE), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    log = build_dir / (src.stem + ".ptxas.log")
    log.write_text(proc.stderr)
    if proc.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{proc.stderr}")
    if verbose:
        print(proc.stderr)
    return obj


def build(force: bool = False, verbose: bool = False) -> Path:
    BUILD.mkdir(exist_ok=True)
    LIB.parent.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    with ThreadPoolExecutor(max_workers=min(len(sources), os.cpu_count() or 4)) as pool:
        objs = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-cudart", "static", "-o", str(LIB), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"link failed:\n{proc.stderr}")
    return LIB


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    args = parser.parse_args(argv)
    print(build(args.force, args.verbose))


if __name__ == "__main__":
    main(sys.argv[1:])
