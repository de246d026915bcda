"""Builds libb200fa.so (the C-ABI library of include/b200fa.h) in-tree with nvcc for sm_100a.

Usage: python build.py [--force] [--verbose] [--trace]
Each .cu file under csrc/ is compiled to an object file (in parallel) and linked into zigfa/libb200fa.so.
A file is rebuilt when it or any header is newer than its object. `--trace` builds the tuning variant instead
(-DB200FA_TRACE -DB200FA_TRACE_SUMS=0: per-role event timelines for zigfa/profile.py) into zigfa/libb200fa_trace.so.
"""
from __future__ import annotations

import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "build"
LIB = ROOT / "zigfa" / "libb200fa.so"
INCLUDE = ROOT.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-Xptxas", "-v",
]
NVCC_FLAGS += os.environ.get("B200FA_NVCC_FLAGS", "").split()  # tuning builds: extra -D switches
if os.environ.get("B200FA_TRACE"):  # tuning build: cycle counters in the backward kernel (see b200fa_set_trace)
    NVCC_FLAGS.append("-DB200FA_TRACE")


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(found).exists():
        raise RuntimeError("nvcc not found; the library cannot be built")
    return found


def newest_header() -> float:
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    return max(path.stat().st_mtime for path in headers)


def compile_one(source: Path, verbose: bool, objects: Path = OBJ, extra: tuple = ()) -> tuple[Path, str]:
    target = objects / (source.stem + ".o")
    command = [nvcc(), *NVCC_FLAGS, *extra, "-I", str(INCLUDE), "-c", str(source), "-o", str(target)]
    result = subprocess.run(command, capture_output=True, text=True)
    log = result.stdout + result.stderr
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{log}")
    (objects / (source.stem + ".ptxas.log")).write_text(log)
    if verbose:
        print(log)
    return target, log


def build(force: bool = False, verbose: bool = False, trace: bool = False) -> Path:
    objects = ROOT / "build_trace" if trace else OBJ
    library = LIB.with_name("libb200fa_trace.so") if trace else LIB
    extra = ("-DB200FA_TRACE", "-DB200FA_TRACE_SUMS=0") if trace else ()
    objects.mkdir(exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    header_time = newest_header()
    stale = []
    for source in sources:
        target = objects / (source.stem + ".o")
        if force or not target.exists() or target.stat().st_mtime < max(source.stat().st_mtime, header_time):
            stale.append(source)
    if stale:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(stale), os.cpu_count() or 1)) as pool:
            for _ in pool.map(lambda source: compile_one(source, verbose, objects, extra), stale):
                pass
    object_files = [objects / (source.stem + ".o") for source in sources]
    if stale or not library.exists():
        command = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(library), *map(str, object_files)]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"link failed:\n{result.stdout}{result.stderr}")
    return library


if __name__ == "__main__":
    parser = argparse.ArgumentParser()
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true")
    parser.add_argument("--trace", action="store_true", help="build the tuning variant zigfa/libb200fa_trace.so")
    options = parser.parse_args()
    print(build(options.force, options.verbose, options.trace))
