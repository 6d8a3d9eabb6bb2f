"""Build ``libmolt_b200.so`` in-tree with nvcc for sm_100a.

    python -m molt_b200.build            # incremental
    python -m molt_b200.build --force    # rebuild everything

The library is plain C ABI (see ``include/molt_b200.h``); it links only the CUDA runtime.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
BUILD_DIR = CSRC / "build"
LIBRARY = PACKAGE_DIR / "libmolt_b200.so"
SOURCES = ["api.cu", "elementwise.cu", "general.cu", "skinny.cu", "gemv.cu", "gemm_sm100_pair.cu", "skinny_sm100.cu", "static_scratch.cu"]
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).exists():
            return candidate
    raise RuntimeError("nvcc was not found; set NVCC or install the CUDA toolkit")


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + [PACKAGE_DIR.parent / "include" / "molt_b200.h"]
    return max(h.stat().st_mtime for h in headers if h.exists())


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile every CUDA source for sm_100a and link the shared library. Returns its path."""
    nvcc = _nvcc()
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    header_time = _newest_header()
    common = [nvcc, "-O3", "-std=c++17", "-lineinfo", *ARCH_FLAGS, "-Xcompiler", "-fPIC,-O3", "--expt-relaxed-constexpr"]
    extra = os.environ.get("MOLT_B200_NVCC_FLAGS", "")  # e.g. -DMOLT_PAIR_TRACE for pipeline timelines
    common += extra.split()
    # objects built with other flags are stale: remember the command line they were built with
    stamp = BUILD_DIR / "flags.txt"
    signature = " ".join(common)
    if verbose:
        common += ["-Xptxas", "-v"]
    if not stamp.exists() or stamp.read_text() != signature:
        force = True
    jobs = []
    objects = []
    for name in SOURCES:
        src = CSRC / name
        obj = BUILD_DIR / (src.stem + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, header_time)
        if stale:
            jobs.append(common + ["-c", str(src), "-o", str(obj)])

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, proc

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            for cmd, proc in pool.map(run, jobs):
                if verbose or proc.returncode != 0:
                    sys.stderr.write(proc.stdout + proc.stderr)
                if proc.returncode != 0:
                    raise RuntimeError("nvcc failed: " + " ".join(cmd))
    stamp.write_text(signature)
    if jobs or not LIBRARY.exists():
        link = [nvcc, "-shared", *ARCH_FLAGS, "-o", str(LIBRARY), *map(str, objects), "-lcudart"]
        proc = subprocess.run(link, capture_output=True, text=True)
        if proc.returncode != 0:
            sys.stderr.write(proc.stdout + proc.stderr)
            raise RuntimeError("linking libmolt_b200.so failed")
    return LIBRARY


def main() -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true", help="pass -Xptxas -v and echo compiler output")
    args = parser.parse_args()
    print(build(force=args.force, verbose=args.verbose))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
