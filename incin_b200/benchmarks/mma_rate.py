"""Cycles per ``tcgen05.mma`` by operand shape, layout and source (one B200).

``python -m incin_b200.benchmarks.mma_rate`` compiles ``csrc/bench/mma_rate.cu`` for sm_100a into
``incin_b200/lib/mma_rate`` (when the binary is older than its sources) and runs it.  The kernel issues 512 products
of M 128, K 16 from one thread with one commit at the end and reports, per variant, the cycles the issuing thread
spent issuing and the cycles until completion, with one CTA and with one CTA on every SM.  The attention kernels'
pipeline (which products may share a tile, what a split into halves costs) is laid out from these figures.
"""
from __future__ import annotations

import subprocess
import sys

from .. import _build


def binary(build: bool = True):
    src = _build.CSRC / "bench" / "mma_rate.cu"
    out = _build.LIBDIR / "mma_rate"
    hdr = _build.CSRC / "kernels" / "sm100" / "ptx.cuh"
    stale = not out.exists() or out.stat().st_mtime < max(src.stat().st_mtime, hdr.stat().st_mtime)
    if build and stale:
        nvcc = _build._nvcc()
        if nvcc is None:
            raise RuntimeError("nvcc not found")
        _build.LIBDIR.mkdir(exist_ok=True)
        _build._run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
                     "-o", str(out), str(src), "-lcuda"])
    return out


def main() -> int:
    exe = binary()
    if "--build-only" in sys.argv:
        print(exe)
        return 0
    return subprocess.run([str(exe)], timeout=120).returncode


if __name__ == "__main__":
    sys.exit(main())
