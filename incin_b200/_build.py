"""In-tree build of the native libraries.

Two shared objects are produced under ``incin_b200/lib``:

* ``libincin_sm100.so`` — every CUDA kernel, compiled by nvcc for
  ``compute_100a/sm_100a`` only (no fat binary, no PTX for other targets).
* ``libincin_host.so``  — the C++ host runtime that needs no GPU: CPU oracle and
  tape autograd (``cpu_ref``), rendezvous and reference transport (``comm``),
  plan-hash digest, batch loader and telemetry sink (``runtime``).

Both export a plain C ABI and are loaded with ``ctypes``; they do not link
against libtorch, so a rebuild takes seconds.  Objects are cached under
``build/`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
LIBDIR = Path(__file__).resolve().parent / "lib"
OBJDIR = ROOT / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O3",
]
# no contraction: the CPU oracle promises the same bits whatever instruction set a multi-versioned loop runs on
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-pthread", "-ffp-contract=off", "-Wall", "-Wno-unused-function"]


def _nvcc() -> str | None:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def cuda_sources() -> list[Path]:
    return sorted((CSRC / "kernels" / "sm100").glob("*.cu")) + sorted((CSRC / "comm").glob("*.cu")) + sorted(
        (CSRC / "runtime").glob("*.cu"))


def host_sources() -> list[Path]:
    out: list[Path] = []
    for sub in ("cpu_ref", "runtime", "comm"):
        out += sorted((CSRC / sub).glob("*.cpp"))
    return out


def _headers_mtime(cuda: bool = True) -> float:
    """Newest header an object of that library can depend on: ``incin_host.h`` declares the host library only, so a
    change there does not rebuild the CUDA objects (and the ``.cuh`` headers do not rebuild the host objects)."""
    cuda_abi = {"incin_b200.h", "incin_comm.h", "incin_b200_noalloc.h"}
    hs = [h for h in CSRC.rglob("*.h") if (h.name in cuda_abi if cuda else h.name not in cuda_abi)]
    hs += list(CSRC.rglob("*.hpp"))
    if cuda:
        hs += list(CSRC.rglob("*.cuh"))
    return max((h.stat().st_mtime for h in hs), default=0.0)


def _stale(obj: Path, src: Path, hdr_mtime: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or hdr_mtime > t


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    if proc.stderr.strip() and os.environ.get("INCIN_BUILD_VERBOSE"):
        sys.stderr.write(proc.stderr)


def build_cuda(force: bool = False, verbose_ptxas: bool = False) -> Path | None:
    nvcc = _nvcc()
    if nvcc is None:
        return None
    OBJDIR.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    hdr = _headers_mtime()
    jobs = []
    objs = []
    for src in cuda_sources():
        obj = OBJDIR / (src.stem + ".cu.o")
        objs.append(obj)
        if force or _stale(obj, src, hdr):
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC / "include"), "-c", str(src), "-o", str(obj)]
            if verbose_ptxas:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    lib = LIBDIR / "libincin_sm100.so"
    if jobs or not lib.exists():
        _run([nvcc, "-shared", "-o", str(lib), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
              "-Xcompiler", "-fPIC"])
    return lib


def build_host(force: bool = False) -> Path | None:
    cxx = shutil.which("g++")
    if cxx is None:
        return None
    srcs = host_sources()
    if not srcs:
        return None
    OBJDIR.mkdir(exist_ok=True)
    LIBDIR.mkdir(exist_ok=True)
    hdr = _headers_mtime(cuda=False)
    jobs, objs = [], []
    for src in srcs:
        obj = OBJDIR / (src.parent.name + "_" + src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, src, hdr):
            jobs.append([cxx, *CXX_FLAGS, "-I", str(CSRC / "include"), "-c", str(src), "-o", str(obj)])
    with cf.ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    lib = LIBDIR / "libincin_host.so"
    if jobs or not lib.exists():
        _run([cxx, "-shared", "-o", str(lib), *map(str, objs), "-pthread"])
    return lib


def build_all(force: bool = False) -> dict[str, str | None]:
    host = build_host(force)
    cuda = build_cuda(force)
    return {"host": str(host) if host else None, "cuda": str(cuda) if cuda else None}


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv))
