"""In-tree build of the native libraries.

Two shared objects are produced under ``fsdp_comm_opt_b200/lib``:

* ``libzc_cpu.so``  - scalar C++ codec (g++ only; no CUDA dependency), used on CPU/gloo ranks.
* ``libzc_cuda.so`` - every sm_100a kernel plus its C launchers (nvcc, ``-gencode
  arch=compute_100a,code=sm_100a``).  Plain C ABI, loaded with ctypes, so no libtorch headers
  are compiled and a full rebuild takes seconds.
* ``libzc_cuda_dbg.so`` - the same sources with ``-DZC_DEBUG_BOUNDS`` (built on demand, loaded when
  ``ZC_DEBUG_BOUNDS=1``): stores into peer memory are checked against the destination's extent and
  an offending store is skipped and recorded in the status words instead of being issued.

The reference builds one pybind11/libtorch extension with setuptools
(reference: zipccl/setup.py:18-71) for sm_90a; there is no sm_100 target there.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib"
OBJ = PKG / "build"

CPU_SOURCES = ["codec_cpu.cpp"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "--use_fast_math",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]


def cuda_sources() -> list[str]:
    return sorted(p.name for p in CSRC.glob("*.cu"))


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def _digest(paths: list[Path], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()


def _stamp_ok(stamp: Path, digest: str, out: Path) -> bool:
    return out.exists() and stamp.exists() and stamp.read_text().strip() == digest


def build_cpu(force: bool = False, verbose: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    out = LIB / "libzc_cpu.so"
    srcs = [CSRC / s for s in CPU_SOURCES]
    hdrs = list(CSRC.glob("*.h"))
    digest = _digest(srcs + hdrs, "cpu-v1")
    stamp = LIB / "libzc_cpu.stamp"
    if not force and _stamp_ok(stamp, digest, out):
        return out
    cmd = ["g++", "-O3", "-std=c++17", "-fPIC", "-shared", "-fopenmp", "-o", str(out)] + [str(s) for s in srcs]
    if verbose:
        print(" ".join(cmd), file=sys.stderr)
    subprocess.run(cmd, check=True)
    stamp.write_text(digest)
    return out


def build_cuda(force: bool = False, verbose: bool = False, ptxas_v: bool = False,
               debug_bounds: bool = False) -> Path | None:
    nvcc = _nvcc()
    if nvcc is None:
        return None
    LIB.mkdir(exist_ok=True)
    obj_dir = PKG / "build_dbg" if debug_bounds else OBJ
    obj_dir.mkdir(exist_ok=True)
    out = LIB / ("libzc_cuda_dbg.so" if debug_bounds else "libzc_cuda.so")
    names = cuda_sources()
    if not names:
        return None
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh"))
    flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if ptxas_v else []) + (["-DZC_DEBUG_BOUNDS"] if debug_bounds else [])
    hdr_digest = _digest(hdrs, " ".join(flags))
    objs: list[Path] = []
    jobs = []
    for name in names:
        src = CSRC / name
        obj = obj_dir / (src.stem + ".o")
        stamp = obj_dir / (src.stem + ".stamp")
        digest = _digest([src], hdr_digest)
        objs.append(obj)
        if force or not _stamp_ok(stamp, digest, obj):
            jobs.append((src, obj, stamp, digest))

    def _compile(job):
        src, obj, stamp, digest = job
        cmd = [nvcc] + flags + ["-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
        if ptxas_v or verbose:
            sys.stderr.write(r.stderr)
        stamp.write_text(digest)

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            list(ex.map(_compile, jobs))
    link_digest = _digest(objs, "link-v1")
    link_stamp = LIB / (out.stem + ".stamp")
    if jobs or force or not _stamp_ok(link_stamp, link_digest, out):
        cmd = [nvcc, "-shared", "-o", str(out)] + [str(o) for o in objs] + ["-Xcompiler", "-fPIC", "-lcuda"]
        # libcuda is only needed for the tensor-map encoder; it is resolved at run time through
        # cudaGetDriverEntryPoint, so do not link it (there is no libcuda on CPU-only hosts).
        cmd = [c for c in cmd if c != "-lcuda"]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        subprocess.run(cmd, check=True)
        link_stamp.write_text(link_digest)
    return out


def build_all(force: bool = False, verbose: bool = False) -> dict:
    return {"cpu": build_cpu(force, verbose), "cuda": build_cuda(force, verbose),
            "cuda_dbg": build_cuda(force, verbose, debug_bounds=True)}


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers/spills/smem per kernel")
    ap.add_argument("--debug-bounds", action="store_true", help="also build libzc_cuda_dbg.so (-DZC_DEBUG_BOUNDS)")
    a = ap.parse_args()
    print(build_cpu(a.force, a.verbose))
    print(build_cuda(a.force, a.verbose, a.ptxas_v))
    if a.debug_bounds:
        print(build_cuda(a.force, a.verbose, a.ptxas_v, debug_bounds=True))
