"""In-tree build of libmatxtract_b200.so (CUDA kernels + C ABI + host helpers) for sm_100a.

Usage: ``python -m matxtract_b200.build`` (or ``build_all()``).  Objects go to ``matxtract_b200/lib/obj``,
the library to ``matxtract_b200/lib/libmatxtract_b200.so``.  nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = LIBDIR / "obj"
LIB = LIBDIR / "libmatxtract_b200.so"
SYNTH_LIB = LIBDIR / "libmx_synth.so"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC,-fopenmp", "-ccbin", "/usr/bin/g++",
                     f"-I{ROOT / 'include'}", f"-I{CSRC}"]


KERNEL_SOURCES = ("csr_resid.cu", "col_slabs.cu", "tile_spmv.cu", "se_spmv.cu", "device_prims.cuh", "mx_internal.h")


def source_hash() -> str:
    """Short hash of the files that hold the SpMV kernels and their launchers (ties an ncu summary to the kernels it
    was captured on; the handle layer, the extraction, file formats and host tools are not part of it)."""
    import hashlib

    hsh = hashlib.sha256()
    files = [CSRC / name for name in KERNEL_SOURCES]
    for f in files:
        hsh.update(f.name.encode())
        hsh.update(f.read_bytes())
    return hsh.hexdigest()[:12]


def _newer(src: Path, dst: Path, extra=()) -> bool:
    if not dst.exists():
        return True
    t = dst.stat().st_mtime
    return any(p.stat().st_mtime > t for p in (src, *extra))


def _run(cmd, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd)}")
    return r.stdout + r.stderr


def build_all(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    OBJDIR.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list((ROOT / "include").glob("*.h"))
    sources = sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJDIR / (src.name + ".o")
        objs.append(obj)
        if force or _newer(src, obj, headers):
            flags = list(NVCC_FLAGS)
            if ptxas_info:
                flags += ["-Xptxas", "-v"]
            if src.suffix == ".cpp":
                flags += ["-x", "cu"] if False else []
            jobs.append([NVCC, *flags, "-c", src, "-o", obj])
    logs = []
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            logs = list(ex.map(lambda c: _run(c, verbose), jobs))
    if ptxas_info:
        print("\n".join(logs))
    if force or jobs or not LIB.exists():
        _run([NVCC, *ARCH, "-shared", "-ccbin", "/usr/bin/g++", "-Xcompiler", "-fPIC,-fopenmp", *objs, "-o", LIB,
              "-lgomp"], verbose)
    # C++ host API shims (include/MatXtract.h) and the drop-in command-line driver, one per precision
    host = CSRC / "host"
    if host.exists():
        for tag, define in (("fp64", ["-Dfp64"]), ("fp16", [])):
            shim = LIBDIR / f"libMatXtract_{tag}.so"
            srcs = [host / "MatXtract_api.cpp", host / "mm_reader.cpp"]
            if any(_newer(s, shim, headers) for s in srcs) or force or _newer(LIB, shim):
                _run(["/usr/bin/g++", "-std=c++17", "-O2", "-fPIC", "-shared", *define, f"-I{ROOT / 'include'}",
                      "-I/usr/local/cuda/include", *srcs, f"-L{LIBDIR}", "-lmatxtract_b200",
                      "-Wl,-rpath,$ORIGIN", "-o", shim], verbose)
            exe = LIBDIR / f"matxtract_perftest_{tag}"
            srcs = [host / "matxtract_perftest.cpp"]
            if all(s.exists() for s in srcs) and (any(_newer(s, exe, headers) for s in srcs) or force or _newer(shim, exe)):
                _run(["/usr/bin/g++", "-std=c++17", "-O2", *define, f"-I{ROOT / 'include'}",
                      "-I/usr/local/cuda/include", *srcs, f"-L{LIBDIR}", f"-lMatXtract_{tag}", "-lmatxtract_b200",
                      "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64",
                      "-o", exe], verbose)
        feat = host / "extract_features.cpp"
        exe = LIBDIR / "extract_features"
        if feat.exists() and (force or _newer(feat, exe, headers) or _newer(LIB, exe)):
            _run(["/usr/bin/g++", "-std=c++17", "-O2", f"-I{ROOT / 'include'}", feat, f"-L{LIBDIR}", "-lmatxtract_b200",
                  "-L/usr/local/cuda/lib64", "-lcudart", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath,/usr/local/cuda/lib64",
                  "-o", exe], verbose)
    # the synthetic-input generator: host code in a library of its own (include/mx_synth.h)
    synth = CSRC / "synth" / "synth.cpp"
    if force or _newer(synth, SYNTH_LIB, [ROOT / "include" / "mx_synth.h"]):
        _run(["/usr/bin/g++", "-std=c++17", "-O2", "-fPIC", "-fopenmp", "-shared", f"-I{ROOT / 'include'}",
              "-I/usr/local/cuda/include", synth, "-o", SYNTH_LIB], verbose)
    return LIB


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(LIB)
