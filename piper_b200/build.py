"""Builds the native library of this package for sm_100a.

Every ``csrc/*.cu`` is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
(cross-compiles without a GPU), ``csrc/*.cpp`` with the host compiler against
the installed PyTorch headers, and everything is linked into
``piper_b200/lib/libpiper_b200.so`` next to the sources, so the library
travels with the source tree.  Objects are rebuilt only when a source or
header is newer than the object.

Usage: ``python -m piper_b200.build [--force] [--verbose]``.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib" / "libpiper_b200.so"
PLAN_SRC = CSRC / "plan" / "plan_executor.cpp"
PLAN_LIB = ROOT / "lib" / "piper_plan.so"          # CPython extension module (pybind11): the launch-plan executor

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _torch_paths():
    import torch
    from torch.utils import cpp_extension as ce

    inc = ce.include_paths("cuda")
    libs = ce.library_paths("cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    return inc, libs, abi


def _newest_header_mtime() -> float:
    hdrs = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
    if verbose and (proc.stdout or proc.stderr):
        print(proc.stdout, proc.stderr, flush=True)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the library if anything is out of date; return its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    inc, libdirs, abi = _torch_paths()
    hdr_mtime = _newest_header_mtime()
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    jobs = []
    objects = []
    for src in sorted(CSRC.glob("*.cu")) + sorted(CSRC.glob("*.cpp")):
        obj = OBJ / (src.name + ".o")
        objects.append(obj)
        stale = force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_mtime)
        if not stale:
            continue
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
        else:
            cmd = ["g++", "-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
                   "-DTORCH_EXTENSION_NAME=piper_c", "-I", str(CSRC)]
            for i in inc:
                cmd += ["-isystem", i]
            cmd += ["-c", str(src), "-o", str(obj)]
        jobs.append(cmd)
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda c: _run(c, verbose), jobs))
    need_link = force or bool(jobs) or not LIB.exists()
    if need_link:
        tmp = LIB.with_name(LIB.name + f".{os.getpid()}.tmp")   # link aside, then rename: readers never see a partial file
        cmd = ["g++", "-shared", "-o", str(tmp), *map(str, objects)]
        for d in libdirs:
            cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
        cmd += ["-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart"]
        try:
            _run(cmd, verbose)
            os.replace(tmp, LIB)
        finally:
            if tmp.exists():
                tmp.unlink()
    build_plan_executor(force=force, verbose=verbose)
    return LIB


def build_plan_executor(force: bool = False, verbose: bool = False) -> Path:
    """The launch-plan executor is a separate CPython extension module: it calls back into Python."""
    import sysconfig

    import pybind11

    if not force and PLAN_LIB.exists() and PLAN_LIB.stat().st_mtime >= PLAN_SRC.stat().st_mtime:
        return PLAN_LIB
    inc, libdirs, abi = _torch_paths()
    tmp = PLAN_LIB.with_name(PLAN_LIB.name + f".{os.getpid()}.tmp")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-fvisibility=hidden",
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    for i in inc:
        cmd += ["-isystem", i]
    cmd += [str(PLAN_SRC), "-o", str(tmp)]
    for d in libdirs:
        cmd += [f"-L{d}", f"-Wl,-rpath,{d}"]
    cmd += ["-lc10", "-lc10_cuda", "-lcudart"]
    try:
        _run(cmd, verbose)
        os.replace(tmp, PLAN_LIB)
    finally:
        if tmp.exists():
            tmp.unlink()
    return PLAN_LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    args = ap.parse_args(argv)
    path = build(force=args.force, verbose=args.verbose)
    print(path)
    return 0


if __name__ == "__main__":
    sys.exit(main())
