"""In-tree native build for dgpp_b200.

Two shared objects are produced under ``dgpp_b200/lib``:

* ``libdgpp_kernels.so`` -- every CUDA kernel plus the launch-program executor,
  compiled by nvcc for sm_100a only and exposed through a plain C ABI (loaded with
  ctypes, no torch headers involved, so a full rebuild takes seconds).
* ``_dgpp_rt*.so`` -- the host runtime (scheduler, paged KV table, prefix cache,
  tokenizer, chat template, grammars, sampler oracle, HTTP server), a pybind11 module
  compiled by g++.

Objects are cached under ``build/`` and rebuilt when a source or header is newer.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
LIB = ROOT / "lib"
BUILD = ROOT.parent / "build"

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
CXX = os.environ.get("CXX", "g++")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wall",
    "-Xcompiler", "-Wno-unused-function", "-I", str(CSRC),
]
# Translation units that must not contract a*b+c into fma (sampler parity with the host oracle).
NO_FMA = {"sample.cu"}

CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-Wno-unused-function", "-pthread", "-ffp-contract=off",
             "-I", str(CSRC)]


def _newest_header() -> float:
    newest = 0.0
    for pat in ("*.h", "*.cuh", "*.hpp"):
        for p in CSRC.rglob(pat):
            newest = max(newest, p.stat().st_mtime)
    return newest


def _needs(obj: Path, src: Path, hdr_time: float) -> bool:
    if not obj.exists():
        return True
    t = obj.stat().st_mtime
    return src.stat().st_mtime > t or hdr_time > t


def _run(cmd: list[str]) -> str:
    p = subprocess.run(cmd, capture_output=True, text=True)
    if p.returncode != 0:
        raise RuntimeError("build failed: %s\n%s\n%s" % (" ".join(cmd), p.stdout, p.stderr))
    return p.stdout + p.stderr


def kernel_sources() -> list[Path]:
    return sorted((CSRC / "kernels").glob("*.cu")) + sorted((CSRC / "engine").glob("*.cu"))


def rt_sources() -> list[Path]:
    return sorted((CSRC / "rt").glob("*.cpp"))


def build_kernels(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    LIB.mkdir(exist_ok=True)
    odir = BUILD / "kernels"
    odir.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    out = LIB / "libdgpp_kernels.so"
    jobs = []
    objs = []
    for src in kernel_sources():
        obj = odir / (src.stem + ".o")
        objs.append(obj)
        if force or _needs(obj, src, hdr):
            flags = list(NVCC_FLAGS)
            if src.name in NO_FMA:
                flags += ["--fmad=false"]
            if ptxas_info:
                flags += ["-Xptxas", "-v"]
            jobs.append([NVCC, *flags, "-c", str(src), "-o", str(obj)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            for log in ex.map(_run, jobs):
                if (verbose or ptxas_info) and log.strip():
                    print(log)
    if jobs or not out.exists():
        _run([NVCC, "-shared", "-o", str(out), *map(str, objs), "-lcudart", "-ldl"])
    return out


def _shared_stdcxx() -> list[str]:
    """Link against the system's shared libstdc++ by file name.  A toolchain wrapper that cannot find
    ``libstdc++.so`` silently links the static archive instead; a second copy of libstdc++ in one process (PyTorch
    loads the shared one) corrupts iostream locale state, so the shared library is named explicitly."""
    for d in ("/usr/lib/x86_64-linux-gnu", "/lib/x86_64-linux-gnu", "/usr/lib64"):
        if (Path(d) / "libstdc++.so.6").exists():
            return ["-L" + d, "-l:libstdc++.so.6"]
    return []


def rt_module_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return LIB / ("_dgpp_rt" + suffix)


def build_rt(verbose: bool = False, force: bool = False) -> Path:
    import pybind11

    LIB.mkdir(exist_ok=True)
    odir = BUILD / "rt"
    odir.mkdir(parents=True, exist_ok=True)
    hdr = _newest_header()
    out = rt_module_path()
    inc = ["-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    jobs = []
    objs = []
    for src in rt_sources():
        obj = odir / (src.stem + ".o")
        objs.append(obj)
        if force or _needs(obj, src, hdr):
            jobs.append([CXX, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)])
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
            for log in ex.map(_run, jobs):
                if verbose and log.strip():
                    print(log)
    if jobs or not out.exists():
        _run([CXX, "-shared", "-o", str(out), *map(str, objs), *_shared_stdcxx(), "-pthread"])
    return out


def build_all(verbose: bool = False, force: bool = False) -> None:
    build_rt(verbose=verbose, force=force)
    build_kernels(verbose=verbose, force=force)


if __name__ == "__main__":
    build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built", LIB)
