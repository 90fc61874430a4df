"""Out-of-tree sm_100a build of the reference's own synthetic decode harness (`apps/gpt_doll.cpp`).

The reference's CMake project targets sm_121a and needs libibverbs / OpenSSL / PCRE2 for its server targets; the
`gpt_doll` harness needs none of that.  This script copies the UNMODIFIED reference sources the harness links
(headers of `src/common`, `src/core`, `src/kernels`; the listed translation units) into `baseline/_ref/`, compiles
each for sm_100a with nvcc / g++ and links `baseline/_ref/build/gpt_doll`.  Nothing of this repository's own engine
is on that path.  `bench.py --impl reference` runs the binary.

    python baseline/build_ref.py [--src /path/to/reference] [--force]

Build graph being reproduced: the reference's CMakeLists.txt targets dgpp_core, dgpp_kernels (the subset gpt_doll
reaches), dgpp_models_doll and gpt_doll (CMakeLists.txt:120-130, 246, 2758-2762).
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
BIN = os.path.join(REF, "build", "gpt_doll")

HEADER_GLOBS = ["src/common/*.hpp", "src/core/*.hpp", "src/kernels/*.hpp", "src/kernels/*.cuh"]
HEADERS = ["src/models/gpt_doll.hpp", "src/models/quant_matrix.hpp", "src/models/exl3_matrix.hpp",
           "src/models/glm/moe.hpp"]
CUDA_UNITS = ["src/models/gpt_doll.cu", "src/kernels/kernels.cu", "src/kernels/doll_attention.cu",
              "src/kernels/bf12_gemv.cu", "src/kernels/bf16_gemv.cu", "src/kernels/mma_gemv.cu",
              "src/kernels/scale_gemm.cu", "src/kernels/fp8w_gemm.cu", "src/kernels/glm_moe.cu",
              "src/kernels/dense_fp4_decode.cu"]
HOST_UNITS = ["src/kernels/gemm_cublaslt.cpp", "src/common/log.cpp", "src/core/trace.cpp", "apps/gpt_doll.cpp"]
EXTRA = ["LICENSE"]

NVCC_FLAGS = ["-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "--extended-lambda",
              "--expt-relaxed-constexpr", "-Xcompiler=-ffp-contract=off", "-Isrc"]
GXX_FLAGS = ["-std=c++20", "-O2", "-ffp-contract=off", "-Isrc", "-I/usr/local/cuda/include"]


def default_source() -> str | None:
    """The reference checkout named by BASELINE.json beside this folder (`reference_path`), when it exists."""
    import json
    try:
        with open(os.path.join(os.path.dirname(HERE), "BASELINE.json")) as f:
            return json.load(f).get("reference_path")
    except (OSError, ValueError):
        return None


def copy_sources(src_root: str) -> None:
    rel = list(HEADERS) + CUDA_UNITS + HOST_UNITS + EXTRA
    for g in HEADER_GLOBS:
        rel += [os.path.relpath(p, src_root) for p in glob.glob(os.path.join(src_root, g))]
    for r in sorted(set(rel)):
        dst = os.path.join(REF, r)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(src_root, r), dst)


def run(cmd) -> None:
    p = subprocess.run(cmd, cwd=REF, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if p.returncode != 0:
        errs = [ln for ln in p.stdout.splitlines() if "error" in ln][:3]
        raise RuntimeError("%s failed: %s" % (" ".join(cmd[:4]), " | ".join(errs) or p.stdout[-400:]))


def build(src_root: str | None = None, force: bool = False) -> str:
    """Returns the path of the harness binary; raises RuntimeError with the first compiler errors otherwise."""
    if os.path.exists(BIN) and not force:
        return BIN
    if src_root and os.path.isdir(src_root):
        copy_sources(src_root)
    if not os.path.exists(os.path.join(REF, "apps", "gpt_doll.cpp")):
        raise RuntimeError("reference sources not found (neither %s nor a copy under baseline/_ref)" % src_root)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found")
    os.makedirs(os.path.join(REF, "build"), exist_ok=True)
    objs = []
    for u in CUDA_UNITS:
        o = os.path.join("build", os.path.basename(u) + ".o")
        run([nvcc] + NVCC_FLAGS + ["-c", u, "-o", o])
        objs.append(o)
    for u in HOST_UNITS:
        o = os.path.join("build", os.path.basename(u) + ".o")
        run(["g++"] + GXX_FLAGS + ["-c", u, "-o", o])
        objs.append(o)
    run(["g++", "-o", os.path.join("build", "gpt_doll")] + objs +
        ["-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64", "-lcudart", "-lcublasLt", "-lcublas", "-lcuda"])
    for o in objs:
        os.remove(os.path.join(REF, o))
    return BIN


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--src", default=default_source())
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    try:
        print(build(a.src, a.force))
    except RuntimeError as e:
        print("build failed:", e, file=sys.stderr)
        sys.exit(1)
