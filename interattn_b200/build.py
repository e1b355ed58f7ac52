"""In-tree build of libinterattn_b200.so (nvcc, sm_100a only).

    python -m interattn_b200.build [--force] [--verbose]
    python -m interattn_b200.build --define IA_SELECT_TRACE --define IA_DECODE_TRACE --output <path>.so

The shared library lands next to this file so that it travels with the source
tree; nothing is installed into site-packages and nothing is JIT-compiled at
import time.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libinterattn_b200.so")
SOURCES = ["capi.cu", "summaries.cu", "select.cu", "select_inst_bf16_d128_range.cu", "select_inst_bf16_d128_diag.cu",
           "select_inst_bf16_d64.cu", "select_inst_f32_d128.cu", "select_inst_f32_d64.cu",
           "select_inst_kbar16_d128.cu", "select_inst_kbar16_d64.cu", "select_inst_bf16_d128_packed.cu",
           "select_inst_bf16_d64_packed.cu", "select_inst_f32_packed.cu", "select_inst_kbar16_packed.cu", "sparse_decode.cu", "sparse_decode_mma.cu",
           "finalize.cu", "llama_step.cu", "skinny_gemm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return exe


def _deps(src: str):
    out = [os.path.join(CSRC, src), os.path.join(HERE, "..", "include", "interattn_b200.h")]
    out += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    return out


def _stale(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, defines=(), output: str = None) -> str:
    """Compile the library.  ``defines`` / ``output`` build a variant beside the normal one (its
    objects in their own folder), e.g. the phase-trace build: ``defines=("IA_SELECT_TRACE",
    "IA_DECODE_TRACE"), output=".../libinterattn_b200_trace.so"``."""
    variant = "_".join(sorted(defines))
    obj_dir = OBJ_DIR if not variant else OBJ_DIR + "_" + variant.lower()
    lib_path = output or LIB_PATH
    if variant and output is None:
        raise ValueError("a variant build needs its own output path")
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    objs = []
    jobs = []
    for src in SOURCES:
        obj = os.path.join(obj_dir, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or _stale(obj, _deps(src)):
            cmd = [nvcc, *NVCC_FLAGS, *[f"-D{d}" for d in defines], "-c", os.path.join(CSRC, src), "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas")
                cmd.insert(2, "-v")
            jobs.append(cmd)

    def run(cmd):
        res = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or res.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
        if res.returncode != 0:
            raise RuntimeError(f"nvcc failed on {cmd[-3]}")

    if jobs:
        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 1)) as pool:
            list(pool.map(run, jobs))
    if jobs or force or _stale(lib_path, objs):
        run([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", lib_path, *objs, "-lcudart"])
    return lib_path


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--define", action="append", default=[], help="preprocessor symbol of a variant build")
    ap.add_argument("--output", default=None, help="where a variant build goes")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose, defines=tuple(a.define), output=a.output))
