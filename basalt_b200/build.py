"""Compiles the CUDA sources under basalt_b200/csrc for sm_100a into basalt_b200/lib/libbasalt_b200.so with nvcc.

The library has no Python or torch dependency: it exports the C ABI declared in include/basalt_b200.h.  nvcc
cross-compiles without a GPU, so this also runs on a CPU-only build box.  Only router_fast.cu gets --use_fast_math.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIB = PKG / "lib" / "libbasalt_b200.so"
OBJ = PKG / "lib" / "obj"

SOURCES = ["router.cu", "router_fast.cu", "dispatch.cu", "experts.cu", "experts_simple.cu", "experts_mma.cu", "experts_kq.cu", "experts_prefill.cu", "router_prefill.cu", "experts_nvf4.cu", "experts_prefill_nvf4.cu", "layout_file.cu", "norm_pack.cu", "layer.cu", "prefill_group.cu", "ep_layer.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC",
         "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]
EXTRA = {"router_fast.cu": ["--use_fast_math"]}


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps)


def build(force: bool = False, verbose: bool = False) -> Path:
    nvcc = os.environ.get("NVCC", "nvcc")
    OBJ.mkdir(parents=True, exist_ok=True)
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.inc")) + [PKG.parent / "include" / "basalt_b200.h"]
    jobs = []
    for s in SOURCES:
        src, obj = CSRC / s, OBJ / (s + ".o")
        if force or _stale(obj, [src] + headers):
            cmd = [nvcc] + FLAGS + EXTRA.get(s, []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", str(src), "-o", str(obj)]
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or verbose:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed: " + cmd[-3])

    with ThreadPoolExecutor(max_workers=8) as ex:
        list(ex.map(run, jobs))
    objs = [OBJ / (s + ".o") for s in SOURCES]
    if force or jobs or _stale(LIB, objs):
        run([nvcc, "-shared", "-o", str(LIB)] + [str(o) for o in objs] + ["-lcudart", "-ldl"])
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
