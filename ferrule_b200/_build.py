"""In-tree build of the native library (CUDA kernels for sm_100a + C++ host runtime).

`build()` compiles every source under `ferrule_b200/csrc` with nvcc for
`compute_100a/sm_100a` and links `ferrule_b200/_lib/libferrule_b200.so`.  nvcc
cross-compiles without a GPU, so this runs on a CPU-only box; the shared object is
git-ignored but travels with the source tree.

Plays the role of the reference's cc-rs + NVCC build script
(crates/ferrule-backend/build.rs:14-126), with one fixed architecture instead of a
detected one.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OUT_DIR = PKG_DIR / "_lib"
LIB_PATH = OUT_DIR / "libferrule_b200.so"

CUDA_SOURCES = [
    "gemm_tcgen05.cu",
    "gemm_fp8.cu",
    "gemm_mxfp4.cu",
    "mla_attention.cu",
    "mla_prefill_tc.cu",
    "elementwise.cu",
    "data_movers.cu",
    "quant.cu",
    "v4_ops.cu",
    "ep_moe.cu",
    "expert_table.cu",
    "comm.cu",
    "comm_mm.cu",
    "no_alloc.cu",
]
CXX_SOURCES = [
    "host/kv_page_manager.cpp",
    "host/direct_reader.cpp",
    "host/host_runtime.cpp",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
    "-diag-suppress", "550",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return cand


def _existing(names):
    return [n for n in names if (CSRC / n).exists()]


def _digest(paths) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        h.update(str(p).encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


def sources():
    cu = [CSRC / n for n in _existing(CUDA_SOURCES)]
    cxx = [CSRC / n for n in _existing(CXX_SOURCES)]
    hdr = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + sorted((CSRC / "host").glob("*.h"))
    return cu, cxx, hdr


def is_current() -> bool:
    cu, cxx, hdr = sources()
    stamp = OUT_DIR / "build.sha256"
    return LIB_PATH.exists() and stamp.exists() and stamp.read_text().strip() == _digest(cu + cxx + hdr)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compile and link the native library; returns its path."""
    cu, cxx, hdr = sources()
    if not force and is_current():
        return LIB_PATH
    OUT_DIR.mkdir(exist_ok=True)
    obj_dir = OUT_DIR / "obj"
    obj_dir.mkdir(exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: Path) -> Path:
        obj = obj_dir / (src.stem + ".o")
        if src.suffix == ".cu":
            cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        else:
            cmd = [nvcc, "-x", "c++", "-std=c++17", "-O2", "-Xcompiler", "-fPIC,-Wall,-pthread",
                   "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
        if verbose:
            print(" ".join(cmd), file=sys.stderr)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compile failed: {src.name}\n{r.stdout}\n{r.stderr}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as ex:
        objs = list(ex.map(compile_one, cu + cxx))
    tmp = LIB_PATH.with_suffix(".so.tmp")
    cmd = [nvcc, "-shared", "-o", str(tmp), *map(str, objs), "-lpthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB_PATH)
    (OUT_DIR / "build.sha256").write_text(_digest(cu + cxx + hdr))
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
