"""Builds the CUDA kernel library in-tree with nvcc for sm_100a.

``build()`` compiles every ``csrc/*.cu`` to an object (in parallel, only when stale) and links
``velogb10_b200/_C.so``. A build id (hash of the sources) is compiled in and checked at load time,
the counterpart of the reference's kernel/source build-ID handshake (reference: build.rs:19-145).
"""
from __future__ import annotations

import hashlib
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from typing import List

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CSRC = os.path.join(ROOT, "csrc")
OBJ_DIR = os.path.join(ROOT, "build", "obj")
LIB_PATH = os.path.join(ROOT, "velogb10_b200", "_C.so")
ID_PATH = os.path.join(ROOT, "build", "build_id.txt")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr"]
if os.environ.get("VELO_TRACE", "0") == "1":        # device timeline stamps (profiling builds only)
    NVCC_FLAGS.append("-DVG_TRACE")


def sources() -> List[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    for f in sorted(os.listdir(CSRC)):
        if f.endswith((".cu", ".cuh", ".h")):
            with open(os.path.join(CSRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()[:16]


def nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def is_fresh() -> bool:
    if not os.path.exists(LIB_PATH) or not os.path.exists(ID_PATH):
        return False
    with open(ID_PATH) as f:
        return f.read().strip() == source_hash()


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> str:
    """Compile and link the library if it is stale. Returns its path."""
    if not force and is_fresh():
        return LIB_PATH
    os.makedirs(OBJ_DIR, exist_ok=True)
    bid = source_hash()
    flags = NVCC_FLAGS + [f'-DVG_BUILD_ID="{bid}"', "-I", CSRC]
    if ptxas_info:
        flags += ["-Xptxas", "-v"]

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        cmd = [nvcc()] + flags + ["-c", src, "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
        if verbose or ptxas_info:
            sys.stderr.write(r.stderr)
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
        objs = list(ex.map(compile_one, sources()))
    cmd = [nvcc(), "-shared", "-o", LIB_PATH] + objs + ["-lcudart_static", "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    with open(ID_PATH, "w") as f:
        f.write(bid)
    return LIB_PATH


if __name__ == "__main__":
    p = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(p)
