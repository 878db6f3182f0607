"""Builds libpkv.so, the sm_100a shared library behind the C ABI of include/pkv.h.

Plain nvcc, in-tree, one object per source so unchanged files are not recompiled.
Usage:  python llm-engine_b200/build.py [--force] [--verbose]
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "libpkv.so")

SOURCES = [
    "host_capi.cpp",
    "kv_cache_manager.cpp",
    "append.cu",
    "copy_blocks.cu",
    "rope_append.cu",
    "step_pack.cu",
    "peer_memory.cu",
    "error_mirror.cu",
    "decode_attn.cu",
    "prefill_attn.cu",
    "engine_shim.cu",
]

NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-fvisibility=default",
          "-I" + os.path.join(ROOT, "include"), "-I" + CSRC]


def _deps_newer(target: str, src: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    deps = [src] + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".hpp", ".cuh", ".h"))]
    deps += [os.path.join(ROOT, "include", f) for f in ("pkv.h", "pkv_kv_cache.hpp")]
    return any(os.path.getmtime(d) > t for d in deps if os.path.exists(d))


def _compile(src: str, force: bool, verbose: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if force or _deps_newer(obj, path):
        cmd = [NVCC, *ARCH, *COMMON, "-Xptxas", "-v" if verbose else "-warn-spills", "-c", path, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    with ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force, verbose), SOURCES))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [NVCC, *ARCH, "-shared", "-o", LIB, *objs, "-cudart", "static"]
        if verbose:
            print(" ".join(cmd))
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("linking libpkv.so failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
