"""Drop-in evidence that needs the reference tree (skipped where it is absent, e.g. on
the GPU box): llm-engine's OWN sources are compiled, unmodified and where they lie,
against this repository's headers and library."""
import os
import subprocess

import pytest

import oracle

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = oracle.reference_root()
LIBDIR = os.path.join(ROOT, "llm-engine_b200")

needs_ref = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "include", "engine")),
                               reason="reference tree not present")


@needs_ref
def test_reference_allocator_tests_pass_against_this_kvcachemanager(pkv, tmp_path):
    """tests/test_block_allocator.cpp of llm-engine (8 cases), with `engine/kv_cache.h` resolved
    to this repository's include/engine/kv_cache.h and the class implemented by libpkv.so."""
    exe = tmp_path / "alloc_tests"
    cmd = ["g++", "-std=c++17", "-O1", "-DMINI_CATCH_MAIN",
           "-I" + os.path.join(ROOT, "tests", "support"), "-I" + os.path.join(ROOT, "include"),
           os.path.join(REF, "tests", "test_block_allocator.cpp"),
           "-L" + LIBDIR, "-lpkv", "-Wl,-rpath," + LIBDIR, "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "cases=8 failures=0" in r.stdout


@needs_ref
def test_reference_launcher_header_links_against_libpkv(pkv, tmp_path):
    """A translation unit that includes llm-engine's include/engine/cuda_kernels.h and takes the
    three KV-path launchers exactly as src/model/cuda/cuda_model.cu:368-377 calls them links
    against libpkv.so: the signatures are the reference's, symbol for symbol."""
    src = tmp_path / "link_probe.cpp"
    src.write_text(r'''
#define ENGINE_CUDA 1
#include "engine/cuda_kernels.h"
#include <cstdio>
int main() {
  // empty steps: the documented no-op path, no device needed
  engine::launch_store_kv(nullptr, nullptr, nullptr, nullptr, nullptr, 0, 128, nullptr);
  engine::launch_attention_decode(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                  0, 14, 2, 64, 16, 0.125f, nullptr);
  engine::launch_attention_decode_gqa(nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr,
                                      0, 14, 2, 64, 16, 0.125f, nullptr);
  std::puts("linked");
  return 0;
}
''')
    exe = tmp_path / "link_probe"
    cmd = ["g++", "-std=c++17", "-I" + os.path.join(REF, "include"), "-I/usr/local/cuda/include", str(src),
           "-L" + LIBDIR, "-lpkv", "-Wl,-rpath," + LIBDIR, "-o", str(exe)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0 and "linked" in r.stdout, r.stdout + r.stderr
