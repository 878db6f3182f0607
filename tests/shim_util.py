"""Builds and binds tests/support/shim_harness.cpp: llm-engine's three launcher symbols, called by
their C++ names from a small shared object, with exceptions turned into return codes."""
import ctypes as C
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "llm-engine_b200")
CUDA_INC = os.environ.get("CUDA_HOME", "/usr/local/cuda") + "/include"


def build_harness(tmp_dir) -> C.CDLL:
    so = os.path.join(str(tmp_dir), "libshim_harness.so")
    cmd = ["g++", "-std=c++17", "-O1", "-shared", "-fPIC", "-I" + CUDA_INC,
           os.path.join(ROOT, "tests", "support", "shim_harness.cpp"), "-L" + LIBDIR, "-lpkv", "-Wl,-rpath," + LIBDIR, "-o", so]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    H = C.CDLL(so)
    H.harness_layer.restype = C.c_int
    H.harness_layer.argtypes = [C.c_int, C.c_int] + [C.c_void_p] * 11 + [C.c_int] * 5 + [C.c_float, C.c_void_p, C.c_char_p, C.c_int]
    return H


def call_layer(H, d, case, use_gqa=False, do_store=True, stream=None):
    """One layer through the harness on the device arrays of `d` (tests.gpu_util.Case.upload).  Returns
    (code, message)."""
    err = C.create_string_buffer(600)
    p = lambda t: t.data_ptr()
    code = H.harness_layer(int(use_gqa), int(do_store), p(d["q"]), p(d["k"]), p(d["v"]), p(d["slots"]), p(d["kc"]), p(d["vc"]),
                           p(d["block_tables"]), p(d["table_offset"]), p(d["token_seq"]), p(d["token_pos"]), p(d["out"]),
                           case.N, case.qh, case.kvh, case.hd, case.bs, C.c_float(case.scale), stream, err, 600)
    return code, err.value.decode()
