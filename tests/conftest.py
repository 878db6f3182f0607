"""Shared fixtures.  Tests marked `gpu` need a B200; everything else runs on CPU."""
import importlib
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _ensure_built():
    lib = os.path.join(ROOT, "llm-engine_b200", "libpkv.so")
    if not os.path.exists(lib):
        spec = importlib.util.spec_from_file_location("pkv_build", os.path.join(ROOT, "llm-engine_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    import oracle
    if not os.path.exists(oracle.ORC_PATH):
        oracle.build()


@pytest.fixture(scope="session")
def pkv():
    """The product package (its directory name has a hyphen, hence import_module)."""
    _ensure_built()
    return importlib.import_module("llm-engine_b200")


@pytest.fixture(scope="session")
def workloads(pkv):
    return importlib.import_module("llm-engine_b200.workloads")


@pytest.fixture(scope="session")
def orc():
    """The plain-C restatement of the reference's CPU path (the checker)."""
    _ensure_built()
    import oracle
    return oracle.load_orc()


@pytest.fixture(scope="session")
def ref():
    """The reference's own sources compiled behind oracle/ref_shim.cpp, or None."""
    import oracle
    if not os.path.exists(oracle.REF_PATH) and os.path.isdir(os.path.join(oracle.reference_root(), "include", "engine")):
        oracle.build()
    return oracle.load_ref()


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch
