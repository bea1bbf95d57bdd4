"""Shared pytest plumbing: the `gpu` marker, the package loader (the package
directory name contains a dot, so it is imported by path) and library fixtures."""
from __future__ import annotations

import importlib.util
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))


def load_package():
    if "evo_cpp_b200" in sys.modules:
        return sys.modules["evo_cpp_b200"]
    pkg_dir = ROOT / "evo.cpp_b200"
    spec = importlib.util.spec_from_file_location(
        "evo_cpp_b200", pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
    module = importlib.util.module_from_spec(spec)
    sys.modules["evo_cpp_b200"] = module
    spec.loader.exec_module(module)
    return module


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def pkg():
    return load_package()


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib

    return oracle_lib.load()


@pytest.fixture(scope="session")
def ops(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return pkg.ops()


@pytest.fixture(autouse=True)
def _release_device_temporaries():
    yield
    for name in ("gpu_util", "oracle_lib"):
        module = sys.modules.get(name)
        if module is not None:
            module.KEEP_ALIVE.clear()
