"""The C-ABI libraries load and export exactly what include/*.h declares
(no compute calls: runs without a GPU)."""
from __future__ import annotations

import ctypes
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared(header: Path, prefix: str) -> set[str]:
    text = re.sub(r"/\*.*?\*/", "", header.read_text(), flags=re.S)
    text = re.sub(r"//[^\n]*", "", text)
    return set(re.findall(rf"\b({prefix}\w+)\s*\(", text))


def exported(library: Path) -> set[str]:
    out = subprocess.run(["nm", "-D", "--defined-only", str(library)], check=True,
                         capture_output=True, text=True).stdout
    return {line.split()[-1].split("@")[0] for line in out.splitlines() if line.strip()}


def test_ops_library_exports_every_declared_symbol(pkg):
    header = ROOT / "include" / "evo_b200_ops.h"
    names = declared(header, "evo_b200_")
    assert len(names) >= 28
    symbols = exported(pkg.OPS_LIBRARY)
    assert names <= symbols, sorted(names - symbols)
    assert {s for s in symbols if s.startswith("evo_b200_")} == names
    lib = ctypes.CDLL(str(pkg.OPS_LIBRARY))
    for name in names:
        assert getattr(lib, name) is not None
    # the Python binding table covers the header too
    bound = {"evo_b200_" + n.removeprefix("evo_b200_") for n in pkg.OPS_SIGNATURES}
    assert bound | set(pkg.OPS_OTHER) == names


def test_missing_library_fails_loudly(pkg, tmp_path):
    with pytest.raises(FileNotFoundError):
        pkg.Ops(tmp_path / "libevo_b200_ops.so")
