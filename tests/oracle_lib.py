"""ctypes binding of oracle/libevo_oracle.so (the CPU checker) with numpy
helpers.  BF16 tensors travel as uint16 bit patterns."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "oracle" / "libevo_oracle.so"

P, Z, F, I = ctypes.c_void_p, ctypes.c_size_t, ctypes.c_float, ctypes.c_int

SIGNATURES = {
    "orc_quantize_bf16": [P, Z, F, P, P],
    "orc_quantize_f32": [P, Z, F, P],
    "orc_qgmma_codes": [P, P, Z, Z, Z, F, P],
    "orc_qgmma_linear": [P, P, Z, Z, Z, F, F, P],
    "orc_e4m3_exact_linear": [P, P, Z, Z, Z, F, F, P],
    "orc_rms_norm": [P, P, Z, Z, F, P],
    "orc_linear_bf16": [P, P, P, P, Z, Z, Z, I, P],
    "orc_gelu": [P, Z, P],
    "orc_gate": [P, P, Z, I, P],
    "orc_add": [P, P, Z, P],
    "orc_split": [P, Z, P, P, P],
    "orc_fir_prefill": [P, P, I, P, I, Z, Z, Z, Z, I, P, P],
    "orc_fir_step": [P, P, I, P, I, Z, Z, Z, Z, I, P, Z, P],
    "orc_gated_fir": [P, P, P, P, I, P, Z, Z, Z, Z, I, P, P, P],
    "orc_hcl_prefill": [P, P, P, P, P, P, Z, Z, Z, I, P, P, P],
    "orc_hcl_decode": [P, P, P, P, P, P, Z, Z, P, P, P],
    "orc_split_rope_append": [P, P, Z, Z, Z, Z, F, I, P, P, P],
    "orc_causal_attention": [P, P, P, Z, Z, Z, Z, P],
    "orc_cached_attention": [P, P, P, Z, Z, Z, Z, P],
    "orc_embedding": [P, P, Z, Z, P],
}


def f32_to_bf16(values) -> np.ndarray:
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
    return rounded.astype(np.uint16).reshape(np.shape(values))


def bf16_to_f32(bits) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


# Arrays built inline in a call expression must outlive the foreign call;
# tests/conftest.py empties this list after every test.
KEEP_ALIVE: list = []


def ptr(array):
    if array is None:
        return None
    assert array.flags["C_CONTIGUOUS"]
    KEEP_ALIVE.append(array)
    return array.ctypes.data


class Oracle:
    def __init__(self, lib):
        self.lib = lib
        lib.orc_e4m3_encode.restype = ctypes.c_uint8
        lib.orc_e4m3_encode.argtypes = [F]
        lib.orc_e4m3_decode.restype = F
        lib.orc_e4m3_decode.argtypes = [ctypes.c_uint8]
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = None
            fn.argtypes = argtypes

    def __getattr__(self, name):
        return getattr(self.lib, "orc_" + name)


def load() -> Oracle:
    source = ROOT / "oracle" / "evo_oracle.cpp"
    if not LIB.exists() or LIB.stat().st_mtime < source.stat().st_mtime:
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "libevo_oracle.so"], check=True,
                       capture_output=True)
    return Oracle(ctypes.CDLL(str(LIB)))
