"""Python test/bench tooling over the B200 StripedHyena2 libraries.

The product is the pair of C-ABI shared libraries built in-tree by
``build.py`` (``libevo_b200_ops.so``: operator level, ``libevo.so``: the
``evo_*`` model/context ABI).  This package only binds them with ctypes for the
tests and the benchmark; torch is used for device memory and streams.  There is
no CPU fallback: a missing library is an error.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
OPS_LIBRARY = PACKAGE_DIR / "libevo_b200_ops.so"
EVO_LIBRARY = PACKAGE_DIR / "libevo.so"

_P = ctypes.c_void_p
_Z = ctypes.c_size_t
_F = ctypes.c_float
_I = ctypes.c_int

# name -> argument types, in the order of include/evo_b200_ops.h
OPS_SIGNATURES: dict[str, list] = {
    "evo_b200_check_async_errors": [_P],
    "evo_b200_software_e4m3_quantize_bf16": [_P, _Z, _F, _P, _P, _P],
    "evo_b200_software_e4m3_quantize_f32_codes": [_P, _Z, _F, _P, _P],
    "evo_b200_software_e4m3_h100_linear": [_P, _P, _Z, _Z, _Z, _F, _F, _P, _P, _P],
    "evo_b200_e4m3_tensorcore_linear": [_P, _P, _Z, _Z, _Z, _F, _F, _P, _P, _P],
    "evo_b200_e4m3_quantize_rows": [_P, _Z, _Z, _P, _P, _P],
    "evo_b200_e4m3_codes_linear": [_P, _P, _P, _P, _P, _Z, _Z, _Z, _F, _I, _I, _P, _P],
    "evo_b200_bf16_linear": [_P, _P, _P, _P, _Z, _Z, _Z, _I, _I, _P, _P],
    "evo_b200_bf16_linear_split_k": [_P, _P, _P, _P, _Z, _Z, _Z, _I, _I, _P, _Z, _P, _P],
    "evo_b200_bf16_gated_up_projection": [_P, _P, _Z, _Z, _Z, _I, _P, _P],
    "evo_b200_interleave_gate_weights": [_P, _P, _Z, _Z, _P, _P],
    "evo_b200_bf16_rms_norm": [_P, _P, _Z, _Z, _F, _P, _P, _F, _P],
    "evo_b200_bf16_gelu": [_P, _Z, _P, _P],
    "evo_b200_bf16_gated_elementwise": [_P, _P, _Z, _I, _P, _P],
    "evo_b200_bf16_add": [_P, _P, _Z, _P, _P],
    "evo_b200_bf16_add_bias_inplace": [_P, _P, _Z, _Z, _P],
    "evo_b200_bf16_row_to_column_major": [_P, _Z, _Z, _P, _P],
    "evo_b200_embedding": [_P, _P, _Z, _Z, _Z, _P, _P],
    "evo_b200_bf16_split_hyena_projection": [_P, _Z, _Z, _P, _P, _P, _P],
    "evo_b200_bf16_fir_prefill_direct": [_P, _P, _I, _P, _Z, _Z, _Z, _Z, _I, _I, _P, _P, _P],
    "evo_b200_bf16_fir_continue_direct": [_P, _P, _I, _P, _Z, _Z, _Z, _Z, _I, _I, _P, _Z, _P, _P],
    "evo_b200_bf16_gated_fir_prefill": [_P, _P, _P, _P, _I, _P, _Z, _Z, _Z, _Z, _I, _P, _P, _P, _P],
    "evo_b200_bf16_gated_fir_prefill_window": [_P, _P, _P, _P, _I, _P, _Z, _Z, _Z, _Z, _Z, _I, _P, _P, _P],
    "evo_b200_bf16_hcl_prefill_window": [_P, _P, _P, _P, _P, _P, _Z, _Z, _Z, _Z, _P, _P, _P, _P],
    "evo_b200_bf16_projection_gated_fir_prefill": [_P, _P, _P, _I, _P, _Z, _Z, _Z, _Z, _I, _P, _P, _P, _P, _P],
    "evo_b200_bf16_hcl_prefill": [_P, _P, _P, _P, _P, _P, _Z, _Z, _Z, _I, _P, _P, _P, _P, _P],
    "evo_b200_bf16_hcl_prefill_noalloc": [_P, _P, _P, _P, _P, _P, _Z, _Z, _Z, _I, _P, _P, _P, _P],
    "evo_b200_bf16_projection_hcl_prefill": [_P, _P, _P, _P, _P, _Z, _Z, _Z, _I, _P, _P, _P, _P, _P, _P],
    "evo_b200_bf16_hcl_decode": [_P, _P, _P, _P, _P, _P, _Z, _Z, _P, _P, _P, _P],
    "evo_b200_bf16_hyena_decode_mixer": [_P, _P, _P, _P, _P, _I, _Z, _Z, _I, _P, _P, _P, _Z, _P, _Z, _P, _P],
    "evo_b200_bf16_split_rope_append": [_P, _P, _Z, _Z, _Z, _Z, _F, _I, _P, _P, _P, _Z, _P],
    "evo_b200_bf16_causal_attention": [_P, _P, _P, _Z, _Z, _Z, _Z, _P, _P],
    "evo_b200_bf16_causal_attention_mma_sync": [_P, _P, _P, _Z, _Z, _Z, _Z, _P, _P],
    "evo_b200_bf16_cached_cross_attention": [_P, _P, _P, _Z, _Z, _Z, _Z, _P, _P],
    "evo_b200_bf16_cached_cross_attention_probabilities": [_P, _P, _P, _Z, _Z, _Z, _Z, _P, _P, _P],
    "evo_b200_linear_executor_create": [_I, ctypes.POINTER(_P)],
    "evo_b200_linear_executor_linear": [_P, _P, _Z, _Z, _P, _I, _Z, _Z, _P, _I, _Z, _P],
    "evo_b200_e4m3_encode_array": [_P, _Z, _F, _P],
    "evo_b200_q8_kv_append": [_P, _P, _P, _P, _P, _P, _Z, _Z, _Z, _Z, _Z, _P],
    "evo_b200_q8_kv_expand": [_P, _P, _P, _P, _Z, _Z, _Z, _Z, _P, _P, _P],
    "evo_b200_q8_attention_decode": [_P, _P, _P, _P, _P, _Z, _Z, _Z, _Z, _Z, _P, _P],
}
# entry points that do not return a status
OPS_OTHER = ("evo_b200_last_error", "evo_b200_hcl_scratch_floats", "evo_b200_linear_executor_free",
             "evo_b200_linear_executor_name", "evo_b200_linear_executor_cached_bytes",
             "evo_b200_e4m3_encode", "evo_b200_e4m3_decode", "evo_b200_e4m3_scaled_roundtrip")


class OpsError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"[{code}] {message}")
        self.code = code


class Ops:
    """ctypes view of libevo_b200_ops.so; calls raise OpsError on failure."""

    def __init__(self, path: Path = OPS_LIBRARY):
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: run `python evo.cpp_b200/build.py` "
                "(there is no CPU fallback)")
        self.lib = ctypes.CDLL(str(path))
        self.lib.evo_b200_last_error.restype = ctypes.c_char_p
        self.lib.evo_b200_hcl_scratch_floats.restype = _Z
        self.lib.evo_b200_hcl_scratch_floats.argtypes = [_Z, _Z, _Z]
        self.lib.evo_b200_linear_executor_free.restype = None
        self.lib.evo_b200_linear_executor_free.argtypes = [_P]
        self.lib.evo_b200_linear_executor_name.restype = ctypes.c_char_p
        self.lib.evo_b200_linear_executor_cached_bytes.restype = _Z
        self.lib.evo_b200_linear_executor_cached_bytes.argtypes = [_P]
        self.lib.evo_b200_e4m3_encode.restype = ctypes.c_uint8
        self.lib.evo_b200_e4m3_encode.argtypes = [_F]
        self.lib.evo_b200_e4m3_decode.restype = _F
        self.lib.evo_b200_e4m3_decode.argtypes = [ctypes.c_uint8]
        self.lib.evo_b200_e4m3_scaled_roundtrip.restype = _F
        self.lib.evo_b200_e4m3_scaled_roundtrip.argtypes = [_F, _F]
        for name, argtypes in OPS_SIGNATURES.items():
            fn = getattr(self.lib, name)
            fn.restype = _I
            fn.argtypes = argtypes

    def last_error(self) -> str:
        return (self.lib.evo_b200_last_error() or b"").decode()

    def call(self, name: str, *args) -> None:
        status = getattr(self.lib, "evo_b200_" + name)(*args)
        if status != 0:
            raise OpsError(status, self.last_error())

    def status(self, name: str, *args) -> int:
        return getattr(self.lib, "evo_b200_" + name)(*args)

    def hcl_scratch_floats(self, length: int, width: int, modes: int) -> int:
        return int(self.lib.evo_b200_hcl_scratch_floats(length, width, modes))


_ops: Ops | None = None


def ops() -> Ops:
    global _ops
    if _ops is None:
        _ops = Ops()
    return _ops


def ptr(tensor) -> int | None:
    """Device (or host) address of a torch tensor / numpy array, None -> NULL."""
    if tensor is None:
        return None
    if hasattr(tensor, "data_ptr"):
        return tensor.data_ptr()
    return tensor.ctypes.data


def current_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
