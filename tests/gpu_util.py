"""Helpers for the GPU parity tests: move BF16 bit patterns / F32 / bytes between
numpy and torch device tensors and call the operator C ABI."""
from __future__ import annotations

import numpy as np
import torch

from oracle_lib import bf16_to_f32, f32_to_bf16


# Device tensors created inline in a call expression must outlive the launch
# (a freed block is handed to the very next allocation); tests/conftest.py
# empties this list after every test.
KEEP_ALIVE: list = []


def _keep(tensor: torch.Tensor) -> torch.Tensor:
    KEEP_ALIVE.append(tensor)
    return tensor


def dev_bits(bits: np.ndarray) -> torch.Tensor:
    """uint16 BF16 bit patterns -> device int16 tensor (same bits)."""
    return _keep(torch.from_numpy(np.ascontiguousarray(bits, dtype=np.uint16).view(np.int16)).cuda())


def dev(array: np.ndarray) -> torch.Tensor:
    array = np.ascontiguousarray(array)
    if array.dtype == np.uint16:
        return dev_bits(array)
    if array.dtype == np.uint32:
        return _keep(torch.from_numpy(array.view(np.int32)).cuda())
    return _keep(torch.from_numpy(array).cuda())


def host_bits(tensor: torch.Tensor) -> np.ndarray:
    return tensor.cpu().numpy().view(np.uint16)


def empty_bits(*shape) -> torch.Tensor:
    return torch.empty(shape, dtype=torch.int16, device="cuda")


def rand_bf16(rng, *shape, scale=1.0) -> np.ndarray:
    return f32_to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def p(tensor):
    if tensor is None:
        return None
    KEEP_ALIVE.append(tensor)
    return tensor.data_ptr()


def ulp_mismatch_report(actual_bits: np.ndarray, expected_bits: np.ndarray):
    """Fraction of differing BF16 values and the largest difference in BF16 ulps
    (adjacent bit patterns of equal sign differ by one)."""
    a = actual_bits.astype(np.int32).ravel()
    e = expected_bits.astype(np.int32).ravel()
    differ = a != e
    if not differ.any():
        return 0.0, 0
    # map sign-magnitude patterns to a monotonic integer line
    mono = lambda x: np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    gap = np.abs(mono(a) - mono(e))
    return float(differ.mean()), int(gap.max())


def assert_close_bits(actual_bits, expected_bits, atol, rtol, min_cosine=None):
    actual = bf16_to_f32(actual_bits).astype(np.float64).ravel()
    expected = bf16_to_f32(expected_bits).astype(np.float64).ravel()
    assert np.all(np.isfinite(actual)), "non-finite output"
    bound = atol + rtol * np.abs(expected)
    worst = np.max(np.abs(actual - expected) - bound)
    assert worst <= 0, f"tolerance exceeded by {worst}"
    if min_cosine is not None:
        cosine = float(actual @ expected / (np.linalg.norm(actual) * np.linalg.norm(expected) + 1e-30))
        assert cosine >= min_cosine, cosine
