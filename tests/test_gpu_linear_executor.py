"""Dense-linear offload with upstream's LinearExecutor contract
(src/linear_executor.hpp:13-28): F32 host activations, F32, BF16 or E4M3 host weights,
optional bias, F32 host output - about 18 bits of the absolute sum from BF16-plane
products on the tensor cores, weights cached by host address."""
from __future__ import annotations

import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
F32, BF16, E4M3 = 0, 1, 2


def to_bf16_bits(values: np.ndarray) -> np.ndarray:
    bits = values.astype(np.float32).view(np.uint32).astype(np.uint64)
    return (((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16) & 0xFFFF).astype(np.uint16)


def widen(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


@pytest.fixture()
def executor(ops):
    handle = ctypes.c_void_p()
    ops.call("linear_executor_create", 0, ctypes.byref(handle))
    yield handle
    ops.lib.evo_b200_linear_executor_free(handle)


def run(ops, executor, x, weight, weight_dtype, bias=None, bias_dtype=F32):
    rows, k = x.shape
    n = weight.shape[0]
    out = np.empty((rows, n), np.float32)
    ops.call("linear_executor_linear", executor, x.ctypes.data, rows, k, weight.ctypes.data, weight_dtype,
             weight.size, n, None if bias is None else bias.ctypes.data, bias_dtype,
             0 if bias is None else bias.size, out.ctypes.data)
    return out


@pytest.mark.parametrize("rows,k,n", [(1, 512, 384), (37, 1000, 200), (300, 4096, 1024), (130, 72, 64)])
@pytest.mark.parametrize("weight_dtype", [BF16, F32])
def test_matches_float64_reference(ops, executor, rows, k, n, weight_dtype):
    rng = np.random.default_rng(rows + k + weight_dtype)
    x = np.ascontiguousarray(rng.standard_normal((rows, k)).astype(np.float32) * 3.0)
    w32 = (rng.standard_normal((n, k)) * 0.05).astype(np.float32)
    if weight_dtype == BF16:
        weight = to_bf16_bits(w32)
        w_value = widen(weight)
        bias = to_bf16_bits((rng.standard_normal(n) * 0.5).astype(np.float32))
        bias_value, bias_dtype = widen(bias), BF16
    else:
        weight, w_value = w32, w32
        bias = (rng.standard_normal(n) * 0.5).astype(np.float32)
        bias_value, bias_dtype = bias, F32
    got = run(ops, executor, x, weight, weight_dtype, bias, bias_dtype)
    want = x.astype(np.float64) @ w_value.astype(np.float64).T + bias_value.astype(np.float64)
    # The operands are represented to ~2^-24; the tensor-core accumulator truncates when it
    # aligns partial sums (768 accumulation steps at k = 4096), which leaves a few 1e-6 of the absolute
    # sum - BF16 activations would leave 4e-3.
    budget = (np.abs(x).astype(np.float64) @ np.abs(w_value).astype(np.float64).T + np.abs(bias_value)) * 4e-6
    worst = float(np.max(np.abs(got - want) / (budget + 1e-7)))
    assert worst <= 1.0, worst
    # without a bias, and again from the cache: identical bits
    first = run(ops, executor, x, weight, weight_dtype)
    cached_before = ops.lib.evo_b200_linear_executor_cached_bytes(executor)
    second = run(ops, executor, x, weight, weight_dtype)
    assert np.array_equal(first, second)
    assert ops.lib.evo_b200_linear_executor_cached_bytes(executor) == cached_before > 0
    assert np.all(np.abs(first - (want - bias_value)) <= budget + 1e-7)


def test_e4m3_weight_views_are_decoded_like_upstreams_executor(ops, executor):
    """The 1B- and 40B-shaped artifacts carry E4M3 projection weights; upstream's Metal executor
    decodes the raw codes without a scale (src/mps/model.mm:42-58).  Every finite code is a BF16
    value, so the product is as exact as with BF16 weights."""
    rng = np.random.default_rng(8)
    rows, k, n = 70, 1920, 320
    x = np.ascontiguousarray(rng.standard_normal((rows, k)).astype(np.float32))
    codes = rng.integers(0, 256, (n, k)).astype(np.uint8)
    codes[(codes & 0x7F) == 0x7F] = 0x38                      # no NaN codes in a weight
    decoded = np.array([ops.lib.evo_b200_e4m3_decode(c) for c in range(256)], np.float32)
    w_value = decoded[codes] * np.float32(1.0)
    bias = (rng.standard_normal(n) * 0.5).astype(np.float32)
    got = run(ops, executor, x, codes, E4M3, bias, F32)
    want = x.astype(np.float64) @ w_value.astype(np.float64).T + bias
    budget = (np.abs(x).astype(np.float64) @ np.abs(w_value).astype(np.float64).T + np.abs(bias)) * 4e-6
    assert np.all(np.abs(got - want) <= budget + 1e-7)


def test_contract_errors(ops, executor):
    assert ops.lib.evo_b200_linear_executor_name() == b"b200-tcgen05-bf16x3"
    x = np.zeros((2, 64), np.float32)
    w = np.zeros((64, 64), np.float32)
    out = np.zeros((2, 64), np.float32)
    # inconsistent dimensions: upstream's "internal" status
    assert ops.status("linear_executor_linear", executor, x.ctypes.data, 2, 64, w.ctypes.data, F32, 100, 64, None,
                      0, 0, out.ctypes.data) == 70
    assert ops.status("linear_executor_linear", executor, x.ctypes.data, 2, 64, w.ctypes.data, 3, w.size, 64, None,
                      0, 0, out.ctypes.data) == 5      # no such weight type
    assert ops.status("linear_executor_linear", executor, x.ctypes.data, 2, 64, w.ctypes.data, F32, w.size, 64,
                      w.ctypes.data, E4M3, 64, out.ctypes.data) == 5   # biases are F32 or BF16
    narrow = np.zeros((8, 64), np.float32)
    assert ops.status("linear_executor_linear", executor, x.ctypes.data, 2, 64, narrow.ctypes.data, F32, narrow.size,
                      8, None, 0, 0, out.ctypes.data) == 5
    assert ops.status("linear_executor_linear", executor, None, 2, 64, w.ctypes.data, F32, w.size, 64, None, 0, 0,
                      out.ctypes.data) == 2
    handle = ctypes.c_void_p()
    assert ops.status("linear_executor_create", 99, ctypes.byref(handle)) == 2
