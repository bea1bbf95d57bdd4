"""GPU parity of the tcgen05 / CUDA-core projections through the C ABI.

Small shapes are checked against the CPU oracle; shapes too large for it are
checked against an F32 matmul of the same BF16 operands (tolerance 0.02 abs +
0.02 rel, the gate upstream applies to its cuBLASLt linear,
tests/test_cuda_ops.cu:252-369)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream
from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu


def _linear(ops, x, w, bias, residual, bias_mode, path):
    rows, inner = x.shape
    columns = w.shape[0]
    out = empty_bits(rows, columns)
    ops.call("bf16_linear", p(x), p(w), p(bias), p(residual), rows, inner, columns, bias_mode,
             path, p(out), stream())
    ops.call("check_async_errors", stream())
    return out


@pytest.mark.parametrize("path", [0, 1])
@pytest.mark.parametrize("rows,inner,columns", [(128, 256, 256), (200, 1920, 640), (16, 4096, 512),
                                               (1, 256, 128), (333, 320, 1000)])
def test_bf16_linear_against_oracle(ops, oracle, rows, inner, columns, path):
    rng = np.random.default_rng(rows + inner + columns)
    x, w = rand_bf16(rng, rows, inner), rand_bf16(rng, columns, inner, scale=0.05)
    bias, residual = rand_bf16(rng, columns), rand_bf16(rng, rows, columns)
    dx, dw, db, dr = dev_bits(x), dev_bits(w), dev_bits(bias), dev_bits(residual)
    for bias_mode, use_residual in [(0, False), (1, False), (2, True), (1, True)]:
        out = _linear(ops, dx, dw, db if bias_mode else None, dr if use_residual else None,
                      bias_mode, path)
        expected = np.empty((rows, columns), np.uint16)
        oracle.linear_bf16(ptr(x), ptr(w), ptr(bias) if bias_mode else None,
                           ptr(residual) if use_residual else None, rows, inner, columns,
                           bias_mode, ptr(expected))
        assert_close_bits(host_bits(out), expected, atol=0.02, rtol=0.02, min_cosine=0.9999)


def test_bf16_linear_tiny_fixture_shapes_use_cuda_core_path(ops, oracle):
    """Width 8 / inner 12 (the 50-layer test fixture) cannot be described to TMA."""
    rng = np.random.default_rng(1)
    for rows, inner, columns in [(4, 8, 24), (9, 12, 8), (1, 8, 512)]:
        x, w = rand_bf16(rng, rows, inner), rand_bf16(rng, columns, inner)
        out = _linear(ops, dev_bits(x), dev_bits(w), None, None, 0, 0)
        expected = np.empty((rows, columns), np.uint16)
        oracle.linear_bf16(ptr(x), ptr(w), None, None, rows, inner, columns, 0, ptr(expected))
        assert_close_bits(host_bits(out), expected, atol=0.02, rtol=0.02)


@pytest.mark.parametrize("rows,inner,columns", [(1024, 4096, 4096), (8192, 4096, 512), (2048, 11264, 4096),
                                               (1000, 1920, 5760)])
def test_bf16_linear_large_against_f32_matmul(ops, rows, inner, columns):
    torch.manual_seed(rows)
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(columns, inner, device="cuda") * 0.02).bfloat16()
    out = torch.empty(rows, columns, device="cuda", dtype=torch.bfloat16)
    ops.call("bf16_linear", p(x), p(w), None, None, rows, inner, columns, 0, 0, p(out), stream())
    ops.call("check_async_errors", stream())
    reference = x.float() @ w.float().T
    error = (out.float() - reference).abs()
    bound = 0.02 + 0.02 * reference.abs()
    assert bool((error <= bound).all()), float((error - bound).max())
    cosine = torch.nn.functional.cosine_similarity(out.float().flatten(), reference.flatten(), dim=0)
    assert float(cosine) > 0.99995


def test_pair_kernel_epilogues_at_ragged_sizes(ops):
    """600 rows (two full pair tiles and a ragged third) x 6400 / 12800 columns run on CTA pairs.
    Gated: the fused up-projection equals two linears and the gate bit for bit (same accumulators,
    same rounding points).  Bias + residual: against an F32 matmul with the BF16 rounding chain."""
    torch.manual_seed(600)
    rows, inner, hidden = 600, 512, 6400
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w1 = (torch.randn(hidden, inner, device="cuda") * 0.08).bfloat16()
    w2 = (torch.randn(hidden, inner, device="cuda") * 0.08).bfloat16()
    packed = torch.empty(2 * hidden, inner, device="cuda", dtype=torch.bfloat16)
    ops.call("interleave_gate_weights", p(w1), p(w2), hidden, inner, p(packed), stream())
    fused = torch.empty(rows, hidden, device="cuda", dtype=torch.bfloat16)
    ops.call("bf16_gated_up_projection", p(x), p(packed), rows, inner, hidden, 0, p(fused), stream())
    first, second = (torch.empty(rows, hidden, device="cuda", dtype=torch.bfloat16) for _ in range(2))
    ops.call("bf16_linear", p(x), p(w1), None, None, rows, inner, hidden, 0, 0, p(first), stream())
    ops.call("bf16_linear", p(x), p(w2), None, None, rows, inner, hidden, 0, 0, p(second), stream())
    unfused = torch.empty_like(fused)
    ops.call("bf16_gated_elementwise", p(first), p(second), rows * hidden, 0, p(unfused), stream())
    ops.call("check_async_errors", stream())
    assert torch.equal(fused.view(torch.int16), unfused.view(torch.int16))
    bias = torch.randn(hidden, device="cuda").bfloat16()
    residual = torch.randn(rows, hidden, device="cuda").bfloat16()
    out = torch.empty(rows, hidden, device="cuda", dtype=torch.bfloat16)
    ops.call("bf16_linear", p(x), p(w1), p(bias), p(residual), rows, inner, hidden, 1, 0, p(out), stream())
    ops.call("check_async_errors", stream())
    reference = ((x.float() @ w1.float().T + bias.float()).bfloat16().float() + residual.float())
    error = (out.float() - reference).abs()
    assert bool((error <= 0.03 + 0.02 * reference.abs()).all()), float(error.max())


def test_gated_up_projection_matches_two_linears_and_gate(ops, oracle):
    rng = np.random.default_rng(11)
    rows, inner, hidden = 150, 256, 384
    x = rand_bf16(rng, rows, inner)
    w1, w2 = rand_bf16(rng, hidden, inner, scale=0.08), rand_bf16(rng, hidden, inner, scale=0.08)
    dx, dw1, dw2 = dev_bits(x), dev_bits(w1), dev_bits(w2)
    packed = empty_bits(2 * hidden, inner)
    ops.call("interleave_gate_weights", p(dw1), p(dw2), hidden, inner, p(packed), stream())
    for activation in (0, 1):
        out = empty_bits(rows, hidden)
        ops.call("bf16_gated_up_projection", p(dx), p(packed), rows, inner, hidden, activation,
                 p(out), stream())
        ops.call("check_async_errors", stream())
        first = _linear(ops, dx, dw1, None, None, 0, 0)
        second = _linear(ops, dx, dw2, None, None, 0, 0)
        unfused = empty_bits(rows, hidden)
        ops.call("bf16_gated_elementwise", p(first), p(second), rows * hidden, activation, p(unfused),
                 stream())
        # same accumulators, same rounding points: identical bits
        mismatch = np.flatnonzero(host_bits(out).ravel() != host_bits(unfused).ravel())
        assert mismatch.size == 0, (activation, mismatch[:8], mismatch.size)
        if activation == 0:
            expected = np.empty((rows, hidden), np.uint16)
            first_bits, second_bits = host_bits(first), host_bits(second)
            oracle.gate(ptr(first_bits), ptr(second_bits), rows * hidden, 0, ptr(expected))
            assert np.array_equal(host_bits(out), expected)


@pytest.mark.parametrize("rows,inner,columns", [(64, 256, 384), (100, 1920, 5760), (16, 4096, 12288)])
def test_e4m3_tensorcore_linear_against_exact_products(ops, oracle, rows, inner, columns):
    rng = np.random.default_rng(columns)
    x = rand_bf16(rng, rows, inner)
    w_f = (rng.standard_normal((columns, inner)) * 0.02).astype(np.float32)
    w_scale = np.float32(448.0 / np.abs(w_f).max())
    w_codes = np.empty((columns, inner), np.uint8)
    oracle.quantize_f32(ptr(w_f), w_f.size, float(w_scale), ptr(w_codes))
    in_scale = np.float32(448.0 / np.abs(bf16_to_f32(x)).max())
    out_scale = float(np.float32(1.0 / in_scale) * np.float32(1.0 / w_scale))
    scratch = torch.empty(rows * inner, dtype=torch.uint8, device="cuda")
    out = empty_bits(rows, columns)
    ops.call("e4m3_tensorcore_linear", p(dev_bits(x)), p(dev(w_codes)), rows, inner, columns,
             float(in_scale), out_scale, p(scratch), p(out), stream())
    ops.call("check_async_errors", stream())
    if rows * inner * columns <= 1.2e9:
        expected = np.empty((rows, columns), np.uint16)
        oracle.e4m3_exact_linear(ptr(x), ptr(w_codes), rows, inner, columns, float(in_scale),
                                 out_scale, ptr(expected))
        # exact E4M3 products, F32 accumulation: only summation-order rounding
        assert_close_bits(host_bits(out), expected, atol=2e-3, rtol=1e-2, min_cosine=0.99999)
    # and the emulation profile stays within the tolerance gate of the tensor-core one
    emulated = empty_bits(rows, columns)
    ops.call("software_e4m3_h100_linear", p(dev_bits(x)), p(dev(w_codes)), rows, inner, columns,
             float(in_scale), out_scale, p(scratch), p(emulated), stream())
    assert_close_bits(host_bits(out), host_bits(emulated), atol=0.02, rtol=0.02, min_cosine=0.9999)


@pytest.mark.parametrize("rows,inner,columns", [(16, 4096, 4096), (32, 4096, 12288), (24, 11264, 4096),
                                               (31, 4096, 512), (9, 2048, 1024), (64, 4096, 4096),
                                               (100, 1920, 5760), (128, 4096, 22528), (128, 11264, 4096),
                                               (48, 4096, 512), (33, 4096, 200)])
def test_split_k_projection_against_f32_matmul(ops, rows, inner, columns):
    """9..128 rows with a workspace: the weights are the 128-row tensor-core operand and the tokens
    the narrow one, K is split over several CTAs per 128 weight rows, F32 partials are added in
    split order; bias, residual and their rounding points as in the one-pass kernel."""
    torch.manual_seed(rows + columns)
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w = (torch.randn(columns, inner, device="cuda") * 0.02).bfloat16()
    bias = (torch.randn(columns, device="cuda") * 0.5).bfloat16()
    residual = torch.randn(rows, columns, device="cuda").bfloat16()
    workspace = torch.empty(8 * rows * columns, device="cuda")
    out = torch.empty(rows, columns, device="cuda", dtype=torch.bfloat16)
    plain = torch.empty_like(out)
    for bias_mode in (1, 2):
        ops.call("bf16_linear_split_k", p(x), p(w), p(bias), p(residual), rows, inner, columns, bias_mode, 0,
                 p(workspace), workspace.numel() * 4, p(out), stream())
        ops.call("bf16_linear", p(x), p(w), p(bias), p(residual), rows, inner, columns, bias_mode, 0, p(plain),
                 stream())
        ops.call("check_async_errors", stream())
        reference = x.float() @ w.float().T + bias.float() + residual.float()
        error = (out.float() - reference).abs()
        assert bool((error <= 0.03 + 0.02 * reference.abs()).all()), float(error.max())
        # the one-pass kernel rounds the same sums: at most a BF16 ulp apart where F32 sums differ
        assert float((out.float() - plain.float()).abs().max()) <= 0.07
        assert float((out != plain).float().mean()) < 0.05
    # a workspace too small for any split falls back to the one-pass kernel: identical bits
    ops.call("bf16_linear_split_k", p(x), p(w), p(bias), p(residual), rows, inner, columns, 2, 0, p(workspace), 64,
             p(out), stream())
    assert torch.equal(out, plain)


def test_split_k_gated_up_projection(ops):
    torch.manual_seed(5)
    for rows, inner, hidden in ((28, 4096, 2048), (100, 4096, 11264)):
        _check_split_k_gated(ops, rows, inner, hidden)


def _check_split_k_gated(ops, rows, inner, hidden):
    x = torch.randn(rows, inner, device="cuda").bfloat16()
    w1 = (torch.randn(hidden, inner, device="cuda") * 0.02).bfloat16()
    w2 = (torch.randn(hidden, inner, device="cuda") * 0.02).bfloat16()
    packed = torch.empty(2 * hidden, inner, device="cuda", dtype=torch.bfloat16)
    ops.call("interleave_gate_weights", p(w1), p(w2), hidden, inner, p(packed), stream())
    workspace = torch.empty(8 * rows * 2 * hidden, device="cuda")
    for activation in (0, 1):
        split = torch.empty(rows, hidden, device="cuda", dtype=torch.bfloat16)
        fused = torch.empty_like(split)
        ops.call("bf16_linear_split_k", p(x), p(packed), None, None, rows, inner, 2 * hidden, 0, activation + 1,
                 p(workspace), workspace.numel() * 4, p(split), stream())
        ops.call("bf16_gated_up_projection", p(x), p(packed), rows, inner, hidden, activation, p(fused), stream())
        ops.call("check_async_errors", stream())
        first = (x.float() @ w1.float().T).bfloat16().float()
        if activation == 1:
            first = torch.nn.functional.gelu(first).bfloat16().float()
        reference = first * (x.float() @ w2.float().T).bfloat16().float()
        # a BF16 ulp of the product where a factor rounded the other way (values reach ~10 at 1.1 M outputs)
        assert bool(((split.float() - reference).abs() <= 0.05 + 0.02 * reference.abs()).all())
        assert bool(((split.float() - fused.float()).abs() <= 0.05 + 0.02 * fused.float().abs()).all())
        assert float((split != fused).float().mean()) < 0.05
