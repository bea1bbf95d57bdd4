"""E4M3 projection GEMMs at the full projection shapes (K = 4096, N = 12,288 /
11,264 / 4,096, M = 16 ... 8,192 tokens), in both modes:

* emulation mode against the oracle's restatement of upstream's software QGMMA
  (src/cuda/ops.cu:353-441; host statement tests/test_cuda_ops.cu:119-187):
  bit-exact.  An output element depends only on its activation row and its
  weight row, so the oracle is run on sampled rows x sampled columns of each
  shape (tile edges, first and last, seeded others) and once on a whole
  16 x 4,096 x 4,096 product;
* tcgen05 mode against the oracle's exact-product reference on the same samples
  (tolerance 2e-3 + 1e-2 |y|: F32 accumulation order and one BF16 rounding);
* the dynamic per-row quantisation of profile b200-fp8 (bit-exact codes and
  scales) and its row-scaled GEMM epilogues.

Activations N(0,1) BF16, weights N(0,0.02), both with per-tensor amax scaling.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import dev, dev_bits, empty_bits, host_bits, p, stream
from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu

K = 4096


def _operands(rows, outer, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, K, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(outer, K, device="cuda", generator=gen) * 0.02).bfloat16().float()
    w_scale = float(np.float32(448.0) / np.float32(w.abs().max().item()))
    codes = (w * w_scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    in_scale = float(np.float32(448.0) / np.float32(x.float().abs().max().item()))
    out_scale = float(np.float32(1.0 / np.float32(in_scale)) * np.float32(1.0 / np.float32(w_scale)))
    return x, codes, in_scale, out_scale


def _samples(rows, outer, seed, row_count=12, column_count=160):
    rng = np.random.default_rng(seed)
    row_edges = [0, 1, 127, 128, 129, 255, 256, rows - 2, rows - 1]
    column_edges = [0, 1, 63, 64, 127, 128, 255, 256, 257, outer - 257, outer - 256, outer - 129, outer - 128,
                    outer - 1]
    pick = lambda edges, limit, count: np.unique(np.concatenate([
        np.array([e for e in edges if 0 <= e < limit]), rng.integers(0, limit, count)]))[: count + len(edges)]
    return pick(row_edges, rows, row_count), pick(column_edges, outer, column_count)


@pytest.mark.parametrize("outer", [12288, 11264, 4096])
@pytest.mark.parametrize("rows", [16, 128, 1024, 8192])
def test_projection_grid_emulation_bit_exact_and_tensor_core_in_tolerance(ops, oracle, rows, outer):
    x, codes, in_scale, out_scale = _operands(rows, outer, rows + outer)
    scratch = torch.empty(rows * K, dtype=torch.uint8, device="cuda")
    emulated, fast = empty_bits(rows, outer), empty_bits(rows, outer)
    ops.call("software_e4m3_h100_linear", p(x), p(codes), rows, K, outer, in_scale, out_scale, p(scratch),
             p(emulated), stream())
    ops.call("e4m3_tensorcore_linear", p(x), p(codes), rows, K, outer, in_scale, out_scale, p(scratch), p(fast),
             stream())
    ops.call("check_async_errors", stream())
    take_rows, take_columns = _samples(rows, outer, rows * 7 + outer)
    x_host = np.ascontiguousarray(x.view(torch.int16).cpu().numpy().view(np.uint16)[take_rows])
    w_host = np.ascontiguousarray(codes.cpu().numpy()[take_columns])
    expected = np.empty((len(take_rows), len(take_columns)), np.uint16)
    oracle.qgmma_linear(ptr(x_host), ptr(w_host), len(take_rows), K, len(take_columns), in_scale, out_scale,
                        ptr(expected))
    got = host_bits(emulated)[np.ix_(take_rows, take_columns)]
    assert np.array_equal(got, expected), (rows, outer)
    exact = np.empty_like(expected)
    oracle.e4m3_exact_linear(ptr(x_host), ptr(w_host), len(take_rows), K, len(take_columns), in_scale, out_scale,
                             ptr(exact))
    a = bf16_to_f32(host_bits(fast)[np.ix_(take_rows, take_columns)]).astype(np.float64)
    e = bf16_to_f32(exact).astype(np.float64)
    assert np.all(np.abs(a - e) <= 2e-3 + 1e-2 * np.abs(e)), np.abs(a - e).max()
    # the two modes agree with each other everywhere within the operator tolerance
    full_a = bf16_to_f32(host_bits(fast)).astype(np.float32)
    full_e = bf16_to_f32(host_bits(emulated)).astype(np.float32)
    assert np.all(np.abs(full_a - full_e) <= 0.02 + 0.02 * np.abs(full_e))


def test_emulation_whole_product_16_rows(ops, oracle):
    rows, outer = 16, 4096
    x, codes, in_scale, out_scale = _operands(rows, outer, 99)
    scratch = torch.empty(rows * K, dtype=torch.uint8, device="cuda")
    emulated = empty_bits(rows, outer)
    ops.call("software_e4m3_h100_linear", p(x), p(codes), rows, K, outer, in_scale, out_scale, p(scratch),
             p(emulated), stream())
    x_host = np.ascontiguousarray(x.view(torch.int16).cpu().numpy().view(np.uint16))
    w_host = np.ascontiguousarray(codes.cpu().numpy())
    expected = np.empty((rows, outer), np.uint16)
    oracle.qgmma_linear(ptr(x_host), ptr(w_host), rows, K, outer, in_scale, out_scale, ptr(expected))
    assert np.array_equal(host_bits(emulated), expected)


@pytest.mark.parametrize("rows,width", [(5, 64), (300, 1920), (1024, 4096), (257, 11264)])
def test_row_quantise_codes_and_scales_bit_exact(ops, oracle, rows, width):
    rng = np.random.default_rng(rows + width)
    values = (rng.standard_normal((rows, width)) * rng.uniform(0.01, 30.0, (rows, 1))).astype(np.float32)
    values[1 % rows] = 0.0                                   # an all-zero row keeps scale 1
    values[2 % rows, ::3] = 0.0
    x = f32_to_bf16(values)
    codes = torch.empty((rows, width), dtype=torch.uint8, device="cuda")
    scales = torch.empty(rows, device="cuda")
    ops.call("e4m3_quantize_rows", p(dev_bits(x)), rows, width, p(codes), p(scales), stream())
    amax = np.abs(bf16_to_f32(x)).max(axis=1)
    quant = np.where(amax > 0, np.float32(448.0) / np.where(amax > 0, amax, 1).astype(np.float32), np.float32(1.0))
    quant = quant.astype(np.float32)
    expected = np.empty((rows, width), np.uint8)
    for r in range(rows):
        oracle.quantize_bf16(ptr(np.ascontiguousarray(x[r])), width, float(quant[r]), ptr(expected[r]), None)
    assert np.array_equal(codes.cpu().numpy(), expected)
    assert np.array_equal(scales.cpu().numpy(), (np.float32(1.0) / quant).astype(np.float32))
    assert expected[1 % rows].max() == 0 and ((expected & 0x7F) == 0x7E).any(axis=1).sum() >= rows - 1


@pytest.mark.parametrize("rows,inner,outer,gate", [(300, 1920, 640, 0), (1024, 4096, 4096, 0), (640, 1024, 2048, 1),
                                                   (130, 512, 512, 2)])
def test_row_scaled_e4m3_linear_epilogues(ops, oracle, rows, inner, outer, gate):
    """codes x codes on the FP8 tensor cores with alpha * row_scale[r], then bias + residual or the
    gate: against float64 products of the decoded codes, rounded where the epilogue rounds."""
    rng = np.random.default_rng(rows + outer + gate)
    decode = np.array([oracle.lib.orc_e4m3_decode(c) for c in range(256)], np.float64)
    x_codes = rng.integers(0, 256, (rows, inner)).astype(np.uint8)
    w_codes = rng.integers(0, 256, (outer, inner)).astype(np.uint8)
    x_codes[(x_codes & 0x7F) > 0x77] &= 0x8F                 # keep magnitudes moderate, no NaN codes
    w_codes[(w_codes & 0x7F) > 0x77] &= 0x8F
    row_scale = rng.uniform(0.001, 0.01, rows).astype(np.float32)
    alpha = 0.37
    product = (decode[x_codes] @ decode[w_codes].T) * alpha * row_scale[:, None].astype(np.float64)
    if gate:
        blocks = product.reshape(rows, outer // 256, 2, 128)
        first, second = blocks[:, :, 0, :].reshape(rows, -1), blocks[:, :, 1, :].reshape(rows, -1)
        rounded = lambda v: bf16_to_f32(f32_to_bf16(v.astype(np.float32))).astype(np.float64)
        if gate == 2:
            activated = np.empty(first.shape, np.uint16)
            oracle.gelu(ptr(f32_to_bf16(first.astype(np.float32))), first.size, ptr(activated))
            first = bf16_to_f32(activated).astype(np.float64)
        else:
            first = rounded(first)
        expected = first * rounded(second)
        out = empty_bits(rows, outer // 2)
        ops.call("e4m3_codes_linear", p(dev(x_codes)), p(dev(row_scale)), p(dev(w_codes)), None, None, rows, inner,
                 outer, alpha, 0, gate, p(out), stream())
    else:
        bias = f32_to_bf16((rng.standard_normal(outer) * 0.5).astype(np.float32))
        residual = f32_to_bf16(rng.standard_normal((rows, outer)).astype(np.float32))
        expected = product + bf16_to_f32(bias) + bf16_to_f32(residual)
        out = empty_bits(rows, outer)
        ops.call("e4m3_codes_linear", p(dev(x_codes)), p(dev(row_scale)), p(dev(w_codes)), p(dev_bits(bias)),
                 p(dev_bits(residual)), rows, inner, outer, alpha, 2, 0, p(out), stream())
    ops.call("check_async_errors", stream())
    got = bf16_to_f32(host_bits(out)).astype(np.float64)
    scale = np.abs(expected).max()
    assert np.all(np.abs(got - expected) <= 0.02 * scale * 0.05 + 0.02 * np.abs(expected)), \
        np.abs(got - expected).max()
