"""GPU parity of the dense / element-wise operators against the CPU oracle,
through the operator C ABI (include/evo_b200_ops.h)."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import (assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16,
                      stream, ulp_mismatch_report)
from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


def test_e4m3_quantise_every_bf16_value_bit_exact(ops, oracle):
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    nan = np.isnan(bf16_to_f32(bits))
    x = dev_bits(bits)
    for scale in (1.0, 5.75, 0.03125, 37.5):
        codes = torch.empty(65536, dtype=torch.uint8, device="cuda")
        dequant = torch.empty(65536, dtype=torch.float32, device="cuda")
        ops.call("software_e4m3_quantize_bf16", p(x), 65536, scale, p(codes), None, stream())
        expected = np.empty(65536, np.uint8)
        expected_dq = np.empty(65536, np.float32)
        oracle.quantize_bf16(ptr(bits), 65536, scale, ptr(expected), ptr(expected_dq))
        got = codes.cpu().numpy()
        assert np.array_equal(got[~nan], expected[~nan])
        assert np.all((got[nan] & 0x7F) == 0x7F)
        # scalar path with the dequantised copy
        ops.call("software_e4m3_quantize_bf16", p(x), 65536, scale, p(codes), p(dequant), stream())
        assert np.array_equal(codes.cpu().numpy()[~nan], expected[~nan])
        assert np.array_equal(dequant.cpu().numpy()[~nan], expected_dq[~nan])
    # F32 input variant
    values = bf16_to_f32(bits)[~nan].copy()
    codes = torch.empty(values.size, dtype=torch.uint8, device="cuda")
    ops.call("software_e4m3_quantize_f32_codes", p(dev(values)), values.size, 3.25, p(codes), stream())
    expected = np.empty(values.size, np.uint8)
    oracle.quantize_f32(ptr(values), values.size, 3.25, ptr(expected))
    assert np.array_equal(codes.cpu().numpy(), expected)


def test_e4m3_quantise_rejects_bad_scale(ops):
    x = dev_bits(np.zeros(16, np.uint16))
    codes = torch.empty(16, dtype=torch.uint8, device="cuda")
    assert ops.status("software_e4m3_quantize_bf16", p(x), 16, 0.0, p(codes), None, stream()) == 2
    assert ops.status("software_e4m3_quantize_bf16", p(x), 16, float("inf"), p(codes), None, stream()) == 2
    assert "invalid_argument" in ops.last_error()


def _emulated(ops, x_bits, w_codes, in_scale, out_scale):
    rows, inner = x_bits.shape
    columns = w_codes.shape[0]
    x, w = dev_bits(x_bits), dev(w_codes)
    scratch = torch.empty(rows * inner, dtype=torch.uint8, device="cuda")
    out = empty_bits(rows, columns)
    ops.call("software_e4m3_h100_linear", p(x), p(w), rows, inner, columns, in_scale, out_scale,
             p(scratch), p(out), stream())
    return host_bits(out)


def test_emulated_qgmma_upstream_test_configuration(ops):
    """rows 3 / K 64 / N 5 and the one-row decode shape of
    tests/test_cuda_ops.cu:433-503, expected values from upstream's Python statement."""
    g = np.load(GOLDEN / "qgmma_golden.npz")
    x_bits = np.ascontiguousarray(g["upstream_test_x_bf16"])
    w = np.ascontiguousarray(g["upstream_test_w"])
    out = _emulated(ops, x_bits, w, 5.75, 0.03125)
    assert np.array_equal(out, g["upstream_test_y"])
    out1 = _emulated(ops, x_bits[:1].copy(), w, 5.75, 0.03125)
    assert np.array_equal(out1, g["upstream_test_y"][:1])
    # K not a multiple of 32 is rejected
    x = dev_bits(x_bits)
    scratch = torch.empty(3 * 64, dtype=torch.uint8, device="cuda")
    out_t = empty_bits(3, 5)
    assert ops.status("software_e4m3_h100_linear", p(x), p(dev(w)), 3, 63, 5, 5.75, 0.03125,
                      p(scratch), p(out_t), stream()) == 2


@pytest.mark.parametrize("case", ["uniform", "small", "sparse", "spread"])
def test_emulated_qgmma_golden_codes(ops, case):
    """Committed golden vectors: codes in, BF16 bits out (scale 1 on the input
    so the quantiser is an identity on E4M3-representable values)."""
    g = np.load(GOLDEN / "qgmma_golden.npz")
    decode = np.load(GOLDEN / "e4m3_exhaustive.npz")["decode"]
    x_bits = f32_to_bf16(decode[g[f"{case}_x"]])  # every E4M3 value is exact in BF16
    out = _emulated(ops, x_bits, np.ascontiguousarray(g[f"{case}_w"]), 1.0, float(g[f"{case}_scale"]))
    assert np.array_equal(out, g[f"{case}_y"])


@pytest.mark.parametrize("rows,inner,columns", [(1, 4096, 96), (70, 96, 130), (128, 1024, 192), (257, 256, 65)])
def test_emulated_qgmma_random_shapes_bit_exact(ops, oracle, rows, inner, columns):
    rng = np.random.default_rng(rows * 7 + columns)
    x_bits = rand_bf16(rng, rows, inner)
    w_f = (rng.standard_normal((columns, inner)) * 0.02).astype(np.float32)
    w_scale = np.float32(448.0 / np.abs(w_f).max())
    w_codes = np.empty((columns, inner), np.uint8)
    oracle.quantize_f32(ptr(w_f), w_f.size, float(w_scale), ptr(w_codes))
    in_scale = np.float32(448.0 / np.abs(bf16_to_f32(x_bits)).max())
    out_scale = np.float32(np.float32(1.0) / in_scale) * np.float32(np.float32(1.0) / w_scale)
    out = _emulated(ops, x_bits, w_codes, float(in_scale), float(out_scale))
    expected = np.empty((rows, columns), np.uint16)
    oracle.qgmma_linear(ptr(x_bits), ptr(w_codes), rows, inner, columns, float(in_scale),
                        float(out_scale), ptr(expected))
    assert np.array_equal(out, expected)


def test_rms_norm_and_fused_codes(ops, oracle):
    rng = np.random.default_rng(3)
    # (3, 4096), (1, 8192), (8, 256): the few-row kernel of decode steps (width a multiple of 256)
    for rows, width in [(5, 1920), (33, 4096), (3, 8), (2, 513), (3, 4096), (1, 8192), (8, 256)]:
        x_bits = rand_bf16(rng, rows, width, scale=2.0)
        scale = (1 + 0.1 * rng.standard_normal(width)).astype(np.float32)
        out = empty_bits(rows, width)
        codes = torch.empty((rows, width), dtype=torch.uint8, device="cuda")
        ops.call("bf16_rms_norm", p(dev_bits(x_bits)), p(dev(scale)), rows, width, 1e-6, p(out),
                 p(codes), 11.5, stream())
        expected = np.empty((rows, width), np.uint16)
        oracle.rms_norm(ptr(x_bits), ptr(scale), rows, width, 1e-6, ptr(expected))
        got = host_bits(out)
        fraction, gap = ulp_mismatch_report(got, expected)
        # rsqrt(width) is a hardware approximation on the device: a row whose
        # BF16 denominator lands on the other side of a rounding boundary may
        # differ by one BF16 ulp.
        assert gap <= 1 and fraction < 0.02, (rows, width, fraction, gap)
        expected_codes = np.empty((rows, width), np.uint8)
        oracle.quantize_bf16(ptr(got), got.size, 11.5, ptr(expected_codes), None)
        assert np.array_equal(codes.cpu().numpy(), expected_codes)


def test_pointwise_bit_exact(ops, oracle):
    rng = np.random.default_rng(5)
    n = 8 * 1000 + 5
    a, b = rand_bf16(rng, n, scale=3.0), rand_bf16(rng, n, scale=3.0)
    da, db = dev_bits(a), dev_bits(b)
    out = empty_bits(n)
    expected = np.empty(n, np.uint16)
    ops.call("bf16_gated_elementwise", p(da), p(db), n, 0, p(out), stream())
    oracle.gate(ptr(a), ptr(b), n, 0, ptr(expected))
    assert np.array_equal(host_bits(out), expected)
    ops.call("bf16_add", p(da), p(db), n, p(out), stream())
    oracle.add(ptr(a), ptr(b), n, ptr(expected))
    assert np.array_equal(host_bits(out), expected)
    # GELU over every finite BF16 input
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite = np.isfinite(bf16_to_f32(bits))
    out = empty_bits(65536)
    ops.call("bf16_gelu", p(dev_bits(bits)), 65536, p(out), stream())
    expected = np.empty(65536, np.uint16)
    oracle.gelu(ptr(bits), 65536, ptr(expected))
    fraction, gap = ulp_mismatch_report(host_bits(out)[finite], expected[finite])
    # device erff vs libm erff: one BF16 ulp, more only in the far negative tail
    # where 1 + erf cancels (the region of upstream's seven pinned inputs)
    assert fraction < 2e-3, fraction
    values = bf16_to_f32(bits)[finite]
    body = np.abs(values) < 2.5
    _, body_gap = ulp_mismatch_report(host_bits(out)[finite][body], expected[finite][body])
    assert body_gap <= 1 and gap <= 16, (body_gap, gap)
    for given, wanted in [(0xC049, 0xBB2D), (0xC081, 0xB8EB), (0xC089, 0xB827), (0xC092, 0xB742),
                          (0xC0A0, 0xB5C8), (0xC0A8, 0xB4FC), (0xC0AB, 0xB4AB)]:
        assert host_bits(out)[given] == wanted


def test_embedding_split_transpose_bias(ops, oracle):
    rng = np.random.default_rng(9)
    table = rand_bf16(rng, 512, 24)
    tokens = rng.integers(0, 512, 37).astype(np.uint32)
    out = empty_bits(37, 24)
    ops.call("embedding", p(dev(tokens)), p(dev_bits(table)), 37, 24, 512, p(out), stream())
    assert np.array_equal(host_bits(out), table[tokens])
    # an id outside the table is not dereferenced: zero row + a sticky invalid_argument
    bad = tokens.copy()
    bad[5] = 512
    bad[20] = 0xFFFFFFFF
    out = empty_bits(37, 24)
    ops.call("embedding", p(dev(bad)), p(dev_bits(table)), 37, 24, 512, p(out), stream())
    with pytest.raises(RuntimeError, match="token ID exceeds model vocabulary"):
        ops.call("check_async_errors", stream())
    got = host_bits(out)
    assert not got[5].any() and not got[20].any()
    keep = np.ones(37, bool)
    keep[[5, 20]] = False
    assert np.array_equal(got[keep], table[tokens[keep]])
    ops.call("check_async_errors", stream())  # reported once, then clear
    proj = rand_bf16(rng, 11, 3 * 10)
    x2, x1, v = empty_bits(11, 10), empty_bits(11, 10), empty_bits(11, 10)
    ops.call("bf16_split_hyena_projection", p(dev_bits(proj)), 11, 10, p(x2), p(x1), p(v), stream())
    triples = proj.reshape(11, 10, 3)
    assert np.array_equal(host_bits(x2), triples[:, :, 0])
    assert np.array_equal(host_bits(x1), triples[:, :, 1])
    assert np.array_equal(host_bits(v), triples[:, :, 2])
    m = rand_bf16(rng, 37, 53)
    out = empty_bits(53, 37)
    ops.call("bf16_row_to_column_major", p(dev_bits(m)), 37, 53, p(out), stream())
    assert np.array_equal(host_bits(out), m.T)
    bias = rand_bf16(rng, 53)
    dm = dev_bits(m)
    ops.call("bf16_add_bias_inplace", p(dm), p(dev_bits(bias)), 37, 53, stream())
    expected = np.empty((37, 53), np.uint16)
    oracle.add(ptr(m), ptr(np.ascontiguousarray(np.broadcast_to(bias, (37, 53)))), 37 * 53, ptr(expected))
    assert np.array_equal(host_bits(dm), expected)
