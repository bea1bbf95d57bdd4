"""Pins the CPU oracle (oracle/evo_oracle.cpp) against upstream's own golden
vectors and against outputs of upstream code captured in tests/golden/
(see tests/golden/make_golden.py).  Runs without a GPU."""
from __future__ import annotations

from pathlib import Path

import numpy as np
import pytest

from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

GOLDEN = Path(__file__).resolve().parent / "golden"

# (value, code) pairs of upstream tests/test_fp8.cpp:21-33.
E4M3_KNOWN = [
    (-448.0, 0xFE), (-432.0, 0xFE), (-416.0, 0xFD), (-1.25, 0xBA), (-1.1875, 0xBA),
    (-1.125, 0xB9), (-1.0625, 0xB8), (-1.0, 0xB8), (-0.5, 0xB0), (-0.015625, 0x88),
    (-0.00390625, 0x82), (-0.001953125, 0x81), (-0.0009765625, 0x80), (-0.0, 0x80),
    (0.0, 0x00), (0.0009765625, 0x00), (0.001953125, 0x01), (0.0029296875, 0x02),
    (0.00390625, 0x02), (0.015625, 0x08), (0.5, 0x30), (1.0, 0x38), (1.0625, 0x38),
    (1.125, 0x39), (1.1875, 0x3A), (1.25, 0x3A), (416.0, 0x7D), (432.0, 0x7E),
    (448.0, 0x7E),
]

# BF16 input -> output bit pairs pinned upstream (src/cuda/ops.cu:125-139).
GELU_PINNED = [(0xC049, 0xBB2D), (0xC081, 0xB8EB), (0xC089, 0xB827), (0xC092, 0xB742),
               (0xC0A0, 0xB5C8), (0xC0A8, 0xB4FC), (0xC0AB, 0xB4AB)]


def test_e4m3_known_answers(oracle):
    for value, code in E4M3_KNOWN:
        assert oracle.lib.orc_e4m3_encode(value) == code, value
    # satfinite and NaN rules (tests/test_fp8.cpp:37-63)
    assert oracle.lib.orc_e4m3_encode(1000.0) == 0x7E
    assert oracle.lib.orc_e4m3_encode(-1000.0) == 0xFE
    assert oracle.lib.orc_e4m3_encode(float("inf")) == 0x7E
    assert oracle.lib.orc_e4m3_encode(float("-inf")) == 0xFE
    assert oracle.lib.orc_e4m3_encode(float("nan")) & 0x7F == 0x7F
    assert oracle.lib.orc_e4m3_decode(0x01) == 0.001953125
    assert oracle.lib.orc_e4m3_decode(0x7E) == 448.0
    assert oracle.lib.orc_e4m3_decode(0xFE) == -448.0
    assert np.isnan(oracle.lib.orc_e4m3_decode(0x7F))


def test_e4m3_exhaustive_against_upstream_encoder(oracle):
    golden = np.load(GOLDEN / "e4m3_exhaustive.npz")
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    for scale in (1.0, 5.75, 0.03125):
        codes = np.empty(65536, np.uint8)
        oracle.quantize_bf16(ptr(bits), 65536, scale, ptr(codes), None)
        expected = golden[f"codes_scale_{scale}"]
        nan = np.isnan(bf16_to_f32(bits))
        assert np.array_equal(codes[~nan], expected[~nan])
        assert np.all((codes[nan] & 0x7F) == 0x7F)
    decoded = np.array([oracle.lib.orc_e4m3_decode(c) for c in range(256)], np.float32)
    assert np.array_equal(decoded[~np.isnan(decoded)], golden["decode"][~np.isnan(golden["decode"])])


@pytest.mark.parametrize("case", ["uniform", "small", "sparse", "spread", "upstream_test"])
def test_qgmma_matches_upstream_python_statement(oracle, case):
    golden = np.load(GOLDEN / "qgmma_golden.npz")
    x, w = golden[f"{case}_x"], golden[f"{case}_w"]
    out = np.empty((x.shape[0], w.shape[0]), np.uint16)
    oracle.qgmma_codes(ptr(x), ptr(w), x.shape[0], x.shape[1], w.shape[0],
                       float(golden[f"{case}_scale"]), ptr(out))
    assert np.array_equal(out, golden[f"{case}_y"])


def test_qgmma_linear_quantises_like_upstream_test(oracle):
    """The BF16 -> code -> emulate chain on the inputs of tests/test_cuda_ops.cu:433-503."""
    golden = np.load(GOLDEN / "qgmma_golden.npz")
    x_bf16 = np.ascontiguousarray(golden["upstream_test_x_bf16"])
    w = golden["upstream_test_w"]
    out = np.empty((3, 5), np.uint16)
    oracle.qgmma_linear(ptr(x_bf16), ptr(w), 3, 64, 5, 5.75, 0.03125, ptr(out))
    assert np.array_equal(out, golden["upstream_test_y"])


def test_gelu_pinned_bits(oracle):
    inputs = np.array([a for a, _ in GELU_PINNED], np.uint16)
    out = np.empty_like(inputs)
    oracle.gelu(ptr(inputs), len(inputs), ptr(out))
    assert out.tolist() == [b for _, b in GELU_PINNED]


def test_hcl_decode_reduction_tree_known_answer(oracle):
    """tests/test_cuda_hyena.cu:775-826: 16 residues, unit state -> -0.240234375."""
    residues = np.array([0.191467106, 3.08442359e-5, 27.5075665, -1.320715e-5, -0.159456432,
                         90.2677231, 5.88860703, 3.43213558, -132.08371, 0.391455323,
                         -6.85143023e-5, 0.891909838, -0.0767612457, -0.0025979632,
                         0.0283694491, 3.48360705], np.float32)
    one = f32_to_bf16(np.array([1.0], np.float32))
    zero = f32_to_bf16(np.array([0.0], np.float32))
    state = np.ones(16, np.float32)
    poles = np.zeros(16, np.float32)
    out = np.empty(1, np.uint16)
    gated = np.empty(1, np.uint16)
    oracle.hcl_decode(ptr(one), ptr(zero), ptr(one), ptr(zero), ptr(poles), ptr(residues),
                      1, 16, ptr(state), ptr(gated), ptr(out))
    assert bf16_to_f32(out)[0] == np.float32(-0.240234375)
    assert bf16_to_f32(gated)[0] == 0.0
    assert np.array_equal(state, np.ones(16, np.float32))


def _close(actual_bits, expected, atol=2e-2, rtol=2e-2):
    actual = bf16_to_f32(actual_bits).astype(np.float64)
    np.testing.assert_allclose(actual, np.asarray(expected, np.float64).reshape(actual.shape),
                               atol=atol, rtol=rtol)


def test_operator_math_against_upstream_cpu_reference(oracle):
    """Oracle ops (BF16 rounding chains) vs upstream's F32 operator
    specification on BF16-representable inputs; differences are the BF16
    roundings themselves."""
    g = np.load(GOLDEN / "ref_cpu_ops.npz")
    rb = lambda a: bf16_to_f32(f32_to_bf16(a))
    keep = []  # temporaries must outlive the foreign call that reads them

    def ptr(array):
        if array is None:
            return None
        array = np.ascontiguousarray(array)
        keep.append(array)
        return array.ctypes.data

    # linear: inputs rounded to BF16, so recompute upstream's F32 result on them
    x, w, b = rb(g["lin_x"]), rb(g["lin_w"]), rb(g["lin_b"])
    out = np.empty((x.shape[0], w.shape[0]), np.uint16)
    oracle.linear_bf16(ptr(f32_to_bf16(x)), ptr(f32_to_bf16(w)), ptr(f32_to_bf16(b)), None,
                       x.shape[0], x.shape[1], w.shape[0], 1, ptr(out))
    _close(out, x.astype(np.float64) @ w.T.astype(np.float64) + b, atol=3e-2)
    _close(out, g["lin_y"], atol=0.12, rtol=5e-2)  # vs unrounded-input upstream output

    # rms norm
    x = g["rms_x"]
    out = np.empty(x.shape, np.uint16)
    oracle.rms_norm(ptr(f32_to_bf16(x)), ptr(np.ascontiguousarray(g["rms_scale"])), x.shape[0],
                    x.shape[1], 1e-6, ptr(out))
    _close(out, g["rms_y"], atol=3e-2, rtol=3e-2)

    # FIR (per-channel filters => groups == channels)
    x = g["fir_x"]
    length, channels = x.shape
    for taps in (3, 7, 128):
        wt, bias = g[f"fir_w_{taps}"], g[f"fir_b_{taps}"]
        for conv in (0, 1):
            for mult in (0, 1):
                out = np.empty(x.shape, np.uint16)
                oracle.fir_prefill(ptr(f32_to_bf16(x)), ptr(f32_to_bf16(wt)), 0,
                                   ptr(f32_to_bf16(bias)), mult, length, channels, channels,
                                   taps, 0 if conv else 1, ptr(out), None)
                _close(out, g[f"fir_y_{taps}_{conv}_{mult}"], atol=0.15, rtol=5e-2)

    # HCL: recurrence contract (mode 1 from a zero state) and FFT-path contract (mode 0)
    x2, x1, v = g["hcl_x2"], g["hcl_x1"], g["hcl_v"]
    length, channels = x2.shape
    modes = g["hcl_lp"].shape[1]
    for mode in (0, 1):
        state = np.zeros((channels, modes), np.float32)
        out = np.empty(x2.shape, np.uint16)
        oracle.hcl_prefill(ptr(f32_to_bf16(x2)), ptr(f32_to_bf16(x1)), ptr(f32_to_bf16(v)),
                           ptr(f32_to_bf16(g["hcl_d"])), ptr(np.ascontiguousarray(g["hcl_lp"])),
                           ptr(np.ascontiguousarray(g["hcl_res"])), length, channels, modes,
                           mode, ptr(state), None, ptr(out))
        _close(out, g["hcl_y"], atol=0.25, rtol=6e-2)
        np.testing.assert_allclose(state, g["hcl_state"], atol=0.1, rtol=3e-2)

    # RoPE (projection-major packing of q|k|v) and attention
    q, k = g["rope_q"], g["rope_k"]
    t, heads, hd = q.shape
    qkv = np.concatenate([q.reshape(t, -1), k.reshape(t, -1), np.zeros((t, heads * hd), np.float32)], 1)
    qo = np.empty((t, heads * hd), np.uint16)
    kc = np.zeros((5 + t, heads * hd), np.uint16)
    vc = np.zeros_like(kc)
    oracle.split_rope_append(ptr(f32_to_bf16(qkv)), ptr(np.ascontiguousarray(g["rope_inv"])), t,
                             heads, hd, 5, 2.0, 0, ptr(qo), ptr(kc), ptr(vc))
    _close(qo, g["rope_qr"].reshape(t, -1), atol=4e-2, rtol=2e-2)
    _close(kc[5:], g["rope_kr"].reshape(t, -1), atol=4e-2, rtol=2e-2)

    q, k, v = g["att_q"], g["att_k"], g["att_v"]
    for fn in (oracle.causal_attention, oracle.cached_attention):
        out = np.empty((t, heads * hd), np.uint16)
        fn(ptr(f32_to_bf16(q.reshape(t, -1))), ptr(f32_to_bf16(k.reshape(t, -1))),
           ptr(f32_to_bf16(v.reshape(t, -1))), t, t, heads, hd, ptr(out))
        _close(out, g["att_y"].reshape(t, -1), atol=5e-2, rtol=3e-2)


def test_product_host_codec_matches_upstream_and_oracle(pkg, oracle):
    """The library's own host E4M3FN codec (csrc/fp8_codec.cpp, upstream
    src/fp8.cpp:26-77) against upstream's 29 known answers, upstream's encoder
    over every BF16 bit pattern, and the oracle over a sweep of F32 patterns."""
    lib = pkg.Ops().lib
    for value, code in E4M3_KNOWN:
        assert lib.evo_b200_e4m3_encode(value) == code, value
    for value, code in [(1000.0, 0x7E), (-1000.0, 0xFE), (float("inf"), 0x7E), (float("-inf"), 0xFE)]:
        assert lib.evo_b200_e4m3_encode(value) == code
    assert lib.evo_b200_e4m3_encode(float("nan")) & 0x7F == 0x7F
    golden = np.load(GOLDEN / "e4m3_exhaustive.npz")
    values = bf16_to_f32(np.arange(65536, dtype=np.uint32).astype(np.uint16))
    finite = ~np.isnan(values)
    for scale in (1.0, 5.75, 0.03125):
        codes = np.empty(65536, np.uint8)
        with np.errstate(over="ignore", invalid="ignore"):
            assert lib.evo_b200_e4m3_encode_array(ptr(np.ascontiguousarray(values)), 65536, scale, ptr(codes)) == 0
        assert np.array_equal(codes[finite], golden[f"codes_scale_{scale}"][finite])
    decoded = np.array([lib.evo_b200_e4m3_decode(c) for c in range(256)], np.float32)
    keep = ~np.isnan(golden["decode"])
    assert np.array_equal(decoded[keep], golden["decode"][keep]) and np.isnan(decoded[0x7F]) and np.isnan(decoded[0xFF])
    # F32 patterns between the BF16 ones: every rounding boundary of the 126 finite
    # codes and its float neighbours, plus a seeded sweep of all exponents
    rng = np.random.default_rng(5)
    sweep = rng.integers(0, 1 << 32, 200000, dtype=np.uint64).astype(np.uint32).view(np.float32)
    grid = np.sort(golden["decode"][:0x7F].astype(np.float64))
    mid = ((grid[1:] + grid[:-1]) / 2).astype(np.float32)
    edges = np.concatenate([np.nextafter(mid, np.float32(0)), mid, np.nextafter(mid, np.float32(1e9))])
    for batch in (sweep, edges, -edges):
        batch = np.ascontiguousarray(batch[~np.isnan(batch)])
        codes = np.empty(batch.size, np.uint8)
        expected = np.empty(batch.size, np.uint8)
        assert lib.evo_b200_e4m3_encode_array(ptr(batch), batch.size, 1.0, ptr(codes)) == 0
        oracle.quantize_f32(ptr(batch), batch.size, 1.0, ptr(expected))
        assert np.array_equal(codes, expected)
    assert lib.evo_b200_e4m3_scaled_roundtrip(0.3, 4.0) == np.float32(lib.evo_b200_e4m3_decode(
        lib.evo_b200_e4m3_encode(np.float32(0.3) * np.float32(4.0)))) * np.float32(0.25)
    assert np.isnan(lib.evo_b200_e4m3_scaled_roundtrip(1.0, 0.0))
    assert lib.evo_b200_e4m3_encode_array(ptr(batch), batch.size, -1.0, ptr(codes)) == 2
