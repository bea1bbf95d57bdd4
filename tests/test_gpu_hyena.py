"""GPU parity of the Hyena FIR / modal operators against the CPU oracle,
through the operator C ABI.  Shapes follow upstream's operator tests
(tests/test_cuda_hyena.cu: L = 19 / 128 / 129, grouped filters, BF16 and F32
medium filters, cache hand-over to decode and continuation)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import (assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream,
                      ulp_mismatch_report)
from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("taps,groups,channels,length", [(3, 24, 24, 19), (7, 4, 16, 129), (128, 2, 6, 200),
                                                        (4, 2, 8, 1)])
def test_fir_prefill_direct_and_cache_bit_exact(ops, oracle, taps, groups, channels, length):
    rng = np.random.default_rng(taps * 100 + length)
    x, w, bias = rand_bf16(rng, length, channels), rand_bf16(rng, groups, taps, scale=0.3), rand_bf16(rng, channels)
    w32 = bf16_to_f32(w).copy()
    for orientation in (0, 1):
        for bias_mode, use_bias in [(0, False), (0, True), (1, True)]:
            for f32_filter in (0, 1):
                out = empty_bits(length, channels)
                cache = torch.full((channels, taps - 1), 7.0, device="cuda")
                ops.call("bf16_fir_prefill_direct", p(dev_bits(x)), p(dev(w32) if f32_filter else dev_bits(w)),
                         f32_filter, p(dev_bits(bias)) if use_bias else None, length, channels, groups,
                         taps, orientation, bias_mode, p(out), p(cache), stream())
                expected = np.empty((length, channels), np.uint16)
                expected_cache = np.empty((channels, taps - 1), np.float32)
                oracle.fir_prefill(ptr(x), ptr(w32) if f32_filter else ptr(w), f32_filter,
                                   ptr(bias) if use_bias else None, bias_mode, length, channels, groups,
                                   taps, 1 if orientation == 0 else 0, ptr(expected), ptr(expected_cache))
                assert np.array_equal(host_bits(out), expected)
                assert np.array_equal(cache.cpu().numpy(), expected_cache)


@pytest.mark.parametrize("taps,groups,channels", [(3, 12, 12), (7, 2, 8), (128, 4, 8)])
def test_fir_continue_and_decode_tree_bit_exact(ops, oracle, taps, groups, channels):
    """Prefill a short prompt (shorter than the filter for k=128), then continue
    with a multi-row chunk and single-row decode steps; outputs and the F32
    cache must match the oracle bit for bit."""
    rng = np.random.default_rng(taps)
    w = rand_bf16(rng, groups, taps, scale=0.3)
    bias = rand_bf16(rng, channels)
    for orientation, bias_mode in [(0, 0), (1, 1)]:
        prompt = rand_bf16(rng, 5, channels)
        out = empty_bits(5, channels)
        cache = torch.zeros((channels, taps - 1), device="cuda")
        ops.call("bf16_fir_prefill_direct", p(dev_bits(prompt)), p(dev_bits(w)), 0, p(dev_bits(bias)), 5,
                 channels, groups, taps, orientation, bias_mode, p(out), p(cache), stream())
        host_cache = np.empty((channels, taps - 1), np.float32)
        scratch = np.empty((5, channels), np.uint16)
        oracle.fir_prefill(ptr(prompt), ptr(w), 0, ptr(bias), bias_mode, 5, channels, groups, taps,
                           1 if orientation == 0 else 0, ptr(scratch), ptr(host_cache))
        cached = min(5, taps - 1)
        for length in (4, 1, 1, 140, 1):
            chunk = rand_bf16(rng, length, channels)
            out = empty_bits(length, channels)
            ops.call("bf16_fir_continue_direct", p(dev_bits(chunk)), p(dev_bits(w)), 0, p(dev_bits(bias)),
                     length, channels, groups, taps, orientation, bias_mode, p(cache), cached, p(out),
                     stream())
            expected = np.empty((length, channels), np.uint16)
            oracle.fir_step(ptr(chunk), ptr(w), 0, ptr(bias), bias_mode, length, channels, groups, taps,
                            1 if orientation == 0 else 0, ptr(host_cache), cached, ptr(expected))
            assert np.array_equal(host_bits(out), expected), (taps, length)
            assert np.array_equal(cache.cpu().numpy(), host_cache)
            cached = min(cached + length, taps - 1)


def _gated_inputs(rng, length, width):
    return rand_bf16(rng, length, width), rand_bf16(rng, length, width), rand_bf16(rng, length, width)


@pytest.mark.parametrize("length,width,groups", [(19, 16, 4), (128, 64, 8), (129, 130, 13), (1000, 256, 16),
                                                 (13, 9, 3)])  # odd width: the three-pass route
def test_hcs_fused_prefill_bit_exact(ops, oracle, length, width, groups):
    """k=7 cross-correlation: same tap order and rounding points as upstream's
    gate -> direct FIR -> gate chain, so the fused kernel is bit-identical."""
    rng = np.random.default_rng(length)
    x2, x1, v = _gated_inputs(rng, length, width)
    h = rand_bf16(rng, groups, 7, scale=0.4)
    out, pregate = empty_bits(length, width), empty_bits(length, width)
    cache = torch.full((width, 6), 3.0, device="cuda")
    ops.call("bf16_gated_fir_prefill", p(dev_bits(x2)), p(dev_bits(x1)), p(dev_bits(v)), p(dev_bits(h)), 0,
             None, length, width, groups, 7, 0, p(pregate), p(cache), p(out), stream())
    expected, expected_u = np.empty((length, width), np.uint16), np.empty((length, width), np.uint16)
    expected_cache = np.empty((width, 6), np.float32)
    oracle.gated_fir(ptr(x2), ptr(x1), ptr(v), ptr(h), 0, None, length, width, groups, 7, 1,
                     ptr(expected_u), ptr(expected_cache), ptr(expected))
    assert np.array_equal(host_bits(pregate), expected_u)
    assert np.array_equal(host_bits(out), expected)
    assert np.array_equal(cache.cpu().numpy(), expected_cache)


@pytest.mark.parametrize("length,width,groups,f32_filter", [(19, 8, 2, 1), (128, 64, 4, 0), (129, 64, 64, 0),
                                                           (700, 192, 12, 1), (19, 15, 5, 1), (129, 15, 5, 0)])
def test_hcm_fused_prefill(ops, oracle, length, width, groups, f32_filter):
    """k=128 causal convolution with the direct term.  Upstream evaluates it by
    FFT (tolerance 0.03 abs + 0.02 rel, cosine >= 0.999 in its own test); the
    direct kernel differs from the oracle's direct sum only by summation order."""
    rng = np.random.default_rng(length + width)
    x2, x1, v = _gated_inputs(rng, length, width)
    h = rand_bf16(rng, groups, 128, scale=0.1)
    h32 = bf16_to_f32(h).copy()
    direct = rand_bf16(rng, width)
    out = empty_bits(length, width)
    cache = torch.zeros((width, 127), device="cuda")
    pregate = empty_bits(length, width) if width % 2 else None  # an odd width runs as three passes and needs it
    ops.call("bf16_gated_fir_prefill", p(dev_bits(x2)), p(dev_bits(x1)), p(dev_bits(v)),
             p(dev(h32) if f32_filter else dev_bits(h)), f32_filter, p(dev_bits(direct)), length, width,
             groups, 128, 1, p(pregate) if pregate is not None else None, p(cache), p(out), stream())
    expected = np.empty((length, width), np.uint16)
    expected_cache = np.empty((width, 127), np.float32)
    oracle.gated_fir(ptr(x2), ptr(x1), ptr(v), ptr(h32) if f32_filter else ptr(h), f32_filter, ptr(direct),
                     length, width, groups, 128, 0, None, ptr(expected_cache), ptr(expected))
    fraction, _ = ulp_mismatch_report(host_bits(out), expected)
    assert fraction < 0.02, fraction  # summation order only
    assert_close_bits(host_bits(out), expected, atol=0.03, rtol=0.02, min_cosine=0.9999)
    assert np.array_equal(cache.cpu().numpy(), expected_cache)


@pytest.mark.parametrize("kind", ["hcs", "hcm"])
def test_projection_fed_fused_prefill_matches_unfused_chain(ops, oracle, kind):
    """Raw interleaved projection in, mixer output out: equals featurizer FIR
    (k=3, per-stream filters) -> split -> gated FIR evaluated by the oracle."""
    rng = np.random.default_rng(17)
    length, width = 300, 96
    taps, groups, orientation = (7, 6, 0) if kind == "hcs" else (128, 6, 1)
    projection = rand_bf16(rng, length, 3 * width)
    short = rand_bf16(rng, 3 * width, 3, scale=0.5)
    h = rand_bf16(rng, groups, taps, scale=0.2)
    direct = rand_bf16(rng, width) if kind == "hcm" else None
    out = empty_bits(length, width)
    inner_cache = torch.zeros((width, taps - 1), device="cuda")
    short_cache = torch.zeros((3 * width, 2), device="cuda")
    ops.call("bf16_projection_gated_fir_prefill", p(dev_bits(projection)), p(dev_bits(short)), p(dev_bits(h)),
             0, p(dev_bits(direct)) if direct is not None else None, length, width, groups, taps,
             orientation, None, p(inner_cache), p(short_cache), p(out), stream())
    filtered = np.empty((length, 3 * width), np.uint16)
    expected_short_cache = np.empty((3 * width, 2), np.float32)
    oracle.fir_prefill(ptr(projection), ptr(short), 0, None, 0, length, 3 * width, 3 * width, 3, 1,
                       ptr(filtered), ptr(expected_short_cache))
    x2, x1, v = (np.empty((length, width), np.uint16) for _ in range(3))
    oracle.split(ptr(filtered), length * width, ptr(x2), ptr(x1), ptr(v))
    expected = np.empty((length, width), np.uint16)
    expected_cache = np.empty((width, taps - 1), np.float32)
    oracle.gated_fir(ptr(x2), ptr(x1), ptr(v), ptr(h), 0, ptr(direct) if direct is not None else None,
                     length, width, groups, taps, 1 if orientation == 0 else 0, None, ptr(expected_cache),
                     ptr(expected))
    if kind == "hcs":
        assert np.array_equal(host_bits(out), expected)
    else:
        fraction, _ = ulp_mismatch_report(host_bits(out), expected)
        assert fraction < 0.02, fraction
        assert_close_bits(host_bits(out), expected, atol=0.03, rtol=0.02, min_cosine=0.9999)
    assert np.array_equal(inner_cache.cpu().numpy(), expected_cache)
    assert np.array_equal(short_cache.cpu().numpy(), expected_short_cache)


@pytest.mark.parametrize("length,width,groups,taps", [(19, 32, 2, 128), (127, 32, 2, 64), (129, 48, 3, 100),
                                                       (257, 16, 1, 33), (1000, 64, 4, 128)])
def test_projection_fed_hcm_on_tensor_cores_ragged_shapes(ops, oracle, length, width, groups, taps):
    """The tcgen05 Toeplitz kernel (groups of 16 channels, 32 < taps <= 128) at lengths below, at and
    across its 128-row tile, filters shorter than the strip, with and without the direct term; outputs
    against the unfused oracle chain, both decode caches bit for bit."""
    rng = np.random.default_rng(length * 7 + taps)
    projection = rand_bf16(rng, length, 3 * width)
    short = rand_bf16(rng, 3 * width, 3, scale=0.5)
    h = rand_bf16(rng, groups, taps, scale=0.2)
    direct = rand_bf16(rng, width) if taps != 64 else None
    out = empty_bits(length, width)
    inner_cache = torch.full((width, taps - 1), 3.0, device="cuda")
    short_cache = torch.zeros((3 * width, 2), device="cuda")
    ops.call("bf16_projection_gated_fir_prefill", p(dev_bits(projection)), p(dev_bits(short)), p(dev_bits(h)),
             0, p(dev_bits(direct)) if direct is not None else None, length, width, groups, taps,
             1, None, p(inner_cache), p(short_cache), p(out), stream())
    filtered = np.empty((length, 3 * width), np.uint16)
    expected_short_cache = np.empty((3 * width, 2), np.float32)
    oracle.fir_prefill(ptr(projection), ptr(short), 0, None, 0, length, 3 * width, 3 * width, 3, 1,
                       ptr(filtered), ptr(expected_short_cache))
    x2, x1, v = (np.empty((length, width), np.uint16) for _ in range(3))
    oracle.split(ptr(filtered), length * width, ptr(x2), ptr(x1), ptr(v))
    expected = np.empty((length, width), np.uint16)
    expected_cache = np.empty((width, taps - 1), np.float32)
    oracle.gated_fir(ptr(x2), ptr(x1), ptr(v), ptr(h), 0, ptr(direct) if direct is not None else None,
                     length, width, groups, taps, 0, None, ptr(expected_cache), ptr(expected))
    fraction, _ = ulp_mismatch_report(host_bits(out), expected)
    assert fraction < 0.02, fraction
    assert_close_bits(host_bits(out), expected, atol=0.03, rtol=0.02, min_cosine=0.9999)
    assert np.array_equal(inner_cache.cpu().numpy(), expected_cache)
    assert np.array_equal(short_cache.cpu().numpy(), expected_short_cache)


def test_projection_fed_hcm_gives_the_same_bits_on_concurrent_streams(ops):
    """The tcgen05 Toeplitz kernel hands tiles between its warps with mbarriers only; with several
    launches sharing the SMs its warps drift apart.  Six threads on six streams, every result equal to
    the one computed alone."""
    import threading

    rng = np.random.default_rng(41)
    width, groups, taps = 256, 16, 128
    jobs = []
    for length in (243, 130, 361, 517, 64, 205):
        tensors = [dev_bits(rand_bf16(rng, length, 3 * width)), dev_bits(rand_bf16(rng, 3 * width, 3, scale=0.5)),
                   dev_bits(rand_bf16(rng, groups, taps, scale=0.2)), dev_bits(rand_bf16(rng, width))]
        alone = empty_bits(length, width)
        ops.call("bf16_projection_gated_fir_prefill", p(tensors[0]), p(tensors[1]), p(tensors[2]), 0, p(tensors[3]),
                 length, width, groups, taps, 1, None, None, None, p(alone), stream())
        jobs.append((length, tensors, alone))
    torch.cuda.synchronize()
    failures = []

    def worker(job):
        length, tensors, alone = job
        own = torch.cuda.Stream()
        with torch.cuda.stream(own):
            out = empty_bits(length, width)
            for iteration in range(300):
                out.zero_()
                ops.call("bf16_projection_gated_fir_prefill", p(tensors[0]), p(tensors[1]), p(tensors[2]), 0,
                         p(tensors[3]), length, width, groups, taps, 1, None, None, None, p(out), own.cuda_stream)
                own.synchronize()
                if not torch.equal(out, alone):
                    failures.append((length, iteration))
                    return

    threads = [threading.Thread(target=worker, args=(job,)) for job in jobs]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    ops.call("check_async_errors", stream())
    assert not failures, failures


def _modal_params(rng, width, modes):
    radius = rng.uniform(0.9, 0.999, (width, modes))
    log_poles = np.log(radius).astype(np.float32)
    residues = (rng.standard_normal((width, modes)) * 0.02).astype(np.float32)
    return log_poles, residues


@pytest.mark.parametrize("length,width,modes", [(19, 8, 2), (128, 64, 16), (129, 64, 16), (1000, 96, 16),
                                                (9, 7, 3), (300, 6, 5), (65, 33, 16)])  # any-shape kernel
def test_hcl_prefill_output_and_state(ops, oracle, length, width, modes):
    """Chunked-scan prefill vs the FFT-path contract (exact convolution with the
    materialised filter, four BF16 roundings).  Upstream's own gate for this
    operator is 0.04 abs + 0.03 rel, cosine >= 0.999, state 1e-5 relative to
    its recurrence (tests/test_cuda_hyena.cu:672-689)."""
    rng = np.random.default_rng(length * 3 + width)
    x2, x1, v = _gated_inputs(rng, length, width)
    direct = rand_bf16(rng, width)
    log_poles, residues = _modal_params(rng, width, modes)
    out, pregate = empty_bits(length, width), empty_bits(length, width)
    state = torch.full((width, modes), 5.0, device="cuda")
    scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
    ops.call("bf16_hcl_prefill", p(dev_bits(x2)), p(dev_bits(x1)), p(dev_bits(v)), p(dev_bits(direct)),
             p(dev(log_poles)), p(dev(residues)), length, width, modes, 0, p(state), p(scratch),
             p(pregate), p(out), stream())
    expected, expected_u = np.empty((length, width), np.uint16), np.empty((length, width), np.uint16)
    expected_state = np.zeros((width, modes), np.float32)
    oracle.hcl_prefill(ptr(x2), ptr(x1), ptr(v), ptr(direct), ptr(log_poles), ptr(residues), length, width,
                       modes, 0, ptr(expected_state), ptr(expected_u), ptr(expected))
    assert np.array_equal(host_bits(pregate), expected_u)
    fraction, _ = ulp_mismatch_report(host_bits(out), expected)
    assert fraction < 0.03, fraction
    assert_close_bits(host_bits(out), expected, atol=0.04, rtol=0.03, min_cosine=0.9999)
    # The scan multiplies by expf(log_pole) once per row (segments of 64 rows or more), as
    # upstream's decode recurrence does; the oracle evaluates every power directly.  The rounding
    # of the pole then shows as ~n * 1e-7 relative on a term n rows old: 1e-4 absolute on states
    # of magnitude 1..15 with cancellation.
    np.testing.assert_allclose(state.cpu().numpy(), expected_state, rtol=2e-5, atol=1e-4)


def test_hcl_continuation_matches_single_pass_and_decode(ops, oracle):
    rng = np.random.default_rng(23)
    length, width, modes = 400, 64, 16
    x2, x1, v = _gated_inputs(rng, length, width)
    direct = rand_bf16(rng, width)
    log_poles, residues = _modal_params(rng, width, modes)
    d = {k: dev_bits(a) for k, a in dict(x2=x2, x1=x1, v=v, direct=direct).items()}
    lp, res = dev(log_poles), dev(residues)
    scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
    state = torch.zeros((width, modes), device="cuda")
    first = 150
    out_a = empty_bits(first, width)
    ops.call("bf16_hcl_prefill", p(d["x2"]), p(d["x1"]), p(d["v"]), p(d["direct"]), p(lp), p(res), first,
             width, modes, 0, p(state), p(scratch), None, p(out_a), stream())
    rest = length - first
    out_b = empty_bits(rest, width)
    offset = first * width * 2
    ops.call("bf16_hcl_prefill", p(d["x2"]) + offset, p(d["x1"]) + offset, p(d["v"]) + offset,
             p(d["direct"]), p(lp), p(res), rest, width, modes, 1, p(state), p(scratch), None, p(out_b),
             stream())
    # oracle: recurrence continuation from the oracle's own state after `first`
    host_state = np.zeros((width, modes), np.float32)
    scratch_out = np.empty((first, width), np.uint16)
    oracle.hcl_prefill(ptr(x2[:first].copy()), ptr(x1[:first].copy()), ptr(v[:first].copy()), ptr(direct),
                       ptr(log_poles), ptr(residues), first, width, modes, 0, ptr(host_state), None,
                       ptr(scratch_out))
    expected_b = np.empty((rest, width), np.uint16)
    oracle.hcl_prefill(ptr(x2[first:].copy()), ptr(x1[first:].copy()), ptr(v[first:].copy()), ptr(direct),
                       ptr(log_poles), ptr(residues), rest, width, modes, 1, ptr(host_state), None,
                       ptr(expected_b))
    assert_close_bits(host_bits(out_b), expected_b, atol=0.04, rtol=0.03, min_cosine=0.9999)
    np.testing.assert_allclose(state.cpu().numpy(), host_state, rtol=3e-5, atol=3e-5)
    # one decode step from the carried state
    row = [rand_bf16(rng, width) for _ in range(3)]
    out = empty_bits(width)
    ops.call("bf16_hcl_decode", p(dev_bits(row[0])), p(dev_bits(row[1])), p(dev_bits(row[2])), p(d["direct"]),
             p(lp), p(res), width, modes, p(state), None, p(out), stream())
    expected = np.empty(width, np.uint16)
    oracle.hcl_decode(ptr(row[0]), ptr(row[1]), ptr(row[2]), ptr(direct), ptr(log_poles), ptr(residues),
                      width, modes, ptr(host_state), None, ptr(expected))
    assert_close_bits(host_bits(out), expected, atol=0.02, rtol=0.02)


def test_hcl_continuation_at_an_odd_width_and_state_size(ops, oracle):
    """Width 7 with 3 modes (the shape of upstream's own operator test) takes the one-thread-per-channel
    kernel; the allocation-free entry needs no scratch for it.  A continuation rounds once."""
    rng = np.random.default_rng(31)
    length, width, modes, first = 40, 7, 3, 9
    x2, x1, v = _gated_inputs(rng, length, width)
    direct = rand_bf16(rng, width)
    log_poles, residues = _modal_params(rng, width, modes)
    state = torch.zeros((width, modes), device="cuda")
    host_state = np.zeros((width, modes), np.float32)
    lp, res, d = dev(log_poles), dev(residues), dev_bits(direct)
    for begin, end, mode in ((0, first, 0), (first, length, 1)):
        rows = end - begin
        part = [np.ascontiguousarray(a[begin:end]) for a in (x2, x1, v)]
        out, pregate = empty_bits(rows, width), empty_bits(rows, width)
        ops.call("bf16_hcl_prefill_noalloc", p(dev_bits(part[0])), p(dev_bits(part[1])), p(dev_bits(part[2])), p(d),
                 p(lp), p(res), rows, width, modes, mode, p(state), p(pregate), p(out), stream())
        expected, expected_u = np.empty((rows, width), np.uint16), np.empty((rows, width), np.uint16)
        oracle.hcl_prefill(ptr(part[0]), ptr(part[1]), ptr(part[2]), ptr(direct), ptr(log_poles), ptr(residues),
                           rows, width, modes, mode, ptr(host_state), ptr(expected_u), ptr(expected))
        assert np.array_equal(host_bits(pregate), expected_u)
        assert_close_bits(host_bits(out), expected, atol=0.04, rtol=0.03, min_cosine=0.9999)
        np.testing.assert_allclose(state.cpu().numpy(), host_state, rtol=3e-5, atol=3e-5)


def test_hcl_decode_reduction_tree_known_answer(ops):
    """tests/test_cuda_hyena.cu:775-826 (log-poles 0 make exp exact)."""
    residues = np.array([0.191467106, 3.08442359e-5, 27.5075665, -1.320715e-5, -0.159456432, 90.2677231,
                         5.88860703, 3.43213558, -132.08371, 0.391455323, -6.85143023e-5, 0.891909838,
                         -0.0767612457, -0.0025979632, 0.0283694491, 3.48360705], np.float32)
    one, zero = dev_bits(f32_to_bf16(np.ones(1, np.float32))), dev_bits(np.zeros(1, np.uint16))
    state = torch.ones(16, device="cuda")
    out, gated = empty_bits(1), empty_bits(1)
    ops.call("bf16_hcl_decode", p(one), p(zero), p(one), p(zero), p(torch.zeros(16, device="cuda")),
             p(dev(residues)), 1, 16, p(state), p(gated), p(out), stream())
    assert bf16_to_f32(host_bits(out))[0] == np.float32(-0.240234375)
    assert bf16_to_f32(host_bits(gated))[0] == 0.0
    assert np.array_equal(state.cpu().numpy(), np.ones(16, np.float32))


@pytest.mark.parametrize("kind", ["hcs", "hcm", "hcm_f32", "hcl"])
def test_fused_decode_mixer_matches_the_unfused_launches_bit_for_bit(ops, kind):
    """One launch per mixer and token (featurizer step, split, gate, inner FIR or modal step,
    cache updates, post-gate) against the separate operators the runtime used before, over
    several consecutive tokens so that the in-place cache updates are exercised too."""
    rng = np.random.default_rng({"hcs": 1, "hcm": 2, "hcm_f32": 3, "hcl": 4}[kind])
    width, modes = 96, 16
    taps = 7 if kind == "hcs" else 128
    groups = 6 if kind != "hcl" else 1
    short_filter = dev_bits(rand_bf16(rng, 3 * width, 3))
    direct = None if kind == "hcs" else dev_bits(rand_bf16(rng, width))
    if kind == "hcm_f32":
        inner = dev((rng.standard_normal((groups, taps)) * 0.1).astype(np.float32))
    else:
        inner = dev_bits(rand_bf16(rng, groups, taps))
    log_poles = dev(np.log(rng.uniform(0.9, 0.999, (width, modes))).astype(np.float32))
    residues = dev((rng.standard_normal((width, modes)) * 0.02).astype(np.float32))
    caches = []
    for _ in range(2):  # fused, unfused: identical starting histories
        seed = np.random.default_rng(99)
        caches.append(dict(short=dev(seed.standard_normal((3 * width, 2)).astype(np.float32)),
                           inner=dev(seed.standard_normal((width, taps - 1)).astype(np.float32)),
                           modal=dev(seed.standard_normal((width, modes)).astype(np.float32))))
    fused, plain = caches
    for step in range(5):
        projection = dev_bits(rand_bf16(rng, 3 * width))
        out_fused, out_plain = empty_bits(width), empty_bits(width)
        if kind == "hcl":
            ops.call("bf16_hyena_decode_mixer", p(projection), p(short_filter), p(fused["short"]), p(direct),
                     None, 0, 0, 0, 0, None, p(log_poles), p(residues), modes, p(fused["modal"]), width,
                     p(out_fused), stream())
        else:
            ops.call("bf16_hyena_decode_mixer", p(projection), p(short_filter), p(fused["short"]), p(direct),
                     p(inner), int(kind == "hcm_f32"), groups, taps, 0 if kind == "hcs" else 1, p(fused["inner"]),
                     None, None, 0, None, width, p(out_fused), stream())
        filtered = empty_bits(3 * width)
        ops.call("bf16_fir_continue_direct", p(projection), p(short_filter), 0, None, 1, 3 * width, 3 * width, 3,
                 0, 0, p(plain["short"]), 2, p(filtered), stream())
        x2, x1, v, u, y = (empty_bits(width) for _ in range(5))
        ops.call("bf16_split_hyena_projection", p(filtered), 1, width, p(x2), p(x1), p(v), stream())
        if kind == "hcl":
            ops.call("bf16_hcl_decode", p(x2), p(x1), p(v), p(direct), p(log_poles), p(residues), width, modes,
                     p(plain["modal"]), None, p(out_plain), stream())
        else:
            ops.call("bf16_gated_elementwise", p(x1), p(v), width, 0, p(u), stream())
            ops.call("bf16_fir_continue_direct", p(u), p(inner), int(kind == "hcm_f32"), p(direct), 1, width,
                     groups, taps, 0 if kind == "hcs" else 1, 1, p(plain["inner"]), taps - 1, p(y), stream())
            ops.call("bf16_gated_elementwise", p(y), p(x2), width, 0, p(out_plain), stream())
        assert np.array_equal(host_bits(out_fused), host_bits(out_plain)), (kind, step)
        for name in ("short", "inner", "modal"):
            assert torch.equal(fused[name], plain[name]), (kind, step, name)
