"""The fused Hyena kernels at the benchmark's own shape.

The model benchmark runs gated_fir_stream_kernel (HCS), gated_fir_mma_kernel
(HCM) and modal_stream_kernel (HCL) on 8,192 x 4,096 activations fed by the
raw [8192, 3 x 4096] projection, as one-wave grids of row segments x column
blocks.  Here the same launches are checked against the CPU oracle on channel
slices over the FULL length, so every segment boundary and every carried state
of the real grid is on the path; each operator is depthwise, so a slice of
channels is an independent problem for the oracle.  Filters are grouped 16
channels to a filter (256 groups), as in the 7B-shaped model.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream, ulp_mismatch_report
from oracle_lib import bf16_to_f32, ptr

pytestmark = pytest.mark.gpu

LENGTH, WIDTH, GROUPS = 8192, 4096, 256
SLICES = [(0, 32), (2032, 32), (4064, 32)]   # first, one straddling a 64-channel block edge, last


def _projection(rng):
    projection = rand_bf16(rng, LENGTH, 3 * WIDTH)
    short = rand_bf16(rng, 3 * WIDTH, 3, scale=0.5)
    return projection, short


def _oracle_featurizer(oracle, projection, short, first, count):
    """Featurizer FIR + split on `count` channels starting at `first`."""
    columns = slice(3 * first, 3 * (first + count))
    sub = np.ascontiguousarray(projection[:, columns])
    sub_short = np.ascontiguousarray(short[columns])
    filtered = np.empty((LENGTH, 3 * count), np.uint16)
    short_cache = np.empty((3 * count, 2), np.float32)
    oracle.fir_prefill(ptr(sub), ptr(sub_short), 0, None, 0, LENGTH, 3 * count, 3 * count, 3, 1, ptr(filtered),
                       ptr(short_cache))
    x2, x1, v = (np.empty((LENGTH, count), np.uint16) for _ in range(3))
    oracle.split(ptr(filtered), LENGTH * count, ptr(x2), ptr(x1), ptr(v))
    return x2, x1, v, short_cache


@pytest.mark.parametrize("kind", ["hcs", "hcm"])
def test_projection_fed_fir_at_8192_by_4096(ops, oracle, kind):
    rng = np.random.default_rng(8192 + (kind == "hcm"))
    projection, short = _projection(rng)
    taps, orientation = (7, 0) if kind == "hcs" else (128, 1)
    h = rand_bf16(rng, GROUPS, taps, scale=0.2 if kind == "hcs" else 0.1)
    direct = rand_bf16(rng, WIDTH) if kind == "hcm" else None
    out = empty_bits(LENGTH, WIDTH)
    inner_cache = torch.zeros((WIDTH, taps - 1), device="cuda")
    short_cache = torch.zeros((3 * WIDTH, 2), device="cuda")
    ops.call("bf16_projection_gated_fir_prefill", p(dev_bits(projection)), p(dev_bits(short)), p(dev_bits(h)), 0,
             p(dev_bits(direct)) if direct is not None else None, LENGTH, WIDTH, GROUPS, taps, orientation, None,
             p(inner_cache), p(short_cache), p(out), stream())
    ops.call("check_async_errors", stream())
    got, got_inner, got_short = host_bits(out), inner_cache.cpu().numpy(), short_cache.cpu().numpy()
    per_group = WIDTH // GROUPS
    for first, count in SLICES:
        x2, x1, v, expected_short = _oracle_featurizer(oracle, projection, short, first, count)
        sub_h = np.ascontiguousarray(h[first // per_group:(first + count) // per_group])
        sub_direct = np.ascontiguousarray(direct[first:first + count]) if direct is not None else None
        expected = np.empty((LENGTH, count), np.uint16)
        expected_cache = np.empty((count, taps - 1), np.float32)
        oracle.gated_fir(ptr(x2), ptr(x1), ptr(v), ptr(sub_h), 0, ptr(sub_direct) if direct is not None else None,
                         LENGTH, count, count // per_group, taps, 1 if orientation == 0 else 0, None,
                         ptr(expected_cache), ptr(expected))
        actual = np.ascontiguousarray(got[:, first:first + count])
        if kind == "hcs":
            assert np.array_equal(actual, expected), first       # bit exact over all 8,192 rows
        else:
            fraction, _ = ulp_mismatch_report(actual, expected)
            assert fraction < 0.02, (first, fraction)            # summation order only
            assert_close_bits(actual, expected, atol=0.03, rtol=0.02, min_cosine=0.9999)
        assert np.array_equal(got_inner[first:first + count], expected_cache)
        assert np.array_equal(got_short[3 * first:3 * (first + count)], expected_short)


def test_projection_fed_modal_scan_at_8192_by_4096(ops, oracle):
    rng = np.random.default_rng(81920)
    modes = 16
    projection, short = _projection(rng)
    direct = rand_bf16(rng, WIDTH)
    log_poles = np.log(rng.uniform(0.9, 0.999, (WIDTH, modes))).astype(np.float32)
    residues = (rng.standard_normal((WIDTH, modes)) * 0.02).astype(np.float32)
    out = empty_bits(LENGTH, WIDTH)
    state = torch.full((WIDTH, modes), 9.0, device="cuda")
    short_cache = torch.zeros((3 * WIDTH, 2), device="cuda")
    scratch = torch.empty(ops.hcl_scratch_floats(LENGTH, WIDTH, modes), device="cuda")
    ops.call("bf16_projection_hcl_prefill", p(dev_bits(projection)), p(dev_bits(short)), p(dev_bits(direct)),
             p(dev(log_poles)), p(dev(residues)), LENGTH, WIDTH, modes, 0, p(state), p(scratch), p(short_cache), None,
             p(out), stream())
    ops.call("check_async_errors", stream())
    got, got_state, got_short = host_bits(out), state.cpu().numpy(), short_cache.cpu().numpy()
    for first, count in SLICES[:2]:
        x2, x1, v, expected_short = _oracle_featurizer(oracle, projection, short, first, count)
        expected = np.empty((LENGTH, count), np.uint16)
        expected_state = np.zeros((count, modes), np.float32)
        oracle.hcl_prefill(ptr(x2), ptr(x1), ptr(v), ptr(np.ascontiguousarray(direct[first:first + count])),
                           ptr(np.ascontiguousarray(log_poles[first:first + count])),
                           ptr(np.ascontiguousarray(residues[first:first + count])), LENGTH, count, modes, 0,
                           ptr(expected_state), None, ptr(expected))
        actual = np.ascontiguousarray(got[:, first:first + count])
        fraction, _ = ulp_mismatch_report(actual, expected)
        assert fraction < 0.03, (first, fraction)
        assert_close_bits(actual, expected, atol=0.04, rtol=0.03, min_cosine=0.9999)
        # the scan multiplies by expf(log_pole) once per row: ~n * 1e-7 relative on a term n rows old
        np.testing.assert_allclose(got_state[first:first + count], expected_state, rtol=2e-5, atol=1e-4)
        assert np.array_equal(got_short[3 * first:3 * (first + count)], expected_short)
