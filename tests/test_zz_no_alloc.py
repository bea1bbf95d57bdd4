"""The allocation-free HCL prefill entry point (evo_b200_bf16_hcl_prefill_noalloc).

It exists for callers that must stay away from the CUDA allocator - a server
that gave all free device memory to its own pool at start-up, or a
latency-critical loop that cannot take cudaMalloc's implicit synchronisation -
and keeps its segment-state scratch in a fixed array inside the library instead
of a caller buffer.  The test calls it through the C ABI twice in a row (the
array is shared and keeps the previous call's contents, so the second call
must not be disturbed by the first) and checks both results against the
ordinary entry point, which takes caller-provided scratch.

The file name sorts last on purpose: a run that stops at the first failure has
then already executed every other test.  It passes alone in a fresh process
(the first call does the per-device set-up) and after the rest of the suite.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream

pytestmark = pytest.mark.gpu


def _case(rng, length, width, modes):
    x2, x1, v = (rand_bf16(rng, length, width) for _ in range(3))
    direct = rand_bf16(rng, width)
    log_poles = np.log(rng.uniform(0.9, 0.999, (width, modes))).astype(np.float32)
    residues = (rng.standard_normal((width, modes)) * 0.02).astype(np.float32)
    return x2, x1, v, direct, log_poles, residues


def _prepare(case, length, width, modes, scratch, mode=0, initial_state=None):
    """Every device buffer of one call, allocated up front: (argument list, out, pregate, state)."""
    x2, x1, v, direct, log_poles, residues = case
    out, pregate = empty_bits(length, width), empty_bits(length, width)
    state = (torch.full((width, modes), -3.0, device="cuda") if initial_state is None
             else torch.from_numpy(initial_state).cuda())
    args = [p(dev_bits(x2)), p(dev_bits(x1)), p(dev_bits(v)), p(dev_bits(direct)), p(dev(log_poles)),
            p(dev(residues)), length, width, modes, mode, p(state)]
    if scratch is not None:
        args.append(p(scratch))
    args += [p(pregate), p(out), stream()]
    return args, out, pregate, state


def _run(ops, entry, case, length, width, modes, scratch, mode=0, initial_state=None):
    args, out, pregate, state = _prepare(case, length, width, modes, scratch, mode, initial_state)
    ops.call(entry, *args)
    torch.cuda.synchronize()
    return host_bits(out), host_bits(pregate), state.cpu().numpy()


def test_noalloc_entry_matches_the_allocating_one_twice_in_a_row(ops):
    rng = np.random.default_rng(77)
    # second shape is larger than the first and leaves stale data beyond/under it
    for length, width, modes in [(300, 64, 16), (1000, 96, 16)]:
        case = _case(rng, length, width, modes)
        scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
        expected = _run(ops, "bf16_hcl_prefill", case, length, width, modes, scratch)
        got = _run(ops, "bf16_hcl_prefill_noalloc", case, length, width, modes, None)
        assert np.array_equal(got[1], expected[1])                       # u = bf16(x1 * v)
        assert_close_bits(got[0], expected[0], atol=0.04, rtol=0.03, min_cosine=0.9999)
        np.testing.assert_allclose(got[2], expected[2], rtol=2e-5, atol=2e-5)
        # same segmentation at these sizes, hence the same bits
        assert np.array_equal(got[0], expected[0])


def test_noalloc_entry_at_model_width_and_rejects_beyond_the_limit(ops):
    rng = np.random.default_rng(78)
    # 4096 channels x 16 modes = 65,536 floats per segment state: the one-wave grid wants ~18
    # segments at this width, the 4 Mi-float array holds 63 - same segmentation, same bits.
    length, width, modes = 2048, 4096, 16
    case = _case(rng, length, width, modes)
    scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
    expected = _run(ops, "bf16_hcl_prefill", case, length, width, modes, scratch)
    got = _run(ops, "bf16_hcl_prefill_noalloc", case, length, width, modes, None)
    assert np.array_equal(got[0], expected[0])
    assert np.array_equal(got[2], expected[2])
    # width * modes alone beyond the array: refused with a message naming the limit
    dummy = empty_bits(16)
    status = ops.status("bf16_hcl_prefill_noalloc", p(dummy), p(dummy), p(dummy), p(dummy), p(dummy),
                        p(dummy), 4, (4 << 20) // 16 + 2, 16, 0, None, None, p(dummy), stream())
    assert status == 2
    assert "fixed scratch of 4194304 floats" in ops.last_error()


def test_noalloc_call_leaves_the_free_device_memory_unchanged(ops):
    """cudaMemGetInfo sees every allocation on the device, whoever makes it.  With all buffers
    of the call allocated beforehand and one earlier call behind us (the per-device set-up),
    the free byte count is the same before and after a call."""
    rng = np.random.default_rng(79)
    length, width, modes = 1500, 256, 16
    case = _case(rng, length, width, modes)
    args, out, _, _ = _prepare(case, length, width, modes, None)
    ops.call("bf16_hcl_prefill_noalloc", *args)
    torch.cuda.synchronize()
    first = host_bits(out).copy()
    free_before = torch.cuda.mem_get_info()[0]
    ops.call("bf16_hcl_prefill_noalloc", *args)
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info()[0] == free_before
    assert np.array_equal(host_bits(out), first)


def test_noalloc_continuation_from_a_carried_state_over_several_segments(ops):
    """mode 1 continues from the state the caller passes in; with more than one row segment the
    carried-in state travels through its own slot of the shared array.  Output and final state
    equal the allocating entry point's bit for bit, on two calls in a row."""
    rng = np.random.default_rng(80)
    for length, width, modes in [(640, 128, 16), (2048, 512, 16)]:
        case = _case(rng, length, width, modes)
        carried = (rng.standard_normal((width, modes)) * 0.5).astype(np.float32)
        scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
        expected = _run(ops, "bf16_hcl_prefill", case, length, width, modes, scratch, 1, carried)
        got = _run(ops, "bf16_hcl_prefill_noalloc", case, length, width, modes, None, 1, carried)
        assert np.array_equal(got[0], expected[0])
        assert np.array_equal(got[1], expected[1])
        assert np.array_equal(got[2], expected[2])
        assert not np.array_equal(got[2], carried)
