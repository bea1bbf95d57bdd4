"""Activation taps inside the blocks (evo_b200_context_prefill_with_dumps /
decode_with_dumps; upstream LayerDumpPoint, include/evo/cuda/model.hpp:22-45,
taken at src/cuda/model.cu:1373-1581 and 1757-1856).

A width-256 fixture with every mixer kind is run with all 22 taps on four
blocks; the taps must be consistent with one another under the block graph's
own arithmetic, evaluated by the CPU oracle one rounding at a time, and asking
for them must not change the logits.
"""
from __future__ import annotations

import importlib

import numpy as np
import pytest

from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu

WIDTH, INNER, LAYERS = 256, 512, 8
KINDS = ["hcs", "hcm", "hcl", "attn"]


@pytest.fixture(scope="module")
def rt(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return importlib.import_module("evo_cpp_b200.runtime")


@pytest.fixture(scope="module")
def model(rt, pkg, tmp_path_factory):
    art = importlib.import_module("evo_cpp_b200.artifact")
    directory = tmp_path_factory.mktemp("dumps")
    spec = art.fixture_spec(width=WIDTH, layers=LAYERS, heads=2, inner=INNER, hcs_groups=16, hcm_groups=16)
    art.write_synthetic(directory / "model.safetensors", spec, seed=5, weight_std=0.05, filter_std=0.3)
    return rt.EvoLibrary(pkg.EVO_LIBRARY).load(directory / "model.safetensors", flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)


def bits(values):
    return f32_to_bf16(np.ascontiguousarray(values, np.float32))


def test_every_tap_is_consistent_with_the_block_graph(rt, model, oracle):
    rng = np.random.default_rng(31)
    sequence = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), 200).tolist())
    rows = len(sequence)
    plain = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA).prefill(sequence)
    layers = [0, 1, 2, 3]                                   # HCS (GELU block), HCM, HCL, attention
    taps = [(layer, name) for layer in layers for name in rt.DUMP_POINTS]
    context = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
    logits, d = context.prefill_with_dumps(sequence, taps)
    assert np.array_equal(logits, plain)                    # taps do not disturb the pass
    assert context.position == rows

    def add(a, b):
        out = np.empty(a.shape, np.uint16)
        oracle.add(ptr(bits(a)), ptr(bits(b)), a.size, ptr(out))
        return bf16_to_f32(out)

    def gate(a, b, gelu=0):
        out = np.empty(a.shape, np.uint16)
        oracle.gate(ptr(bits(a)), ptr(bits(b)), a.size, gelu, ptr(out))
        return bf16_to_f32(out)

    for layer in layers:
        kind = KINDS[layer % 4]
        get = lambda name: d[(layer, name)]
        for name in ("block_output", "pre_norm", "mixer_output", "mixer_projection", "mixer_residual", "post_norm",
                     "mlp_output", "mixer_x2", "mixer_x1", "mixer_value"):
            assert get(name).shape == (rows, WIDTH), (layer, name)
        assert get("mixer_input_projection").shape == (rows, 3 * WIDTH)
        for name in ("mlp_l1", "mlp_l2", "mlp_gated"):
            assert get(name).shape == (rows, INNER)
        # the residual stream: block input + projection, then + MLP output
        if layer > 0:
            block_input = d[(layer - 1, "block_output")]
            assert np.array_equal(get("mixer_residual"), add(get("mixer_projection"), block_input))
        assert np.array_equal(get("block_output"), add(get("mlp_output"), get("mixer_residual")))
        # the gated MLP
        if layer == 0:
            activated = np.empty((rows, INNER), np.uint16)
            oracle.gelu(ptr(bits(get("mlp_l1"))), rows * INNER, ptr(activated))
            assert np.array_equal(get("mlp_activation"), bf16_to_f32(activated))
            assert np.array_equal(get("mlp_gated"), gate(get("mlp_l1"), get("mlp_l2"), 1))
        else:
            assert (layer, "mlp_activation") not in d       # only the GELU block has it
            assert np.array_equal(get("mlp_gated"), gate(get("mlp_l1"), get("mlp_l2")))
        # post-norm of the residual stream (unit scales in the fixture); rsqrtf vs libm: <= 1 BF16 ulp
        normed = np.empty((rows, WIDTH), np.uint16)
        oracle.rms_norm(ptr(bits(get("mixer_residual"))), ptr(np.ones(WIDTH, np.float32)), rows, WIDTH, 1e-6,
                        ptr(normed))
        gap = np.abs(bits(get("post_norm")).astype(np.int32) - normed.astype(np.int32))
        assert gap.max() <= 1 and (gap != 0).mean() < 0.01
        if kind == "attn":
            for name in ("mixer_short_filter", "mixer_pregate", "mixer_state", "mixer_filter", "mixer_inner_state"):
                assert (layer, name) not in d
            # V is the last third of the projection, untouched by the rotation
            assert np.array_equal(get("mixer_value"), get("mixer_input_projection")[:, 2 * WIDTH:])
            continue
        # Hyena: featurizer -> split -> pre-gate
        filtered = get("mixer_short_filter")
        assert filtered.shape == (rows, 3 * WIDTH)
        triples = filtered.reshape(rows, WIDTH, 3)
        assert np.array_equal(get("mixer_x2"), triples[:, :, 0])
        assert np.array_equal(get("mixer_x1"), triples[:, :, 1])
        assert np.array_equal(get("mixer_value"), triples[:, :, 2])
        assert np.array_equal(get("mixer_pregate"), gate(get("mixer_x1"), get("mixer_value")))
        # histories: the last raw projection rows and the last pre-gate rows, per channel
        short_state = get("mixer_short_state")
        assert short_state.shape == (3 * WIDTH, 2)
        assert np.array_equal(short_state, get("mixer_input_projection")[-2:].T)
        if kind in ("hcs", "hcm"):
            taps_k = 7 if kind == "hcs" else 128
            inner = get("mixer_inner_state")
            assert inner.shape == (WIDTH, taps_k - 1)
            assert np.array_equal(inner, get("mixer_pregate")[-(taps_k - 1):].T)
            assert (layer, "mixer_state") not in d
        else:
            state, h, conv = get("mixer_state"), get("mixer_filter"), get("mixer_convolution")
            assert state.shape == (WIDTH, 16) and h.shape == (rows, WIDTH) and conv.shape == (rows, WIDTH)
            # the tapped convolution is the tapped filter applied to the tapped pre-gate
            u = get("mixer_pregate").astype(np.float64)
            for channel in (0, 77, WIDTH - 1):
                expected = np.convolve(u[:, channel], h[:, channel].astype(np.float64))[:rows]
                np.testing.assert_allclose(conv[:, channel], expected, rtol=2e-4, atol=2e-4)


def test_decode_taps_and_error_paths(rt, model):
    rng = np.random.default_rng(32)
    sequence = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), 150).tolist())
    context = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
    reference = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
    logits = context.prefill(sequence)
    reference.prefill(sequence)
    token = int(logits[-1].argmax())
    taps = [(layer, name) for layer in (1, 2, 3) for name in
            ("block_output", "mixer_short_filter", "mixer_pregate", "mixer_output", "mixer_state", "mixer_inner_state")]
    step, d = context.decode_with_dumps(token, taps)
    # the tapped step runs the unfused decode operators, which are bit-identical to the fused ones
    assert np.array_equal(step, reference.decode(token))
    assert d[(1, "block_output")].shape == (1, WIDTH)
    assert d[(1, "mixer_inner_state")].shape == (WIDTH, 127)
    assert d[(1, "mixer_inner_state")][:, -1].tolist() == d[(1, "mixer_pregate")][0].tolist()
    assert d[(2, "mixer_state")].shape == (WIDTH, 16)
    assert (3, "mixer_pregate") not in d and (3, "block_output") in d
    assert context.position == len(sequence) + 1
    # bad requests
    with pytest.raises(rt.EvoError) as bad:
        model.context(512).prefill_with_dumps(sequence[:8], [(LAYERS, "block_output")])
    assert bad.value.code == 2
    with pytest.raises(rt.EvoError) as long:
        model.context(512).prefill_with_dumps(sequence, [(0, "block_output")])   # 8-row fixture arena
    assert long.value.code == 5
    # a consumer that returns an error aborts the pass and poisons the context
    failing = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
    with pytest.raises(rt.EvoError) as aborted:
        failing.prefill_with_dumps(sequence, [(0, "block_output")], consume=lambda *a: 3)
    assert aborted.value.code == 3
    with pytest.raises(rt.EvoError):
        failing.prefill(sequence)
