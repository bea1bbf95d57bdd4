"""Row-window (chunked-prefill) forms of the fused Hyena operators and the
chunk-wavefront layer pipeline built on them.

Window property: producing rows [0, a) and then [a, L) with the earlier rows as
history must give what one pass over [0, L) gives - bit for bit for the FIR
operators (same arithmetic per output), at scan tolerance for the modal
operator (the carried state enters through a different but equivalent sum)."""
from __future__ import annotations

import importlib
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import (assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream,
                      ulp_mismatch_report)

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("taps,groups,orientation,f32", [(7, 8, 0, 0), (128, 8, 1, 0), (128, 16, 1, 1)])
def test_fir_windows_equal_single_pass(ops, taps, groups, orientation, f32):
    rng = np.random.default_rng(taps + f32)
    length, width = 1500, 128
    x2, x1, v = (dev_bits(rand_bf16(rng, length, width)) for _ in range(3))
    h_bits = rand_bf16(rng, groups, taps, scale=0.2)
    h = dev((h_bits.astype(np.uint32) << 16).view(np.float32)) if f32 else dev_bits(h_bits)
    direct = dev_bits(rand_bf16(rng, width)) if orientation == 1 else None
    whole = empty_bits(length, width)
    cache_whole = torch.zeros((width, taps - 1), device="cuda")
    ops.call("bf16_gated_fir_prefill", p(x2), p(x1), p(v), p(h), f32, p(direct), length, width, groups,
             taps, orientation, None, p(cache_whole), p(whole), stream())
    pieces = torch.zeros((length, width), dtype=torch.int16, device="cuda")
    cache = torch.zeros((width, taps - 1), device="cuda")
    # The middle window is shorter than k-1.  Window starts are multiples of 16:
    # the tensor-core path groups taps by 16-row tiles anchored at the window
    # start, so other starts change its summation order (not its value set).
    for begin, end in [(0, 512), (512, 608), (608, 1500)]:
        ops.call("bf16_gated_fir_prefill_window", p(x2), p(x1), p(v), p(h), f32, p(direct), begin, end,
                 width, groups, taps, orientation, p(cache), p(pieces), stream())
    assert np.array_equal(host_bits(pieces), host_bits(whole))
    assert np.array_equal(cache.cpu().numpy(), cache_whole.cpu().numpy())


def test_modal_windows_match_single_pass(ops):
    rng = np.random.default_rng(5)
    length, width, modes = 1400, 96, 16
    x2, x1, v = (dev_bits(rand_bf16(rng, length, width)) for _ in range(3))
    direct = dev_bits(rand_bf16(rng, width))
    log_poles = dev(np.log(rng.uniform(0.9, 0.999, (width, modes))).astype(np.float32))
    residues = dev((rng.standard_normal((width, modes)) * 0.02).astype(np.float32))
    scratch = torch.empty(ops.hcl_scratch_floats(length, width, modes), device="cuda")
    whole = empty_bits(length, width)
    state_whole = torch.zeros((width, modes), device="cuda")
    ops.call("bf16_hcl_prefill", p(x2), p(x1), p(v), p(direct), p(log_poles), p(residues), length, width,
             modes, 0, p(state_whole), p(scratch), None, p(whole), stream())
    pieces = torch.zeros((length, width), dtype=torch.int16, device="cuda")
    state = torch.zeros((width, modes), device="cuda")
    ops.call("bf16_hcl_prefill", p(x2), p(x1), p(v), p(direct), p(log_poles), p(residues), 512, width,
             modes, 0, p(state), p(scratch), None, p(pieces), stream())
    for begin, end in [(512, 700), (700, 1400)]:
        ops.call("bf16_hcl_prefill_window", p(x2), p(x1), p(v), p(direct), p(log_poles), p(residues), begin,
                 end, width, modes, p(state), p(scratch), p(pieces), stream())
    # first window: the same arithmetic per row, split into segments at other rows (F32 summation
    # order of the carried state differs); later windows: continuation rounding (single BF16 rounding)
    fraction, worst = ulp_mismatch_report(host_bits(pieces)[:512], host_bits(whole)[:512])
    assert fraction < 0.01, (fraction, worst)
    assert_close_bits(host_bits(pieces), host_bits(whole), atol=0.04, rtol=0.03, min_cosine=0.9999)
    np.testing.assert_allclose(state.cpu().numpy(), state_whole.cpu().numpy(), rtol=3e-5, atol=1e-4)


def test_wavefront_pipeline_matches_single_gpu(pkg, tmp_path_factory):
    """2 GPUs: 1,300-token prompt -> 512-row chunks flowing through two stages."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("wave")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    art.write_synthetic(directory / "model.safetensors", spec, seed=4, weight_std=0.05, filter_std=0.3)
    rng = np.random.default_rng(1003)
    sequence = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), 1300).tolist())
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    single_model = evo.load(directory / "model.safetensors", devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    single = single_model.context(2048, flags)
    expected = single.prefill(sequence)
    piped_model = evo.load(directory / "model.safetensors", devices=[0, 1], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    piped = piped_model.context(2048, flags)
    logits = piped.prefill(sequence)
    a, e = logits.astype(np.float64), expected.astype(np.float64)
    cosine = (a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e))
    assert cosine > 0.9995 and np.abs(a - e).mean() < 0.05, (cosine, np.abs(a - e).mean())
    # decode continues from the caches and state the wavefront left behind
    token = int(expected[-1].argmax())
    for _ in range(3):
        step_single, step_piped = single.decode(token), piped.decode(token)
        assert np.abs(step_single - step_piped).mean() < 0.05
        token = int(step_single.argmax())


def test_chunk_continuation_matches_single_prefill(pkg, tmp_path_factory):
    """A prompt fed as 700 + 512 + 100 + 188 rows (continuation chunks run through
    the fused kernels as row windows behind their carried history) against the
    same prompt in one pass; decode continues from either."""
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    pipe = importlib.import_module("evo_cpp_b200.pipeline")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("chunks")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    art.write_synthetic(directory / "model.safetensors", spec, seed=9, weight_std=0.05, filter_std=0.3)
    rng = np.random.default_rng(31)
    host_tokens = rng.choice(np.frombuffer(b"ACGT", np.uint8), 1500)
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    model = evo.load(directory / "model.safetensors", devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    whole = model.context(2048, flags)
    expected = whole.prefill(bytes(host_tokens.tolist()))
    tokens = torch.from_numpy(host_tokens.astype(np.int32)).cuda()
    chunked = model.context(2048, flags)
    chunked.prefill_device(tokens.data_ptr(), 700, stateless=False)
    begin = 700
    for count in (512, 100, 188):
        logits_address = chunked.continue_device(tokens.data_ptr() + 4 * begin, count)
        chunked.synchronize()
        raw = torch.as_tensor(pipe.DeviceRows(logits_address, count, 512), device="cuda")
        got = ((raw.to(torch.int32) & 0xFFFF) << 16).view(torch.float32).cpu().numpy().astype(np.float64)
        want = expected[begin:begin + count].astype(np.float64)
        cosine = (got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want))
        assert cosine > 0.9995 and np.abs(got - want).mean() < 0.05, (begin, cosine, np.abs(got - want).mean())
        begin += count
    assert chunked.position == 1500
    token = int(expected[-1].argmax())
    for _ in range(3):
        a, b = whole.decode(token), chunked.decode(token)
        assert np.abs(a - b).mean() < 0.05
        token = int(a.argmax())


def test_decode_graph_replay_is_bit_identical(pkg, tmp_path_factory, monkeypatch):
    """Cached decode is recorded once as a CUDA graph and replayed (position read
    from device memory); the same steps with ordinary launches give the same bits."""
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("graph")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    art.write_synthetic(directory / "model.safetensors", spec, seed=12, weight_std=0.05, filter_std=0.3)
    model = evo.load(directory / "model.safetensors", devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    prompt = bytes(np.random.default_rng(3).choice(np.frombuffer(b"ACGT", np.uint8), 300).tolist())
    for flags in (rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8, rt.CONTEXT_FLAG_FULL_ARENA):
        monkeypatch.setenv("EVO_B200_DECODE_GRAPH", "0")
        plain = model.context(1024, flags)
        monkeypatch.delenv("EVO_B200_DECODE_GRAPH")
        replayed = model.context(1024, flags)
        token = int(plain.prefill(prompt)[-1].argmax())
        assert int(replayed.prefill(prompt)[-1].argmax()) == token
        for _ in range(12):
            a, b = plain.decode(token), replayed.decode(token)
            assert np.array_equal(a, b)
            token = int(a.argmax())
        assert plain.position == replayed.position == 312


def test_decode_with_dependent_launches_is_bit_identical(pkg, tmp_path_factory, monkeypatch):
    """One-row projections start under the kernel in front of them (programmatic stream
    serialisation: they pull their weights into L2, then wait for that kernel before reading its
    output).  Same logits, bit for bit, as plain launches - in the captured graph and without it."""
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("pdl")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    art.write_synthetic(directory / "model.safetensors", spec, seed=31, weight_std=0.05, filter_std=0.3)
    model = evo.load(directory / "model.safetensors", devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    prompt = bytes(np.random.default_rng(8).choice(np.frombuffer(b"ACGT", np.uint8), 150).tolist())
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    for graph in ("1", "0"):
        monkeypatch.setenv("EVO_B200_DECODE_GRAPH", graph)
        monkeypatch.setenv("EVO_B200_DECODE_PDL", "0")
        plain = model.context(1024, flags)
        monkeypatch.delenv("EVO_B200_DECODE_PDL")
        dependent = model.context(1024, flags)
        token = int(plain.prefill(prompt)[-1].argmax())
        assert int(dependent.prefill(prompt)[-1].argmax()) == token
        for _ in range(16):
            a, b = plain.decode(token), dependent.decode(token)
            assert np.array_equal(a, b)
            token = int(a.argmax())


def test_continuation_after_decode_steps_uses_current_state(pkg, tmp_path_factory):
    """prefill -> a few decode steps -> a 100-row continuation chunk: the decode steps do not
    update the fused kernels' carried projection history, so the chunk must fall back to the step
    kernels and still agree with one pass over the whole sequence."""
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    pipe = importlib.import_module("evo_cpp_b200.pipeline")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("mixed")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    art.write_synthetic(directory / "model.safetensors", spec, seed=21, weight_std=0.05, filter_std=0.3)
    model = evo.load(directory / "model.safetensors", devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    rng = np.random.default_rng(8)
    sequence = rng.choice(np.frombuffer(b"ACGT", np.uint8), 403)
    expected = model.context(1024, flags).prefill(bytes(sequence.tolist()))
    context = model.context(1024, flags)
    context.prefill(bytes(sequence[:300].tolist()))
    for token in sequence[300:303]:
        context.decode(int(token))
    tokens = torch.from_numpy(sequence.astype(np.int32)).cuda()
    address = context.continue_device(tokens.data_ptr() + 4 * 303, 100)
    context.synchronize()
    raw = torch.as_tensor(pipe.DeviceRows(address, 100, 512), device="cuda")
    got = ((raw.to(torch.int32) & 0xFFFF) << 16).view(torch.float32).cpu().numpy().astype(np.float64)
    want = expected[303:403].astype(np.float64)
    cosine = (got * want).sum() / (np.linalg.norm(got) * np.linalg.norm(want))
    assert cosine > 0.9995 and np.abs(got - want).mean() < 0.05, (cosine, np.abs(got - want).mean())
