"""Whole-model parity on the 1B-shaped configuration: 25 blocks, width 1920,
15 heads, inner 5120, seeded random-init weights (seed 0), 1,024 uniform-ACGT
tokens.

* BF16 twin against upstream's own CPU backend: tests/golden/model_1b_1024.npz
  holds its logits and every block's output at sampled positions (made by
  tests/golden/make_model_golden.py from oracle/_ref/libevo_ref.so; this test
  only reads the file).  Reported per block and on the logits: max-abs error,
  relative L2 error, cosine; asserted: upstream's CPU-vs-CUDA profile gate
  (docs/execution-profiles.md there: cosine >= 0.999, logit MAE <= 0.1) and the
  same top-1 token wherever upstream's winner leads by more than the noise.
* E4M3 artifact: the bit-exact emulation profile (`exact`) against the tcgen05
  FP8 profile (`b200-tc`) on the same 1,024 tokens: per-block and per-logit
  error, identical top-1.

With EVO_B200_REPORT_DIR set, the per-block tables are also written there as
JSON.
"""
from __future__ import annotations

import importlib
import importlib.util
import json
import os
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
GOLDEN = ROOT / "tests" / "golden" / "model_1b_1024.npz"
LAYERS, WIDTH = 25, 1920


def _generator():
    spec = importlib.util.spec_from_file_location("make_model_golden", ROOT / "tests" / "golden" / "make_model_golden.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


@pytest.fixture(scope="module")
def rt(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return importlib.import_module("evo_cpp_b200.runtime")


@pytest.fixture(scope="module")
def evo(rt, pkg):
    return rt.EvoLibrary(pkg.EVO_LIBRARY)


def _report(name, payload):
    directory = os.environ.get("EVO_B200_REPORT_DIR")
    if directory:
        Path(directory).mkdir(parents=True, exist_ok=True)
        (Path(directory) / f"{name}.json").write_text(json.dumps(payload, indent=1))


def _errors(actual, expected):
    a, e = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    diff = np.abs(a - e)
    return {"max_abs": float(diff.max()), "mean_abs": float(diff.mean()),
            "rel_l2": float(np.linalg.norm(a - e) / (np.linalg.norm(e) + 1e-30)),
            "cosine": float((a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e) + 1e-30))}


def _top1(actual, expected, margin):
    """Agreement of the arg-max token overall and on the rows where `expected`'s winner leads
    its runner-up by more than `margin`."""
    ordered = np.sort(expected, axis=-1)
    decided = (ordered[:, -1] - ordered[:, -2]) > margin
    agree = actual.argmax(-1) == expected.argmax(-1)
    return float(agree.mean()), float(agree[decided].mean()) if decided.any() else 1.0, int(decided.sum())


def _block_outputs(context, sequence, rows_wanted):
    """Sampled rows and whole-tensor statistics of every block output, taken through the tap
    interface one block at a time as the pass produces them."""
    sampled, stats = {}, np.zeros((LAYERS, 3))

    def consume(layer, name, values):
        full = values.astype(np.float64)
        sampled[layer] = values[rows_wanted].copy()
        stats[layer] = [np.sqrt((full ** 2).mean()), np.abs(full).mean(), np.abs(full).max()]
        return 0

    logits, _ = context.prefill_with_dumps(sequence, [(layer, "block_output") for layer in range(LAYERS)],
                                           consume=consume)
    return logits, sampled, stats


def test_1b_shaped_bf16_twin_against_upstream_cpu_backend(rt, evo, tmp_path_factory):
    if not GOLDEN.exists():
        pytest.skip("tests/golden/model_1b_1024.npz is missing")
    golden = np.load(GOLDEN)
    gen = _generator()
    sequence = gen.prompt()
    assert np.array_equal(np.frombuffer(sequence, np.uint8), golden["tokens"])
    path = gen.write_artifact(tmp_path_factory.mktemp("model_1b_bf16"))
    model = evo.load(path)
    assert (model.layers, model.width) == (LAYERS, WIDTH)
    rows_wanted = golden["block_rows"]
    logits, sampled, stats = _block_outputs(model.context(1024), sequence, rows_wanted)
    expected_logits = golden["logits"].astype(np.float32)
    table = []
    for layer in range(LAYERS):
        entry = _errors(sampled[layer], golden[f"block_{layer}"].astype(np.float32))
        entry["layer"] = layer
        entry["rms"] = float(stats[layer, 0])
        entry["rms_upstream"] = float(golden["block_stats"][layer, 0])
        table.append(entry)
    on_logits = _errors(logits, expected_logits)
    overall, decided, count = _top1(logits, expected_logits, 0.1)
    on_logits.update(top1=overall, top1_decided=decided, decided_rows=count)
    _report("parity_1b_bf16_vs_upstream_cpu", {"blocks": table, "logits": on_logits})
    for entry in table:
        # BF16 activations against an F32 graph: each block adds rounding noise to the residual stream
        assert entry["cosine"] >= 0.999 and entry["rel_l2"] <= 0.04, entry
        assert abs(entry["rms"] / entry["rms_upstream"] - 1.0) <= 0.01, entry
    assert on_logits["cosine"] >= 0.999 and on_logits["mean_abs"] <= 0.1, on_logits
    # Random-init logits are nearly flat (median top-2 margin 0.13 for this prompt) while a BF16 graph
    # differs from the F32 one by up to ~0.17 per logit, so a winner can only be compared where it
    # leads by more than the error: identical top-1 on every row whose upstream margin exceeds
    # twice the largest per-logit difference, >= 99 % where it exceeds 0.1, >= 90 % over all rows.
    _, beyond_error, beyond_count = _top1(logits, expected_logits, 2.0 * on_logits["max_abs"])
    assert beyond_error == 1.0 and beyond_count >= 50, (on_logits, beyond_count)
    assert decided >= 0.99 and count >= 100, on_logits
    assert overall >= 0.90, on_logits


def test_1b_shaped_e4m3_exact_profile_against_tensor_core_profile(rt, evo, tmp_path_factory):
    gen = _generator()
    sequence = gen.prompt()
    path = gen.write_artifact(tmp_path_factory.mktemp("model_1b_fp8"), fp8=True)
    model = evo.load(path)
    rows_wanted = np.arange(0, 1024, 8)
    exact = model.context(1024)
    fast = model.context(1024, flags=rt.CONTEXT_FLAG_TENSORCORE_FP8)
    assert (exact.profile, fast.profile) == ("exact", "b200-tc")
    logits_exact, blocks_exact, _ = _block_outputs(exact, sequence, rows_wanted)
    logits_fast, blocks_fast, _ = _block_outputs(fast, sequence, rows_wanted)
    table = []
    for layer in range(LAYERS):
        entry = _errors(blocks_fast[layer], blocks_exact[layer])
        entry["layer"] = layer
        table.append(entry)
    on_logits = _errors(logits_fast, logits_exact)
    overall, decided, count = _top1(logits_fast, logits_exact, 4.0 * on_logits["max_abs"])
    on_logits.update(top1=overall, top1_decided=decided, decided_rows=count)
    _report("parity_1b_e4m3_exact_vs_b200_tc", {"blocks": table, "logits": on_logits})
    for entry in table:
        assert entry["cosine"] >= 0.9995 and entry["rel_l2"] <= 0.03, entry
    # upstream's CUDA model gate is 0.08 abs + 0.06 rel on a 4-token prompt of its tiny fixture
    # (tests/test_cuda_model.cu:236-281); 25 blocks x 1,024 tokens accumulate more: 0.15 + 0.06 rel
    assert np.all(np.abs(logits_fast - logits_exact) <= 0.15 + 0.06 * np.abs(logits_exact)), on_logits
    assert on_logits["cosine"] >= 0.9995, on_logits
    # a flip needs two logits closer than twice the per-logit error: none outside that band
    flipped = logits_fast.argmax(-1) != logits_exact.argmax(-1)
    top = np.take_along_axis(logits_exact, logits_exact.argmax(-1)[:, None], 1)[:, 0]
    chosen = np.take_along_axis(logits_exact, logits_fast.argmax(-1)[:, None], 1)[:, 0]
    assert np.all((top - chosen)[flipped] <= 2.0 * on_logits["max_abs"]), on_logits
    assert decided == 1.0, on_logits
    # the emulation profile is deterministic
    assert np.array_equal(model.context(1024).prefill(sequence), logits_exact)


def test_1b_shaped_fp8_ffn_profile_error_budget(rt, evo, tmp_path_factory):
    """Profile b200-fp8 (output and MLP projections in E4M3 with per-row activation scales, on top of
    the tensor-core Hyena projections) on the same 1,024 tokens against `exact`.

    What the profile guarantees is the error of ONE product: E4M3 operands carry 2^-4 relative
    rounding each, which shows as ~3.8 % relative L2 error on a projection's output (checked on
    block 0, whose inputs are identical in both profiles).  On random-init weights that noise is
    not damped: the mixer path contributes almost nothing, the gated MLP dominates the residual
    stream and doubles relative perturbations block after block, so the logits of this synthetic
    model differ by tens of percent and the profile makes no top-1 claim here.  The test pins the
    per-product budget and records the rest."""
    gen = _generator()
    sequence = gen.prompt()
    path = gen.write_artifact(tmp_path_factory.mktemp("model_1b_fp8_ffn"), fp8=True)
    model = evo.load(path)
    taps = [(0, name) for name in ("post_norm", "mlp_l1", "mlp_l2", "mlp_gated", "mlp_output")]
    taps += [(layer, "block_output") for layer in range(LAYERS)]
    fast_context = model.context(1024, flags=rt.CONTEXT_FLAG_FP8_FFN)
    assert fast_context.profile == "b200-fp8"
    logits_exact, exact = model.context(1024).prefill_with_dumps(sequence, taps)
    logits_fast, fast = fast_context.prefill_with_dumps(sequence, taps)
    assert np.isfinite(logits_fast).all()
    assert _errors(fast[(0, "post_norm")], exact[(0, "post_norm")])["rel_l2"] <= 1e-3   # same operand going in
    budget = {name: _errors(fast[(0, name)], exact[(0, name)]) for name in ("mlp_l1", "mlp_l2", "mlp_gated", "mlp_output")}
    for name in ("mlp_l1", "mlp_l2"):
        assert 0.02 <= budget[name]["rel_l2"] <= 0.05, budget           # one E4M3 x E4M3 product
    assert budget["mlp_gated"]["rel_l2"] <= 0.075 and budget["mlp_output"]["rel_l2"] <= 0.09, budget
    table = []
    for layer in range(LAYERS):
        entry = _errors(fast[(layer, "block_output")], exact[(layer, "block_output")])
        entry["layer"] = layer
        table.append(entry)
    on_logits = _errors(logits_fast, logits_exact)
    overall, decided, count = _top1(logits_fast, logits_exact, 0.1)
    on_logits.update(top1=overall, top1_decided_margin_0p1=decided, decided_rows=count)
    _report("parity_1b_b200_fp8_profile", {"first_block_products": budget, "blocks": table, "logits": on_logits})
    assert on_logits["cosine"] >= 0.85, on_logits                           # sanity only, see above
