"""Layer pipeline across GPUs of one process (evo_model_params.devices), after
upstream's tests/test_cuda_pipeline.cu: the same tiny model on 1, 2 and 4 GPUs,
stage layout 25/25 and 13/13/12/12, identical logits, decode and chunked
continuation across the hand-off.  Degrades by device count like upstream's
test (skips what the box cannot run)."""
from __future__ import annotations

import importlib
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
TINY = ROOT / "tests" / "golden" / "tiny" / "tiny.safetensors"
CHUNKED = bytes([2, 5, 7, 3, 9, 11, 13, 17, 19])


@pytest.fixture(scope="module")
def setup(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    rt = importlib.import_module("evo_cpp_b200.runtime")
    return rt, rt.EvoLibrary(pkg.EVO_LIBRARY), torch.cuda.device_count()


def outputs(rt, evo, devices):
    model = evo.load(TINY, devices=devices, flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    context = model.context(64)
    logits = context.prefill(CHUNKED)          # 8-row prefill + 1-row continuation per stage
    step = context.decode(9)
    stages = [(s.device, s.layer_begin, s.layer_end) for s in context.stages()]
    embedding = model.context(64).embed(bytes([2, 5, 7, 3]), 30)   # captured on a later stage
    return logits, step, stages, embedding


@pytest.mark.parametrize("count", [2, 4])
def test_pipeline_matches_single_gpu(setup, count):
    rt, evo, available = setup
    if available < count:
        pytest.skip(f"needs {count} GPUs, box has {available}")
    single = outputs(rt, evo, [0])
    assert single[2] == [(0, 0, 50)]
    devices = list(range(count))
    piped = outputs(rt, evo, devices)
    expected_layers = {2: [(0, 25), (25, 50)], 4: [(0, 13), (13, 26), (26, 38), (38, 50)]}[count]
    assert [(b, e) for _, b, e in piped[2]] == expected_layers
    assert [d for d, _, _ in piped[2]] == devices
    # same kernels, same order, same data: bit-identical across the hand-offs
    assert np.array_equal(piped[0], single[0])
    assert np.array_equal(piped[1], single[1])
    assert np.array_equal(piped[3], single[3])
    # reversed device order works too (stage 0 owns embedding and head)
    reverse = outputs(rt, evo, devices[::-1])
    assert np.array_equal(reverse[0], single[0])


def test_pipeline_rejects_bad_device_lists(setup):
    rt, evo, available = setup
    with pytest.raises(rt.EvoError) as err:
        evo.load(TINY, devices=[0, 0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    assert err.value.code == 2
    with pytest.raises(rt.EvoError) as err:
        evo.load(TINY, devices=[available + 3], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    assert err.value.code == 2
    with pytest.raises(rt.EvoError):
        evo.load(TINY, devices=list(range(9)), flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
