"""One pipeline stage per process: the slice calls of the runtime library.

On one GPU the stages of a 3-slice split run as three contexts of one process
with device-to-device copies standing in for the hand-off; with two or more GPUs
two ranks are spawned and hand the rows over with NCCL send/recv, as the
benchmark does under torchrun."""
from __future__ import annotations

import importlib
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def write_model(pkg, directory):
    art = importlib.import_module("evo_cpp_b200.artifact")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16, fp8=True)
    path = directory / "model.safetensors"
    art.write_synthetic(path, spec, seed=4, weight_std=0.05, filter_std=0.3)
    return path


def bf16_rows(address_tensor):
    return (address_tensor.cpu().numpy().astype(np.uint32) << 16).view(np.float32)


def test_three_slices_on_one_gpu_match_the_whole_model(pkg, tmp_path_factory):
    rt = importlib.import_module("evo_cpp_b200.runtime")
    pipe = importlib.import_module("evo_cpp_b200.pipeline")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    path = write_model(pkg, tmp_path_factory.mktemp("slices"))
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    rng = np.random.default_rng(77)
    rows, width = 1300, 256
    host_tokens = rng.choice(np.frombuffer(b"ACGT", np.uint8), rows)
    whole = evo.load(path, devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC).context(2048, flags)
    expected = whole.prefill(bytes(host_tokens.tolist()))

    tokens = torch.from_numpy(host_tokens.astype(np.int32)).cuda()
    slices = [evo.load_slice(path, 0, index, 3, rt.MODEL_FLAG_ALLOW_SYNTHETIC) for index in range(3)]
    contexts = [model.context(2048, flags) for model in slices]
    assert [(s.layer_begin, s.layer_end) for c in contexts for s in c.stages()] == [(0, 3), (3, 6), (6, 8)]
    hidden = [pipe.alias_hidden_rows(c, 2048, width, "cuda") for c in contexts]
    for _ in range(2):  # a second prompt through the same contexts restarts the state
        for begin, count in pipe.window_plan(rows, 3, chunk=512):
            contexts[0].slice_embed(tokens.data_ptr() + 4 * begin, begin, count)
            for index, context in enumerate(contexts):
                if index > 0:
                    contexts[index - 1].synchronize()
                    with torch.cuda.stream(torch.cuda.ExternalStream(context.stream())):
                        hidden[index][begin:begin + count].copy_(hidden[index - 1][begin:begin + count])
                context.slice_run(begin, count)
        logits_address = contexts[2].slice_head(0, rows)
        contexts[2].synchronize()
    raw = torch.as_tensor(pipe.DeviceRows(logits_address, rows, 512), device="cuda")
    logits = bf16_rows(raw.view(torch.int16).to(torch.int32) & 0xFFFF)
    a, e = logits.astype(np.float64), expected.astype(np.float64)
    cosine = (a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e))
    assert cosine > 0.9995 and np.abs(a - e).mean() < 0.05, (cosine, np.abs(a - e).mean())

    # a prompt longer than the activation capacity (8 rows for fixtures without the
    # full-arena flag): every window wraps around to the same rows
    small = [model.context(64, rt.CONTEXT_FLAG_TENSORCORE_FP8) for model in slices]
    small_hidden = [pipe.alias_hidden_rows(c, 8, width, "cuda") for c in small]
    short_expected = evo.load(path, devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC).context(
        64, rt.CONTEXT_FLAG_TENSORCORE_FP8).prefill(bytes(host_tokens[:50].tolist()))
    collected = np.zeros((50, 512), np.float32)
    for begin in range(0, 50, 8):
        count = min(8, 50 - begin)
        small[0].slice_embed(tokens.data_ptr() + 4 * begin, begin, count)
        for index, context in enumerate(small):
            if index > 0:
                small[index - 1].synchronize()
                with torch.cuda.stream(torch.cuda.ExternalStream(context.stream())):
                    small_hidden[index][:count].copy_(small_hidden[index - 1][:count])
            context.slice_run(begin, count)
        address = small[2].slice_head(begin, count)
        small[2].synchronize()
        window = torch.as_tensor(pipe.DeviceRows(address, 8, 512), device="cuda")[:count]
        collected[begin:begin + count] = bf16_rows(window.to(torch.int32) & 0xFFFF)
    a, e = collected.astype(np.float64), short_expected.astype(np.float64)
    assert (a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e)) > 0.9995 and np.abs(a - e).mean() < 0.05

    # misuse is refused with a clear status, and leaves the context usable
    with pytest.raises(rt.EvoError):
        contexts[1].slice_embed(tokens.data_ptr(), 0, 16)       # not the first slice
    with pytest.raises(rt.EvoError):
        contexts[0].slice_head(0, 16)                            # not the last slice
    with pytest.raises(rt.EvoError):
        contexts[0].slice_run(700, 16)                           # not contiguous with the last window
    with pytest.raises(rt.EvoError):
        contexts[0].prefill(b"ACGT")                             # whole-model call on a slice
    with pytest.raises(rt.EvoError):
        evo.load_slice(path, 0, 3, 3, rt.MODEL_FLAG_ALLOW_SYNTHETIC)


RANK = r"""
import sys, importlib, importlib.util
import numpy as np, torch, torch.distributed as dist
root, port, rank, world, model_path, out_path = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5], sys.argv[6]
spec = importlib.util.spec_from_file_location("evo_cpp_b200", root + "/evo.cpp_b200/__init__.py",
                                              submodule_search_locations=[root + "/evo.cpp_b200"])
pkg = importlib.util.module_from_spec(spec); sys.modules["evo_cpp_b200"] = pkg; spec.loader.exec_module(pkg)
rt = importlib.import_module("evo_cpp_b200.runtime"); pipe = importlib.import_module("evo_cpp_b200.pipeline")
torch.cuda.set_device(rank)
dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
model = evo.load_slice(model_path, rank, rank, world, rt.MODEL_FLAG_ALLOW_SYNTHETIC)
context = model.context(2048, rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8)
rows = 1300
host_tokens = np.random.default_rng(77).choice(np.frombuffer(b"ACGT", np.uint8), rows)
tokens = torch.from_numpy(host_tokens.astype(np.int32)).cuda()
stage = pipe.ContextStage(context, tokens)
driver = pipe.StagePipeline(stage, pipe.alias_hidden_rows(context, 2048, 256, "cuda"), rank, world, chunk=512)
with torch.cuda.stream(torch.cuda.ExternalStream(context.stream())):
    for _ in range(3):
        driver.step(rows)
    driver.drain()
context.synchronize()
if rank == world - 1:
    raw = torch.as_tensor(pipe.DeviceRows(stage.logits_address, rows, 512), device="cuda")
    np.save(out_path, raw.cpu().numpy())
dist.barrier(device_ids=[rank])
dist.destroy_process_group()
"""


def test_two_ranks_hand_rows_over_nccl(pkg, tmp_path_factory):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    rt = importlib.import_module("evo_cpp_b200.runtime")
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    directory = tmp_path_factory.mktemp("ranks")
    path = write_model(pkg, directory)
    host_tokens = np.random.default_rng(77).choice(np.frombuffer(b"ACGT", np.uint8), 1300)
    flags = rt.CONTEXT_FLAG_FULL_ARENA | rt.CONTEXT_FLAG_TENSORCORE_FP8
    expected = evo.load(path, devices=[0], flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC).context(2048, flags).prefill(
        bytes(host_tokens.tolist()))
    port = 29700 + (hash(str(directory)) % 200)
    out = directory / "logits.npy"
    procs = [subprocess.Popen([sys.executable, "-c", RANK, str(ROOT), str(port), str(rank), "2", str(path), str(out)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for rank in range(2)]
    outputs = [p.communicate(timeout=600) for p in procs]
    assert all(p.returncode == 0 for p in procs), outputs
    bits = np.load(out).astype(np.uint16)
    logits = (bits.astype(np.uint32) << 16).view(np.float32)
    a, e = logits.astype(np.float64), expected.astype(np.float64)
    cosine = (a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e))
    assert cosine > 0.9995 and np.abs(a - e).mean() < 0.05, (cosine, np.abs(a - e).mean())
