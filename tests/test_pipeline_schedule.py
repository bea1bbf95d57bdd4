"""Host logic of the per-process layer pipeline (CPU, gloo).

The schedule is exercised with a stand-in stage whose "blocks" are a causal
running sum carried from window to window, so a wrong window order, a missing
hand-off or a lost carry changes the result."""
from __future__ import annotations

import importlib
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_window_plan_covers_the_prompt(pkg):
    pipeline = importlib.import_module("evo_cpp_b200.pipeline")
    for rows, stages in [(8192, 1), (8192, 2), (8192, 8), (1300, 2), (513, 4), (100, 2), (65536, 8)]:
        plan = pipeline.window_plan(rows, stages)
        assert plan[0][0] == 0 and sum(count for _, count in plan) == rows
        assert all(plan[i][0] + plan[i][1] == plan[i + 1][0] for i in range(len(plan) - 1))
        assert all(count % 256 == 0 and 512 <= count <= 2048 for _, count in plan[:-1])
    assert pipeline.window_plan(8192, 2) == [(i * 2048, 2048) for i in range(4)]
    assert pipeline.window_plan(8192, 4) == [(i * 1024, 1024) for i in range(8)]
    assert pipeline.window_plan(8192, 8) == [(i * 1024, 1024) for i in range(8)]
    assert pipeline.window_plan(4096, 8) == [(i * 512, 512) for i in range(8)]
    assert all(8192 % count == 0 for _, count in pipeline.window_plan(131072, 8))
    assert pipeline.window_plan(1000, 2, chunk=300) == [(0, 300), (300, 300), (600, 300), (900, 100)]
    with pytest.raises(ValueError):
        pipeline.window_plan(0, 2)


WORKER = r"""
import sys, importlib.util
import torch, torch.distributed as dist
root, port, rank, world = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
spec = importlib.util.spec_from_file_location("evo_cpp_b200", root + "/evo.cpp_b200/__init__.py",
                                              submodule_search_locations=[root + "/evo.cpp_b200"])
module = importlib.util.module_from_spec(spec); sys.modules["evo_cpp_b200"] = module; spec.loader.exec_module(module)
from evo_cpp_b200.pipeline import StagePipeline
dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)

class RunningSumStage:
    # blocks of this stage: y[t] = (rank + 2) * x[t] + carry, carry += sum of the window's inputs
    def __init__(self, hidden, tokens):
        self.hidden, self.tokens, self.carry, self.calls, self.logits = hidden, tokens, 0.0, [], None
    # position p lives at hidden row p % capacity (prompts longer than the buffer wrap around)
    def embed(self, begin, count):
        row = begin % len(self.hidden)
        self.hidden[row:row + count] = self.tokens[begin:begin + count, None].to(self.hidden.dtype)
    def run(self, begin, count):
        if begin == 0:
            self.carry, self.logits = 0.0, torch.zeros(len(self.tokens), self.hidden.shape[1], dtype=torch.float64)
        row = begin % len(self.hidden)
        rows = self.hidden[row:row + count]
        total = float(rows.sum())
        rows.mul_(rank + 2).add_(self.carry)
        self.carry += total
        self.calls.append((begin, count))
    def head(self, begin, count):
        row = begin % len(self.hidden)
        self.logits[begin:begin + count] = self.hidden[row:row + count]

rows, width = 1300, 3
tokens = torch.arange(rows, dtype=torch.float64) % 7
hidden = torch.zeros(1024, width, dtype=torch.float64)   # shorter than the prompt: the third window wraps
stage = RunningSumStage(hidden, tokens)
pipe = StagePipeline(stage, hidden, rank, world, chunk=512)
for _ in range(2):  # two prompts back to back: rows still in flight must not be overwritten
    pipe.step(rows)
pipe.drain()
assert stage.calls == [(0, 512), (512, 512), (1024, 276)] * 2, stage.calls
if rank == world - 1:
    # sequential restatement over the whole prompt, stage after stage
    expected = tokens[:, None].repeat(1, width)
    for r in range(world):
        carry, out = 0.0, torch.empty_like(expected)
        for begin in (0, 512, 1024):
            window = expected[begin:begin + 512]
            out[begin:begin + 512] = window * (r + 2) + carry
            carry += float(window.sum())
        expected = out
    assert torch.equal(stage.logits, expected)
    print("ok")
dist.barrier()
dist.destroy_process_group()
"""


@pytest.mark.parametrize("world", [2, 3])
def test_wavefront_schedule_over_gloo(world):
    port = 29950 + world + (hash(str(ROOT)) % 300)
    procs = [subprocess.Popen([sys.executable, "-c", WORKER, str(ROOT), str(port), str(rank), str(world)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for rank in range(world)]
    outputs = [p.communicate(timeout=240) for p in procs]
    assert all(p.returncode == 0 for p in procs), outputs
    assert outputs[-1][0].strip().endswith("ok")
