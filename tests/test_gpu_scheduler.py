"""Request scheduler over shared-weight contexts (evo_b200_scheduler_*; upstream's serving loop:
DynamicScheduler, src/scheduler.cpp:49-201, on contexts sharing one copy of the weights,
src/cuda/model.cu:2596-2691).  Requests run concurrently on a pool of long-lived contexts;
every result must equal what one context alone computes for the same input, bit for bit."""
from __future__ import annotations

import importlib
import json
import subprocess
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def rt(pkg):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return importlib.import_module("evo_cpp_b200.runtime")


@pytest.fixture(scope="module")
def fixture_path(pkg, tmp_path_factory):
    art = importlib.import_module("evo_cpp_b200.artifact")
    directory = tmp_path_factory.mktemp("scheduler")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16)
    art.write_synthetic(directory / "model.safetensors", spec, seed=9, weight_std=0.05, filter_std=0.3)
    return directory / "model.safetensors"


def log_softmax_score(logits: np.ndarray, sequence: bytes) -> list[float]:
    out = []
    for t in range(len(sequence) - 1):
        row = logits[t].astype(np.float64)
        peak = float(logits[t].max())
        out.append(float(row[sequence[t + 1]] - peak - np.log(np.exp(row - peak).sum())))
    return out


def test_concurrent_requests_equal_single_context_results(rt, pkg, fixture_path):
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    model = evo.load(fixture_path, flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    rng = np.random.default_rng(4)
    sequences = [bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), int(n)).tolist())
                 for n in rng.integers(2, 400, 24)]
    scheduler = rt.Scheduler(model, workers=4, maximum_queue=64, context_size=512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
    tickets = [scheduler.score(s) for s in sequences]
    prompt = sequences[3][:40]
    greedy = scheduler.generate(prompt, 6)
    sampled = scheduler.generate(prompt, 6, temperature=0.8, top_k=4, top_p=0.9, seed=7)
    assert all(tickets) and greedy and sampled
    scheduler.wait_idle()
    metrics = scheduler.metrics()
    unfinished = {t: (r["status"], r["error"], r["cancelled"]) for t, r in scheduler.results.items()
                  if r["status"] != 0 or r["cancelled"]}
    assert metrics["submitted"] == metrics["completed"] == 26 and metrics["failed"] == metrics["rejected"] == 0, \
        (metrics, unfinished)
    assert metrics["queued"] == metrics["active"] == 0 and 1 <= metrics["active_peak"] <= 4
    for ticket, sequence in zip(tickets, sequences):
        result = scheduler.results[ticket]
        assert result["status"] == 0 and not result["cancelled"] and result["scored_tokens"] == len(sequence) - 1
        logits = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA).prefill(sequence)
        expected = log_softmax_score(logits, sequence)
        assert np.allclose(result["token_log_likelihoods"], expected, rtol=0, atol=1e-12)
        assert abs(result["log_likelihood"] - sum(expected)) < 1e-9
    # generation: the same tokens as one context decoding greedily / with the same sampler seed
    for ticket, kwargs in ((greedy, {}), (sampled, dict(temperature=0.8, top_k=4, top_p=0.9, seed=7))):
        context = model.context(512, flags=rt.CONTEXT_FLAG_FULL_ARENA)
        sampler = rt.Sampler(evo, **kwargs)
        row, produced = context.prefill(prompt)[-1], []
        for step in range(6):
            token = sampler.sample(row)
            if token > 255:          # not a byte: generation ends (vocabulary 512, upstream token_to_byte)
                break
            produced.append(token)
            if step < 5:
                row = context.decode(token)
        assert scheduler.results[ticket]["generated"] == bytes(produced)
    # the model may be freed while the scheduler still holds its weights
    model.close()
    late = scheduler.score(sequences[0])
    scheduler.wait_idle()
    assert scheduler.results[late]["log_likelihood"] == scheduler.results[tickets[0]]["log_likelihood"]
    scheduler.close()


def test_queue_limit_cancellation_and_request_errors(rt, pkg, fixture_path):
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    model = evo.load(fixture_path, flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    with pytest.raises(rt.EvoError):
        rt.Scheduler(model, workers=4, maximum_queue=2, context_size=128)          # queue smaller than the pool
    scheduler = rt.Scheduler(model, workers=1, maximum_queue=2, context_size=2048)
    long_sequence = b"ACGT" * 400                          # 1,600 tokens in 8-row chunks: hundreds of steps
    first = scheduler.score(long_sequence)
    tickets = [scheduler.score(b"ACGTACGT") for _ in range(6)]
    accepted = [t for t in tickets if t]
    assert first and 1 <= len(accepted) <= 2 and tickets.count(0) >= 4      # at most two wait in the queue
    assert scheduler.cancel(accepted[-1]) and scheduler.cancel(first)
    scheduler.wait_idle()
    assert scheduler.results[first]["cancelled"] and scheduler.results[accepted[-1]]["cancelled"]
    metrics = scheduler.metrics()
    assert metrics["rejected"] == tickets.count(0) and metrics["cancelled"] == 2
    assert metrics["submitted"] == 1 + len(accepted) and metrics["queue_peak"] <= 2
    assert not scheduler.cancel(first)                                        # finished: nothing to cancel
    scheduler.close()
    # request-level errors come back through the completion, the worker's context stays usable
    scheduler = rt.Scheduler(model, workers=1, maximum_queue=8, context_size=2048)
    too_long = scheduler.score(b"A" * 3000)
    single = scheduler.score(b"A")
    bad_sampler = scheduler.generate(b"ACGT", 4, temperature=-1.0, top_k=3)
    fine = scheduler.score(b"ACGTACGT")
    scheduler.wait_idle()
    assert scheduler.results[too_long]["status"] == 2 and "context capacity" in scheduler.results[too_long]["error"]
    assert scheduler.results[single]["status"] == 2 and "two tokens" in scheduler.results[single]["error"]
    assert scheduler.results[bad_sampler]["status"] == 2
    assert scheduler.results[fine]["status"] == 0 and scheduler.results[fine]["scored_tokens"] == 7
    scheduler.close()


def test_serve_command_answers_jsonl_requests(pkg, fixture_path, tmp_path):
    requests = "\n".join([
        json.dumps({"id": "s1", "op": "score", "sequence": "ACGTACGTAC"}),
        json.dumps({"id": "g1", "op": "generate", "prompt": "ACGT", "tokens": 5}),
        json.dumps({"id": "bad", "op": "translate"}),
        json.dumps({"op": "score", "sequence": "GGGGCCCC"}),
    ]) + "\n"
    result = subprocess.run([str(pkg.PACKAGE_DIR / "evo"), "serve", "-m", str(fixture_path),
                             "--allow-test-fixture", "--workers", "2", "--ctx", "64"], input=requests.encode(),
                            capture_output=True, check=True)
    rows = {row["id"]: row for row in map(json.loads, result.stdout.decode().splitlines())}
    assert set(rows) == {"s1", "g1", "bad", "4"}
    assert rows["bad"]["error"]["code"] == "invalid_argument"
    assert rows["s1"]["scored_tokens"] == 9 and rows["4"]["scored_tokens"] == 7 and len(rows["g1"]["generated"]) <= 5
    raw = tmp_path / "s1.txt"
    raw.write_bytes(b"ACGTACGTAC")
    scored = json.loads(subprocess.run([str(pkg.PACKAGE_DIR / "evo"), "score", "-m", str(fixture_path),
                                        "--allow-test-fixture", "--input", str(raw), "--ctx", "64"],
                                       capture_output=True, check=True).stdout.decode())
    assert rows["s1"]["log_likelihood"] == scored["log_likelihood"]
    totals = [json.loads(line) for line in result.stderr.decode().splitlines() if line.startswith('{"scheduler"')]
    assert totals and totals[0]["scheduler"]["submitted"] == totals[0]["scheduler"]["completed"] == 3
    assert totals[0]["scheduler"]["workers"] == 2
