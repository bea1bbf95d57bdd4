#!/usr/bin/env python3
"""Headline benchmark: Evo 2 7B-shaped StripedHyena2 batch-1 prefill on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--tokens T] [--impl reference]

One "step" is one stateless prefill of T uniform-ACGT tokens (default 8192,
the activation-arena size) through the 32-block 7B-shaped model with E4M3 Hyena
projections on the tcgen05 profile and every other projection in BF16.  Weights
are random-init (seeded) in the evo2-runtime-v1 Safetensors format and are
loaded through the same evo_model_load call a user makes.

Printed JSON line (rank 0):
  value      tokens/s with the token ids already resident in HBM, timed with
             CUDA events on the context's stream, max over ranks
  e2e        tokens/s through evo_context_prefill with host bytes in and host
             F32 logits out (H2D + D2H inside the timed region)
  roofline   dominant kernel class (tcgen05 BF16 GEMM): algorithmic FLOPs per
             step / its summed launch time, from per-operator CUDA events
  cpu_baseline  upstream's own CPU backend (oracle/_ref/libevo_ref.so) on a
             bounded sample of the same workload, one core
  parity     outside the timed region: the profile that was timed against the
             bit-exact `exact` profile of the same artifact on the first 1,024
             tokens (top-1 agreement, max-abs error); with N > 1 the pipeline's
             logits against a one-GPU prefill of the same prompt
  prefill_by_length  the same batch-1 prefill at 16 / 128 / 1,024 tokens
With --gpus N > 1 (torchrun, one rank per GPU) the ranks form the layer
pipeline of ONE model: rank r holds stage r of the block split and the prompt
flows through them as a chunk wavefront, hidden rows handed over with NCCL
send/recv (strong scaling: total work per step is fixed).  `value` is the
batch-1 figure: one prompt at a time, a barrier between prompts.  `streamed`
is the K prompts issued back to back, so that a stage starts prompt k+1 while
later stages finish prompt k.  --multi-gpu replicas instead gives every rank a
full replica and its own sequence (weak scaling, no data-path exchange).

--impl reference times upstream's CPU implementation (rank 0 only).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
METRIC = "evo2_7b_shaped_batch1_prefill_tokens_per_second"
SEED = 1  # the 7B-shaped configuration uses random-init weights from seed 1
MODEL_ID = "evo2_7b"
# GEMM FLOPs per token of the 7B shape (D=4096, I=11264, 32 blocks, vocab 512)
WIDTH, INNER, LAYERS, VOCAB, HEADS = 4096, 11264, 32, 512, 32
ATTENTION_LAYERS = 5
SHAPE_TEXT = "Evo 2 7B-shaped StripedHyena2 (32 blocks, d_model 4096, FFN 11264, vocab 512)"

# --model: the other shapes (seed 2: 50 blocks, E4M3 Hyena projections; seed 0: 25 blocks)
MODELS = {
    "evo2_7b": dict(seed=1, width=4096, inner=11264, layers=32, heads=32, attention_layers=5, label="7B"),
    "evo2_40b": dict(seed=2, width=8192, inner=22528, layers=50, heads=64, attention_layers=8, label="40B"),
    "evo2_1b_base": dict(seed=0, width=1920, inner=5120, layers=25, heads=15, attention_layers=4, label="1B"),
}


def select_model(name: str) -> None:
    global METRIC, SEED, MODEL_ID, WIDTH, INNER, LAYERS, HEADS, ATTENTION_LAYERS, SHAPE_TEXT
    m = MODELS[name]
    MODEL_ID, SEED = name, m["seed"]
    WIDTH, INNER, LAYERS, HEADS, ATTENTION_LAYERS = m["width"], m["inner"], m["layers"], m["heads"], m["attention_layers"]
    METRIC = f"{name}_shaped_batch1_prefill_tokens_per_second"
    SHAPE_TEXT = (f"Evo 2 {m['label']}-shaped StripedHyena2 ({LAYERS} blocks, d_model {WIDTH}, FFN {INNER}, "
                  f"vocab {VOCAB})")


def load_package():
    if "evo_cpp_b200" in sys.modules:
        return sys.modules["evo_cpp_b200"]
    pkg_dir = ROOT / "evo.cpp_b200"
    spec = importlib.util.spec_from_file_location(
        "evo_cpp_b200", pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
    module = importlib.util.module_from_spec(spec)
    sys.modules["evo_cpp_b200"] = module
    spec.loader.exec_module(module)
    return module


def artifact_dir(kind: str) -> Path:
    base = Path(os.environ.get("EVO_B200_ARTIFACT_DIR", tempfile.gettempdir())) / "evo_b200_artifacts"
    return base / f"{MODEL_ID}-{kind}-seed{SEED}"


def ensure_artifact(kind: str, device: str | None) -> Path:
    """Writes the 7B-shaped artifact once per box (kind: 'fp8' or 'bf16')."""
    import importlib

    load_package()
    art = importlib.import_module("evo_cpp_b200.artifact")
    directory = artifact_dir(kind)
    marker = directory / "COMPLETE"
    if not marker.exists():
        directory.mkdir(parents=True, exist_ok=True)
        spec = art.with_fp8_projections(art.load_spec(MODEL_ID), kind == "fp8")
        art.write_synthetic(directory / "model.safetensors", spec, SEED, device=device)
        marker.write_text("ok\n")
    return model_entry(directory)


def model_entry(directory: Path) -> Path:
    """The file a loader is pointed at: the shard index, or the single file."""
    index = directory / "model.safetensors.index.json"
    return index if index.exists() else directory / "model.safetensors"


def tokens_for(rank: int, count: int):
    import numpy as np

    rng = np.random.default_rng(SEED + 1000 + rank)
    return rng.choice(np.frombuffer(b"ACGT", np.uint8), count).astype(np.uint8)


def max_over_ranks(value: float, device: str, distributed: bool) -> float:
    """The slowest rank's time: every multi-rank figure is computed from it."""
    import torch

    holder = torch.tensor([value], dtype=torch.float64, device=device)
    if distributed:
        import torch.distributed as dist

        dist.all_reduce(holder, op=dist.ReduceOp.MAX)
    return float(holder.item())


def aggregate_throughput(world: int, tokens_per_rank: int, seconds: float) -> float:
    """Whole-job tokens/s of `world` replicas that each process tokens_per_rank
    tokens per step (weak scaling: per-rank work is fixed)."""
    return world * tokens_per_rank / seconds


def gemm_flops_per_token(tokens: int) -> float:
    per_block = 2.0 * (3 * WIDTH * WIDTH + WIDTH * WIDTH + 3 * WIDTH * INNER)
    return per_block * LAYERS + 2.0 * WIDTH * VOCAB


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.stop_flag, self.thread = index, [], threading.Event(), None

    def _run(self):
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                      "-i", str(self.index)], capture_output=True, text=True, timeout=5).stdout
                fields = [f.strip() for f in out.strip().split(",")]
                if len(fields) >= 6:
                    self.samples.append(fields)
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def __enter__(self):
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()
        return self

    def __exit__(self, *exc):
        self.stop_flag.set()
        self.thread.join(timeout=6)

    def summary(self) -> dict:
        clocks = sorted(int(s[0]) for s in self.samples if s[0].isdigit())
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": int(self.samples[0][1]) if self.samples and self.samples[0][1].isdigit() else None,
                "reasons": reasons, "samples": len(self.samples)}


def run_reference(args, rank: int, world: int) -> None:
    """Upstream's CPU backend on the same model shape (BF16 twin of the seeded
    weights: its registry only admits BF16 projections for this shape)."""
    if rank != 0:
        return
    import importlib

    load_package()
    rt = importlib.import_module("evo_cpp_b200.runtime")
    library_path = ROOT / "oracle" / "_ref" / "libevo_ref.so"
    line = {"impl": "reference", "metric": METRIC, "unit": "tokens/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16 weights, f32 math", "data": "synthetic"}
    if not library_path.exists():
        line["unavailable"] = "oracle/_ref/libevo_ref.so was not built (make -C oracle ref needs the upstream tree)"
        print(json.dumps(line))
        return
    import torch

    directory = ensure_artifact("bf16", "cuda" if torch.cuda.is_available() else None)
    model = rt.EvoLibrary(library_path).load(directory, backend=rt.BACKEND_CPU)
    sample = args.reference_tokens
    sequence = bytes(tokens_for(0, sample).tolist())
    times = []
    for step in range(args.warmup + args.steps):
        context = model.context(max(sample, 16))
        start = time.perf_counter()
        context.prefill(sequence)
        elapsed = time.perf_counter() - start
        context.close()
        if step >= args.warmup:
            times.append(elapsed)
    mean = sum(times) / len(times)
    value = sample / mean
    # the backend runs one sequence on one thread; all host cores = independent contexts side by side
    cores = max(1, len(os.sched_getaffinity(0)))
    finished = []

    def one_replica():
        context = model.context(max(sample, 16))
        context.prefill(sequence)
        context.close()
        finished.append(1)

    threads = [threading.Thread(target=one_replica) for _ in range(cores)]
    begin = time.perf_counter()
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    replicas_seconds = time.perf_counter() - begin
    line["all_cores_replicas"] = {"cores": cores, "contexts": len(finished),
                                  "tokens_per_second": len(finished) * sample / replicas_seconds,
                                  "note": "independent batch-1 contexts, one per core; not a batch-1 latency"}
    line.update({
        "value": value, "ms_per_step": mean * 1e3,
        "config": {"workload": f"7B-shaped StripedHyena2 prefill, {sample}-token sample of the "
                               f"{args.tokens}-token prompt (per-token cost is length-independent on this backend)",
                   "model_id": MODEL_ID, "seed": SEED},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 1, "kind": "reference",
                         "sample": f"{sample}-token prefill per step, upstream cpu-f32 backend (single-threaded)"},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    })
    print(json.dumps(line))


def measure_fp8_library_peak(seconds: float = 1.5) -> dict | None:
    """Denominator for the E4M3 GEMMs: a library FP8 GEMM (torch._scaled_mm, cuBLASLt) at
    8192^3, timed like the BF16 figures of MEASURED_PEAKS.json - best single launch (burst)
    and back to back for `seconds` (sustained, under the power cap)."""
    import torch

    try:
        n = 8192
        a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
        one = torch.ones((), device="cuda")
        run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        flops = 2.0 * n ** 3
        best = float("inf")
        for _ in range(10):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            run()
            stop.record()
            torch.cuda.synchronize()
            best = min(best, start.elapsed_time(stop))
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        count = max(10, int(seconds * 1e3 / best))
        start.record()
        for _ in range(count):
            run()
        stop.record()
        torch.cuda.synchronize()
        return {"fp8_tflops": flops / best / 1e9, "fp8_tflops_sustained": flops * count / start.elapsed_time(stop) / 1e9,
                "how": f"torch._scaled_mm e4m3 8192^3, best of 10 and {count} launches back to back"}
    except Exception as error:  # the library path is only a denominator
        return {"fp8_tflops": None, "fp8_tflops_sustained": None, "how": f"unavailable: {error}"}


def profile_flags(rt, name: str) -> int:
    return {"exact": 0, "b200-tc": rt.CONTEXT_FLAG_TENSORCORE_FP8, "b200-fp8": rt.CONTEXT_FLAG_FP8_FFN}[name]


def flop_classes(tokens: int, profile: str) -> dict:
    """Algorithmic GEMM FLOPs of one prefill, by the operator class that runs them."""
    hyena_layers = LAYERS - ATTENTION_LAYERS
    projection = 2.0 * tokens * WIDTH * 3 * WIDTH * hyena_layers              # E4M3 Hyena input projections
    ffn = 2.0 * tokens * (WIDTH * WIDTH + 3 * WIDTH * INNER) * LAYERS         # output + MLP projections
    total = gemm_flops_per_token(tokens) * tokens
    if profile == "b200-fp8" and tokens > 128:
        return {"gemm_e4m3_tcgen05": projection, "gemm_e4m3_ffn_tcgen05": ffn, "gemm_bf16_tcgen05": total - projection - ffn}
    return {"gemm_e4m3_tcgen05": projection, "gemm_e4m3_ffn_tcgen05": 0.0, "gemm_bf16_tcgen05": total - projection}


def compare_logits(actual, expected) -> dict:
    """Agreement of two [rows, vocab] logit matrices: top-1 overall and on the rows whose winner
    in `expected` leads by more than four times the largest per-logit difference."""
    import numpy as np

    a, e = np.asarray(actual, np.float64), np.asarray(expected, np.float64)
    diff = np.abs(a - e)
    ordered = np.sort(e, axis=-1)
    decided = (ordered[:, -1] - ordered[:, -2]) > 4.0 * diff.max()
    agree = a.argmax(-1) == e.argmax(-1)
    return {"rows": int(a.shape[0]), "top1_agreement": float(agree.mean()),
            "top1_agreement_decided": float(agree[decided].mean()) if decided.any() else 1.0,
            "decided_rows": int(decided.sum()), "max_abs": float(diff.max()), "mean_abs": float(diff.mean()),
            "cosine": float((a * e).sum() / (np.linalg.norm(a) * np.linalg.norm(e) + 1e-30))}


def run_ours(args, rank: int, world: int, local_rank: int) -> None:
    import importlib

    import numpy as np
    import torch

    load_package()
    rt = importlib.import_module("evo_cpp_b200.runtime")
    torch.cuda.set_device(local_rank)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    # one rank writes the artifact, the others wait for it
    if rank == 0:
        ensure_artifact("fp8", "cuda")
    if distributed:
        dist.barrier()
    directory = model_entry(artifact_dir("fp8"))
    library = rt.EvoLibrary(ROOT / "evo.cpp_b200" / "libevo.so")
    load_start = time.perf_counter()
    model = library.load(directory, devices=[local_rank])
    load_seconds = time.perf_counter() - load_start
    tokens = args.tokens
    flags = profile_flags(rt, args.profile)
    context = model.context(tokens, flags)
    host_tokens = tokens_for(rank, tokens)
    device_tokens = torch.from_numpy(host_tokens.astype(np.int32)).cuda()
    stream = torch.cuda.ExternalStream(context.stream())

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident throughput
    for _ in range(args.warmup):
        context.prefill_device(device_tokens.data_ptr(), tokens, True)
    context.synchronize()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clocks:
        start.record(stream)
        for _ in range(args.steps):
            context.prefill_device(device_tokens.data_ptr(), tokens, True)
        stop.record(stream)
        context.synchronize()
    barrier()
    ms_per_step = max_over_ranks(start.elapsed_time(stop), "cuda", distributed) / args.steps
    value = aggregate_throughput(world, tokens, ms_per_step * 1e-3)

    # ---- per-operator timing (separate pass; events cost a few us per launch)
    context.profile_enable(True)
    for _ in range(args.steps):
        context.prefill_device(device_tokens.data_ptr(), tokens, True)
    context.synchronize()
    profile = context.profile_read()
    context.profile_enable(False)
    # operator calls of the runtime; the modal scan is two kernels per call, plus the embedding
    launches_per_step = (sum(n for _, n in profile.values()) + profile.get("hcl_modal_scan", (0, 0))[1]) \
        // args.steps + 1
    classes = flop_classes(tokens, args.profile)
    class_tflops = {name: (flops * args.steps / (profile[name][0] * 1e-3) / 1e12 if profile.get(name, (0, 0))[0] else None)
                    for name, flops in classes.items()}
    peaks = {}
    peaks_file = ROOT / "MEASURED_PEAKS.json"
    if peaks_file.exists():
        peaks = json.loads(peaks_file.read_text())
    bf16_peak = peaks.get("bf16_tflops_sustained", 1400.0)
    fp8_library = measure_fp8_library_peak() if rank == 0 else None
    fp8_peak = (fp8_library or {}).get("fp8_tflops_sustained") or 2.0 * bf16_peak
    # the class that holds most of the step's time is the one the roofline line is about
    dominant = max(("gemm_bf16_tcgen05", "gemm_e4m3_ffn_tcgen05"), key=lambda name: profile.get(name, (0, 0))[0])
    fp8_dominant = dominant == "gemm_e4m3_ffn_tcgen05"
    achieved = class_tflops[dominant]
    peak = fp8_peak if fp8_dominant else bf16_peak
    fp8_rates = [class_tflops[n] for n in ("gemm_e4m3_tcgen05", "gemm_e4m3_ffn_tcgen05") if class_tflops[n]]
    roofline = {"bound": "tensor",
                "kernel": ("gemm_tcgen05_pair_kernel<e4m3> (output and MLP projections of a step)" if fp8_dominant else
                           "gemm_tcgen05_pair_kernel<bf16> (all BF16 projections of a step; CTA pairs on 256 x 256 tiles)"),
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                "peak_source": ("library E4M3 GEMM 8192^3 measured in this run, sustained (of measured)"
                                if fp8_dominant and (fp8_library or {}).get("fp8_tflops_sustained") else
                                "2 x MEASURED_PEAKS.json bf16_tflops_sustained (of measured)" if fp8_dominant else
                                "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)" if peaks else
                                "fallback 1.4 PFLOP/s sustained (of fallback)"),
                "class_tflops": class_tflops,
                "fp8_library_peak": fp8_library,
                "fp8_frac_of_measured": {n: class_tflops[n] / fp8_peak for n in
                                         ("gemm_e4m3_tcgen05", "gemm_e4m3_ffn_tcgen05") if class_tflops[n]},
                "fp8_frac_of_datasheet_4500": {n: class_tflops[n] / 4500.0 for n in
                                               ("gemm_e4m3_tcgen05", "gemm_e4m3_ffn_tcgen05") if class_tflops[n]},
                "bf16_frac_of_measured": class_tflops["gemm_bf16_tcgen05"] / bf16_peak
                if class_tflops["gemm_bf16_tcgen05"] else None,
                # DRAM read + write of one launch of this kernel from an ncu capture
                # (M=8192 K=4096 N=8192: 256 MB algorithmic); the step's launches have other shapes
                "traffic": 337.1e6,
                "traffic_case": "ncu capture of gemm_tcgen05_pair_kernel<bf16> at M=8192 K=4096 N=8192: "
                                "223.2 MB read + 113.9 MB written against 256 MB algorithmic",
                "fp8_projection_tflops": class_tflops["gemm_e4m3_tcgen05"],
                "operator_ms_per_step": {k: v[0] / args.steps for k, v in profile.items() if v[1]}}

    # ---- end to end through the public C ABI: host bytes in, host F32 logits out
    sequence = bytes(host_tokens.tolist())
    e2e_times = []
    for step in range(min(args.warmup, 2) + args.steps):
        fresh = model.context(tokens, flags)
        torch.cuda.synchronize()
        begin = time.perf_counter()
        logits = fresh.prefill(sequence)
        e2e_times.append(time.perf_counter() - begin)
        fresh.close()
    e2e_times = e2e_times[min(args.warmup, 2):]
    e2e_value = aggregate_throughput(
        world, tokens, max_over_ranks(sum(e2e_times) / len(e2e_times), "cuda", distributed))
    assert logits.shape == (tokens, VOCAB) and np.isfinite(logits).all()

    # ---- parity of what was timed (outside every timed region): the bit-exact emulation profile of
    # the same artifact on the first 1,024 tokens; attention and the Hyena operators are causal, so
    # the first rows of the long prefill must also agree with the short one
    parity = None
    if rank == 0:
        head = min(tokens, 1024)
        exact_context = model.context(head, 0)
        exact_logits = exact_context.prefill(sequence[:head])
        exact_context.close()
        fast_context = model.context(head, flags)
        fast_logits = fast_context.prefill(sequence[:head])
        fast_context.close()
        parity = {"reference": "profile exact (bit-exact software-QGMMA emulation) of the same artifact, "
                               f"first {head} tokens of the timed prompt",
                  "timed_profile_vs_exact": compare_logits(fast_logits, exact_logits),
                  "timed_prefill_prefix_vs_short_prefill": compare_logits(logits[:head], fast_logits)}
        checked = parity["timed_profile_vs_exact"]
        parity["ok"] = bool(checked["top1_agreement_decided"] == 1.0 and checked["cosine"] >= 0.999)

    # ---- the other prompt lengths of the metric, device-resident like `value`
    by_length = None
    if rank == 0:
        by_length = {}
        for length in (16, 128, 1024):
            if length >= tokens:
                continue
            short = model.context(length, flags)
            short_stream = torch.cuda.ExternalStream(short.stream())
            for _ in range(3):
                short.prefill_device(device_tokens.data_ptr(), length, True)
            short.synchronize()
            begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            repeats = 10
            begin_event.record(short_stream)
            for _ in range(repeats):
                short.prefill_device(device_tokens.data_ptr(), length, True)
            end_event.record(short_stream)
            short.synchronize()
            ms = begin_event.elapsed_time(end_event) / repeats
            by_length[str(length)] = {"ms": ms, "tokens_per_second": length / (ms * 1e-3)}
            short.close()

    # ---- the opt-in profile with E4M3 output / MLP projections, measured beside the headline one
    # (same prompt, device-resident tokens; its parity against `exact` is reported, not claimed)
    other_profile = None
    if rank == 0 and args.profile == "b200-tc" and tokens > 128 and not args.skip_fp8_profile:
        fp8_context = model.context(tokens, rt.CONTEXT_FLAG_FP8_FFN)
        fp8_stream = torch.cuda.ExternalStream(fp8_context.stream())
        for _ in range(3):
            fp8_context.prefill_device(device_tokens.data_ptr(), tokens, True)
        fp8_context.synchronize()
        begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin_event.record(fp8_stream)
        for _ in range(args.steps):
            fp8_context.prefill_device(device_tokens.data_ptr(), tokens, True)
        end_event.record(fp8_stream)
        fp8_context.synchronize()
        fp8_ms = begin_event.elapsed_time(end_event) / args.steps
        fp8_context.profile_enable(True)
        fp8_context.prefill_device(device_tokens.data_ptr(), tokens, True)
        fp8_context.synchronize()
        fp8_profile = fp8_context.profile_read()
        fp8_context.close()
        head = min(tokens, 1024)
        short = model.context(head, rt.CONTEXT_FLAG_FP8_FFN)
        fp8_logits = short.prefill(sequence[:head])
        short.close()
        ffn_flops = flop_classes(tokens, "b200-fp8")["gemm_e4m3_ffn_tcgen05"]
        ffn_tflops = ffn_flops / (fp8_profile["gemm_e4m3_ffn_tcgen05"][0] * 1e-3) / 1e12
        other_profile = {
            "profile": "b200-fp8", "ms_per_step": fp8_ms, "tokens_per_second": tokens / (fp8_ms * 1e-3),
            "ffn_gemm_tflops": ffn_tflops, "ffn_gemm_frac_of_measured_fp8": ffn_tflops / fp8_peak,
            "ffn_gemm_frac_of_datasheet_4500": ffn_tflops / 4500.0,
            "operator_ms_per_step": {k: v[0] for k, v in fp8_profile.items() if v[1]},
            "vs_exact_first_1024_tokens": compare_logits(fp8_logits, exact_logits),
            "note": "E4M3 rounding of every output / MLP projection operand (~3.8 % per product) is amplified "
                    "by the gated MLPs of a random-init model; this profile is not parity-green on synthetic weights"}

    # ---- cached decode after a 1,024-token prompt (greedy, host sampler, one
    # evo_context_decode call per token: logits come back to the host each step)
    decode = None
    if rank == 0 and args.decode_tokens > 0:
        decode = {}
        for name, decode_flags in ((args.profile, flags), ("exact", 0)):
            ctx = model.context(min(tokens, 1024) + args.decode_tokens + 16, decode_flags)
            prompt_logits = ctx.prefill(sequence[:min(tokens, 1024)])
            token = int(prompt_logits[-1].argmax())
            for _ in range(4):
                token = int(ctx.decode(token).argmax())
            torch.cuda.synchronize()
            begin = time.perf_counter()
            for _ in range(args.decode_tokens):
                token = int(ctx.decode(token).argmax())
            seconds = time.perf_counter() - begin
            decode[name] = {"tokens_per_second": args.decode_tokens / seconds,
                            "ms_per_token": seconds / args.decode_tokens * 1e3}
            ctx.close()

    # ---- a prompt longer than the activation capacity: 8,192-row chunks, the
    # first as a prefill, the rest as continuations (KV caches and Hyena state
    # carried); token ids resident on the device, one timed pass after a warm-up
    long_prompt = None
    if rank == 0 and args.long_tokens > tokens:
        total = args.long_tokens
        long_tokens = torch.from_numpy(tokens_for(7, total).astype(np.int32)).cuda()
        ctx = model.context(total, flags)
        long_stream = torch.cuda.ExternalStream(ctx.stream())

        def run_long():
            ctx.prefill_device(long_tokens.data_ptr(), tokens, False)
            for begin in range(tokens, total, tokens):
                ctx.continue_device(long_tokens.data_ptr() + 4 * begin, min(tokens, total - begin))

        run_long()
        ctx.synchronize()
        begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin_event.record(long_stream)
        run_long()
        end_event.record(long_stream)
        ctx.synchronize()
        long_ms = begin_event.elapsed_time(end_event)
        long_prompt = {"tokens": total, "chunk": tokens, "ms": long_ms, "tokens_per_second": total / (long_ms * 1e-3)}
        ctx.close()

    # ---- layer pipeline of ONE sequence over several GPUs of this process
    # (chunk wavefront, stream-ordered peer copies; strong scaling of batch 1)
    pipeline = None
    if world == 1 and args.pipeline_gpus > 1 and torch.cuda.device_count() >= args.pipeline_gpus:
        context.close()
        model.close()
        piped_model = library.load(directory, devices=list(range(args.pipeline_gpus)))
        piped = piped_model.context(tokens, flags)
        for _ in range(args.warmup):
            piped.prefill_device(device_tokens.data_ptr(), tokens, True)
        piped.synchronize()
        piped_stream = torch.cuda.ExternalStream(piped.stream())
        begin_event, end_event = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin_event.record(piped_stream)
        for _ in range(args.steps):
            piped.prefill_device(device_tokens.data_ptr(), tokens, True)
        end_event.record(piped_stream)
        piped.synchronize()
        piped_ms = begin_event.elapsed_time(end_event) / args.steps
        pipeline = {"gpus": args.pipeline_gpus, "ms_per_step": piped_ms,
                    "tokens_per_second": tokens / (piped_ms * 1e-3),
                    "speedup_over_one_gpu": ms_per_step / piped_ms,
                    "stages": [[s.device, s.layer_begin, s.layer_end] for s in piped.stages()]}
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if world == 1 else "weak", "vs_baseline": None,
            "dtype": ("bf16 activations, e4m3 Hyena / output / MLP projections (tcgen05), f32 accumulate"
                      if args.profile == "b200-fp8" else
                      "bf16 activations, e4m3 Hyena projections (tcgen05), f32 accumulate"),
            "data": "synthetic",
            "config": {"workload": f"{SHAPE_TEXT}, "
                                   f"batch-1 stateless prefill of {tokens} uniform-ACGT tokens, profile {args.profile}",
                       "profile": args.profile,
                       "model_id": MODEL_ID, "seed": SEED, "tokens": tokens,
                       "parallelism": "1 GPU" if world == 1 else f"{world} independent replicas (one sequence per GPU)",
                       "l2_policy": "weights (12 GB) and activations exceed the 126 MB L2 every step; no flush needed",
                       "model_load_seconds": load_seconds},
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": 4 * tokens,
                    "d2h_bytes_per_step": 2 * tokens * VOCAB},
            "gpu_launches": launches_per_step * args.steps,
            "gflop_per_token": gemm_flops_per_token(tokens) / 1e9,
            "model_tflops": gemm_flops_per_token(tokens) * tokens / (ms_per_step * 1e-3) / 1e12,
            "roofline": roofline, "clocks": clocks.summary(),
            "parity": parity, "prefill_by_length": by_length, "fp8_ffn_profile": other_profile,
            "cached_decode_after_1024_token_prompt": decode,
            "layer_pipeline": pipeline,
            "long_prompt_chunked_prefill": long_prompt,
        }
        if world == 1 and not args.skip_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args, rt)
        print(json.dumps(line))
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


def run_pipeline(args, rank: int, world: int, local_rank: int) -> None:
    """One pipeline stage per rank; see the module docstring."""
    import importlib

    import numpy as np
    import torch
    import torch.distributed as dist

    load_package()
    rt = importlib.import_module("evo_cpp_b200.runtime")
    pipe = importlib.import_module("evo_cpp_b200.pipeline")
    torch.cuda.set_device(local_rank)
    # no device_id: point-to-point pairs then get their own communicators, so a
    # stage's send to its successor never queues behind its receive
    dist.init_process_group("nccl")

    def barrier():
        dist.barrier(device_ids=[local_rank])
        torch.cuda.synchronize()

    if rank == 0:
        ensure_artifact("fp8", "cuda")
    barrier()
    directory = model_entry(artifact_dir("fp8"))
    library = rt.EvoLibrary(ROOT / "evo.cpp_b200" / "libevo.so")
    load_start = time.perf_counter()
    model = library.load_slice(directory, local_rank, rank, world)
    load_seconds = time.perf_counter() - load_start
    tokens = args.tokens
    flags = profile_flags(rt, args.profile)
    context = model.context(tokens, flags)
    host_tokens = tokens_for(0, tokens)
    pinned_tokens = torch.from_numpy(host_tokens.astype(np.int32)).pin_memory()
    device_tokens = pinned_tokens.cuda()
    pinned_logits = torch.empty((tokens, VOCAB), dtype=torch.int16).pin_memory()
    stage = pipe.ContextStage(context, device_tokens)
    driver = pipe.StagePipeline(stage, pipe.alias_hidden_rows(context, tokens, WIDTH, "cuda"), rank, world,
                                chunk=args.pipeline_chunk)
    stream = torch.cuda.ExternalStream(context.stream())
    last = rank == world - 1

    def elapsed_max(start, stop) -> float:
        return max_over_ranks(start.elapsed_time(stop), "cuda", True)

    with torch.cuda.stream(stream):
        for _ in range(args.warmup):
            driver.step(tokens)
        context.synchronize()
        barrier()
        # ---- K prompts streamed back to back
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with ClockSampler(local_rank) as clocks:
            start.record(stream)
            for _ in range(args.steps):
                driver.step(tokens)
            stop.record(stream)
            context.synchronize()
        barrier()
        ms_per_step = elapsed_max(start, stop) / args.steps
        # ---- one prompt at a time (latency of a single batch-1 prefill)
        isolated = []
        for _ in range(args.steps):
            barrier()
            start.record(stream)
            driver.step(tokens)
            stop.record(stream)
            context.synchronize()
            isolated.append(elapsed_max(start, stop))
        single_ms = sum(isolated) / len(isolated)
        # ---- per-operator timing
        barrier()
        context.profile_enable(True)
        for _ in range(args.steps):
            driver.step(tokens)
        context.synchronize()
        profile = context.profile_read()
        context.profile_enable(False)
        # ---- end to end: pinned host tokens in on rank 0, logits out to pinned
        # host memory on the last rank, one prompt at a time like `value`
        e2e_total = 0.0
        for _ in range(args.steps):
            barrier()
            begin = time.perf_counter()
            if rank == 0:
                device_tokens.copy_(pinned_tokens, non_blocking=True)
            driver.step(tokens)
            if last:
                raw = torch.as_tensor(pipe.DeviceRows(stage.logits_address, tokens, VOCAB), device="cuda")
                pinned_logits.copy_(raw, non_blocking=True)
            driver.drain()
            context.synchronize()
            e2e_total += max_over_ranks(time.perf_counter() - begin, "cuda", True)
        barrier()
        e2e_seconds = e2e_total / args.steps
    parity = None
    if last:
        bits = pinned_logits.numpy().astype(np.uint16).astype(np.uint32) << 16
        piped_logits = bits.view(np.float32)
        assert np.isfinite(piped_logits).all()
        # the same prompt through the whole model on this rank's GPU alone (outside every timed
        # region): windows change the modal scan's carry and the tile shapes, nothing else
        whole = library.load(directory, devices=[local_rank])
        whole_context = whole.context(tokens, flags)
        single_gpu_logits = whole_context.prefill(bytes(host_tokens.tolist()))
        whole_context.close()
        whole.close()
        parity = {"reference": "one-GPU prefill of the same prompt and profile on the last rank's GPU",
                  "pipeline_vs_one_gpu": compare_logits(piped_logits, single_gpu_logits),
                  "note": "windowed results are within tolerance of the one-GPU logits, not bit-equal"}
        checked = parity["pipeline_vs_one_gpu"]
        parity["ok"] = bool(checked["top1_agreement_decided"] == 1.0 and checked["cosine"] >= 0.999)
    gathered = [None] * world
    dist.all_gather_object(gathered, parity)
    parity = gathered[-1]

    # ---- a prompt longer than the activation capacity through the same pipeline:
    # windows wrap around the hidden-row buffers, state is carried per stage
    long_prompt = None
    if args.long_tokens > tokens:
        total = args.long_tokens
        long_context = model.context(total, flags)
        long_device_tokens = torch.from_numpy(tokens_for(7, total).astype(np.int32)).cuda()
        long_stage = pipe.ContextStage(long_context, long_device_tokens)
        long_driver = pipe.StagePipeline(long_stage, pipe.alias_hidden_rows(long_context, tokens, WIDTH, "cuda"),
                                         rank, world, chunk=args.pipeline_chunk)
        long_stream = torch.cuda.ExternalStream(long_context.stream())
        with torch.cuda.stream(long_stream):
            long_driver.step(total)
            long_driver.drain()
            long_context.synchronize()
            barrier()
            start.record(long_stream)
            long_driver.step(total)
            long_driver.drain()
            stop.record(long_stream)
            long_context.synchronize()
            long_ms = elapsed_max(start, stop)
        long_prompt = {"tokens": total, "ms": long_ms, "tokens_per_second": total / (long_ms * 1e-3),
                       "windows": len(pipe.window_plan(total, world, args.pipeline_chunk))}

    totals = torch.tensor([sum(n for _, n in profile.values()) + (1 if rank == 0 else 0) * args.steps,
                           profile["gemm_bf16_tcgen05"][0], profile["gemm_e4m3_tcgen05"][0],
                           profile["gemm_e4m3_ffn_tcgen05"][0]],
                          dtype=torch.float64, device="cuda")
    dist.all_reduce(totals)
    per_operator = torch.tensor([profile[name][0] for name in sorted(profile)], dtype=torch.float64, device="cuda")
    dist.all_reduce(per_operator)
    layout = [None] * world
    info = context.stages()[0]
    dist.all_gather_object(layout, [rank, int(info.layer_begin), int(info.layer_end),
                                    round(info.weight_bytes / 2**30, 2)])
    if rank == 0:
        launches, gemm_ms, fp8_ms, ffn_ms = (float(x) for x in totals.tolist())
        classes = flop_classes(tokens, args.profile)
        flops_fp8 = classes["gemm_e4m3_tcgen05"]
        peaks_file = ROOT / "MEASURED_PEAKS.json"
        peaks = json.loads(peaks_file.read_text()) if peaks_file.exists() else {}
        fp8_dominant = ffn_ms > gemm_ms
        # window sizes exceed 128 rows, so the FP8 FFN profile applies in every window
        achieved = (classes["gemm_e4m3_ffn_tcgen05"] * args.steps / (ffn_ms * 1e-3) / 1e12 if fp8_dominant else
                    classes["gemm_bf16_tcgen05"] * args.steps / (gemm_ms * 1e-3) / 1e12)
        peak = peaks.get("bf16_tflops_sustained", 1400.0) * (2.0 if fp8_dominant else 1.0)
        line = {
            "metric": METRIC, "value": tokens / (single_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": single_ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None,
            "dtype": ("bf16 activations, e4m3 Hyena / output / MLP projections (tcgen05), f32 accumulate"
                      if args.profile == "b200-fp8" else
                      "bf16 activations, e4m3 Hyena projections (tcgen05), f32 accumulate"), "data": "synthetic",
            "config": {"workload": f"{SHAPE_TEXT}, "
                                   f"batch-1 stateless prefill of {tokens} uniform-ACGT tokens, profile {args.profile}",
                       "profile": args.profile,
                       "model_id": MODEL_ID, "seed": SEED, "tokens": tokens,
                       "parallelism": f"pp{world}: one pipeline stage per rank, chunk wavefront, NCCL send/recv of "
                                      f"hidden rows; one prompt at a time (batch 1), barrier between prompts",
                       "stages": layout, "windows": pipe.window_plan(tokens, world, args.pipeline_chunk),
                       "l2_policy": "weights and activations exceed the 126 MB L2 every step; no flush needed",
                       "model_load_seconds": load_seconds},
            "streamed": {"ms_per_prompt": ms_per_step, "tokens_per_second": tokens / (ms_per_step * 1e-3),
                         "note": f"the {args.steps} timed prompts issued back to back: stage r starts prompt k+1 "
                                 "while later stages finish prompt k (several prompts in flight, not batch-1 latency)"},
            "parity": parity,
            "e2e": {"value": tokens / e2e_seconds, "unit": "tokens/s", "h2d_bytes_per_step": 4 * tokens,
                    "d2h_bytes_per_step": 2 * tokens * VOCAB},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor",
                         "kernel": ("gemm_tcgen05_kernel / gemm_tcgen05_pair_kernel <e4m3> (output and MLP projections, "
                                    "all ranks)" if fp8_dominant
                                    else "gemm_tcgen05_kernel / gemm_tcgen05_pair_kernel <bf16> (all BF16 projections, "
                                         "all ranks; pairs from 48 tiles per window on)"),
                         "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": ("2 x MEASURED_PEAKS.json bf16_tflops_sustained (of measured)" if fp8_dominant
                                         else "MEASURED_PEAKS.json bf16_tflops_sustained (of measured)") if peaks else
                                        "fallback 1.4 PFLOP/s sustained (of fallback)",
                         "traffic": None,
                         "fp8_projection_tflops": flops_fp8 * args.steps / (fp8_ms * 1e-3) / 1e12 if fp8_ms else None,
                         "operator_ms_per_step_summed_over_ranks": {
                             name: ms / args.steps for name, ms in zip(sorted(profile), per_operator.tolist()) if ms}},
            "clocks": clocks.summary(),
            "long_prompt_chunked_prefill": long_prompt,
        }
        print(json.dumps(line))
    barrier()
    dist.destroy_process_group()


def cpu_baseline(args, rt) -> dict:
    library_path = ROOT / "oracle" / "_ref" / "libevo_ref.so"
    if not library_path.exists():
        return {"value": None, "unit": "tokens/s", "cores": 1, "kind": "reference",
                "sample": "unavailable: oracle/_ref/libevo_ref.so was not built"}
    directory = ensure_artifact("bf16", "cuda")
    model = rt.EvoLibrary(library_path).load(directory, backend=rt.BACKEND_CPU)
    sample = args.reference_tokens
    sequence = bytes(tokens_for(0, sample).tolist())
    context = model.context(max(sample, 16))
    begin = time.perf_counter()
    context.prefill(sequence)
    seconds = time.perf_counter() - begin
    return {"value": sample / seconds, "unit": "tokens/s", "cores": 1, "kind": "reference",
            "sample": f"one {sample}-token prefill of the BF16 twin of the same seeded 7B-shaped weights on "
                      f"upstream's cpu-f32 backend (single-threaded; {seconds:.1f} s)"}


def main() -> None:
    # NCCL prints its version banner on stdout at NCCL_DEBUG=VERSION; stdout carries the JSON line only
    if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
        os.environ["NCCL_DEBUG"] = "WARN"
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=5)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--tokens", type=int, default=8192)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--reference-tokens", type=int, default=8,
                        help="tokens per CPU step (about 0.5 tokens/s/core on this shape)")
    parser.add_argument("--skip-cpu-baseline", action="store_true")
    parser.add_argument("--pipeline-gpus", type=int, default=0,
                        help="also time the same prefill as a layer pipeline over this many GPUs of "
                             "one process (needs that many visible GPUs; only with --gpus 1)")
    parser.add_argument("--multi-gpu", default="pipeline", choices=["pipeline", "replicas"],
                        help="what --gpus N > 1 ranks do: stages of one layer pipeline (default) or "
                             "independent full replicas")
    parser.add_argument("--pipeline-chunk", type=int, default=0,
                        help="rows per wavefront window (0: about two windows per stage, 512..2048)")
    parser.add_argument("--model", default="evo2_7b", choices=sorted(MODELS),
                        help="model shape (the headline metric is quoted on evo2_7b)")
    parser.add_argument("--long-tokens", type=int, default=0,
                        help="also time a chunked prefill of this many tokens (> --tokens; 0 disables)")
    parser.add_argument("--profile", default="b200-tc", choices=["b200-tc", "b200-fp8"],
                        help="execution profile that is timed (b200-fp8 also runs the output and MLP "
                             "projections in E4M3)")
    parser.add_argument("--skip-fp8-profile", action="store_true",
                        help="do not also time the opt-in b200-fp8 profile")
    parser.add_argument("--decode-tokens", type=int, default=64,
                        help="cached-decode steps timed after a 1,024-token prompt (0 disables)")
    args = parser.parse_args()
    select_model(args.model)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    elif world > 1 and args.multi_gpu == "pipeline":
        run_pipeline(args, rank, world, local_rank)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
