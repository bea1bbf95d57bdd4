#!/usr/bin/env python3
"""Operator microbenchmarks through the operator C ABI (one GPU).

    python evo.cpp_b200/kernel_bench.py gemm   --rows 8192 --inner 4096 --outer 12288 [--type bf16|e4m3|emulated]
    python evo.cpp_b200/kernel_bench.py hyena  --length 8192 --channels 4096 [--op hcs|hcm|hcl|all]
    python evo.cpp_b200/kernel_bench.py norm   --rows 8192 --width 4096
    python evo.cpp_b200/kernel_bench.py attention --rows 8192 --heads 32
    python evo.cpp_b200/kernel_bench.py sweep      # the operator shapes of the reference workloads
    python evo.cpp_b200/kernel_bench.py grid       # E4M3 projection grid: M x {12288, 11264, 4096}, K = 4096, all modes
    python evo.cpp_b200/kernel_bench.py fp8peak    # library E4M3 GEMM 8192^3 (the FP8 denominator)

Inputs are seeded synthetic tensors with the shapes and value distributions of
the reference workloads (BF16 N(0,1) activations, N(0,0.02) weights, modal poles
with radius U[0.9,0.999)).  Every timed launch is preceded by an L2 flush (a
256 MiB write, then a 256 MiB read so that no dirty lines are left) and timed with CUDA events on the launching stream; the median
of --iters launches is reported as one JSON line per operator with the
algorithmic bytes or FLOPs and the fraction of the measured peak
(MEASURED_PEAKS.json at the repository root when present).
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import sys
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent


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


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, iters: int, warmup: int = 3):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
        self.clean = torch.zeros(64 << 20, dtype=torch.int32, device="cuda")

    def __call__(self, launch) -> float:
        """Median milliseconds of `launch()` (which enqueues on the current stream)."""
        for _ in range(self.warmup):
            launch()
        torch.cuda.synchronize()
        times = []
        for _ in range(self.iters):
            # Cold L2 without pending write-backs: the write pass evicts everything,
            # the read pass then replaces its dirty lines with clean ones (a timed
            # kernel that evicts 126 MB of dirty lines pays ~15 us of DRAM writes
            # that are not its own).
            self.flush.zero_()
            self.clean.sum()
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            launch()
            stop.record()
            torch.cuda.synchronize()
            times.append(start.elapsed_time(stop))
        times.sort()
        return times[len(times) // 2]


def p(tensor):
    return None if tensor is None else tensor.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def report(name: str, ms: float, *, bytes_moved: float | None = None, flops: float | None = None, **extra):
    pk = peaks()
    line = {"operator": name, "ms": ms, **extra}
    if bytes_moved is not None:
        line["algorithmic_bytes"] = bytes_moved
        line["gb_per_s"] = bytes_moved / ms / 1e6
        line["frac_of_hbm_copy_peak"] = line["gb_per_s"] / pk["hbm_gbs"]
    if flops is not None:
        line["flops"] = flops
        line["tflop_per_s"] = flops / ms / 1e9
        line["frac_of_bf16_gemm_peak"] = line["tflop_per_s"] / pk["bf16_tflops"]
    line["peak_source"] = pk["source"]
    print(json.dumps(line), flush=True)
    return line


def bench_gemm(ops, timer, rows, inner, outer, kind):
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, inner, device="cuda", generator=gen).bfloat16()
    out = torch.empty(rows, outer, device="cuda", dtype=torch.bfloat16)
    flops = 2.0 * rows * inner * outer
    if kind == "bf16":
        w = (torch.randn(outer, inner, device="cuda", generator=gen) * 0.02).bfloat16()
        if 8 < rows <= 128:
            # few tokens: the runtime hands every projection a 64 MiB partial-sum workspace
            workspace = torch.empty(16 << 20, device="cuda")
            ms = timer(lambda: ops.call("bf16_linear_split_k", p(x), p(w), None, None, rows, inner, outer, 0, 0,
                                        p(workspace), workspace.numel() * 4, p(out), stream()))
        else:
            ms = timer(lambda: ops.call("bf16_linear", p(x), p(w), None, None, rows, inner, outer, 0, 0, p(out),
                                        stream()))
        ops.call("check_async_errors", stream())
        return report("gemm_tcgen05_bf16", ms, flops=flops, rows=rows, inner=inner, outer=outer)
    w = torch.randn(outer, inner, device="cuda", generator=gen) * 0.02
    w_scale = 448.0 / float(w.abs().max())
    codes = (w * w_scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    in_scale = 448.0 / float(x.float().abs().max())
    out_scale = (1.0 / in_scale) * (1.0 / w_scale)
    scratch = torch.empty(rows * inner, dtype=torch.uint8, device="cuda")
    entry = "e4m3_tensorcore_linear" if kind == "e4m3" else "software_e4m3_h100_linear"
    ms = timer(lambda: ops.call(entry, p(x), p(codes), rows, inner, outer, in_scale, out_scale, p(scratch),
                                p(out), stream()))
    ops.call("check_async_errors", stream())
    name = "quantise+gemm_tcgen05_e4m3" if kind == "e4m3" else "quantise+qgmma_emulation"
    return report(name, ms, flops=flops, rows=rows, inner=inner, outer=outer,
                  weight_gb_per_s=outer * inner / ms / 1e6)


def bench_codes_gemm(ops, timer, rows, inner, outer):
    """The E4M3 GEMM alone (operands already codes, per-row scales in the epilogue)."""
    gen = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(rows, inner, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(outer, inner, device="cuda", generator=gen) * 0.02).bfloat16()
    x_codes = torch.empty(rows, inner, dtype=torch.uint8, device="cuda")
    scales = torch.empty(rows, device="cuda")
    ops.call("e4m3_quantize_rows", p(x), rows, inner, p(x_codes), p(scales), stream())
    w_scale = 448.0 / float(w.float().abs().max())
    w_codes = (w.float() * w_scale).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    out = torch.empty(rows, outer, device="cuda", dtype=torch.bfloat16)
    ms = timer(lambda: ops.call("e4m3_codes_linear", p(x_codes), p(scales), p(w_codes), None, None, rows, inner,
                                outer, 1.0 / w_scale, 0, 0, p(out), stream()))
    ops.call("check_async_errors", stream())
    line = report("gemm_tcgen05_e4m3_codes", ms, flops=2.0 * rows * inner * outer, rows=rows, inner=inner, outer=outer,
                  weight_gb_per_s=outer * inner / ms / 1e6)
    ms = timer(lambda: ops.call("e4m3_quantize_rows", p(x), rows, inner, p(x_codes), p(scales), stream()))
    report("e4m3_quantize_rows", ms, bytes_moved=3.0 * rows * inner, rows=rows, width=inner)
    return line


def fp8_library_peak(seconds: float = 2.0):
    n = 8192
    a = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device="cuda").to(torch.float8_e4m3fn).t()
    one = torch.ones((), device="cuda")
    run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(10):
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        run()
        stop.record()
        torch.cuda.synchronize()
        best = min(best, start.elapsed_time(stop))
    count = max(10, int(seconds * 1e3 / best))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(count):
        run()
    stop.record()
    torch.cuda.synchronize()
    flops = 2.0 * n ** 3
    print(json.dumps({"operator": "library_e4m3_gemm_8192^3 (torch._scaled_mm)", "ms_best": best,
                      "fp8_tflops": flops / best / 1e9,
                      "fp8_tflops_sustained": flops * count / start.elapsed_time(stop) / 1e9, "launches": count}),
          flush=True)


def bench_hyena_projection(ops, timer, length, channels, which):
    """The forms the model runs: fed by the interleaved [length, 3*channels]
    projection, 3-tap featurizer applied on the fly, decode caches written."""
    gen = torch.Generator(device="cuda").manual_seed(1)
    projection = torch.randn(length, 3 * channels, device="cuda", generator=gen).bfloat16()
    short = (torch.randn(3 * channels, 3, device="cuda", generator=gen) * 0.3).bfloat16()
    out = torch.empty(length, channels, device="cuda", dtype=torch.bfloat16)
    short_cache = torch.zeros(3 * channels, 2, device="cuda")
    groups = max(1, channels // 16)
    fused_bytes = 8.0 * length * channels
    lines = []
    for name, taps, orientation in (("hcs", 7, 0), ("hcm", 128, 1)):
        if which not in (name, "all"):
            continue
        h = (torch.randn(groups, taps, device="cuda", generator=gen) * 0.02).bfloat16()
        d = (torch.randn(channels, device="cuda", generator=gen) * 0.02).bfloat16() if orientation else None
        cache = torch.zeros(channels, taps - 1, device="cuda")
        ms = timer(lambda: ops.call("bf16_projection_gated_fir_prefill", p(projection), p(short), p(h), 0, p(d),
                                    length, channels, groups, taps, orientation, None, p(cache), p(short_cache),
                                    p(out), stream()))
        lines.append(report(f"{name}_projection_fed_k{taps}", ms, bytes_moved=fused_bytes,
                            flops=2.0 * taps * length * channels, length=length, channels=channels))
    if which in ("hcl", "all"):
        modes = 16
        d = (torch.randn(channels, device="cuda", generator=gen) * 0.02).bfloat16()
        log_poles = (torch.rand(channels, modes, device="cuda", generator=gen) * 0.099 + 0.9).log().float()
        residues = (torch.randn(channels, modes, device="cuda", generator=gen) * 0.02).float()
        scratch = torch.empty(ops.hcl_scratch_floats(length, channels, modes), device="cuda")
        state = torch.zeros(channels, modes, device="cuda")
        ms = timer(lambda: ops.call("bf16_projection_hcl_prefill", p(projection), p(short), p(d), p(log_poles),
                                    p(residues), length, channels, modes, 0, p(state), p(scratch), p(short_cache),
                                    None, p(out), stream()))
        lines.append(report("hcl_projection_fed_modal_scan", ms, bytes_moved=fused_bytes,
                            flops=64.0 * length * channels, length=length, channels=channels))
    return lines


def bench_hyena(ops, timer, length, channels, which):
    gen = torch.Generator(device="cuda").manual_seed(1)
    x2, x1, v = (torch.randn(length, channels, device="cuda", generator=gen).bfloat16() for _ in range(3))
    out = torch.empty(length, channels, device="cuda", dtype=torch.bfloat16)
    groups = max(1, channels // 16)
    fused_bytes = 8.0 * length * channels
    lines = []
    if which in ("hcs", "all"):
        h = (torch.randn(groups, 7, device="cuda", generator=gen) * 0.02).bfloat16()
        ms = timer(lambda: ops.call("bf16_gated_fir_prefill", p(x2), p(x1), p(v), p(h), 0, None, length, channels,
                                    groups, 7, 0, None, None, p(out), stream()))
        lines.append(report("hcs_gated_fir_k7", ms, bytes_moved=fused_bytes, flops=2.0 * 7 * length * channels,
                            length=length, channels=channels))
    if which in ("hcm", "all"):
        h = (torch.randn(groups, 128, device="cuda", generator=gen) * 0.02).bfloat16()
        d = (torch.randn(channels, device="cuda", generator=gen) * 0.02).bfloat16()
        ms = timer(lambda: ops.call("bf16_gated_fir_prefill", p(x2), p(x1), p(v), p(h), 0, p(d), length, channels,
                                    groups, 128, 1, None, None, p(out), stream()))
        lines.append(report("hcm_gated_fir_k128", ms, bytes_moved=fused_bytes, flops=2.0 * 128 * length * channels,
                            length=length, channels=channels))
    if which in ("hcl", "all"):
        modes = 16
        d = (torch.randn(channels, device="cuda", generator=gen) * 0.02).bfloat16()
        radius = torch.rand(channels, modes, device="cuda", generator=gen) * 0.099 + 0.9
        log_poles = radius.log().float()
        residues = (torch.randn(channels, modes, device="cuda", generator=gen) * 0.02).float()
        scratch = torch.empty(ops.hcl_scratch_floats(length, channels, modes), device="cuda")
        state = torch.zeros(channels, modes, device="cuda")
        ms = timer(lambda: ops.call("bf16_hcl_prefill", p(x2), p(x1), p(v), p(d), p(log_poles), p(residues), length,
                                    channels, modes, 0, p(state), p(scratch), None, p(out), stream()))
        lines.append(report("hcl_modal_scan", ms, bytes_moved=fused_bytes, flops=64.0 * length * channels,
                            length=length, channels=channels))
    return lines


def bench_norm(ops, timer, rows, width):
    x = torch.randn(rows, width, device="cuda").bfloat16()
    scale = torch.ones(width, device="cuda")
    out = torch.empty_like(x)
    codes = torch.empty(rows, width, dtype=torch.uint8, device="cuda")
    ms = timer(lambda: ops.call("bf16_rms_norm", p(x), p(scale), rows, width, 1e-6, p(out), None, 1.0, stream()))
    a = report("rms_norm", ms, bytes_moved=4.0 * rows * width, rows=rows, width=width)
    ms = timer(lambda: ops.call("bf16_rms_norm", p(x), p(scale), rows, width, 1e-6, None, p(codes), 32.0, stream()))
    b = report("rms_norm+e4m3_codes", ms, bytes_moved=3.0 * rows * width, rows=rows, width=width)
    return [a, b]


def bench_attention(ops, timer, rows, heads):
    width = heads * 128
    q, k, v = (torch.randn(rows, width, device="cuda").bfloat16() for _ in range(3))
    out = torch.empty_like(q)
    ms = timer(lambda: ops.call("bf16_causal_attention", p(q), p(k), p(v), rows, rows, heads, 128, p(out), stream()))
    return report("flash_causal_attention", ms, flops=2.0 * rows * rows * width, rows=rows, heads=heads)


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("what", choices=["gemm", "hyena", "norm", "attention", "sweep", "grid", "fp8peak"])
    parser.add_argument("--rows", type=int, default=8192)
    parser.add_argument("--inner", type=int, default=4096)
    parser.add_argument("--outer", type=int, default=12288)
    parser.add_argument("--type", default="bf16", choices=["bf16", "e4m3", "emulated"])
    parser.add_argument("--length", type=int, default=8192)
    parser.add_argument("--channels", type=int, default=4096)
    parser.add_argument("--op", default="all", choices=["hcs", "hcm", "hcl", "all"])
    parser.add_argument("--fed", default="separate", choices=["separate", "projection"],
                        help="hyena: separate x2/x1/v inputs, or the interleaved projection as in the model")
    parser.add_argument("--width", type=int, default=4096)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--iters", type=int, default=10)
    args = parser.parse_args()
    ops = load_package().ops()
    timer = Timer(args.iters)
    if args.what == "gemm":
        bench_gemm(ops, timer, args.rows, args.inner, args.outer, args.type)
    elif args.what == "hyena":
        (bench_hyena_projection if args.fed == "projection" else bench_hyena)(
            ops, timer, args.length, args.channels, args.op)
    elif args.what == "norm":
        bench_norm(ops, timer, args.rows, args.width)
    elif args.what == "attention":
        bench_attention(ops, timer, args.rows, args.heads)
    elif args.what == "fp8peak":
        fp8_library_peak()
    elif args.what == "grid":
        for rows in (16, 128, 1024, 8192):
            for outer in (12288, 11264, 4096):
                for kind in ("emulated", "e4m3", "bf16"):
                    line = bench_gemm(ops, timer, rows, 4096, outer, kind)
                if rows > 128:
                    bench_codes_gemm(ops, timer, rows, 4096, outer)
    else:
        for rows in (16, 128, 1024, 8192):
            for outer in (12288, 11264, 4096):
                bench_gemm(ops, timer, rows, 4096, outer, "bf16")
                bench_gemm(ops, timer, rows, 4096, outer, "e4m3")
            if rows <= 1024:
                bench_gemm(ops, timer, rows, 4096, 12288, "emulated")
        for length in (8192, 131072):
            bench_hyena(ops, timer, length, 4096, "all")
        bench_norm(ops, timer, 8192, 4096)
        for rows in (1024, 8192):
            bench_attention(ops, timer, rows, 32)


if __name__ == "__main__":
    main()
