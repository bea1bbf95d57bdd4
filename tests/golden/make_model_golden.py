#!/usr/bin/env python3
"""Golden fixture of a whole 1B-shaped model from upstream's own CPU library.

    python tests/golden/make_model_golden.py <scratch dir> [--workers N]

Writes tests/golden/model_1b_1024.npz.  The artifact is the 1B-shaped
StripedHyena2 stack (25 blocks, width 1920, 15 heads, inner 5120; shapes from
evo.cpp_b200/shapes/evo2_1b_base.json) with BF16 projections and seeded
random-init weights (seed 0, host RNG, so any machine re-creates the same
bytes); the prompt is 1,024 tokens drawn uniformly from A/C/G/T with
numpy default_rng(1000).  Upstream's CPU backend (oracle/_ref/libevo_ref.so,
built by `make -C oracle ref` from the upstream sources) is driven through its
stock C ABI: evo_context_prefill for the logits and evo_context_embed(layer)
for every block output.  One forward takes minutes on one core, so the 26
passes are spread over worker processes.

Stored (float16 holds these values to ~5e-4 relative, far inside the
tolerances the tests use):
  tokens            uint8 [1024]
  logits            float16 [1024, 512]
  block_rows        int32 [R]   the sampled sequence positions
  block_<i>         float16 [R, 1920]  block i output at those positions
  block_stats       float64 [25, 3]    rms, mean |x|, max |x| of the full
                                       [1024, 1920] block output
Only this script needs the upstream library; tests read the .npz.
"""
from __future__ import annotations

import argparse
import importlib.util
import multiprocessing
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
MODEL_ID, SEED, TOKENS, TOKEN_SEED = "evo2_1b_base", 0, 1024, 1000
BLOCK_ROWS = [0, 1, 2, 6, 7, 63, 127, 128, 129, 255, 511, 512, 767, 1000, 1022, 1023]


def _package():
    pkg_dir = ROOT / "evo.cpp_b200"
    if "evo_cpp_b200" not in sys.modules:
        spec = importlib.util.spec_from_file_location(
            "evo_cpp_b200", pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
        module = importlib.util.module_from_spec(spec)
        sys.modules["evo_cpp_b200"] = module
        spec.loader.exec_module(module)
    return sys.modules["evo_cpp_b200"]


def prompt() -> bytes:
    rng = np.random.default_rng(TOKEN_SEED)
    return bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), TOKENS).tolist())


def write_artifact(directory: Path, fp8: bool = False) -> Path:
    """The seeded 1B-shaped artifact (BF16 projections unless fp8)."""
    _package()
    art = importlib.import_module("evo_cpp_b200.artifact")
    path = directory / ("model_fp8.safetensors" if fp8 else "model.safetensors")
    if not path.exists():
        spec = art.with_fp8_projections(art.load_spec(MODEL_ID), fp8)
        art.write_synthetic(path, spec, seed=SEED)
    return path


def _task(args):
    model_path, layer = args
    _package()
    rt = importlib.import_module("evo_cpp_b200.runtime")
    lib = rt.EvoLibrary(ROOT / "oracle" / "_ref" / "libevo_ref.so")
    model = lib.load(model_path, backend=rt.BACKEND_CPU)
    context = model.context(TOKENS)
    start = time.time()
    if layer < 0:
        values = context.prefill(prompt())
    else:
        values = context.embed(prompt(), layer)
    print(f"layer {layer}: {time.time() - start:.0f} s", flush=True)
    if layer < 0:
        return layer, values.astype(np.float16), None
    full = values.astype(np.float64)
    stats = np.array([np.sqrt((full ** 2).mean()), np.abs(full).mean(), np.abs(full).max()])
    return layer, values[BLOCK_ROWS].astype(np.float16), stats


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("scratch", type=Path)
    parser.add_argument("--workers", type=int, default=6)
    args = parser.parse_args()
    args.scratch.mkdir(parents=True, exist_ok=True)
    model_path = write_artifact(args.scratch)
    _package()
    rt = importlib.import_module("evo_cpp_b200.runtime")
    layers = 25
    tasks = [(str(model_path), layer) for layer in range(-1, layers)]
    out = {"tokens": np.frombuffer(prompt(), np.uint8), "block_rows": np.array(BLOCK_ROWS, np.int32)}
    stats = np.zeros((layers, 3))
    with multiprocessing.get_context("spawn").Pool(args.workers) as pool:
        for layer, values, layer_stats in pool.imap_unordered(_task, tasks):
            if layer < 0:
                out["logits"] = values
            else:
                out[f"block_{layer}"] = values
                stats[layer] = layer_stats
    out["block_stats"] = stats
    np.savez_compressed(HERE / "model_1b_1024.npz", **out)
    print("written", HERE / "model_1b_1024.npz")


if __name__ == "__main__":
    main()
