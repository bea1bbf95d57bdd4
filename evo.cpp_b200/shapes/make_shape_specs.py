#!/usr/bin/env python3
"""Writes evo.cpp_b200/shapes/<model_id>.json from the upstream tree.

Each file records, for one official Evo 2 shape, the typed Safetensors metadata
and the ordered tensor manifest (name, dtype, shape) that upstream's own
converter tooling (tools/evo/model_config.py: load_config, container_manifest,
config_metadata; tools/evo/format.py: encode_metadata) would write, so that
artifact.py can produce random-init artifacts that upstream's loader accepts.
Needs the upstream tree (its path is the first argument); the JSON files it writes are
committed and are all that is needed afterwards.
"""
import json
import os
import sys
from pathlib import Path

if len(sys.argv) < 2 and "EVO_UPSTREAM_ROOT" not in os.environ:
    sys.exit("usage: pass the upstream source tree as the first argument (or set EVO_UPSTREAM_ROOT)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["EVO_UPSTREAM_ROOT"])
sys.path.insert(0, str(REF / "tools"))
from evo import format as fmt  # noqa: E402
from evo import model_config as mc  # noqa: E402

HERE = Path(__file__).resolve().parent
CONFIGS = ["evo2-1b-8k", "evo2-7b-1m", "evo2-7b-8k", "evo2-40b-1m", "evo2-40b-8k"]

for name in CONFIGS:
    cfg = mc.load_config(REF / "configs" / f"{name}.yml")
    meta = mc.config_metadata(cfg, "synthetic-random-init", 0)
    meta["hcm_filter_dtype"] = "BF16"
    if cfg.use_fp8_input_projections:
        meta["fp8.reference"] = "TransformerEngine-2.3-HYBRID"
    encoded = fmt.encode_metadata(meta, artifact_profile=fmt.EVO2_PROFILE_VALUE)
    manifest = [[s.name, s.dtype, list(s.shape)] for s in mc.container_manifest(cfg)]
    out = {"model_id": cfg.model_id, "metadata": encoded, "manifest": manifest}
    (HERE / f"{cfg.model_id}.json").write_text(json.dumps(out, indent=0, sort_keys=True) + "\n")
    print(cfg.model_id, len(manifest), "tensors")
