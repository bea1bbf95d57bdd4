"""Random-init StripedHyena2 artifacts in the evo2-runtime-v1 Safetensors format.

Test and benchmark tooling: real Evo 2 checkpoints are not available offline,
so seeded synthetic weights with the checkpoints' shapes, dtypes and value
scales stand in for them.  Official shapes come from shapes/<model_id>.json
(metadata + manifest exactly as upstream's converter writes them, see
shapes/make_shape_specs.py); `fixture_spec` builds free-form test-fixture
shapes (architecture StripedHyena2Test).

Container layout (upstream docs/model-format.md:31-49): 8-byte little-endian
header length, JSON header padded with spaces to 8 bytes, dense payload in
manifest order; shards of <= max_shard_bytes plus model.safetensors.index.json.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path
from typing import Iterable, Iterator

import numpy as np

SHAPES = Path(__file__).resolve().parent / "shapes"
DTYPE_NAMES = {"F32": "F32", "BF16": "BF16", "E4M3_SW": "F8_E4M3"}
DTYPE_BYTES = {"F32": 4, "BF16": 2, "E4M3_SW": 1}
PROFILE = "evo2-runtime-v1"


def typed(value) -> str:
    """Typed metadata string (s:/u:/f:/b:/l: prefixes, docs/model-format.md:109-127)."""
    if isinstance(value, bool):
        return f"b:{int(value)}"
    if isinstance(value, int):
        return f"u:{value}"
    if isinstance(value, float):
        return "f:" + struct.pack(">d", value).hex()
    if isinstance(value, (list, tuple)):
        return "l:" + ",".join(str(int(v)) for v in value)
    return f"s:{value}"


def load_spec(model_id: str) -> dict:
    return json.loads((SHAPES / f"{model_id}.json").read_text())


def with_fp8_projections(spec: dict, enabled: bool) -> dict:
    """Variant of an official spec with E4M3 (or BF16) Hyena projections."""
    spec = json.loads(json.dumps(spec))
    meta = spec["metadata"]
    manifest = []
    for name, dtype, shape in spec["manifest"]:
        if name.endswith("projections.fp8_runtime_scales"):
            continue
        if name.endswith("projections.weight"):
            if enabled:
                manifest.append([name.replace("projections.weight", "projections.fp8_runtime_scales"), "F32", [2]])
            manifest.append([name, "E4M3_SW" if enabled else "BF16", shape])
        else:
            manifest.append([name, dtype, shape])
    spec["manifest"] = manifest
    meta["hyena_projection_dtype"] = typed("E4M3_SW" if enabled else "BF16")
    meta["config.use_fp8_input_projections"] = typed(enabled)
    if enabled:
        meta["fp8.reference"] = typed("TransformerEngine-2.3-HYBRID")
    else:
        meta.pop("fp8.reference", None)
    return spec


def fixture_spec(*, width: int, layers: int, heads: int, inner: int, state: int = 16,
                 hcs_taps: int = 7, hcm_taps: int = 128, hcs_groups: int | None = None,
                 hcm_groups: int | None = None, fp8: bool = False, hcm_filter_f32: bool = False,
                 rope_scale: float = 1.0, vocab: int = 512) -> dict:
    """A synthetic-architecture fixture: blocks cycle HCS, HCM, HCL, attention."""
    kinds = ["hcs", "hcm", "hcl", "attn"]
    idx = {k: [i for i in range(layers) if kinds[i % 4] == k] for k in kinds}
    hcs_groups = hcs_groups or width
    hcm_groups = hcm_groups or width
    meta = {
        "runtime.abi": "evo2-safetensors-v1", "model.name": "fixture",
        "model.architecture": "StripedHyena2Test", "fixture.synthetic": True,
        "config.vocab_size": vocab, "config.hidden_size": width, "config.num_layers": layers,
        "config.num_attention_heads": heads, "config.state_size": state,
        "config.inner_mlp_size": inner, "config.short_filter_length": 3,
        "config.hcs_filter_length": hcs_taps, "config.hcm_filter_length": hcm_taps,
        "config.hcs_filter_groups": hcs_groups, "config.hcm_filter_groups": hcm_groups,
        "config.hcs_layer_idxs": idx["hcs"], "config.hcm_layer_idxs": idx["hcm"],
        "config.hcl_layer_idxs": idx["hcl"], "config.attn_layer_idxs": idx["attn"],
        "config.eps": 1e-6, "config.rotary_emb_scaling_factor": float(rope_scale),
        "config.tie_embeddings": True, "config.column_split_hyena": False,
        "config.interleave": True, "config.hyena_flip_x1x2": False,
        "config.use_fp8_input_projections": fp8,
        "hyena_projection_dtype": "E4M3_SW" if fp8 else "BF16",
        "hcm_filter_dtype": "F32" if hcm_filter_f32 else "BF16",
        "evo2.profile": PROFILE,
    }
    manifest = [["embedding_layer.weight", "BF16", [vocab, width]],
                ["unembed.weight", "BF16", [vocab, width]], ["norm.scale", "F32", [width]]]
    head_dim = width // heads
    for layer in range(layers):
        p = f"blocks.{layer}"
        manifest.append([f"{p}.pre_norm.scale", "F32", [width]])
        kind = kinds[layer % 4]
        if kind == "attn":
            manifest += [[f"{p}.inner_mha_cls.out_proj.bias", "BF16", [width]],
                         [f"{p}.inner_mha_cls.out_proj.weight", "BF16", [width, width]],
                         [f"{p}.inner_mha_cls.Wqkv.weight", "BF16", [3 * width, width]],
                         [f"{p}.inner_mha_cls.rotary_emb.inv_freq", "F32", [head_dim // 2]]]
        else:
            manifest += [[f"{p}.out_filter_dense.bias", "BF16", [width]],
                         [f"{p}.out_filter_dense.weight", "BF16", [width, width]]]
            if fp8:
                manifest.append([f"{p}.projections.fp8_runtime_scales", "F32", [2]])
            manifest.append([f"{p}.projections.weight", "E4M3_SW" if fp8 else "BF16", [3 * width, width]])
            manifest.append([f"{p}.filter.short_filter_weight", "BF16", [3 * width, 1, 3]])
            if kind == "hcs":
                manifest.append([f"{p}.filter.h", "BF16", [hcs_groups, 1, hcs_taps]])
            elif kind == "hcm":
                manifest += [[f"{p}.filter.D", "BF16", [width]],
                             [f"{p}.filter.h", "F32" if hcm_filter_f32 else "BF16", [hcm_groups, 1, hcm_taps]]]
            else:
                manifest += [[f"{p}.filter.D", "BF16", [width]],
                             [f"{p}.filter.log_poles", "F32", [width, state, 1]],
                             [f"{p}.filter.residues", "F32", [width, state]]]
        manifest += [[f"{p}.mlp.l1.weight", "BF16", [inner, width]],
                     [f"{p}.mlp.l2.weight", "BF16", [inner, width]],
                     [f"{p}.mlp.l3.weight", "BF16", [width, inner]],
                     [f"{p}.post_norm.scale", "F32", [width]]]
    return {"model_id": "", "metadata": {k: typed(v) for k, v in meta.items()}, "manifest": manifest}


def _bf16_bytes(values: np.ndarray) -> bytes:
    bits = np.ascontiguousarray(values, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16).tobytes()


def _e4m3_codes(scaled: np.ndarray) -> np.ndarray:
    import torch

    t = torch.from_numpy(np.ascontiguousarray(scaled, dtype=np.float32)).clamp(-448.0, 448.0)
    return t.to(torch.float8_e4m3fn).view(torch.uint8).numpy()


def synthetic_tensors(spec: dict, seed: int, *, weight_std: float = 0.02,
                      filter_std: float | None = None, input_scale: float = 32.0,
                      rope_base: float = 10000.0, device: str | None = None
                      ) -> Iterator[tuple[str, str, list[int], bytes]]:
    """Yields (name, dtype, shape, payload) in manifest order.

    BF16 weights ~ N(0, weight_std); filters ~ N(0, filter_std or weight_std);
    norm scales 1; inv_freq = base^(-2i/d); log_poles = ln U[0.9, 0.999);
    residues ~ N(0, filter_std or weight_std) (F32).  E4M3 projections: per-tensor
    scale 448/amax(bf16 w), codes of clamp(w*s, +-448), runtime scales
    [input_scale, (1/input_scale)*(1/s_w)] (upstream tools/evo/checkpoint.py:73-112).
    With device="cuda" large tensors are drawn by torch on the GPU (faster; a
    different but equally seeded stream).
    """
    filter_std = weight_std if filter_std is None else filter_std
    rng = np.random.default_rng(seed)
    torch_gen = None
    if device is not None:
        import torch

        torch_gen = torch.Generator(device=device)
        torch_gen.manual_seed(seed)

    def normal(shape, std):
        count = math.prod(shape)
        if torch_gen is not None and count >= 1 << 16:
            import torch

            return (torch.randn(count, generator=torch_gen, device=device) * std).cpu().numpy().reshape(shape)
        return (rng.standard_normal(shape) * std).astype(np.float32)

    pending_scale: list | None = None
    for name, dtype, shape in spec["manifest"]:
        if name.endswith("fp8_runtime_scales"):
            pending_scale = [name, shape]
            continue
        if name.endswith(".scale"):
            payload = np.ones(shape, np.float32).tobytes()
        elif name.endswith("inv_freq"):
            half = shape[0]
            payload = (rope_base ** (-np.arange(half, dtype=np.float64) * 2.0 / (2 * half))).astype(np.float32).tobytes()
        elif name.endswith("log_poles"):
            payload = np.log(rng.uniform(0.9, 0.999, shape)).astype(np.float32).tobytes()
        elif name.endswith("residues"):
            payload = normal(shape, filter_std).astype(np.float32).tobytes()
        elif ".filter." in name:
            values = normal(shape, filter_std)
            payload = values.astype(np.float32).tobytes() if dtype == "F32" else _bf16_bytes(values)
        elif torch_gen is not None and dtype in ("E4M3_SW", "BF16") and math.prod(shape) >= 1 << 16:
            # large dense weights: draw, round and (for E4M3) quantise on the device
            import torch

            values = (torch.randn(math.prod(shape), generator=torch_gen, device=device) * weight_std).bfloat16()
            if dtype == "BF16":
                payload = values.view(torch.int16).cpu().numpy().tobytes()
            else:
                rounded = values.float()
                w_scale = np.float32(448.0) / np.float32(rounded.abs().max().item())
                codes = (rounded * float(w_scale)).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
                if pending_scale is not None:
                    scales = np.array([input_scale, np.float32(np.float32(1.0) / np.float32(input_scale)) *
                                       np.float32(np.float32(1.0) / w_scale)], np.float32)
                    yield pending_scale[0], "F32", pending_scale[1], scales.tobytes()
                    pending_scale = None
                payload = codes.view(torch.uint8).cpu().numpy().tobytes()
        elif dtype == "E4M3_SW":
            values = normal(shape, weight_std)
            rounded = (np.frombuffer(_bf16_bytes(values), np.uint16).astype(np.uint32) << 16).view(np.float32)
            w_scale = np.float32(448.0) / np.float32(np.abs(rounded).max())
            codes = _e4m3_codes(rounded * w_scale)
            if pending_scale is not None:
                scales = np.array([input_scale, np.float32(np.float32(1.0) / np.float32(input_scale)) *
                                   np.float32(np.float32(1.0) / w_scale)], np.float32)
                yield pending_scale[0], "F32", pending_scale[1], scales.tobytes()
                pending_scale = None
            payload = codes.tobytes()
        elif dtype == "BF16":
            payload = _bf16_bytes(normal(shape, weight_std))
        else:
            payload = normal(shape, weight_std).astype(np.float32).tobytes()
        yield name, dtype, shape, payload


def write_model(path: Path, metadata: dict[str, str], tensors: Iterable[tuple[str, str, list[int], bytes]],
                *, max_shard_bytes: int = 4 << 30) -> list[Path]:
    """Writes `path` (a .safetensors file) or, when the payload exceeds
    max_shard_bytes, standard shard files plus model.safetensors.index.json in
    path's directory.  Returns the files written."""
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)

    def write_one(target: Path, items) -> None:
        header = {"__metadata__": dict(sorted(metadata.items()))}
        offset = 0
        for name, dtype, shape, payload in items:
            header[name] = {"dtype": DTYPE_NAMES[dtype], "shape": list(shape),
                            "data_offsets": [offset, offset + len(payload)]}
            offset += len(payload)
        text = json.dumps(header, separators=(",", ":")).encode()
        text += b" " * (-len(text) % 8)
        with open(target, "wb") as out:
            out.write(struct.pack("<Q", len(text)))
            out.write(text)
            for _, _, _, payload in items:
                out.write(payload)

    # Shards are flushed as they fill so that only one is held in memory.
    parts: list[tuple[Path, list[str], int]] = []
    current: list = []
    size = 0

    def flush() -> None:
        nonlocal current, size
        if not current:
            return
        target = path.parent / f".shard-{len(parts)}.tmp"
        write_one(target, current)
        parts.append((target, [item[0] for item in current], size))
        current, size = [], 0

    for item in tensors:
        nbytes = len(item[3])
        assert nbytes == math.prod(item[2]) * DTYPE_BYTES[item[1]], item[0]
        if current and size + nbytes > max_shard_bytes:
            flush()
        current.append(item)
        size += nbytes
    flush()
    if len(parts) == 1:
        parts[0][0].replace(path)
        return [path]
    written, weight_map, total = [], {}, 0
    for index, (temporary, names, nbytes) in enumerate(parts, 1):
        name = f"model-{index:05d}-of-{len(parts):05d}.safetensors"
        temporary.replace(path.parent / name)
        written.append(path.parent / name)
        for tensor_name in names:
            weight_map[tensor_name] = name
        total += nbytes
    index_path = path.parent / "model.safetensors.index.json"
    index_path.write_text(json.dumps({"metadata": {"total_size": total}, "weight_map": weight_map}))
    written.append(index_path)
    return written


def write_synthetic(path: Path, spec: dict, seed: int, **kwargs) -> list[Path]:
    shard = kwargs.pop("max_shard_bytes", 4 << 30)
    return write_model(path, spec["metadata"], synthetic_tensors(spec, seed, **kwargs), max_shard_bytes=shard)
