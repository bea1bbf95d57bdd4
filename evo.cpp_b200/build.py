"""In-tree build of the sm_100a libraries (nvcc cross-compiles without a GPU).

    python evo.cpp_b200/build.py            # build what is out of date
    python evo.cpp_b200/build.py --force

Outputs, next to this file:
    libevo_b200_ops.so   operator-level C ABI (include/evo_b200_ops.h)
    libevo.so            model-level C ABI (include/evo/evo.h), when its
                         sources are present
"""
from __future__ import annotations

import concurrent.futures
import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = HERE / "build"
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3",
    "-std=c++17", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--threads", "2",
]

KERNEL_SOURCES = [
    "errors.cu", "elementwise.cu", "qgmma_emulation.cu", "gemm_tcgen05.cu", "gemv.cu",
    "hyena_fir.cu", "hyena_fir_fused.cu", "hyena_fir_tcgen05.cu", "hyena_modal.cu", "hyena_decode.cu", "attention.cu", "attention_flash.cu", "attention_tcgen05.cu", "attention_tcgen05_k64.cu", "attention_decode.cu", "kv_q8.cu", "linear_executor.cu", "fp8_codec.cpp",
]
OPS_SOURCES = KERNEL_SOURCES + ["ops_api.cu"]
RUNTIME_SOURCES = KERNEL_SOURCES + [
    "runtime/safetensors.cpp", "runtime/model_load.cpp", "runtime/model_weights.cpp",
    "runtime/model.cu", "runtime/sampler.cpp", "runtime/variant.cpp", "runtime/variant_io.cpp", "runtime/scheduler.cpp", "runtime/c_api.cpp",
]


def _newest_header() -> float:
    headers = list(CSRC.rglob("*.hpp")) + list(CSRC.rglob("*.cuh")) + list(
        (HERE.parent / "include").rglob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(source: str, force: bool, header_time: float) -> Path:
    src = CSRC / source
    obj = OBJ / (source.replace("/", "_") + ".o")
    if (not force and obj.exists() and obj.stat().st_mtime > src.stat().st_mtime
            and obj.stat().st_mtime > header_time):
        return obj
    cmd = [NVCC, *FLAGS, "-I", str(CSRC), "-I", str(HERE.parent / "include"),
           "-x", "cu", "-c", str(src), "-o", str(obj)]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source}:\n{result.stdout}\n{result.stderr}")
    return obj


def _link(objects: list[Path], output: Path, extra: list[str]) -> None:
    cmd = [NVCC, "-shared", "-o", str(output), *[str(o) for o in objects],
           "-Xlinker", "--no-undefined", "-lcudart", *extra]
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed for {output.name}:\n{result.stdout}\n{result.stderr}")


def build(force: bool = False) -> dict[str, Path]:
    OBJ.mkdir(exist_ok=True)
    header_time = _newest_header()
    sources = list(OPS_SOURCES)
    have_runtime = all((CSRC / s).exists() for s in RUNTIME_SOURCES)
    if have_runtime:
        sources += [s for s in RUNTIME_SOURCES if s not in sources]
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objects = dict(zip(sources, pool.map(
            lambda s: _compile(s, force, header_time), sources)))
    outputs = {}
    ops_lib = HERE / "libevo_b200_ops.so"
    ops_objects = [objects[s] for s in OPS_SOURCES]
    if force or not ops_lib.exists() or any(
            o.stat().st_mtime > ops_lib.stat().st_mtime for o in ops_objects):
        _link(ops_objects, ops_lib, [])
    outputs["ops"] = ops_lib
    if have_runtime:
        lib = HERE / "libevo.so"
        rt_objects = [objects[s] for s in RUNTIME_SOURCES]
        if force or not lib.exists() or any(
                o.stat().st_mtime > lib.stat().st_mtime for o in rt_objects):
            _link(rt_objects, lib, [
                "-lz", "-Xlinker", f"--version-script={CSRC / 'runtime' / 'evo.map'}",
                "-Xlinker", "-soname=libevo.so.1"])
        outputs["evo"] = lib
        soname = HERE / "libevo.so.1"
        if not soname.exists():
            soname.symlink_to("libevo.so")
        # command-line driver: links only against the public C ABI of libevo.so
        cli_source = CSRC / "runtime" / "cli_main.cpp"
        cli = HERE / "evo"
        if cli_source.exists() and (force or not cli.exists()
                                    or cli.stat().st_mtime < max(cli_source.stat().st_mtime,
                                                                 lib.stat().st_mtime)):
            cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++17", "-o", str(cli), str(cli_source),
                   f"-L{HERE}", "-l:libevo.so", "-Wl,-rpath,$ORIGIN"]
            result = subprocess.run(cmd, capture_output=True, text=True)
            if result.returncode != 0:
                raise RuntimeError(f"CLI build failed:\n{result.stdout}\n{result.stderr}")
        outputs["cli"] = cli
    return outputs


if __name__ == "__main__":
    built = build(force="--force" in sys.argv)
    for name, path in built.items():
        print(f"{name}: {path}")
