"""Upstream evo.cpp's own CUDA operator tests as acceptance tests of the drop-in boundary.

`oracle/Makefile` (target `operator_tests`) compiles upstream's tests/test_cuda_ops.cu,
tests/test_cuda_hyena.cu and tests/test_cuda_attention.cu unmodified, from the upstream source tree,
against upstream's headers, and links them with the `evo::cuda` source-compatibility layer
(`evo.cpp_b200/compat/`) over this build's operator library.  Each binary prints one `FAIL: <what>`
line per failed check and exits non-zero if there was any.

Every check must pass except the one listed in KNOWN: a known answer that hashes the bits of a cuBLAS
GEMM's summation order on the reference stack, for a product this build sums in another order (within
the tolerance its own parity tests state).
"""
import pathlib
import subprocess

import pytest

pytestmark = pytest.mark.gpu

BINARIES = pathlib.Path(__file__).resolve().parent.parent / "oracle" / "_ref"

KNOWN = {
    "ops": set(),
    "hyena": set(),
    "attention": {
        # upstream tests/test_cuda_attention.cu:341-393: FNV-1a hashes of raw BF16 bytes from PyTorch on the
        # reference stack, five context lengths.  The five probability tensors match bit for bit and so do
        # four of the five outputs; at 10,240 keys the F32 sum of probabilities x values rounds differently
        # in one of its 16 BF16 results than the library GEMM behind the reference bytes.
        "cached cross-attention output is bit exact to PyTorch",
    },
}


def run(name, *arguments):
    binary = BINARIES / f"upstream_test_cuda_{name}"
    if not binary.exists():
        pytest.skip(f"{binary.name} was not built (the upstream source tree was absent at build time)")
    done = subprocess.run([str(binary), *arguments], capture_output=True, text=True, timeout=600)
    failed = [line[len("FAIL: "):].strip() for line in done.stderr.splitlines() if line.startswith("FAIL: ")]
    return done, failed


@pytest.mark.parametrize("name", ["ops", "hyena", "attention"])
def test_upstream_operator_tests_pass_against_the_compatibility_layer(name):
    done, failed = run(name)
    unexpected = sorted(set(failed) - KNOWN[name])
    assert not unexpected, f"unexpected failures: {unexpected}\nstdout: {done.stdout[-2000:]}\nstderr: {done.stderr[-4000:]}"
    if not failed:
        assert done.returncode == 0, done.stderr[-2000:]
        assert "tests passed" in done.stdout
    else:
        # only the documented known-answer check failed, once; the binary still ran to its end
        assert "test(s) failed" in done.stderr, done.stderr[-2000:]
        assert len(failed) == 1, failed


def test_upstream_c_api_test_passes_against_libevo():
    """Upstream's tests/test_cuda_c_api.c, compiled as C against upstream's include/evo/evo.h and linked with
    this build's libevo.so, on the strict tiny fixture its own driver generates (tools/generate_tiny_model.py;
    the committed copy under tests/golden/tiny): shared-weight contexts, the exact and fast-q8-kv profiles,
    embeddings of an inner layer, byte-deterministic prefill and decode, callback abort poisoning."""
    model = pathlib.Path(__file__).resolve().parent / "golden" / "tiny" / "tiny.safetensors"
    done, failed = run("c_api", str(model))
    assert not failed, f"{failed}\n{done.stderr[-2000:]}"
    assert done.returncode == 0 and "CUDA C API tests passed" in done.stdout, done.stderr[-2000:]
