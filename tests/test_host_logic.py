"""Host-side logic that needs no GPU: the model-level ABI's symbol table, the
pipeline stage planner, the Safetensors reader's refusals, the sampler, and
the multi-rank aggregation used by the benchmark (gloo, world size 2)."""
from __future__ import annotations

import ctypes
import importlib
import json
import re
import struct
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parent.parent

# The 39 symbols of upstream's stable C ABI (tests/test_c_api_symbols.py:12-52 there).
UPSTREAM_SYMBOLS = """evo_abi_version evo_version_string evo_status_name evo_backend_name evo_last_error
evo_model_default_params evo_context_default_params evo_sampler_default_params
evo_embedding_default_options evo_model_load evo_model_free evo_model_backend evo_model_id
evo_model_architecture evo_model_profile evo_model_vocab_size evo_model_max_context
evo_model_embedding_width evo_model_layer_count evo_model_encode evo_model_decode_token
evo_context_create evo_context_free evo_context_position evo_context_capacity evo_context_profile
evo_context_prefill evo_context_decode evo_context_embed evo_context_embed_ex evo_batch_create
evo_batch_free evo_batch_clear evo_batch_add_sequence evo_batch_sequence_count
evo_batch_token_count evo_sampler_create evo_sampler_free evo_sampler_sample""".split()


@pytest.fixture(scope="module")
def rt(pkg):
    return importlib.import_module("evo_cpp_b200.runtime")


@pytest.fixture(scope="module")
def evo(rt, pkg):
    return rt.EvoLibrary(pkg.EVO_LIBRARY)


def test_libevo_exports_upstream_abi_and_declared_extensions(pkg):
    assert len(UPSTREAM_SYMBOLS) == 39
    out = subprocess.run(["nm", "-D", "--defined-only", str(pkg.EVO_LIBRARY)], check=True,
                         capture_output=True, text=True).stdout
    exported = {line.split()[-1].split("@")[0] for line in out.splitlines() if line.strip()}
    header = (ROOT / "include" / "evo" / "evo.h").read_text()
    declared = set(re.findall(r"\b(evo_\w+)\s*\(", re.sub(r"/\*.*?\*/", "", header, flags=re.S)))
    declared -= {"evo_logits_callback", "evo_embedding_callback", "evo_embedding_ex_callback",
                 "evo_status"}  # callback typedefs: `typedef evo_status (*name)(...)`
    assert declared == set(UPSTREAM_SYMBOLS)
    extensions = set(re.findall(r"\b(evo_b200_\w+)\s*\(", re.sub(
        r"/\*.*?\*/", "", (ROOT / "include" / "evo" / "evo_b200.h").read_text(), flags=re.S)))
    assert exported == set(UPSTREAM_SYMBOLS) | extensions, exported ^ (set(UPSTREAM_SYMBOLS) | extensions)
    lib = ctypes.CDLL(str(pkg.EVO_LIBRARY))
    lib.evo_abi_version.restype = ctypes.c_uint32
    assert lib.evo_abi_version() == (1 << 24) | (5 << 16)
    lib.evo_status_name.restype = ctypes.c_char_p
    assert [lib.evo_status_name(c) for c in (0, 2, 3, 4, 5, 6, 7, 70)] == [
        b"ok", b"invalid_argument", b"io", b"model_format", b"unsupported", b"cuda", b"mps", b"internal"]


def plan(evo, layer_bytes, stages, even):
    n = len(layer_bytes)
    sizes = (ctypes.c_size_t * n)(*layer_bytes)
    begins, ends = (ctypes.c_size_t * stages)(), (ctypes.c_size_t * stages)()
    fn = evo.lib.evo_b200_plan_stages
    fn.argtypes = [ctypes.c_void_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p]
    status = fn(sizes, n, stages, int(even), begins, ends)
    return status, list(zip(begins, ends))


def test_stage_planner(evo):
    # fixtures: equal counts, remainder to the first stages (upstream
    # tests/test_cuda_pipeline.cu:178-209: 50 layers -> 25/25 and 13/13/12/12)
    assert plan(evo, [1] * 50, 2, True) == (0, [(0, 25), (25, 50)])
    assert plan(evo, [1] * 50, 4, True) == (0, [(0, 13), (13, 26), (26, 38), (38, 50)])
    # byte-balanced greedy split: contiguous, at least one layer each, covers everything
    rng = np.random.default_rng(0)
    for stages in range(1, 9):
        sizes = rng.integers(1, 100, 32).tolist()
        status, stage_list = plan(evo, sizes, stages, False)
        assert status == 0 and stage_list[0][0] == 0 and stage_list[-1][1] == 32
        assert all(b < e for b, e in stage_list)
        assert all(stage_list[i][1] == stage_list[i + 1][0] for i in range(stages - 1))
        loads = [sum(sizes[b:e]) for b, e in stage_list]
        assert max(loads) <= sum(sizes) / stages + 2 * max(sizes)
    # uniform 7B-like blocks over 4 stages: 8 each
    assert plan(evo, [10] * 32, 4, False)[1] == [(0, 8), (8, 16), (16, 24), (24, 32)]
    assert plan(evo, [1, 1], 3, False)[0] == 2 and plan(evo, [1] * 9, 9, False)[0] == 2


def test_model_reader_refusals(evo, rt, tmp_path):
    """Bad containers are refused before any device work (status codes as upstream)."""
    with pytest.raises(rt.EvoError) as err:
        evo.load(tmp_path / "missing.safetensors")
    assert err.value.code == 3
    truncated = tmp_path / "short.safetensors"
    truncated.write_bytes(b"\x10")
    with pytest.raises(rt.EvoError) as err:
        evo.load(truncated)
    assert err.value.code == 4
    header = json.dumps({"__metadata__": {"evo2.profile": "s:evo2-runtime-v1"},
                         "t": {"dtype": "F16", "shape": [2], "data_offsets": [0, 4]}}).encode()
    header += b" " * (-len(header) % 8)
    bad_dtype = tmp_path / "dtype.safetensors"
    bad_dtype.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 4)
    with pytest.raises(rt.EvoError) as err:
        evo.load(bad_dtype)
    assert err.value.code == 4 and "dtype" in str(err.value)
    header = json.dumps({"t": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}).encode()
    header += b" " * (-len(header) % 8)
    trailing = tmp_path / "trailing.safetensors"
    trailing.write_bytes(struct.pack("<Q", len(header)) + header + b"\0" * 12)
    with pytest.raises(rt.EvoError) as err:
        evo.load(trailing)
    assert err.value.code == 4
    with pytest.raises(rt.EvoError) as err:   # the CPU backend is not part of this library
        evo.load(ROOT / "tests" / "golden" / "tiny" / "tiny.safetensors", backend=rt.BACKEND_CPU)
    assert err.value.code == 5


def mt19937_64_first_output(seed: int) -> int:
    """First output of the 64-bit Mersenne Twister (the generator the C++
    standard fixes as std::mt19937_64), from its published recurrence."""
    mask = (1 << 64) - 1
    state = [seed & mask]
    for i in range(1, 312):
        state.append((6364136223846793005 * (state[-1] ^ (state[-1] >> 62)) + i) & mask)
    for i in range(312):
        x = (state[i] & 0xFFFFFFFF80000000) | (state[(i + 1) % 312] & 0x7FFFFFFF)
        state[i] = state[(i + 156) % 312] ^ (x >> 1) ^ (0xB5026F5AA96619E9 if x & 1 else 0)
    y = state[0]
    y ^= (y >> 29) & 0x5555555555555555
    y ^= (y << 17) & 0x71D67FFFEDA60000
    y ^= (y << 37) & 0xFFF7EEE000000000
    y ^= y >> 43
    return y & mask


def test_model_configuration_is_read_without_a_device(evo, rt):
    """evo_b200_read_model_config on upstream's 50-block tiny fixture: the fields upstream's own model test checks
    (tests/test_cuda_model.cu:175-191) and the refusal of a synthetic fixture without permission."""
    path = ROOT / "tests" / "golden" / "tiny" / "tiny.safetensors"
    with pytest.raises(rt.EvoError):
        evo.read_model_config(path, allow_test_fixture=False)
    config, mixers = evo.read_model_config(path, allow_test_fixture=True)
    assert (config.layers, config.vocab_size, config.width) == (50, 512, 8)
    assert config.architecture == b"StripedHyena2Test" and config.test_fixture == 1
    assert len(mixers) == 50 and mixers.count(3) == 8 and set(mixers) == {0, 1, 2, 3}
    assert config.hyena_projection_e4m3 == 0 and config.hcm_filter_f32 == 1
    assert (config.heads, config.hcm_filter_length, config.short_filter_length) == (2, 4, 3)


def test_model_configuration_reader_refuses_what_the_loader_refuses(evo, rt, pkg, tmp_path):
    """The three refusals of upstream's configuration reader that its model test pins
    (tests/test_cuda_model.cu:195-208), from evo_b200_read_model_config: no device is involved."""
    import importlib

    art = importlib.import_module("evo_cpp_b200.artifact")
    base = dict(width=64, layers=4, heads=1, inner=128, hcs_groups=8, hcm_groups=8)

    def write(name, mutate, extra=None):
        spec = art.fixture_spec(**base)
        mutate(spec)
        tensors = list(art.synthetic_tensors(spec, seed=1))
        if extra is not None:
            tensors.append(extra)
        path = tmp_path / f"{name}.safetensors"
        art.write_model(path, spec["metadata"], tensors)
        return path

    good = write("good", lambda s: None)
    config, mixers = evo.read_model_config(good, allow_test_fixture=True)
    assert (config.layers, config.width, config.inner_width) == (4, 64, 128) and len(mixers) == 4
    for path, code, fragment in (
            (write("disagrees", lambda s: s["metadata"].update({"hyena_projection_dtype": art.typed("E4M3_SW")})), 4,
             "disagrees"),
            (write("dtype", lambda s: s["metadata"].update({"hyena_projection_dtype": art.typed("INT8")})), 5,
             "unsupported Hyena projection dtype: INT8"),
            (write("extra", lambda s: None, ("blocks.0.surplus", "F32", [4], bytes(16))), 4,
             "unknown tensor for model profile")):
        with pytest.raises(rt.EvoError) as refused:
            evo.read_model_config(path, allow_test_fixture=True)
        assert refused.value.code == code and fragment in str(refused.value), str(refused.value)


def test_cli_refuses_bad_diagnostic_flags_before_any_device_work():
    """Option errors of the generation / scoring diagnostics (upstream src/cli.cpp:654-667, 737-762, 1049-1051):
    exit code 2 and upstream's wording, decided while parsing."""
    import subprocess

    binary = ROOT / "evo.cpp_b200" / "evo"

    def refused(*arguments):
        done = subprocess.run([str(binary), *arguments], capture_output=True, timeout=60)
        assert done.returncode == 2, (arguments, done.returncode, done.stderr)
        return done.stderr.decode()

    for bad in ("0", "-3", "1048577", "ten", ""):
        assert "--force-prompt-threshold must be an integer in [1, 1048576]" in refused(
            "run", "-m", "x", "-p", "AC", "--force-prompt-threshold", bad)
    assert "only valid for generation" in refused("score", "-m", "x", "--input", "y", "--force-prompt-threshold", "3")
    for bad in ("17", ":path", "17:", "x:path", "-1:path"):
        assert "--dump-layer must be a nonnegative INDEX:PATH" in refused("run", "-m", "x", "-p", "AC", "--dump-layer", bad)
    assert "--dump-logits path must not be empty" in refused("run", "-m", "x", "-p", "AC", "--dump-logits", "")
    assert "generation and scoring only" in refused("bench", "-m", "x", "--input", "y", "--dump-logits", "z.npy")


def test_sampler_matches_upstream_rule(evo, rt):
    assert mt19937_64_first_output(5489) == 14514284786278117030  # the standard's check value seed
    logits = np.array([0.5, 2.0, 2.0, -1.0, 1.5], np.float32)
    assert rt.Sampler(evo).sample(logits) == 1                     # argmax, lowest index on ties
    for seed in (0, 7):
        sampler = rt.Sampler(evo, temperature=0.7, top_k=0, top_p=0.9, seed=seed)
        order = sorted(range(5), key=lambda i: (-logits[i], i))
        weights = [float(np.exp(np.float64(logits[i]) / np.float64(np.float32(0.7)) -
                                np.float64(logits[order[0]]) / np.float64(np.float32(0.7)))) for i in order]
        total, cumulative, keep = sum(weights), 0.0, 0
        while keep < len(weights) and cumulative / total < float(np.float32(0.9)):
            cumulative += weights[keep]
            keep += 1
        first = mt19937_64_first_output(seed)
        draw = (first >> 11) * 2.0 ** -53 * cumulative
        running, expected = 0.0, order[keep - 1]
        for i in range(keep):
            running += weights[i]
            if draw < running:
                expected = order[i]
                break
        assert sampler.sample(logits) == expected
    with pytest.raises(rt.EvoError):
        rt.Sampler(evo, temperature=0.0)
    with pytest.raises(rt.EvoError):
        rt.Sampler(evo, top_k=9).sample(logits)


WORKER = """
import sys, importlib.util
sys.path.insert(0, {root!r})
spec = importlib.util.spec_from_file_location("bench", {root!r} + "/bench.py")
bench = importlib.util.module_from_spec(spec); spec.loader.exec_module(bench)
import torch.distributed as dist
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank={rank}, world_size=2)
slowest = bench.max_over_ranks([10.0, 14.0][{rank}], "cpu", True)
value = bench.aggregate_throughput(2, 8192, slowest * 1e-3)
assert slowest == 14.0, slowest
print(value)
dist.destroy_process_group()
"""


def test_two_rank_aggregation_over_gloo():
    """Replica ranks report the slowest rank's time; throughput is the sum of
    what all ranks processed in that time."""
    port = 29500 + (hash(str(ROOT)) % 400)
    procs = [subprocess.Popen([sys.executable, "-c", WORKER.format(root=str(ROOT), port=port, rank=rank)],
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for rank in range(2)]
    outputs = [p.communicate(timeout=180) for p in procs]
    assert all(p.returncode == 0 for p in procs), outputs
    for out, _ in outputs:
        assert abs(float(out.strip().splitlines()[-1]) - 2 * 8192 / 0.014) < 1e-6


def _variant_window(evo, sequence, position, ref, alt, maximum):
    class Window(ctypes.Structure):
        _fields_ = [(name, ctypes.c_size_t) for name in (
            "struct_size", "reference_start", "reference_end", "variant_offset", "reference_length",
            "alternate_length")]
    fn = evo.lib.evo_b200_variant_window_make
    fn.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_char_p, ctypes.c_size_t,
                   ctypes.c_char_p, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_void_p, ctypes.c_char_p,
                   ctypes.c_char_p, ctypes.c_size_t]
    window = Window(struct_size=ctypes.sizeof(Window))
    capacity = max(maximum, 1)
    reference, alternate = ctypes.create_string_buffer(capacity), ctypes.create_string_buffer(capacity)
    status = fn(sequence, len(sequence), position, ref, len(ref), alt, len(alt), maximum,
                ctypes.byref(window), reference, alternate, capacity)
    if status != 0:
        evo.lib.evo_last_error.restype = ctypes.c_char_p
        return status, evo.lib.evo_last_error().decode()
    return 0, (reference.raw[:window.reference_length], alternate.raw[:window.alternate_length],
               window.reference_start, window.reference_end, window.variant_offset)


def _reverse_complement(evo, sequence):
    fn = evo.lib.evo_b200_reverse_complement
    fn.argtypes = [ctypes.c_char_p, ctypes.c_size_t, ctypes.c_char_p]
    out = ctypes.create_string_buffer(max(len(sequence), 1))
    status = fn(sequence, len(sequence), out)
    if status != 0:
        evo.lib.evo_last_error.restype = ctypes.c_char_p
        return status, evo.lib.evo_last_error().decode()
    return 0, out.raw[:len(sequence)]


def test_variant_windows_match_upstream_known_answers(evo):
    """The known answers of upstream's tests/test_frontend.cpp:400-433."""
    assert _reverse_complement(evo, b"ACGTN") == (0, b"NACGT")
    assert _reverse_complement(evo, b"RYSWKMBDHVN") == (0, b"NBDHVKMWSRY")
    assert _reverse_complement(evo, b"acgt") == (0, b"acgt")
    status, message = _reverse_complement(evo, b"ACGU")
    assert status == 2 and "offset 3" in message
    assert _variant_window(evo, b"AACCGGTT", 3, b"C", b"T", 6) == (0, (b"AACCGG", b"AATCGG", 0, 6, 2))
    assert _variant_window(evo, b"AACCGG", 3, b"C", b"CTT", 5) == (0, (b"ACC", b"ACTTC", 1, 4, 1))
    status, message = _variant_window(evo, b"AACCGG", 3, b"G", b"T", 5)
    assert status == 2 and "does not match" in message
    status, message = _variant_window(evo, b"A", 1, b"A", b"T", 2)
    assert status == 2 and "two tokens" in message


def test_variant_window_properties(evo):
    """Seeded random loci: the window contains the allele at the stated offset, never exceeds
    the budget, uses the whole budget when the sequence allows it, and the flanks of the two
    windows are the same bytes of the input."""
    rng = np.random.default_rng(11)
    for _ in range(300):
        length = int(rng.integers(2, 60))
        sequence = bytes(rng.choice(np.frombuffer(b"ACGTNacgt", np.uint8), length).tolist())
        start = int(rng.integers(0, length))
        ref = sequence[start:start + int(rng.integers(1, min(4, length - start) + 1))]
        alt = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), int(rng.integers(1, 5))).tolist())
        maximum = int(rng.integers(1, 40))
        status, result = _variant_window(evo, sequence, start + 1, ref, alt, maximum)
        core = max(len(ref), len(alt))
        if maximum < core or maximum < 2:
            assert status == 2
            continue
        if status != 0:  # only a window of fewer than two tokens may still be refused
            assert "two tokens" in result
            continue
        reference, alternate, begin, end, offset = result
        assert reference == sequence[begin:end] and begin + offset == start
        assert alternate == sequence[begin:start] + alt + sequence[start + len(ref):end]
        assert max(len(reference), len(alternate)) <= maximum
        flank = (end - begin) - len(ref)
        assert flank == min(maximum - core, length - len(ref))
        # a side gives up budget only when it runs out of sequence
        left, right = offset, end - (start + len(ref))
        if left < (maximum - core) // 2:
            assert begin == 0 or right == length - (start + len(ref))


def test_modal_scratch_size_is_monotonic_and_bounded(pkg):
    """The HCL scratch holds one state per row segment of the one-wave grid plus the carried-in
    slot: it grows with the length until the grid is full, never shrinks (a buffer sized for a
    prompt serves every window of it), and stays far below one state per 64 rows for long prompts."""
    lib = ctypes.CDLL(str(pkg.OPS_LIBRARY))
    fn = lib.evo_b200_hcl_scratch_floats
    fn.restype = ctypes.c_size_t
    fn.argtypes = [ctypes.c_size_t] * 3
    for width, modes in ((4096, 16), (8192, 16), (96, 16), (64, 2)):
        previous = 0
        for length in (0, 1, 63, 64, 65, 128, 1000, 8192, 8336, 131072, 1 << 20):
            floats = fn(length, width, modes)
            assert floats >= previous, (width, length)
            previous = floats
            if length:
                assert floats >= 3 * width * modes                     # at least one segment and the slot
                assert floats <= (length // 64 + 3) * width * modes    # never more than a state per 64 rows
        assert fn(1 << 20, width, modes) == fn(131072, width, modes)   # bounded by the grid, not by the length
    assert fn(1 << 20, 4096, 16) * 4 <= 16 << 20                      # 7B shape: below the 16 MiB static array


# ---- file inputs of the variant driver (VCF stream, indexed reference FASTA): host-only
class _VcfRecord(ctypes.Structure):
    _fields_ = [("struct_size", ctypes.c_size_t), ("contig", ctypes.c_char_p), ("id", ctypes.c_char_p),
                ("reference", ctypes.c_char_p), ("alternate", ctypes.c_char_p), ("position_1based", ctypes.c_size_t),
                ("record_index", ctypes.c_size_t), ("allele_index", ctypes.c_size_t), ("line_number", ctypes.c_size_t)]


_VCF_CALLBACK = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.POINTER(_VcfRecord), ctypes.c_void_p)


def _stream_vcf(evo, path, stop_at=None):
    records = []

    @_VCF_CALLBACK
    def on_record(record, _user):
        r = record.contents
        records.append((r.contig, r.position_1based, r.id, r.reference, r.alternate, r.record_index, r.allele_index,
                        r.line_number))
        return 3 if stop_at is not None and len(records) == stop_at else 0

    fn = evo.lib.evo_b200_vcf_stream
    fn.argtypes = [ctypes.c_char_p, _VCF_CALLBACK, ctypes.c_void_p]
    status = fn(str(path).encode(), on_record, None)
    return status, records, (evo.lib.evo_last_error() or b"").decode()


VCF_HEADER = "##fileformat=VCFv4.2\n#CHROM\tPOS\tID\tREF\tALT\tQUAL\tFILTER\tINFO\n"


def test_vcf_stream_one_callback_per_alt_allele(evo, tmp_path):
    import gzip

    text = VCF_HEADER + "chr1\t5\trs1\tA\tG,TT\t.\t.\t.\nchr2\t12\t.\tacg\tA\t50\tPASS\tX=1\tGT\t0/1\r\n"
    plain = tmp_path / "a.vcf"
    plain.write_text(text)
    packed = tmp_path / "a.vcf.gz"
    packed.write_bytes(gzip.compress(text.encode()))
    expected = [(b"chr1", 5, b"rs1", b"A", b"G", 0, 0, 3), (b"chr1", 5, b"rs1", b"A", b"TT", 0, 1, 3),
                (b"chr2", 12, b".", b"acg", b"A", 1, 0, 4)]
    for path in (plain, packed):
        status, records, _ = _stream_vcf(evo, path)
        assert status == 0 and records == expected
    status, records, message = _stream_vcf(evo, plain, stop_at=2)      # a consumer's error stops the stream
    assert status == 3 and len(records) == 2
    cases = {
        "chr1\t5\t.\tA\tG\t.\t.\t.\n": "before the #CHROM header",
        VCF_HEADER: "contains no records",
        VCF_HEADER + "chr1\t0\t.\tA\tG\t.\t.\t.\n": "POS must be a positive integer at line 3",
        VCF_HEADER + "chr1\t5\t.\tA\t<DEL>\t.\t.\t.\n": "VCF ALT",
        VCF_HEADER + "chr1\t5\t.\tA\n": "fewer than 8 valid fields at line 3",
        VCF_HEADER + "\nchr1\t5\t.\tA\tG\t.\t.\t.\n": "empty line at 3",
        VCF_HEADER + VCF_HEADER.splitlines()[1] + "\n": "repeats the #CHROM header",
        "##x\n#CHROM\tPOS\n": "unsupported header at line 2",
    }
    for index, (body, fragment) in enumerate(cases.items()):
        path = tmp_path / f"bad{index}.vcf"
        path.write_text(body)
        status, _, message = _stream_vcf(evo, path)
        assert status == 2 and fragment in message, (body, message)
    assert _stream_vcf(evo, tmp_path / "missing.vcf")[0] == 3


def _reference(evo, path):
    handle = ctypes.c_void_p()
    fn = evo.lib.evo_b200_reference_open
    fn.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    status = fn(str(path).encode(), ctypes.byref(handle))
    return status, handle, (evo.lib.evo_last_error() or b"").decode()


def _window(evo, handle, contig, position, ref, alt, maximum):
    fn = evo.lib.evo_b200_reference_window
    Z = ctypes.c_size_t
    fn.argtypes = [ctypes.c_void_p, ctypes.c_char_p, Z, ctypes.c_char_p, Z, ctypes.c_char_p, Z, Z,
                   ctypes.POINTER(Z), ctypes.POINTER(Z), ctypes.POINTER(Z), ctypes.c_char_p, Z]
    start, end, length = Z(), Z(), Z()
    buffer = ctypes.create_string_buffer(max(maximum, 1))
    status = fn(handle, contig, position, ref, len(ref), alt, len(alt), maximum, ctypes.byref(start),
                ctypes.byref(end), ctypes.byref(length), buffer, maximum)
    if status != 0:
        return status, (evo.lib.evo_last_error() or b"").decode()
    return 0, (buffer.raw[:end.value - start.value], start.value, end.value, length.value)


def test_reference_fasta_index_and_scoring_windows(evo, tmp_path):
    rng = np.random.default_rng(21)
    contigs = {b"chrA": bytes(rng.choice(np.frombuffer(b"ACGTacgtN", np.uint8), 137).tolist()),
               b"chrB": bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), 60).tolist()),
               b"tiny": b"ACG"}
    evo.lib.evo_b200_reference_free.argtypes = [ctypes.c_void_p]
    for width, newline in ((10, b"\n"), (60, b"\r\n"), (7, b"\n")):
        path = tmp_path / f"genome{width}.fa"
        with open(path, "wb") as out:
            for name, bases in contigs.items():
                out.write(b">" + name + b" description text" + newline)
                for begin in range(0, len(bases), width):
                    out.write(bases[begin:begin + width] + newline)
        status, handle, message = _reference(evo, path)
        assert status == 0, message
        for _ in range(200):
            name = [b"chrA", b"chrB", b"tiny"][int(rng.integers(0, 3))]
            bases = contigs[name]
            start = int(rng.integers(0, len(bases)))
            ref = bases[start:start + int(rng.integers(1, min(4, len(bases) - start) + 1))]
            alt = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), int(rng.integers(1, 5))).tolist())
            maximum = int(rng.integers(2, 50))
            core = max(len(ref), len(alt))
            status, result = _window(evo, handle, name, start + 1, ref, alt, maximum)
            if maximum < core:
                assert status == 2 and "two tokens" in result
                continue
            assert status == 0, result
            sequence, begin, end, length = result
            assert length == len(bases) and sequence == bases[begin:end] and begin <= start and start + len(ref) <= end
            assert (end - begin) - len(ref) == min(maximum - core, len(bases) - len(ref))   # the whole budget
            left, right = start - begin, end - (start + len(ref))
            if left < (maximum - core) // 2:
                assert begin == 0 or right == len(bases) - (start + len(ref))
        assert _window(evo, handle, b"chrB", 3, b"N" if contigs[b"chrB"][2:3] != b"N" else b"A", b"T", 20)[1].startswith(
            "invalid_argument: VCF REF does not match reference contig 'chrB' at 1-based position 3")
        assert "extends beyond" in _window(evo, handle, b"tiny", 3, b"GT", b"T", 20)[1]
        assert "has no contig 'chrZ'" in _window(evo, handle, b"chrZ", 1, b"A", b"T", 20)[1]
        evo.lib.evo_b200_reference_free(handle)
    # refusals at open
    def refused(name, payload, code, fragment):
        path = tmp_path / name
        path.write_bytes(payload)
        status, _, message = _reference(evo, path)
        assert status == code and fragment in message, message

    refused("dup.fa", b">a\nAC\n>a\nGT\n", 2, "duplicate contig 'a'")
    refused("ragged.fa", b">a\nACGT\nAC\nACGT\n", 2, "differ in width")
    refused("blank.fa", b">a\nACGT\n\nACGT\n", 2, "differ in width")
    refused("space.fa", b">a\nAC GT\n", 2, "whitespace at line 2")
    refused("nohdr.fa", b"ACGT\n", 2, "before a header")
    refused("empty.fa", b"", 2, "not FASTA")
    import gzip
    refused("packed.fa.gz", gzip.compress(b">a\nACGT\n"), 5, "gzip-compressed")
    assert _reference(evo, tmp_path / "absent.fa")[0] == 3
