#!/usr/bin/env python3
"""Regenerates the committed golden fixtures from the upstream project.

Run where the upstream tree is present (its path is the first argument) and
the upstream CPU libraries built by `make -C oracle ref`.  Nothing at test or
bench time needs the upstream tree; only this script does.

Outputs (all under tests/golden/):
  e4m3_exhaustive.npz   upstream encode_e4m3fn over every BF16 bit pattern at
                        three scales, plus decode of all 256 codes
  qgmma_golden.npz      upstream's pure-Python H100 QGMMA statement
                        (tests/test_triton_fp8.py:51-115) on seeded E4M3
                        operands, incl. zeros, subnormals and a wide exponent
                        spread, plus the case of tests/test_cuda_ops.cu:433-503
  ref_cpu_ops.npz       upstream src/cpu_reference.cpp operators on seeded
                        inputs (rms_norm, linear, gated_mlp, fir, hcl, rope,
                        attention)
  tiny/                 upstream's 50-layer tiny StripedHyena2 fixture and the
                        logits of its pure-Python BF16 oracle
                        (tools/generate_tiny_model.py)
"""
from __future__ import annotations

import ctypes
import importlib.util
import subprocess
import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
if len(sys.argv) < 2 and "EVO_UPSTREAM_ROOT" not in os.environ:
    sys.exit("usage: pass the upstream source tree as the first argument (or set EVO_UPSTREAM_ROOT)")
REF = Path(sys.argv[1] if len(sys.argv) > 1 else os.environ["EVO_UPSTREAM_ROOT"])


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(values: np.ndarray) -> np.ndarray:
    return torch.from_numpy(np.ascontiguousarray(values, dtype=np.float32)).to(
        torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def ref_ops():
    lib = ctypes.CDLL(str(ROOT / "oracle" / "_ref" / "libevo_ref_ops.so"))
    lib.ref_encode_e4m3fn.restype = ctypes.c_uint8
    lib.ref_encode_e4m3fn.argtypes = [ctypes.c_float]
    lib.ref_decode_e4m3fn.restype = ctypes.c_float
    lib.ref_decode_e4m3fn.argtypes = [ctypes.c_uint8]
    P, Z, F, I = ctypes.POINTER(ctypes.c_float), ctypes.c_size_t, ctypes.c_float, ctypes.c_int
    lib.ref_rms_norm.argtypes = [P, Z, Z, P, F, P]
    lib.ref_linear.argtypes = [P, Z, Z, P, Z, P, P]
    lib.ref_gated_mlp.argtypes = [P, Z, Z, Z, P, P, P, I, P]
    lib.ref_fir.argtypes = [P, Z, Z, P, Z, P, I, I, P]
    lib.ref_hcl_recurrence.argtypes = [P, P, P, Z, Z, P, P, P, Z, P, P]
    lib.ref_rope.argtypes = [P, P, Z, Z, Z, P, Z, F]
    lib.ref_attention.argtypes = [P, P, P, Z, Z, Z, P]
    return lib


def fptr(a: np.ndarray):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def make_e4m3(lib) -> None:
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    values = bf16_bits_to_f32(bits)
    out = {}
    for scale in (1.0, 5.75, 0.03125):
        with np.errstate(over="ignore", invalid="ignore"):
            scaled = (values * np.float32(scale)).astype(np.float32)
        out[f"codes_scale_{scale}"] = np.array(
            [lib.ref_encode_e4m3fn(float(v)) for v in scaled], dtype=np.uint8)
    out["decode"] = np.array([lib.ref_decode_e4m3fn(c) for c in range(256)], dtype=np.float32)
    np.savez_compressed(HERE / "e4m3_exhaustive.npz", **out)


def make_qgmma(lib) -> None:
    sys.path.insert(0, str(REF / "tools"))
    spec = importlib.util.spec_from_file_location("ref_triton_test", REF / "tests" / "test_triton_fp8.py")
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    oracle = module.h100_qgmma_oracle
    decode = np.array([lib.ref_decode_e4m3fn(c) for c in range(256)], dtype=np.float32)
    rng = np.random.default_rng(20250)
    cases = {}

    def run(name, x_codes, w_codes, scale):
        x = torch.from_numpy(decode[x_codes])
        w = torch.from_numpy(decode[w_codes])
        expected = oracle(x, w, scale).view(torch.int16).numpy().view(np.uint16)
        cases[f"{name}_x"] = x_codes
        cases[f"{name}_w"] = w_codes
        cases[f"{name}_scale"] = np.float32(scale)
        cases[f"{name}_y"] = expected

    def finite_codes(shape, low=0, high=0x7f):
        magnitude = rng.integers(low, high, size=shape, dtype=np.uint8)  # excludes NaN 0x7f
        sign = rng.integers(0, 2, size=shape, dtype=np.uint8) << 7
        return (magnitude | sign).astype(np.uint8)

    run("uniform", finite_codes((5, 128)), finite_codes((7, 128)), 0.001953125)
    run("small", finite_codes((4, 96), 0, 0x20), finite_codes((6, 96), 0, 0x18), 3.0)
    x = finite_codes((4, 160)); w = finite_codes((5, 160))
    x[rng.random(x.shape) < 0.4] = 0; w[rng.random(w.shape) < 0.3] = 0x80
    x[0, :32] = 0  # a whole zero group
    run("sparse", x, w, 0.0625)
    # one huge product among tiny ones, then cancellation
    x = finite_codes((3, 64), 0, 0x10); w = finite_codes((4, 64), 0, 0x10)
    x[:, 5] = 0x7e; w[:, 5] = 0x7e; x[:, 40] = 0xfe; w[:, 40] = 0x7e
    run("spread", x, w, 1.0)
    # the configuration of upstream's CUDA operator test
    def values(count, offset, divisor):
        idx = np.arange(count)
        return ((((idx + offset) * 37 + 11) % 29) - 14).astype(np.float32) / np.float32(divisor)
    xin = bf16_bits_to_f32(f32_to_bf16_bits(values(3 * 64, 41, 13.0)))
    win = bf16_bits_to_f32(f32_to_bf16_bits(values(5 * 64, 73, 17.0)))
    xc = np.array([lib.ref_encode_e4m3fn(float(v)) for v in xin * np.float32(5.75)], dtype=np.uint8).reshape(3, 64)
    wc = np.array([lib.ref_encode_e4m3fn(float(v)) for v in win * np.float32(3.25)], dtype=np.uint8).reshape(5, 64)
    run("upstream_test", xc, wc, 0.03125)
    cases["upstream_test_x_bf16"] = f32_to_bf16_bits(xin).reshape(3, 64)
    np.savez_compressed(HERE / "qgmma_golden.npz", **cases)


def make_cpu_ops(lib) -> None:
    rng = np.random.default_rng(7)
    out = {}
    f = lambda *s: rng.standard_normal(s).astype(np.float32)
    rows, width, inner = 5, 24, 40
    x = f(rows, width); scale = (1 + 0.1 * f(width)).astype(np.float32)
    y = np.empty_like(x)
    assert lib.ref_rms_norm(fptr(x), rows, width, fptr(scale), 1e-6, fptr(y)) == 0
    out.update(rms_x=x, rms_scale=scale, rms_y=y)
    w = f(inner, width); b = f(inner); y = np.empty((rows, inner), np.float32)
    assert lib.ref_linear(fptr(x), rows, width, fptr(w), inner, fptr(b), fptr(y)) == 0
    out.update(lin_x=x, lin_w=w, lin_b=b, lin_y=y)
    l1 = f(inner, width) * 0.3; l2 = f(inner, width) * 0.3; l3 = f(width, inner) * 0.3
    for gelu in (0, 1):
        y = np.empty((rows, width), np.float32)
        assert lib.ref_gated_mlp(fptr(x), rows, width, inner, fptr(l1), fptr(l2), fptr(l3), gelu, fptr(y)) == 0
        out[f"mlp_y_{gelu}"] = y
    out.update(mlp_l1=l1, mlp_l2=l2, mlp_l3=l3)
    length, channels = 19, 6
    xin = f(length, channels)
    for taps in (3, 7, 128):
        wt = f(channels, taps); bias = f(channels)
        for conv in (0, 1):
            for mult in (0, 1):
                y = np.empty_like(xin)
                assert lib.ref_fir(fptr(xin), length, channels, fptr(wt), taps, fptr(bias), conv, mult, fptr(y)) == 0
                out[f"fir_y_{taps}_{conv}_{mult}"] = y
        out[f"fir_w_{taps}"] = wt; out[f"fir_b_{taps}"] = bias
    out["fir_x"] = xin
    modes = 4
    x2, x1, v = f(length, channels), f(length, channels), f(length, channels)
    direct = f(channels); lp = -np.abs(f(channels, modes)) * 0.2; res = f(channels, modes)
    state = np.zeros((channels, modes), np.float32); y = np.empty((length, channels), np.float32)
    assert lib.ref_hcl_recurrence(fptr(x2), fptr(x1), fptr(v), length, channels, fptr(direct), fptr(lp),
                                  fptr(res), modes, fptr(state), fptr(y)) == 0
    out.update(hcl_x2=x2, hcl_x1=x1, hcl_v=v, hcl_d=direct, hcl_lp=lp, hcl_res=res, hcl_state=state, hcl_y=y)
    heads, hd, t = 3, 8, 9
    q, k, vv = f(t, heads, hd), f(t, heads, hd), f(t, heads, hd)
    inv = (10000.0 ** (-np.arange(hd // 2) * 2.0 / hd)).astype(np.float32)
    qr, kr = q.copy(), k.copy()
    assert lib.ref_rope(fptr(qr), fptr(kr), t, heads, hd, fptr(inv), 5, 2.0) == 0
    out.update(rope_q=q, rope_k=k, rope_inv=inv, rope_qr=qr, rope_kr=kr)
    y = np.empty_like(q)
    assert lib.ref_attention(fptr(q), fptr(k), fptr(vv), t, heads, hd, fptr(y)) == 0
    out.update(att_q=q, att_k=k, att_v=vv, att_y=y)
    np.savez_compressed(HERE / "ref_cpu_ops.npz", **out)


def make_tiny() -> None:
    tiny = HERE / "tiny"
    tiny.mkdir(exist_ok=True)
    env = {"PYTHONPATH": str(REF / "tools")}
    subprocess.run([sys.executable, str(REF / "tools" / "generate_tiny_model.py"),
                    "--model", str(tiny / "tiny.safetensors"),
                    "--expected-logits", str(tiny / "logits.f32"),
                    "--expected-decode", str(tiny / "decode.f32"),
                    "--expected-layer", str(tiny / "layer17.f32"),
                    "--expected-chunked", str(tiny / "chunked.f32")],
                   check=True, env=env)


if __name__ == "__main__":
    lib = ref_ops()
    make_e4m3(lib)
    make_qgmma(lib)
    make_cpu_ops(lib)
    make_tiny()
    print("golden fixtures written under", HERE)
