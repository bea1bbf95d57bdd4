"""Quantised KV cache of the fast-q8-kv profile (upstream docs/execution-profiles.md:96-127,
src/cuda/attention.cu:798-866 and 1072-1141): per (token, head) vector scale = max|v| / 127,
codes clamp(rint(v / scale), +-127), fixed pages; attention reads code * scale.

Operator level: codes and scales bit-exact against the same F32 arithmetic in numpy, the BF16
image of the pages, and decode attention straight from the pages against an F32 reference on the
dequantised values.  Model level: the profile against `exact` on a synthetic fixture, gated like
upstream's own plumbing check (there: min per-row cosine 0.9999, logit MAE 0.01, top-1 agreement
1.0 on its fixture; this fixture's larger weights measure 0.99987 / 0.004, so the cosine gate is
0.9995 here) with identical top-1 on every row that is decided beyond the per-logit error."""
from __future__ import annotations

import importlib

import numpy as np
import pytest
import torch

from gpu_util import dev_bits, empty_bits, host_bits, p, rand_bf16, stream
from oracle_lib import bf16_to_f32, f32_to_bf16

pytestmark = pytest.mark.gpu

HEAD_DIM = 128


class Pages:
    def __init__(self, page_tokens, page_count, heads, head_dim=HEAD_DIM):
        self.page_tokens, self.heads, self.head_dim = page_tokens, heads, head_dim
        self.codes = [[torch.zeros(page_tokens * heads * head_dim, dtype=torch.int8, device="cuda")
                       for _ in range(page_count)] for _ in range(2)]
        self.scales = [[torch.zeros(page_tokens * heads, device="cuda") for _ in range(page_count)] for _ in range(2)]
        self.tables = [torch.tensor([t.data_ptr() for t in group], dtype=torch.int64, device="cuda")
                       for group in (self.codes[0], self.codes[1], self.scales[0], self.scales[1])]

    def args(self):
        return [p(t) for t in self.tables] + [self.page_tokens]

    def host(self, which, count):
        codes = torch.cat(self.codes[which]).cpu().numpy().reshape(-1, self.heads, self.head_dim)[:count]
        scales = torch.cat(self.scales[which]).cpu().numpy().reshape(-1, self.heads)[:count]
        return codes, scales


def reference_quantise(bits):
    values = bf16_to_f32(bits)                                       # [rows, heads, 128]
    largest = np.abs(values).max(axis=-1)
    scale = np.where(largest == 0, np.float32(1.0), (largest / np.float32(127.0)).astype(np.float32)).astype(np.float32)
    codes = np.clip(np.rint((values / scale[..., None]).astype(np.float32)), -127, 127).astype(np.int8)
    return codes, scale


@pytest.mark.parametrize("heads,page_tokens", [(2, 16), (15, 64), (32, 16384)])
def test_append_expand_and_decode_from_pages(ops, heads, page_tokens):
    rng = np.random.default_rng(heads)
    total = 150 if page_tokens < 16384 else 700
    pages = Pages(page_tokens, (total + page_tokens - 1) // page_tokens, heads)
    key = rand_bf16(rng, total, heads, HEAD_DIM)
    value = rand_bf16(rng, total, heads, HEAD_DIM, scale=3.0)
    key[5, 0] = 0                                                    # a zero vector keeps scale 1
    # appended in three pieces that straddle page edges
    for begin, end in ((0, 17), (17, 18), (18, total)):
        ops.call("q8_kv_append", p(dev_bits(key[begin:end])), p(dev_bits(value[begin:end])), *pages.args(), begin,
                 end - begin, heads, HEAD_DIM, stream())
    for which, source in ((0, key), (1, value)):
        codes, scales = pages.host(which, total)
        expected_codes, expected_scales = reference_quantise(source)
        assert np.array_equal(scales, expected_scales)
        assert np.array_equal(codes, expected_codes)
    assert pages.host(0, total)[1][5, 0] == 1.0
    image_k, image_v = empty_bits(total, heads, HEAD_DIM), empty_bits(total, heads, HEAD_DIM)
    ops.call("q8_kv_expand", *pages.args(), total, heads, HEAD_DIM, p(image_k), p(image_v), stream())
    for which, image in ((0, image_k), (1, image_v)):
        codes, scales = pages.host(which, total)
        assert np.array_equal(host_bits(image), f32_to_bf16(codes.astype(np.float32) * scales[..., None]))
    # decode rows against every prefix length class: reference in F32 on code * scale
    kq, ks = pages.host(0, total)
    vq, vs = pages.host(1, total)
    k = kq.astype(np.float32) * ks[..., None]
    v = vq.astype(np.float32) * vs[..., None]
    for rows in (1, 3, 8):
        query = rand_bf16(rng, rows, heads, HEAD_DIM)
        out = empty_bits(rows, heads, HEAD_DIM)
        ops.call("q8_attention_decode", p(dev_bits(query)), *pages.args(), rows, total, heads, HEAD_DIM, p(out),
                 stream())
        q = bf16_to_f32(query).astype(np.float64)
        expected = np.empty((rows, heads, HEAD_DIM))
        for r in range(rows):
            visible = total - rows + r + 1
            scores = np.einsum("hd,thd->ht", q[r], k[:visible].astype(np.float64)) / np.sqrt(HEAD_DIM)
            weights = np.exp(scores - scores.max(axis=1, keepdims=True))
            weights /= weights.sum(axis=1, keepdims=True)
            expected[r] = np.einsum("ht,thd->hd", weights, v[:visible].astype(np.float64))
        got = bf16_to_f32(host_bits(out)).astype(np.float64)
        assert np.all(np.abs(got - expected) <= 0.02 + 0.02 * np.abs(expected)), np.abs(got - expected).max()


@pytest.mark.parametrize("heads,head_dim,page_tokens", [(2, 32, 3), (3, 6, 5), (1, 200, 4)])
def test_append_and_expand_at_other_head_sizes(ops, heads, head_dim, page_tokens):
    """Append and expand take any head size (upstream's own paged-cache test uses 32); same codes and scales."""
    rng = np.random.default_rng(head_dim)
    total = 11
    pages = Pages(page_tokens, (total + page_tokens - 1) // page_tokens, heads, head_dim)
    key, value = rand_bf16(rng, total, heads, head_dim), rand_bf16(rng, total, heads, head_dim, scale=3.0)
    key[2, 0] = 0
    for begin, end in ((0, 4), (4, total)):
        ops.call("q8_kv_append", p(dev_bits(key[begin:end])), p(dev_bits(value[begin:end])), *pages.args(), begin,
                 end - begin, heads, head_dim, stream())
    image_k, image_v = empty_bits(total, heads, head_dim), empty_bits(total, heads, head_dim)
    ops.call("q8_kv_expand", *pages.args(), total, heads, head_dim, p(image_k), p(image_v), stream())
    for which, source, image in ((0, key, image_k), (1, value, image_v)):
        codes, scales = pages.host(which, total)
        expected_codes, expected_scales = reference_quantise(source)
        assert np.array_equal(scales, expected_scales)
        assert np.array_equal(codes, expected_codes)
        assert np.array_equal(host_bits(image), f32_to_bf16(codes.astype(np.float32) * scales[..., None]))
    query, out = rand_bf16(rng, 1, heads, head_dim), empty_bits(1, heads, head_dim)
    assert ops.status("q8_attention_decode", p(dev_bits(query)), *pages.args(), 1, total, heads, head_dim, p(out),
                      stream()) == 2  # reading the pages directly stays a head-size-128 kernel


def test_profile_against_exact_with_upstreams_gates(pkg, tmp_path_factory):
    rt = importlib.import_module("evo_cpp_b200.runtime")
    art = importlib.import_module("evo_cpp_b200.artifact")
    directory = tmp_path_factory.mktemp("q8")
    spec = art.fixture_spec(width=256, layers=8, heads=2, inner=512, hcs_groups=16, hcm_groups=16)
    art.write_synthetic(directory / "model.safetensors", spec, seed=3, weight_std=0.05, filter_std=0.3)
    evo = rt.EvoLibrary(pkg.EVO_LIBRARY)
    model = evo.load(directory / "model.safetensors", flags=rt.MODEL_FLAG_ALLOW_SYNTHETIC)
    rng = np.random.default_rng(12)
    sequence = bytes(rng.choice(np.frombuffer(b"ACGT", np.uint8), 600).tolist())
    full = rt.CONTEXT_FLAG_FULL_ARENA
    exact = model.context(1024, flags=full)
    fast = model.context(1024, flags=full | rt.CONTEXT_FLAG_FAST_Q8_KV)
    assert (exact.profile, fast.profile) == ("exact", "fast-q8-kv")
    a, b = exact.prefill(sequence[:400]), fast.prefill(sequence[:400])
    outputs = [(a, b)]
    # a continuation chunk (attends to pages written by the prefill), then decode steps from the pages
    import torch as _torch
    tokens = _torch.tensor(list(sequence[400:600]), dtype=_torch.int32, device="cuda")
    for context in (exact, fast):
        context.continue_device(tokens.data_ptr(), 200)
        context.synchronize()
    token = int(a[-1].argmax())
    steps_exact, steps_fast = [], []
    for _ in range(6):
        step_exact, step_fast = exact.decode(token), fast.decode(token)
        steps_exact.append(step_exact)
        steps_fast.append(step_fast)
        token = int(step_exact.argmax())
    outputs.append((np.stack(steps_exact), np.stack(steps_fast)))
    for reference, candidate in outputs:
        r, c = reference.astype(np.float64), candidate.astype(np.float64)
        cosine = (r * c).sum(-1) / (np.linalg.norm(r, axis=-1) * np.linalg.norm(c, axis=-1))
        assert cosine.min() >= 0.9995, cosine.min()
        assert np.abs(r - c).mean() <= 0.01
        ordered = np.sort(r, axis=-1)
        decided = (ordered[:, -1] - ordered[:, -2]) > 2.0 * np.abs(r - c).max()
        assert (r.argmax(-1) == c.argmax(-1))[decided].all() and (r.argmax(-1) == c.argmax(-1)).mean() >= 0.95
    # the same through the chunked public prefill (8-row arena: every chunk but the first attends to pages)
    chunked = model.context(1024, flags=rt.CONTEXT_FLAG_FAST_Q8_KV).prefill(sequence[:100])
    close = np.abs(chunked.astype(np.float64) - a[:100]) <= 0.08 + 0.06 * np.abs(a[:100])
    assert close.all()
