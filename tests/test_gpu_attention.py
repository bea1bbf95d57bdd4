"""GPU parity of the attention stripe operators against the CPU oracle through
the operator C ABI (shapes after upstream's tests/test_cuda_attention.cu:
prefix + chunk, tile boundaries, long-context RoPE positions)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import (assert_close_bits, dev, dev_bits, empty_bits, host_bits, p, rand_bf16, stream,
                      ulp_mismatch_report)
from oracle_lib import bf16_to_f32, f32_to_bf16, ptr

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("head_major", [0, 1])
@pytest.mark.parametrize("rows,heads,head_dim,offset,scale", [(9, 3, 8, 5, 2.0), (4, 2, 128, 0, 1.0),
                                                             (3, 2, 128, 1048573, 128.0)])
def test_split_rope_append(ops, oracle, rows, heads, head_dim, offset, scale, head_major):
    rng = np.random.default_rng(rows + offset % 97)
    width = heads * head_dim
    qkv = rand_bf16(rng, rows, 3 * width)
    inv = (10000.0 ** (-np.arange(head_dim // 2) * 2.0 / head_dim)).astype(np.float32)
    base = max(0, offset - 2)           # keep the cache small: it starts at `base`
    local = offset - base
    capacity = local + rows
    q = empty_bits(rows, width)
    kc, vc = torch.zeros((capacity, width), dtype=torch.int16, device="cuda"), \
        torch.zeros((capacity, width), dtype=torch.int16, device="cuda")
    # position_offset is also the cache row; shift the cache pointers so that row
    # `offset` lands at local row `local`.
    shift = base * width * 2
    ops.call("bf16_split_rope_append", p(dev_bits(qkv)), p(dev(inv)), rows, heads, head_dim, offset,
             scale, head_major, p(q), p(kc) - shift, p(vc) - shift, offset + rows, stream())
    eq = np.empty((rows, width), np.uint16)
    ek = np.zeros((offset + rows, width), np.uint16) if offset < 4096 else None
    if ek is None:
        # oracle writes at absolute rows; give it a window the same way
        ek_window = np.zeros((capacity, width), np.uint16)
        ev_window = np.zeros((capacity, width), np.uint16)
        oracle.split_rope_append(ptr(qkv), ptr(inv), rows, heads, head_dim, offset, scale, head_major,
                                 ptr(eq), ek_window.ctypes.data - shift, ev_window.ctypes.data - shift)
        ek_rows, ev_rows = ek_window[local:], ev_window[local:]
    else:
        ev = np.zeros_like(ek)
        oracle.split_rope_append(ptr(qkv), ptr(inv), rows, heads, head_dim, offset, scale, head_major,
                                 ptr(eq), ptr(ek), ptr(ev))
        ek_rows, ev_rows = ek[offset:], ev[offset:]
    assert np.array_equal(host_bits(vc)[local:], ev_rows)
    for got, want in ((host_bits(q), eq), (host_bits(kc)[local:], ek_rows)):
        # device sincosf vs libm sin/cos and FMA contraction choices: 1 BF16 ulp
        # away from cancellation, tiny absolute differences where a*cos ~ b*sin
        assert_close_bits(got, want, atol=4e-3, rtol=8e-3)
        fraction, _ = ulp_mismatch_report(got, want)
        assert fraction < 0.05, fraction


@pytest.mark.parametrize("rows,prefix,heads,head_dim", [
    (64, 0, 2, 128), (200, 0, 3, 128), (129, 37, 2, 128), (16, 300, 2, 128), (700, 0, 1, 128),
    (9, 0, 3, 8), (5, 11, 2, 4), (1, 40, 2, 128), (1, 2000, 3, 128), (5, 1000, 2, 128), (8, 0, 2, 128),
    (3, 5, 1, 128)])
def test_causal_attention(ops, oracle, rows, prefix, heads, head_dim):
    """Tensor-core flash kernel (head 128, >= 16 rows) and the row-wise kernel.
    Upstream gates its FlashAttention path against CPU attention at tolerance
    (tests/test_cuda_attention.cu:265-339); so does this test."""
    rng = np.random.default_rng(rows * 5 + prefix)
    width = heads * head_dim
    total = prefix + rows
    q = rand_bf16(rng, rows, width)
    k, v = rand_bf16(rng, total, width), rand_bf16(rng, total, width)
    out = empty_bits(rows, width)
    ops.call("bf16_causal_attention", p(dev_bits(q)), p(dev_bits(k)), p(dev_bits(v)), rows, total, heads,
             head_dim, p(out), stream())
    expected = np.empty((rows, width), np.uint16)
    oracle.causal_attention(ptr(q), ptr(k), ptr(v), rows, total, heads, head_dim, ptr(expected))
    assert_close_bits(host_bits(out), expected, atol=0.02, rtol=0.02, min_cosine=0.9995)


@pytest.mark.parametrize("rows,prefix,heads", [(128, 0, 1), (1024, 0, 3), (2048, 512, 2), (1000, 77, 2),
                                               (4096, 0, 1), (300, 1300, 2)])
def test_tcgen05_attention_matches_warp_mma_kernel(ops, rows, prefix, heads):
    """>= 128 rows of head size 128 run on the tcgen05 kernel; the warp-level MMA
    kernel computes the same contract with different tiling and summation order."""
    gen = torch.Generator(device="cuda").manual_seed(rows + prefix)
    width, total = heads * 128, prefix + rows
    q = torch.randn(rows, width, device="cuda", generator=gen).bfloat16()
    k = torch.randn(total, width, device="cuda", generator=gen).bfloat16()
    v = torch.randn(total, width, device="cuda", generator=gen).bfloat16()
    out, check = torch.full_like(q, 7.0), torch.full_like(q, -7.0)
    ops.call("bf16_causal_attention", p(q), p(k), p(v), rows, total, heads, 128, p(out), stream())
    ops.call("bf16_causal_attention_mma_sync", p(q), p(k), p(v), rows, total, heads, 128, p(check), stream())
    ops.call("check_async_errors", stream())
    a, b = out.float(), check.float()
    assert torch.isfinite(a).all()
    assert (a - b).abs().max().item() < 0.03, (a - b).abs().max().item()
    assert torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item() > 0.9999
    # and against plain F32 softmax attention for the first head
    scores = (q[:, :128].float() @ k[:, :128].float().T) / 128 ** 0.5
    visible = torch.arange(total, device="cuda")[None, :] <= (prefix + torch.arange(rows, device="cuda"))[:, None]
    reference = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1) @ v[:, :128].float()
    assert (a[:, :128] - reference).abs().max().item() < 0.03


@pytest.mark.parametrize("rows,prefix,growth", [(1024, 0, 2.0), (1024, 0, 0.05), (640, 384, 0.02)])
def test_tcgen05_attention_with_growing_scores(ops, rows, prefix, growth):
    """Scores that climb with the key position, at a different rate per query row: the row maximum
    keeps moving, so the accumulated output has to be rescaled again and again (the two-CTA kernel
    keeps it in tensor memory and rescales only rows whose reference moved by more than 2^8, other
    rows of the same warp multiply by one).  Against F32 softmax attention."""
    gen = torch.Generator(device="cuda").manual_seed(int(rows + prefix + growth * 100))
    total = prefix + rows
    direction = torch.sign(torch.randn(128, device="cuda", generator=gen)) / 128 ** 0.5
    # row i looks along `direction` with strength i % 5 (0: flat scores), key j lies growth * j along it
    strength = (torch.arange(rows, device="cuda") % 5).float()[:, None]
    q = (strength * direction[None, :] * 128 ** 0.5 + 0.3 * torch.randn(rows, 128, device="cuda", generator=gen))
    k = (growth * torch.arange(total, device="cuda").float()[:, None] * direction[None, :]
         + 0.3 * torch.randn(total, 128, device="cuda", generator=gen))
    v = torch.randn(total, 128, device="cuda", generator=gen)
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    out = torch.full_like(q, 7.0)
    ops.call("bf16_causal_attention", p(q), p(k), p(v), rows, total, 1, 128, p(out), stream())
    ops.call("check_async_errors", stream())
    scores = (q.float() @ k.float().T) / 128 ** 0.5
    visible = torch.arange(total, device="cuda")[None, :] <= (prefix + torch.arange(rows, device="cuda"))[:, None]
    reference = torch.softmax(scores.masked_fill(~visible, float("-inf")), dim=-1) @ v.float()
    got = out.float()
    assert torch.isfinite(got).all()
    assert (got - reference).abs().max().item() < 0.04, (got - reference).abs().max().item()
    assert torch.nn.functional.cosine_similarity(got.flatten(), reference.flatten(), dim=0).item() > 0.9995


def test_tcgen05_attention_gives_the_same_bits_on_concurrent_streams(ops):
    """Six host threads, each with its own stream, run the attention operator over and over on
    prompts of 151..361 rows.  With several kernels sharing the SMs the warps of a CTA drift far
    apart, which is when a hand-over that is only safe at similar speeds shows (two did: a warp that
    skipped phases of a barrier read the accumulator two phases early, or waited for a phase that had
    long passed).  Every result must equal the one computed alone, bit for bit."""
    import threading

    gen = torch.Generator(device="cuda").manual_seed(11)
    jobs = []
    for rows in (243, 233, 361, 151, 348, 205):
        q, k, v = (torch.randn(rows, 256, device="cuda", generator=gen).bfloat16() for _ in range(3))
        alone = torch.empty_like(q)
        ops.call("bf16_causal_attention", p(q), p(k), p(v), rows, rows, 2, 128, p(alone), stream())
        jobs.append((rows, q, k, v, alone))
    torch.cuda.synchronize()
    failures = []

    def worker(job):
        rows, q, k, v, alone = job
        own = torch.cuda.Stream()
        with torch.cuda.stream(own):
            out = torch.empty_like(q)
            for iteration in range(400):
                out.zero_()
                ops.call("bf16_causal_attention", p(q), p(k), p(v), rows, rows, 2, 128, p(out), own.cuda_stream)
                own.synchronize()
                if not torch.equal(out, alone):
                    failures.append((rows, iteration, int((out != alone).any(dim=1).nonzero()[0])))
                    return

    # two more threads keep every SM busy with large projections (persistent CTA pairs): attention CTAs
    # then start late and their warps see very different delays
    x = torch.randn(1024, 4096, device="cuda", generator=gen).bfloat16()
    w = (torch.randn(12288, 4096, device="cuda", generator=gen) * 0.05).bfloat16()
    product = torch.empty(1024, 12288, device="cuda", dtype=torch.bfloat16)
    ops.call("bf16_linear", p(x), p(w), None, None, 1024, 4096, 12288, 0, 0, p(product), stream())
    torch.cuda.synchronize()

    def load():
        own = torch.cuda.Stream()
        with torch.cuda.stream(own):
            out = torch.empty_like(product)
            for iteration in range(150):
                ops.call("bf16_linear", p(x), p(w), None, None, 1024, 4096, 12288, 0, 0, p(out), own.cuda_stream)
                own.synchronize()
                if not torch.equal(out, product):
                    failures.append(("projection", iteration))
                    return

    threads = [threading.Thread(target=worker, args=(job,)) for job in jobs]
    threads += [threading.Thread(target=load) for _ in range(2)]
    for thread in threads:
        thread.start()
    for thread in threads:
        thread.join()
    ops.call("check_async_errors", stream())
    assert not failures, failures


@pytest.mark.parametrize("rows,prefix,heads,head_dim", [(1, 0, 2, 128), (1, 2048, 2, 128), (9, 0, 3, 8),
                                                       (40, 100, 2, 128), (1, 10240, 1, 128)])
def test_cached_cross_attention(ops, oracle, rows, prefix, heads, head_dim):
    rng = np.random.default_rng(rows + prefix)
    width = heads * head_dim
    total = prefix + rows
    q = rand_bf16(rng, rows, width)
    k, v = rand_bf16(rng, total, width), rand_bf16(rng, total, width)
    out = empty_bits(rows, width)
    ops.call("bf16_cached_cross_attention", p(dev_bits(q)), p(dev_bits(k)), p(dev_bits(v)), rows, total,
             heads, head_dim, p(out), stream())
    expected = np.empty((rows, width), np.uint16)
    oracle.cached_attention(ptr(q), ptr(k), ptr(v), rows, total, heads, head_dim, ptr(expected))
    # same BF16 materialisation points; only F32 summation order differs
    assert_close_bits(host_bits(out), expected, atol=0.01, rtol=0.02, min_cosine=0.9999)


@pytest.mark.parametrize("rows,prefix,heads,head_dim", [(1, 2048, 2, 8), (5, 300, 3, 16), (1, 10240, 2, 8)])
def test_cached_cross_attention_writes_its_probabilities(ops, rows, prefix, heads, head_dim):
    """The BF16 probabilities [heads, rows, keys] upstream materialises between its two GEMMs
    (include/evo/cuda/attention.hpp:131-140), zeros behind the causal boundary, and the same output bits as
    the entry that does not write them.  Reference: the same materialisation points in numpy (BF16 scaled
    keys, BF16 scores, F32 softmax); its sums run in another order, so a probability may differ by one
    BF16 step where the quotient sits on a rounding boundary."""
    rng = np.random.default_rng(prefix + head_dim)
    width, total = heads * head_dim, prefix + rows
    q = rand_bf16(rng, rows, width)
    k, v = rand_bf16(rng, total, width), rand_bf16(rng, total, width)
    out, plain = empty_bits(rows, width), empty_bits(rows, width)
    probabilities = torch.full((heads, rows, total), 0x7fc0, dtype=torch.int16, device="cuda")
    ops.call("bf16_cached_cross_attention_probabilities", p(dev_bits(q)), p(dev_bits(k)), p(dev_bits(v)), rows, total,
             heads, head_dim, p(probabilities), p(out), stream())
    ops.call("bf16_cached_cross_attention", p(dev_bits(q)), p(dev_bits(k)), p(dev_bits(v)), rows, total, heads,
             head_dim, p(plain), stream())
    assert np.array_equal(host_bits(out), host_bits(plain))
    got = bf16_to_f32(probabilities.cpu().numpy().view(np.uint16))
    rbf = lambda x: bf16_to_f32(f32_to_bf16(np.asarray(x, np.float32)))
    scale = np.float32(1.0 / np.sqrt(head_dim))
    qf = bf16_to_f32(q).reshape(rows, heads, head_dim)
    kf = rbf(bf16_to_f32(k).reshape(total, heads, head_dim) * scale)
    for r in range(rows):
        visible = prefix + r + 1
        assert not got[:, r, visible:].any()
        scores = rbf(np.einsum("hd,thd->ht", qf[r].astype(np.float64), kf[:visible].astype(np.float64)))
        e = np.exp(scores - scores.max(axis=1, keepdims=True), dtype=np.float32)
        expected = rbf(e / e.sum(axis=1, keepdims=True, dtype=np.float32))
        # a score on a BF16 rounding boundary (F32 against F64 dot product) moves a probability by ~1 %
        np.testing.assert_allclose(got[:, r, :visible], expected, rtol=0.03, atol=1e-30)
        off = np.abs(got[:, r, :visible] - expected) > 2.0 ** -7 * np.abs(expected)
        assert off.mean() < 1e-3, off.mean()
        np.testing.assert_allclose(got[:, r, :visible].astype(np.float64).sum(axis=1), 1.0, atol=0.01)


def test_attention_rejects_bad_arguments(ops):
    q = empty_bits(4, 256)
    assert ops.status("bf16_causal_attention", p(q), p(q), p(q), 4, 2, 2, 128, p(q), stream()) == 2
    assert ops.status("bf16_split_rope_append", p(q), p(q), 4, 2, 128, 10, 1.0, 0, p(q), p(q), p(q), 8,
                      stream()) == 2
