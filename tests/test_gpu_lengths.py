"""Key lengths and decode through the C ABI: tests/hardware/ops/test_attention_lengths.py
and test_flash_kv_lengths.py, with the split-K decode kernel checked against both the
float64 ruler and the general kernel."""

import pytest
import torch

import kohaku_tt_b200 as ktt
from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, qkv, rel

pytestmark = pytest.mark.gpu

# (B, H, Hk, S, D, lengths, causal): test_attention_lengths.py:16-35.
CASES = [
    (4, 2, 2, 33, 32, [1, 32, 33, 17], False), (4, 2, 2, 33, 32, [1, 32, 33, 17], True),
    (2, 4, 2, 197, 64, [197, 64], False), (4, 4, 2, 70, 64, [1, 33, 70, 64], True),
    (3, 2, 2, 128, 64, [96, 1, 128], False),
]


@pytest.mark.parametrize("b,h,hk,s,d,lengths,causal", CASES)
def test_key_lengths_forward_and_gradients(cuda, b, h, hk, s, d, lengths, causal):
    q, k, v, do = qkv(b, h, hk, s, s, d, 40 + b + s, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, lengths=lengths, causal=causal)
    qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
    out = ktt.sdpa(qc, kc, vc, key_lengths=lengths, is_causal=causal)
    assert rel(out, ruler) <= FWD_BOUND
    out.backward(do.to(cuda))
    for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
        assert rel(got, want) <= 2.5e-2
    for i, n in enumerate(lengths):  # exact zeros past each length
        if n < s:
            assert kc.grad[i, :, n:].abs().max() == 0
            assert vc.grad[i, :, n:].abs().max() == 0


def test_garbage_past_the_lengths_changes_nothing(cuda):
    # test_attention_lengths.py:107-124: inf past the lengths => bit-equal outputs.
    b, h, hk, s, d, lengths = 3, 4, 2, 128, 64, [96, 1, 128]
    q, k, v = qkv(b, h, hk, s, s, d, 5)
    k2, v2 = k.clone(), v.clone()
    for i, n in enumerate(lengths):
        k2[i, :, n:] = float("inf")
        v2[i, :, n:] = float("inf")
    ln = torch.tensor(lengths, dtype=torch.int32, device=cuda)
    a = ktt.sdpa(q.to(cuda), k.to(cuda), v.to(cuda), key_lengths=ln)
    b_ = ktt.sdpa(q.to(cuda), k2.to(cuda), v2.to(cuda), key_lengths=ln)
    assert torch.equal(a, b_)
    # Each forward kernel by name (the tcgen05 one blanks the value rows past a length in
    # its tile; NaN there as well), causal and not, against the float64 ruler too.
    v3 = v2.clone()
    for i, n in enumerate(lengths):
        v3[i, :, n:] = float("nan")
    for kernel in ("mma", "flash"):
        for causal in (False, True):
            clean, lse = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), key_lengths=ln, causal=causal, kernel=kernel)
            dirty, lse2 = ops.sdpa_forward(q.to(cuda), k2.to(cuda), v3.to(cuda), key_lengths=ln, causal=causal, kernel=kernel)
            assert torch.equal(clean, dirty) and torch.equal(lse, lse2), (kernel, causal)
            assert rel(clean, ao.ruler_lengths(q, k, v, lengths, causal=causal)) <= FWD_BOUND, (kernel, causal)
    # Decode shape (one query row): the split-K kernel.
    q1 = q[:, :, :1].contiguous()
    a = ktt.sdpa(q1.to(cuda), k.to(cuda), v.to(cuda), key_lengths=ln)
    b_ = ktt.sdpa(q1.to(cuda), k2.to(cuda), v2.to(cuda), key_lengths=ln)
    assert torch.equal(a, b_)


@pytest.mark.parametrize("kernel", ["mma", "flash"])
@pytest.mark.parametrize("d,causal", [(64, False), (128, True)])
def test_key_length_gradients_on_each_kernel_ignore_garbage(cuda, kernel, d, causal):
    """Gradients with key lengths on the warp-MMA and on the tcgen05 backward: against
    float64, exact zeros past each length, and bit-equal when the cache holds inf / NaN past
    the lengths (test_attention_lengths.py:107-124 carried to the backward)."""
    b, h, hk, s, lengths = 3, 4, 2, 300, [300, 1, 170]
    q, k, v, do = qkv(b, h, hk, s, s, d, 50 + d, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, lengths=lengths, causal=causal)
    ln = torch.tensor(lengths, dtype=torch.int32, device=cuda)
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.sdpa_forward(qc, kc, vc, key_lengths=ln, causal=causal)
    gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, key_lengths=ln, causal=causal, kernel=kernel)
    for name, got, want in (("dq", gq, dq), ("dk", gk, dk), ("dv", gv, dv)):
        assert rel(got, want) <= 2.5e-2, name
    k2, v2 = k.clone(), v.clone()
    for i, n in enumerate(lengths):
        if n < s:
            assert gk[i, :, n:].abs().max() == 0 and gv[i, :, n:].abs().max() == 0
        k2[i, :, n:] = float("inf")
        v2[i, :, n:] = float("nan")
    hq, hk_, hv = ops.sdpa_backward(doc, qc, k2.to(cuda), v2.to(cuda), out, lse, key_lengths=ln, causal=causal, kernel=kernel)
    assert torch.equal(hq, gq) and torch.equal(hk_, gk) and torch.equal(hv, gv)
    torch.cuda.synchronize()
    _lib.device_status()


def test_full_lengths_equal_plain_attention(cuda):
    # test_attention_lengths.py:127-139 (same kernel, so bit for bit).
    q, k, v = qkv(2, 4, 2, 197, 197, 64, 6)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    plain, _ = ops.sdpa_forward(qc, kc, vc, kernel="mma")
    full, _ = ops.sdpa_forward(qc, kc, vc, key_lengths=torch.full((2,), 197, dtype=torch.int32, device=cuda),
                               kernel="mma")
    assert torch.equal(plain, full)
    plain, _ = ops.sdpa_forward(qc, kc, vc, kernel="flash")
    full, _ = ops.sdpa_forward(qc, kc, vc, key_lengths=torch.full((2,), 197, dtype=torch.int32, device=cuda),
                               kernel="flash")
    assert torch.equal(plain, full)


def test_bad_lengths_raise(cuda):
    # test_attention_lengths.py:169-174.
    q, k, v = (t.to(cuda) for t in qkv(2, 2, 2, 16, 16, 32, 1))
    with pytest.raises(ValueError):
        ktt.sdpa(q, k, v, key_lengths=[0, 4])
    with pytest.raises(ValueError):
        ktt.sdpa(q, k, v, key_lengths=[1, 17])
    with pytest.raises(ValueError):
        ktt.sdpa(q, k, v, key_lengths=[1, 2, 3])


# Decode with a growing KV length: test_flash_kv_lengths.py:22-56.
@pytest.mark.parametrize("hk,d,sq", [(8, 64, 1), (2, 128, 1), (8, 64, 16)])
def test_decode_growing_kv(cuda, hk, d, sq):
    b, h, cap = 2, 8, 512
    q, k, v = qkv(b, h, hk, sq, cap, d, d + hk)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    before = ktt.counters()["attention_decode"]
    for n in (100, 101, 127, 128, 129, 383, 384, 385, 417, 500):
        ln = torch.full((b,), n, dtype=torch.int32, device=cuda)
        out = ktt.sdpa(qc, kc, vc, key_lengths=ln)
        ruler = ao.ruler_dense(q, k[:, :, :n], v[:, :, :n])
        assert rel(out, ruler) <= FWD_BOUND, n
    grouped_rows = (h // hk) * sq
    if grouped_rows <= 16:
        assert ktt.counters()["attention_decode"] == before + 10


# (b, h, hk, sq, sk, causal): test_flash_kv_lengths.py:78-98.
@pytest.mark.parametrize("b,h,hk,sq,sk,causal", [
    (1, 14, 14, 1, 500, False), (2, 32, 8, 1, 700, False), (1, 8, 8, 16, 200, True),
    (1, 4, 4, 8, 5, True), (1, 4, 4, 64, 20, True),
])
def test_decode_lanes(cuda, b, h, hk, sq, sk, causal):
    q, k, v = qkv(b, h, hk, sq, sk, 64, sk)
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal)
    assert rel(out, ao.ruler_dense(q, k, v, causal=causal)) <= FWD_BOUND
    if not causal:
        dec, _ = ops.decode(q.to(cuda), k.to(cuda), v.to(cuda))
        assert rel(dec, ao.ruler_dense(q, k, v)) <= FWD_BOUND


def test_decode_random_lengths_match_the_general_kernel(cuda):
    """The benchmark's decode shape, reduced: GQA 16 / 2, D 128, random lengths; the
    split-K kernel against the float64 ruler and against the general kernel."""
    b, h, hk, d, cap = 16, 16, 2, 128, 1024
    q, k, v = qkv(b, h, hk, 1, cap, d, 0)
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(1, cap + 1, (b,), generator=g, dtype=torch.int32)
    lengths[0], lengths[1], lengths[2] = 1, cap, 64
    qc, kc, vc, ln = q.to(cuda), k.to(cuda), v.to(cuda), lengths.to(cuda)
    out, lse = ops.decode(qc, kc, vc, key_lengths=ln, need_lse=True)
    ruler = ao.ruler_lengths(q, k, v, lengths)
    assert rel(out, ruler) <= FWD_BOUND
    general, glse = ops.sdpa_forward(qc, kc, vc, key_lengths=ln, kernel="mma")
    assert (out.float() - general.float()).abs().max() <= 2e-2
    assert (lse - glse).abs().max() <= 1e-3
    for splits in (1, 2, 7):
        again, _ = ops.decode(qc, kc, vc, key_lengths=ln, splits=splits)
        assert rel(again, ruler) <= FWD_BOUND, splits
    # Run to run the kernel is deterministic (fixed merge order, no atomics).
    assert torch.equal(out, ops.decode(qc, kc, vc, key_lengths=ln)[0])


def test_decode_without_lengths_and_strided_cache(cuda):
    b, h, hk, d, cap = 3, 8, 2, 64, 300
    q, k, v = qkv(b, h, hk, 2, cap, d, 9)
    big_k = torch.zeros(b, hk, cap + 40, d, dtype=torch.bfloat16, device=cuda)
    big_v = torch.zeros_like(big_k)
    big_k[:, :, :cap], big_v[:, :, :cap] = k.to(cuda), v.to(cuda)
    out, _ = ops.decode(q.to(cuda), big_k[:, :, :cap], big_v[:, :, :cap])
    assert rel(out, ao.ruler_dense(q, k, v)) <= FWD_BOUND
    with pytest.raises(_lib.UnsupportedAttention):
        ops.decode(q.to(cuda)[..., :32], big_k[..., :32], big_v[..., :32])


def test_decode_calls_of_different_shapes_share_one_scratch(cuda):
    """The cached scratch is reused by calls of any shape: the ticket counters sit in a
    fixed area that no call's partials reach."""
    shapes = [(5, 4, 4, 200, 64), (64, 16, 2, 1024, 128), (3, 14, 2, 300, 64), (64, 16, 2, 1024, 128)]
    for i, (b, h, hk, smax, d) in enumerate(shapes):
        q, k, v = ao.make_inputs([(b, h, 1, d), (b, hk, smax, d), (b, hk, smax, d)], 40 + i)
        lengths = torch.randint(1, smax + 1, (b,), generator=torch.Generator().manual_seed(i)).tolist()
        n = torch.tensor(lengths, dtype=torch.int32, device=cuda)
        out, _ = ops.decode(q.to(cuda), k.to(cuda), v.to(cuda), key_lengths=n)
        assert rel(out, ao.ruler_lengths(q, k, v, lengths)) <= FWD_BOUND, (i, b, h)
