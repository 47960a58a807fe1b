"""Packed variable-length attention through the C ABI against the per-sequence float64
loop: the reference's suites tests/hardware/ops/test_flash_varlen.py and
test_flash_varlen_gaps.py."""

import pytest
import torch

import kohaku_tt_b200 as ktt
from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, VARLEN_GRAD_BOUND, cu, cumulative, packed, rel

pytestmark = pytest.mark.gpu

MIXED = [1, 31, 33, 5, 64, 100]
# (lengths, h, hk, d, causal): test_flash_varlen.py:18-43.
FORWARD = [
    ([32], 1, 1, 32, False), ([40], 1, 1, 32, False), (MIXED, 2, 2, 64, False),
    (MIXED, 4, 2, 64, True), ([3] * 50, 2, 1, 64, True), ([32, 64, 96], 4, 4, 128, False),
    ([32, 64, 96], 4, 4, 128, True), ([201] * 8, 12, 12, 64, False),
    ([700, 13, 1500], 4, 2, 64, True), ([700, 13, 1500], 4, 2, 64, False),
    (MIXED, 2, 2, 96, True), ([40], 2, 2, 256, False), ([201] * 8, 4, 1, 128, True),
]


def _run_forward(cuda, q, k, v, lq, lk, causal, kernel="auto", **kw):
    return ops.varlen_forward(q.to(cuda), k.to(cuda), v.to(cuda), cu(lq, cuda), cu(lk, cuda),
                              max(lq), max(lk), causal=causal, kernel=kernel, **kw)


@pytest.mark.parametrize("lengths,h,hk,d,causal", FORWARD)
def test_forward_sets(cuda, lengths, h, hk, d, causal):
    q, k, v = packed(lengths, lengths, h, hk, d, len(lengths) + h + d)
    c = cumulative(lengths)
    ruler = ao.ruler_varlen(q, k, v, c, c, causal=causal)
    kernels = ["mma", "flash"] if d in (64, 128) else ["mma"]
    for kernel in kernels:
        # Packed D 64 / 128 operands are aligned: a tcgen05 refusal raises and fails here.
        out, lse = _run_forward(cuda, q, k, v, lengths, lengths, causal, kernel)
        assert out.shape == ruler.shape
        assert rel(out, ruler) <= FWD_BOUND, kernel
        for b in range(len(lengths)):  # per sequence: 3e-2 (test_flash_varlen.py:86-93)
            sl = slice(c[b], c[b + 1])
            assert rel(out[sl], ruler[sl]) <= 3e-2, (kernel, b)


def test_lse_layout_and_values(cuda):
    # test_flash_varlen.py:314-341: [H, Tq] against float64 logsumexp, max abs 3e-2.
    lengths = MIXED
    q, k, v = packed(lengths, lengths, 4, 2, 64, 7)
    c = cumulative(lengths)
    for causal in (False, True):
        out, lse = _run_forward(cuda, q, k, v, lengths, lengths, causal)
        want = ao.lse_varlen(q, k, v, c, c, causal=causal)
        assert lse.shape == (4, sum(lengths))
        assert (lse.cpu().double() - want).abs().max() <= 3e-2


def test_different_key_offsets(cuda):
    # test_flash_varlen.py:171-184 and the gaps file: cu_seq_k != cu_seq_q, causal Lk > Lq.
    lq, lk = [40, 7, 90], [50, 20, 100]
    q, k, v = packed(lq, lk, 2, 2, 64, 33)
    for causal in (False, True):
        ruler = ao.ruler_varlen(q, k, v, cumulative(lq), cumulative(lk), causal=causal)
        out, _ = _run_forward(cuda, q, k, v, lq, lk, causal)
        assert rel(out, ruler) <= FWD_BOUND


def test_neighbours_do_not_matter(cuda):
    # test_flash_varlen.py:118-135,269-284: replace every other sequence's data; the kept
    # sequences' outputs and gradients are bit-identical.
    lengths = [5, 40, 3, 33, 70, 1, 31]
    c = cumulative(lengths)
    q, k, v, do = packed(lengths, lengths, 2, 2, 64, 11, extra=1)
    q2, k2, v2, do2 = packed(lengths, lengths, 2, 2, 64, 12, extra=1)
    keep = [1, 3, 5]
    for t, t2 in ((q, q2), (k, k2), (v, v2), (do, do2)):
        for b in keep:
            t2[c[b]:c[b + 1]] = t[c[b]:c[b + 1]]
    results = []
    for tq, tk, tv, tdo in ((q, k, v, do), (q2, k2, v2, do2)):
        tq, tk, tv, tdo = (t.to(cuda) for t in (tq, tk, tv, tdo))
        out, lse = ops.varlen_forward(tq, tk, tv, cu(lengths, cuda), cu(lengths, cuda),
                                      max(lengths), max(lengths), causal=True)
        grads = ops.varlen_backward(tdo, tq, tk, tv, out, lse, cu(lengths, cuda), cu(lengths, cuda),
                                    max(lengths), max(lengths), causal=True)
        results.append((out, *grads))
    for a, b_ in zip(*results):
        for b in keep:
            assert torch.equal(a[c[b]:c[b + 1]], b_[c[b]:c[b + 1]])


# (lq, lk, h, hk, d, causal): test_flash_varlen.py:188-248.
BACKWARD = [
    ([32], None, 1, 1, 32, False), ([40], None, 1, 1, 32, False),
    (MIXED, None, 2, 2, 64, False), (MIXED, None, 4, 2, 64, True),
    ([3] * 50, None, 2, 1, 64, True), ([40, 7, 90], [25, 70, 33], 2, 2, 64, False),
    ([40, 0, 90], [25, 70, 33], 2, 1, 64, False), ([201] * 8, None, 12, 12, 64, False),
    ([700, 13, 1500], None, 2, 2, 64, True),
]


@pytest.mark.parametrize("lq,lk,h,hk,d,causal", BACKWARD)
def test_backward_sets(cuda, lq, lk, h, hk, d, causal):
    lk = lq if lk is None else lk
    q, k, v, do = packed(lq, lk, h, hk, d, len(lq) + h + d, extra=1)
    cq, ck = cumulative(lq), cumulative(lk)
    ruler, dq, dk, dv = ao.ruler_varlen(q, k, v, cq, ck, causal=causal, dout=do)
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.varlen_forward(qc, kc, vc, cu(lq, cuda), cu(lk, cuda), max(lq), max(lk), causal=causal)
    assert rel(out, ruler) <= FWD_BOUND
    for kernel in (["mma", "flash"] if d in (64, 128) else ["mma"]):
        gq, gk, gv = ops.varlen_backward(doc, qc, kc, vc, out, lse, cu(lq, cuda), cu(lk, cuda),
                                         max(lq), max(lk), causal=causal, kernel=kernel)
        for name, got, want in (("dq", gq, dq), ("dk", gk, dk), ("dv", gv, dv)):
            assert rel(got, want) <= VARLEN_GRAD_BOUND, (kernel, name)
        for b, n in enumerate(lq):
            if n == 0:  # a sequence without queries: its keys get exact zeros
                assert gk[ck[b]:ck[b + 1]].abs().max() == 0
                assert gv[ck[b]:ck[b + 1]].abs().max() == 0


def _poison_free_memory(cuda, like):
    """Leaves NaN patterns in freed blocks the size of the gradients, so that a row the
    backward does not write shows (torch.empty hands such blocks back)."""
    junk = [torch.full(t.shape, float("nan"), dtype=t.dtype, device=cuda) for t in like for _ in range(2)]
    torch.cuda.synchronize()
    del junk


@pytest.mark.parametrize("kernel", ["mma", "flash"])
def test_rows_outside_the_offsets_get_zero_gradients(cuda, kernel):
    # The gradients are not cleared by the caller: rows of sequences are written by their
    # owners, rows before the first offset and after the last are zeroed by the library.
    lq, lk = [40, 0, 90], [25, 70, 33]
    q, k, v, do = packed(lq + [17], lk + [9], 2, 1, 64, 77, extra=1)   # 17 / 9 rows no offset covers
    cq, ck = cumulative(lq), cumulative(lk)
    tq, tk = cq[-1], ck[-1]
    _, dq, dk, dv = ao.ruler_varlen(q[:tq], k[:tk], v[:tk], cq, ck, causal=False, dout=do[:tq])
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.varlen_forward(qc, kc, vc, cu(lq, cuda), cu(lk, cuda), max(lq), max(lk), kernel=kernel)
    _poison_free_memory(cuda, (qc, kc, vc))
    gq, gk, gv = ops.varlen_backward(doc, qc, kc, vc, out, lse, cu(lq, cuda), cu(lk, cuda),
                                     max(lq), max(lk), kernel=kernel)
    torch.cuda.synchronize()
    _lib.device_status()
    for got, want, n in ((gq, dq, tq), (gk, dk, tk), (gv, dv, tk)):
        assert torch.isfinite(got.float()).all()
        assert rel(got[:n], want) <= VARLEN_GRAD_BOUND
        assert got[n:].abs().max() == 0
    assert gk[ck[1]:ck[2]].abs().max() == 0 and gv[ck[1]:ck[2]].abs().max() == 0


def test_edge_sets(cuda):
    # test_flash_varlen_gaps.py:120-308: one long sequence, a long + short pair, Dv != D,
    # an explicit scale, 40 different lengths.
    for lengths, d, dv, causal, scale in (
        ([4200], 64, 64, False, None), ([4100, 100], 64, 64, True, None),
        ([70, 33], 64, 32, False, None), ([70, 33], 32, 128, True, None),
        ([130, 61], 256, 256, True, None), ([90, 41], 64, 64, False, 0.05),
        (list(range(33, 73)), 64, 64, True, None),
    ):
        q, k, v = packed(lengths, lengths, 2, 2, d, 31 + len(lengths), dv=dv)
        c = cumulative(lengths)
        ruler = ao.ruler_varlen(q, k, v, c, c, causal=causal, scale=scale)
        out, _ = ops.varlen_forward(q.to(cuda), k.to(cuda), v.to(cuda), cu(lengths, cuda),
                                    cu(lengths, cuda), max(lengths), max(lengths), causal=causal,
                                    scale=scale)
        assert rel(out, ruler) <= FWD_BOUND, (lengths[:3], d, dv)


def test_key_mask(cuda):
    # test_flash_varlen.py:398-458: a key mask [Tk], bool or additive, with gradients.
    lengths = [40, 7, 90]
    c = cumulative(lengths)
    q, k, v, do = packed(lengths, lengths, 2, 2, 64, 21, extra=1)
    g = torch.Generator().manual_seed(3)
    keep = torch.rand(sum(lengths), generator=g) > 0.3
    for b in range(3):
        keep[c[b]] = True
    add = torch.randn(sum(lengths), generator=g)
    for mask in (keep, add):
        ruler, dq, dk, dv = ao.ruler_varlen(q, k, v, c, c, key_mask=mask, dout=do)
        qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
        out = ktt.sdpa_varlen(qc, kc, vc, c, attn_mask=mask)
        assert rel(out, ruler) <= FWD_BOUND
        out.backward(do.to(cuda))
        for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
            assert rel(got, want) <= VARLEN_GRAD_BOUND


def test_rejections(cuda):
    # test_flash_varlen.py:525-534.
    q = torch.zeros(9, 2, 64, dtype=torch.bfloat16, device=cuda)
    with pytest.raises(RuntimeError):
        ktt.sdpa_varlen(q, q, q, [0, 4, 8])
    with pytest.raises(ValueError):
        ktt.sdpa_varlen(q, q, q, [0, 4, 9], attn_mask=torch.ones(2, 9, device=cuda))
    with pytest.raises(ValueError):
        ktt.sdpa_varlen(q, q, q, [0, 4, 9], attn_mask=torch.ones(8, device=cuda))
