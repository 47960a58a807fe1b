"""Dense attention through the C ABI against the float64 ruler: the reference's own shape
suite (tests/hardware/ops/test_flash.py, test_flash_key_mask.py, test_flash_fp32_causal.py),
run on each kernel that takes the shape."""

import math

import pytest
import torch

from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, GRAD_BOUND, LSE_RMS, qkv, rel, rms

pytestmark = pytest.mark.gpu

# (b, h, hk, s, d, causal): test_flash.py:18-32.
FORWARD = [
    (1, 2, 2, 32, 32, False), (1, 2, 2, 256, 64, False), (2, 4, 4, 512, 64, True),
    (1, 4, 2, 96, 96, False), (3, 4, 1, 300, 128, False), (1, 4, 4, 1000, 64, False),
    (1, 4, 4, 1000, 64, True), (1, 8, 8, 1024, 128, True), (4, 8, 4, 640, 128, False),
    (1, 16, 4, 1024, 128, True), (8, 16, 16, 256, 64, False), (1, 2, 1, 1100, 256, False),
    (2, 2, 2, 96, 256, True),
]


def _kernels_for(d, dv=None):
    dv = d if dv is None else dv
    if d != dv or d not in (64, 128):
        return ["mma"]
    # Head dim 64 has two tcgen05 forwards: 'flash' (two streams per SM) and 'flash_wide'.
    return ["mma", "flash", "flash_wide"] if d == 64 else ["mma", "flash"]


def _forward(kernel, q, k, v, **kw):
    """Every shape these tests hand the tcgen05 kernel (D == Dv in {64, 128}, aligned
    contiguous operands, no mask or a one-row mask) is one it must take: a refusal raises
    and fails the test."""
    return ops.sdpa_forward(q, k, v, kernel=kernel, **kw)


@pytest.mark.parametrize("b,h,hk,s,d,causal", FORWARD)
def test_forward_shapes(cuda, b, h, hk, s, d, causal):
    q, k, v = qkv(b, h, hk, s, s, d, b + h + s + d)
    ruler = ao.ruler_dense(q, k, v, causal=causal)
    for kernel in _kernels_for(d):
        out, lse = _forward(kernel, q.to(cuda), k.to(cuda), v.to(cuda), causal=causal)
        assert out.shape == ruler.shape and out.dtype == torch.bfloat16
        assert rel(out, ruler) <= FWD_BOUND, kernel
        assert rms(lse, ao.ruler_lse(q, k, v, causal=causal)) <= LSE_RMS, kernel


# (b, h, hk, s, d, kind): test_flash.py:36-41,86-117. Even batches right-padded at 0.7 s,
# odd ones left-padded at 0.4 s.
MASKS = [
    (2, 4, 4, 512, 64, "row"), (2, 4, 4, 256, 64, "head"),
    (2, 8, 2, 1024, 128, "bcast"), (2, 4, 4, 300, 64, "bool"),
]


def _padding_keep(b, s):
    keep = torch.ones(b, s, dtype=torch.bool)
    for i in range(b):
        if i % 2 == 0:
            keep[i, int(0.7 * s):] = False
        else:
            keep[i, :int(0.4 * s)] = False
    return keep


@pytest.mark.parametrize("b,h,hk,s,d,kind", MASKS)
def test_masks(cuda, b, h, hk, s, d, kind):
    q, k, v = qkv(b, h, hk, s, s, d, b + h + s + d + 1)
    keep = _padding_keep(b, s)
    if kind == "bool":
        mask = keep[:, None, None, :]
    else:
        add = torch.zeros(b, s).masked_fill(~keep, -math.inf)
        if kind == "row":
            mask = add[:, None, None, :].expand(b, 1, s, s).contiguous()
        elif kind == "head":
            mask = add[:, None, None, :].expand(b, h, s, s).contiguous()
        else:
            mask = add[:, None, None, :]
    ruler = ao.ruler_dense(q, k, v, mask=mask)
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), mask=mask.to(cuda))
    assert rel(out, ruler) <= FWD_BOUND


# (b, h, hk, sq, sk, d, mb, mh, kind): test_flash_key_mask.py:19-65.
ONE_ROW = [
    (2, 4, 4, 256, 256, 64, 2, 1, "bool"), (2, 8, 2, 197, 197, 64, 2, 1, "bool"),
    (2, 4, 4, 300, 300, 80, 2, 1, "inf"), (1, 4, 4, 33, 1000, 128, 1, 1, "finfo"),
    (2, 4, 4, 128, 160, 64, 1, 4, "values"), (3, 2, 2, 64, 77, 32, 3, 2, "values"),
]


@pytest.mark.parametrize("b,h,hk,sq,sk,d,mb,mh,kind", ONE_ROW)
def test_one_row_masks(cuda, b, h, hk, sq, sk, d, mb, mh, kind):
    q, k, v = qkv(b, h, hk, sq, sk, d, sq + sk + d)
    g = torch.Generator().manual_seed(sq + sk)
    keep = torch.rand(mb, mh, 1, sk, generator=g) > 0.3
    keep[..., 0] = True
    if kind == "bool":
        mask = keep
    elif kind == "inf":
        mask = torch.zeros(mb, mh, 1, sk).masked_fill(~keep, -math.inf)
    elif kind == "finfo":
        mask = torch.zeros(mb, mh, 1, sk).masked_fill(~keep, torch.finfo(torch.bfloat16).min).to(torch.bfloat16)
    else:
        mask = torch.randn(mb, mh, 1, sk, generator=g)
    ruler = ao.ruler_dense(q, k, v, mask=mask if kind != "finfo" else keep)
    # A mask of one row per (batch, head) is also taken by the tcgen05 kernel.
    for kernel in _kernels_for(d):
        out, lse = _forward(kernel, q.to(cuda), k.to(cuda), v.to(cuda), mask=mask.to(cuda))
        assert rel(out, ruler) <= FWD_BOUND, kernel
        assert rms(lse, ao.ruler_lse(q, k, v, mask=mask if kind != "finfo" else keep)) <= LSE_RMS, kernel


@pytest.mark.parametrize("masked_logit", [1e3, 1e4, 3e4, 1e5])
@pytest.mark.parametrize("kind", ["bool", "inf"])
def test_masked_keys_with_huge_logits_get_zero_weight(cuda, masked_logit, kind):
    # test_flash.py:120-145: masked keys hold values whose logits would dominate.
    b, h, s, d = 2, 2, 128, 64
    q, k, v = qkv(b, h, h, s, s, d, int(masked_logit))
    keep = torch.ones(b, 1, 1, s, dtype=torch.bool)
    keep[..., 96:] = False
    k = k.clone()
    k[:, :, 96:] = (q[:, :, :1] * (masked_logit / d)).to(torch.bfloat16).expand(-1, -1, 32, -1)
    mask = keep if kind == "bool" else torch.zeros(b, 1, 1, s).masked_fill(~keep, -math.inf)
    ruler = ao.ruler_dense(q, k, v, mask=mask)
    for kernel in _kernels_for(d):
        out, _ = _forward(kernel, q.to(cuda), k.to(cuda), v.to(cuda), mask=mask.to(cuda))
        assert torch.isfinite(out).all(), kernel
        assert rel(out, ruler) <= FWD_BOUND, kernel


# (b, h, hk, sq, sk, d): top-left causal with Sq != Sk, test_flash_fp32_causal.py:74-104.
RECT = [(1, 4, 4, 1, 77, 64), (2, 8, 2, 64, 300, 64), (1, 4, 4, 300, 128, 80),
        (1, 8, 8, 1024, 512, 64), (1, 2, 2, 300, 290, 64), (1, 2, 2, 290, 300, 64)]


@pytest.mark.parametrize("b,h,hk,sq,sk,d", RECT)
def test_rectangular_causal_is_top_left(cuda, b, h, hk, sq, sk, d):
    q, k, v = qkv(b, h, hk, sq, sk, d, sq + sk)
    ruler = ao.ruler_dense(q, k, v, causal=True)
    for kernel in _kernels_for(d):
        out, _ = _forward(kernel, q.to(cuda), k.to(cuda), v.to(cuda), causal=True)
        assert rel(out, ruler) <= FWD_BOUND, kernel


# (b, h, hk, s, d, causal): test_flash.py:232-254 and the ragged set :259-300.
BACKWARD = [
    (1, 2, 2, 32, 32, False), (2, 4, 4, 256, 64, False), (2, 4, 4, 512, 64, True),
    (1, 8, 2, 512, 128, False), (1, 8, 2, 384, 64, True), (2, 4, 1, 256, 64, False),
    (1, 4, 4, 1024, 128, True), (1, 2, 2, 256, 256, False),
    (1, 2, 2, 40, 32, False), (1, 2, 2, 40, 32, True), (1, 2, 2, 31, 64, False),
    (2, 12, 12, 201, 64, False), (1, 4, 4, 201, 64, True),
]


@pytest.mark.parametrize("b,h,hk,s,d,causal", BACKWARD)
def test_backward_shapes(cuda, b, h, hk, s, d, causal):
    q, k, v, do = qkv(b, h, hk, s, s, d, b + h + s + d + 3, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=causal)
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.sdpa_forward(qc, kc, vc, causal=causal)
    assert rel(out, ruler) <= FWD_BOUND
    for kernel in ("mma", "flash") if d in (64, 128) else ("mma",):
        gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, causal=causal, kernel=kernel)
        assert gk.shape == k.shape and gv.shape == v.shape
        for name, got, want in (("dq", gq, dq), ("dk", gk, dk), ("dv", gv, dv)):
            assert rel(got, want) <= GRAD_BOUND, (kernel, name)


@pytest.mark.parametrize("kernel", ["mma", "flash"])
@pytest.mark.parametrize("d,kind", [(64, "bool"), (128, "bool"), (64, "values")])
def test_masked_backward(cuda, kernel, d, kind):
    # Masked calls train through the same fused backward here (the reference recomputes
    # with separate ops, aten_attention.cpp:781-811): key-padding masks of one row per
    # (batch, head) on both kernel families.
    b, h, hk, s = 2, 4, 2, 200
    q, k, v, do = qkv(b, h, hk, s, s, d, 77 + d, extra=1)
    keep = _padding_keep(b, s)[:, None, None, :]
    mask = keep
    if kind == "values":   # an additive row per (batch, head), -inf where dropped
        mask = torch.randn(b, h, 1, s, generator=torch.Generator().manual_seed(5)).masked_fill(~keep, -math.inf)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, mask=mask)
    qc, kc, vc, doc, mc = (t.to(cuda) for t in (q, k, v, do, mask))
    out, lse = ops.sdpa_forward(qc, kc, vc, mask=mc)
    gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, mask=mc, kernel=kernel)
    for name, got, want in (("dq", gq, dq), ("dk", gk, dk), ("dv", gv, dv)):
        assert rel(got, want) <= GRAD_BOUND, name
    # Keys every row masks get exactly zero gradients (flash.md "exact zeros").
    dropped = ~keep[:, 0, 0, :]
    for i in range(b):
        assert gk[i][:, dropped[i].to(cuda)].abs().max() == 0
        assert gv[i][:, dropped[i].to(cuda)].abs().max() == 0
    torch.cuda.synchronize()
    _lib.device_status()


def test_masks_that_differ_between_rows_train_on_the_general_kernel(cuda):
    b, h, s, d = 1, 2, 130, 64
    q, k, v, do = qkv(b, h, h, s, s, d, 78, extra=1)
    mask = torch.randn(b, 1, s, s, generator=torch.Generator().manual_seed(6))
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, mask=mask)
    qc, kc, vc, doc, mc = (t.to(cuda) for t in (q, k, v, do, mask))
    out, lse = ops.sdpa_forward(qc, kc, vc, mask=mc)
    gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, mask=mc)
    assert rel(out, ruler) <= FWD_BOUND
    for got, want in ((gq, dq), (gk, dk), (gv, dv)):
        assert rel(got, want) <= GRAD_BOUND
    with pytest.raises(_lib.UnsupportedAttention):
        ops.sdpa_backward(doc, qc, kc, vc, out, lse, mask=mc, kernel="flash")


def test_exact_zero_gradients(cuda):
    # test_flash.py:333-346: causal, dO[:, :, 80:] = 0 => dk, dv, dq [:, :, 80:] == 0.
    q, k, v, do = qkv(2, 4, 4, 256, 256, 64, 11, extra=1)
    do = do.clone()
    do[:, :, 80:] = 0
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.sdpa_forward(qc, kc, vc, causal=True)
    for kernel in ("mma", "flash"):
        gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, causal=True, kernel=kernel)
        for g in (gq, gk, gv):
            assert g[:, :, 80:].abs().max() == 0, kernel


def test_no_mixing_across_batch_head_pairs(cuda):
    # test_flash.py:349-361,580-590: V scaled by 1 + pair index; each pair checked alone.
    b, h, s, d = 8, 16, 512, 64
    q, k, v = qkv(b, h, h, s, s, d, 7)
    pair = torch.arange(b * h, dtype=torch.float32).reshape(b, h, 1, 1)
    v = (v.float() * (1 + pair)).to(torch.bfloat16)
    ruler = ao.ruler_dense(q, k, v)
    for kernel in ("mma", "flash"):
        out, _ = _forward(kernel, q.to(cuda), k.to(cuda), v.to(cuda))
        for i in range(0, b, 3):
            for j in range(0, h, 5):
                assert rel(out[i, j], ruler[i, j]) <= FWD_BOUND


def test_head_views_are_read_in_place_and_output_follows(cuda):
    # The pitched route (aten_attention.cpp:605-628): q/k/v as view(B,S,H,D).transpose(1,2)
    # of [B,S,C] storages; the output comes back laid out [B,S,H*Dv].
    b, s, h, d = 2, 300, 10, 64
    x = ao.make_inputs([(b, s, 3 * h * d)], 5)[0]
    qkv_cpu = x.view(b, s, 3, h, d)
    q, k, v = (qkv_cpu[:, :, i].transpose(1, 2) for i in range(3))
    ruler = ao.ruler_dense(q, k, v)
    xc = x.to(cuda).view(b, s, 3, h, d)
    qc, kc, vc = (xc[:, :, i].transpose(1, 2) for i in range(3))
    for kernel in ("mma", "flash"):
        out, _ = _forward(kernel, qc, kc, vc)
        assert out.transpose(1, 2).is_contiguous()
        assert rel(out, ruler) <= FWD_BOUND


def test_other_head_dims(cuda):
    # test_flash_head_pad.py: D in {40, 72, 80, 100, 120, 200}; and Dv != D.
    for d in (40, 72, 80, 100, 120, 200):
        q, k, v = qkv(1, 2, 2, 150, 150, d, d)
        out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda))
        assert rel(out, ao.ruler_dense(q, k, v)) <= FWD_BOUND, d
    q, k, v = qkv(1, 2, 2, 130, 130, 64, 3, dv=32)
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda))
    assert out.shape[-1] == 32 and rel(out, ao.ruler_dense(q, k, v)) <= FWD_BOUND


def test_explicit_scale(cuda):
    q, k, v, do = qkv(1, 4, 2, 160, 160, 64, 36, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, scale=0.05)
    qc, kc, vc, doc = (t.to(cuda) for t in (q, k, v, do))
    out, lse = ops.sdpa_forward(qc, kc, vc, scale=0.05)
    assert rel(out, ruler) <= FWD_BOUND
    gq, gk, gv = ops.sdpa_backward(doc, qc, kc, vc, out, lse, scale=0.05)
    for got, want in ((gq, dq), (gk, dk), (gv, dv)):
        assert rel(got, want) <= GRAD_BOUND


def test_large_logits_stay_finite(cuda):
    # test_flash.py:72-83,559-577.
    q, k, v = qkv(1, 2, 2, 256, 256, 64, 1)
    q = (q.float() * 30).to(torch.bfloat16)
    out, lse = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda))
    assert torch.isfinite(out).all() and torch.isfinite(lse).all()
    assert rel(out, ao.ruler_dense(q, k, v)) <= 2e-2


# Long causal work lists: many key blocks per item and several items per CTA let the two
# softmax groups and the MMA warp drift apart by more than one block, which is what the
# per-buffer barriers of the tcgen05 kernel are for. The full float64 score matrix is too
# large here: whole output against the warp-MMA kernel, sampled rows against float64.
@pytest.mark.parametrize("b,h,hk,s,d", [(2, 16, 16, 4096, 128), (2, 14, 2, 4096, 64)])
def test_long_causal_work_lists(cuda, b, h, hk, s, d):
    q, k, v = qkv(b, h, hk, s, s, d, b + h + s + d)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    for _ in range(3):  # repeated: the drift differs from launch to launch
        out, lse = ops.sdpa_forward(qc, kc, vc, causal=True, kernel="flash")
    torch.cuda.synchronize()
    _lib.device_status()
    ref, ref_lse = ops.sdpa_forward(qc, kc, vc, causal=True, kernel="mma")
    assert rel(out.float(), ref.float()) <= 4e-3
    assert (lse - ref_lse).abs().max().item() <= 2e-3
    rows = torch.tensor([0, 1, 127, 128, 1000, 2047, 2048, 3000, s - 1])
    group = h // hk
    for bi, hi in ((0, 0), (b - 1, h - 1)):
        kk, vv = k[bi, hi // group].double(), v[bi, hi // group].double()
        scores = (q[bi, hi, rows].double() @ kk.T) / math.sqrt(d)
        scores = scores.masked_fill(torch.arange(s)[None, :] > rows[:, None], float("-inf"))
        ruler = torch.softmax(scores, dim=-1) @ vv
        assert rel(out[bi, hi, rows.to(cuda)].cpu(), ruler) <= FWD_BOUND


def test_counter_driven_work_gives_the_same_bits(cuda):
    """Which CTA draws an item does not touch the item's arithmetic: with the work counter
    the one-CTA-per-SM tcgen05 forward returns exactly what the fixed deal returns (dense,
    packed-style ragged sizes)."""
    old = ops.dynamic_work(False)
    try:
        for b, h, hk, s, d, causal in [(2, 8, 2, 1000, 64, True), (1, 16, 16, 2048, 128, True), (3, 4, 4, 300, 64, False)]:
            q, k, v = (t.to(cuda) for t in qkv(b, h, hk, s, s, d, b + h + s + d))
            kernel = "flash_wide" if d == 64 else "flash"
            want, want_lse = ops.sdpa_forward(q, k, v, causal=causal, kernel=kernel)
            ops.dynamic_work(True, 0)
            got, got_lse = ops.sdpa_forward(q, k, v, causal=causal, kernel=kernel)
            ops.dynamic_work(False)
            again, _ = ops.sdpa_forward(q, k, v, causal=causal, kernel=kernel, dynamic=True)
            assert torch.equal(got, want) and torch.equal(got_lse, want_lse) and torch.equal(again, want)
        torch.cuda.synchronize()
        _lib.device_status()
    finally:
        ops.dynamic_work(old["on"], old["min_items_per_sm"])


# The reference's bench shapes (src/kohakutt/bench/ops.py:189-209): [3, 24, s, 128], plain and
# causal, judged by their statistics against float64 (on two (batch, head) pairs: the full
# float64 score matrices of the longest shape would not fit).
@pytest.mark.parametrize("s", [279, 1043, 1615, 4379])
@pytest.mark.parametrize("causal", [False, True])
def test_bench_shapes_statistics(cuda, s, causal):
    import kohaku_tt_b200 as ktt

    q, k, v = qkv(3, 24, 24, s, s, 128, 0)
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), causal=causal)
    for bi, hi in ((0, 0), (2, 23)):
        sl = (slice(bi, bi + 1), slice(hi, hi + 1))
        ruler = ao.ruler_dense(q[sl], k[sl], v[sl], causal=causal)
        st = ktt.diff_stats(out[sl], ruler)
        assert st["nonfinite"] == 0 and st["rel_median"] <= 1e-2 and st["abs_max"] <= 2e-2, (s, causal, st)
