"""The head-dim-64 forward kernel (two streams per SM; on small launches the two streams of
a CTA share a query tile, half of its key blocks each) against the float64 ruler and the
warp-MMA kernel, at the benchmark's own sizes."""

import math

import pytest
import torch

from kohaku_tt_b200 import _lib, ops
from tests.gpu_util import FWD_BOUND, LSE_RMS, qkv, rel, rms

pytestmark = pytest.mark.gpu


def _sampled_rows_ruler(q, k, v, bi, hi, rows, causal):
    """float64 attention of a few query rows of one (batch, head)."""
    group = q.shape[1] // k.shape[1]
    kk, vv = k[bi, hi // group].double(), v[bi, hi // group].double()
    scores = (q[bi, hi, rows].double() @ kk.T) / math.sqrt(q.shape[-1])
    if causal:
        scores = scores.masked_fill(torch.arange(k.shape[2])[None, :] > rows[:, None], float("-inf"))
    return torch.softmax(scores, dim=-1) @ vv, torch.logsumexp(scores, dim=-1)


def test_two_streams_fit_one_sm(cuda):
    assert _lib.lib().ktt_b200_forward_streams_per_sm() == 2


# (b, h, hk, s, causal): the headline shape (tiles are cut: 224 tiles on 296 CTA slots), its
# batch-8 form (whole tiles, several per CTA), SDXL self-attention's shape, ragged sizes.
@pytest.mark.parametrize("b,h,hk,s,causal", [
    (1, 14, 2, 2048, True), (8, 14, 2, 2048, True), (2, 10, 10, 4096, False),
    (1, 4, 4, 1000, True), (3, 4, 1, 300, False), (1, 2, 2, 129, True),
])
def test_against_the_warp_mma_kernel_and_float64_rows(cuda, b, h, hk, s, causal):
    q, k, v = qkv(b, h, hk, s, s, 64, b + h + s)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    for _ in range(3):  # repeated: which CTA draws which unit differs from launch to launch
        out, lse = ops.sdpa_forward(qc, kc, vc, causal=causal, kernel="flash")
    torch.cuda.synchronize()
    _lib.device_status()
    ref, ref_lse = ops.sdpa_forward(qc, kc, vc, causal=causal, kernel="mma")
    assert rel(out.float(), ref.float()) <= 4e-3
    assert (lse - ref_lse).abs().max().item() <= 2e-3
    rows = torch.tensor(sorted({0, 1, 127, 128, s // 2, s - 129 if s > 129 else 0, s - 1}))
    for bi, hi in ((0, 0), (b - 1, h - 1)):
        ruler, ruler_lse = _sampled_rows_ruler(q, k, v, bi, hi, rows, causal)
        assert rel(out[bi, hi, rows.to(cuda)].cpu(), ruler) <= FWD_BOUND
        assert rms(lse[bi, hi, rows.to(cuda)], ruler_lse) <= LSE_RMS


def _full_ruler(q, k, v, causal):
    """float64 attention of every row (small sizes)."""
    group = q.shape[1] // k.shape[1]
    kk = k.double().repeat_interleave(group, dim=1)
    vv = v.double().repeat_interleave(group, dim=1)
    scores = q.double() @ kk.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if causal:
        sq, sk = q.shape[2], k.shape[2]
        hidden = torch.arange(sk)[None, :] > torch.arange(sq)[:, None] + (sk - sq)
        scores = scores.masked_fill(hidden, float("-inf"))
    return torch.softmax(scores, dim=-1) @ vv, torch.logsumexp(scores, dim=-1)


# How the keys' magnitude runs along the sequence. The kernel rescales a row's running sum
# and output lazily, only when a block's maximum exceeds the reference by more than 2^8, and
# the row's two threads agree on each block's maximum through a 16-bit exchange. `rising` and
# `steps` move the reference in every block by hundreds, `falling` leaves the first reference
# far above everything after it, `spike` puts one huge key in the middle of a late block,
# `halves` makes the two threads of a row see very different maxima.
@pytest.mark.parametrize("profile", ["rising", "falling", "steps", "spike", "halves"])
@pytest.mark.parametrize("s,causal", [(640, False), (640, True), (2048, True)])
def test_references_that_move_inside_a_block(cuda, profile, s, causal):
    q, k, v = qkv(1, 4, 2, s, s, 64, 11 + s)
    pos = torch.arange(s, dtype=torch.float32)
    if profile == "rising":
        gain = 1.0 + pos * (60.0 / s)
    elif profile == "falling":
        gain = 60.0 - pos * (59.0 / s)
    elif profile == "steps":
        gain = 1.0 + 40.0 * ((pos // 16) % 5)
    elif profile == "spike":
        gain = torch.ones(s)
        gain[s - 150] = 300.0
        gain[200] = 80.0
    else:
        gain = torch.where((pos // 64) % 2 == 1, 50.0, 1.0)
    k = (k.float() * gain[None, None, :, None]).to(torch.bfloat16)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    out, lse = ops.sdpa_forward(qc, kc, vc, causal=causal, kernel="flash")
    again, again_lse = ops.sdpa_forward(qc, kc, vc, causal=causal, kernel="flash", dynamic=False)
    torch.cuda.synchronize()
    _lib.device_status()
    assert torch.equal(out, again) and torch.equal(lse, again_lse)
    assert torch.isfinite(out.float()).all() and torch.isfinite(lse).all()
    ruler, ruler_lse = _full_ruler(q, k, v, causal)
    assert rel(out.cpu(), ruler) <= FWD_BOUND
    # lse grows with the logits here (hundreds): compare relative to its size.
    assert ((lse.cpu().double() - ruler_lse).abs() / ruler_lse.abs().clamp_min(1.0)).max().item() <= 1e-5
    ref, _ = ops.sdpa_forward(qc, kc, vc, causal=causal, kernel="mma")
    assert rel(out.float(), ref.float()) <= 4e-3


def test_shared_tiles_give_the_same_bits_every_time(cuda):
    # 224 tiles on 148 SMs: every tile is shared by the two streams of a CTA. Which CTA draws
    # which tile differs from launch to launch; the bits must not.
    q, k, v = (t.to(cuda) for t in qkv(1, 14, 2, 2048, 2048, 64, 5))
    first, first_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    for _ in range(6):
        out, lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
        assert torch.equal(out, first) and torch.equal(lse, first_lse)
    # The fixed deal (no workspace) shares the tiles the same way: the same bits again.
    fixed, fixed_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash", dynamic=False)
    assert torch.equal(fixed, first) and torch.equal(fixed_lse, first_lse)
    torch.cuda.synchronize()
    _lib.device_status()


def test_drawn_work_equals_the_fixed_deal_for_whole_tiles(cuda):
    # 1,792 tiles: each stream takes whole tiles; who draws a tile does not touch its arithmetic.
    q, k, v = (t.to(cuda) for t in qkv(8, 14, 2, 2048, 2048, 64, 6))
    drawn, drawn_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    fixed, fixed_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash", dynamic=False)
    assert torch.equal(drawn, fixed) and torch.equal(drawn_lse, fixed_lse)


def test_fixed_deal_is_reproducible_over_thousands_of_tiles(cuda):
    # 4,096 tiles without a workspace: every stream walks its own list of tiles and the warps
    # of a stream drift apart by up to a tile. What two warps exchange through shared memory
    # must stay inside their own words whatever the others do (the row sums of one pair of
    # warps once lay over the maxima of another pair: sixteen rows of a tile in a few hundred
    # came out wrong, differently on every run). Two runs give the same bits, and the same
    # bits as the drawn order.
    g = torch.Generator(device=cuda).manual_seed(11)
    q, k, v = (torch.randn((8, 16, 4096, 64), generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16) for _ in range(3))
    first, first_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash", dynamic=False)
    second, second_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash", dynamic=False)
    drawn, drawn_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    torch.cuda.synchronize()
    _lib.device_status()
    assert torch.equal(first, second) and torch.equal(first_lse, second_lse)
    assert torch.equal(first, drawn) and torch.equal(first_lse, drawn_lse)


@pytest.mark.parametrize("d", [64, 128])
def test_tiles_grouped_by_kv_head_when_kv_exceeds_l2(cuda, d):
    # 268 MB of K / V: with a workspace the tiles of one (batch, head)
    # are drawn together so that those in flight share K / V in L2. The order a tile is drawn
    # in does not touch its arithmetic: the same bits as the fixed deal, and float64 rows.
    b, h, s = (8 if d == 64 else 4), 16, 8192
    g = torch.Generator(device=cuda).manual_seed(3 + d)
    q, k, v = (torch.randn((b, h, s, d), generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16) for _ in range(3))
    out, lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    again, again_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    fixed, fixed_lse = ops.sdpa_forward(q, k, v, causal=True, kernel="flash", dynamic=False)
    torch.cuda.synchronize()
    _lib.device_status()
    assert torch.equal(out, again) and torch.equal(lse, again_lse)
    assert torch.equal(out, fixed) and torch.equal(lse, fixed_lse)
    rows = torch.tensor([0, 127, 128, 4095, 8191])
    for bi, hi in ((0, 0), (b - 1, h - 1)):
        kk, vv = k[bi, hi].double().cpu(), v[bi, hi].double().cpu()
        scores = (q[bi, hi].cpu()[rows].double() @ kk.T) / math.sqrt(d)
        scores = scores.masked_fill(torch.arange(s)[None, :] > rows[:, None], float("-inf"))
        ruler = torch.softmax(scores, dim=-1) @ vv
        assert rel(out[bi, hi].cpu()[rows], ruler) <= FWD_BOUND
        assert rms(lse[bi, hi].cpu()[rows], torch.logsumexp(scores, dim=-1)) <= LSE_RMS


def test_the_workspace_is_left_zeroed(cuda):
    q, k, v = (t.to(cuda) for t in qkv(1, 14, 2, 2048, 2048, 64, 7))
    ops.drop_forward_workspaces()
    ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    torch.cuda.synchronize()
    (buf,) = ops._FORWARD_WORKSPACE.values()
    assert int(buf.to(torch.int32).abs().sum()) == 0


def test_key_lengths_and_one_row_masks_on_shared_tiles(cuda):
    import kohaku_tt_b200 as ktt
    from oracle import attention_oracle as ao

    b, h, hk, s = 2, 4, 2, 1500
    q, k, v = qkv(b, h, hk, s, s, 64, 8)
    lengths = [1500, 700]
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), kernel="flash",
                              key_lengths=torch.tensor(lengths, dtype=torch.int32, device=cuda))
    assert rel(out, ao.ruler_lengths(q, k, v, lengths)) <= FWD_BOUND
    keep = torch.rand(b, 1, 1, s, generator=torch.Generator().manual_seed(3)) > 0.3
    keep[..., 0] = True
    out, _ = ops.sdpa_forward(q.to(cuda), k.to(cuda), v.to(cuda), mask=keep.to(cuda), kernel="flash")
    assert rel(out, ao.ruler_dense(q, k, v, mask=keep)) <= FWD_BOUND
    assert ktt.counters()["attention_flash"] > 0


# Both tcgen05 forward kernels and the tcgen05 backward, launched three times on the same
# inputs, with and without a workspace (drawn and fixed order of the tiles): every launch gives
# the same bits. Which CTA takes which tile, and how far the warps of a CTA drift apart,
# differs from launch to launch; nothing in the arithmetic may depend on it.
@pytest.mark.parametrize("b,h,hk,s,d,causal", [
    (8, 14, 2, 2048, 64, True), (4, 16, 4, 4096, 64, True), (2, 10, 10, 4096, 64, False),
    (8, 16, 4, 2048, 128, True), (3, 8, 2, 1500, 128, False),
])
def test_every_launch_gives_the_same_bits(cuda, b, h, hk, s, d, causal):
    g = torch.Generator(device=cuda).manual_seed(b * 1000 + s + d)
    q, k, v, do = (torch.randn((b, n, s, d), generator=g, device=cuda, dtype=torch.float32).to(torch.bfloat16) for n in (h, hk, hk, h))
    runs = []
    for _ in range(3):
        runs.append(ops.sdpa_forward(q, k, v, causal=causal, kernel="flash"))
        runs.append(ops.sdpa_forward(q, k, v, causal=causal, kernel="flash", dynamic=False))
    out, lse = runs[0]
    grads = [ops.sdpa_backward(do, q, k, v, out, lse, causal=causal) for _ in range(3)]
    torch.cuda.synchronize()
    _lib.device_status()
    for other, other_lse in runs[1:]:
        assert torch.equal(out, other) and torch.equal(lse, other_lse)
    for other in grads[1:]:
        assert all(torch.equal(x, y) for x, y in zip(grads[0], other))


# The dump of one query tile (the counterpart of the reference's _debug_flash_dump,
# aten_attention.cpp:814-831) against float64: a tile the CTA's two streams share (small
# launch) and a whole tile of one stream (1,792 tiles).
@pytest.mark.parametrize("b,h,hk,s,tile", [(1, 4, 2, 512, (0, 3, 3)), (1, 4, 2, 512, (0, 1, 0)), (8, 14, 2, 2048, (5, 9, 11))])
def test_debug_dump_of_one_query_tile(cuda, b, h, hk, s, tile):
    import kohaku_tt_b200 as ktt

    q, k, v = (t.to(cuda) for t in qkv(b, h, hk, s, s, 64, 21))
    bi, hi, ti = tile
    tiles = s // 128
    d = ktt.debug_flash_dump(q, k, v, True, (bi * h + hi) * tiles + ti)
    assert (d["batch"], d["head"], d["q_tile"]) == tile
    nblk = ti + 1
    x, pr, m = d["x"].double().cpu(), d["p"].double().cpu(), d["m"].double().cpu()
    assert torch.isnan(x[nblk:]).all() and not torch.isnan(x[:nblk]).any()
    assert torch.equal(m[:nblk, 0], m[:nblk, 1])   # the two halves of a row agree on the reference
    qq = q[bi, hi, ti * 128:(ti + 1) * 128].double().cpu()
    kk = k[bi, hi // (h // hk)].double().cpu()
    logit2 = (qq @ kk.T) / math.sqrt(64) * math.log2(math.e)   # [128, s]
    rows = torch.arange(128)[:, None] + ti * 128
    l_ref = torch.zeros(128, dtype=torch.float64)
    m_row, l_row = d["m_row"].double().cpu(), d["l_row"].double().cpu()
    for j in range(nblk):
        cols = torch.arange(128)[None, :] + j * 128
        seen = cols <= rows
        want = logit2[:, j * 128:(j + 1) * 128] - m[j, 0][:, None]
        assert (x[j][~seen] == float("-inf")).all() and (pr[j][~seen] == 0).all()
        assert (x[j][seen] - want[seen]).abs().max() <= 2e-3
        # P is 2^x rounded to bf16 (MUFU or the cubic: both well inside bf16's 2^-9)
        assert ((pr[j][seen] - torch.exp2(x[j][seen])).abs() <= 6e-3 * torch.exp2(x[j][seen]) + 1e-30).all()
        l_ref += (torch.exp2(x[j] + m[j, 0][:, None] - m_row[:, None]) * seen).sum(dim=1)
    assert ((l_row - l_ref).abs() <= 1e-3 * l_ref).all()
    lse = d["lse"][bi, hi, ti * 128:(ti + 1) * 128].double().cpu()
    assert (lse - math.log(2.0) * (m_row + torch.log2(l_row))).abs().max() <= 1e-4
    out = d["out"][bi, hi, ti * 128:(ti + 1) * 128].double().cpu()
    assert rel(out, d["o"].double().cpu() / l_row[:, None]) <= 3e-3   # the output is this, rounded to bf16
    ruler = torch.softmax((logit2 * math.log(2.0)).masked_fill(torch.arange(s)[None, :] > rows, float("-inf")), dim=-1) @ v[bi, hi // (h // hk)].double().cpu()
    assert rel(out, ruler) <= FWD_BOUND
    # a launch after the request was cleared leaves the buffer alone and gives the same output
    again, _ = ops.sdpa_forward(q, k, v, causal=True, kernel="flash")
    assert torch.equal(again, d["out"])
