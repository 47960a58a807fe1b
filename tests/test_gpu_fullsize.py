"""The benchmark's own configurations at their full sizes, each compared with the float64
ruler (sampled (batch, head) pairs / query rows / whole sequences where the full float64
score matrices would not fit a host): BASELINE's tolerance, median relative error <= 1e-2 and
maximum absolute error <= 2e-2, plus the reference's rel-RMS bounds."""

import pytest
import torch

import bench
from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, GRAD_BOUND, VARLEN_GRAD_BOUND, rel

pytestmark = pytest.mark.gpu


def _within_baseline(st):
    return st["nonfinite"] == 0 and st["rel_median"] <= 1e-2 and st["abs_max"] <= 2e-2


def test_decode_config_at_full_size(cuda):
    # C3: batch 64, 16 / 2 heads, D 128, lengths U[512, 4096] (seed 0), cache capacity 4096.
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    k = bench.device_randn((64, 2, 4096, 128), 1, cuda)
    v = bench.device_randn((64, 2, 4096, 128), 2, cuda)
    q = bench.seeded([(64, 16, 1, 128)], 3, cuda)[0]
    out, lse = ops.decode(q, k, v, key_lengths=lengths.to(cuda), need_lse=True)
    torch.cuda.synchronize()
    pairs = [(0, 0), (0, 15), (17, 3), (31, 8), (63, 15), (int(lengths.argmax()), 5), (int(lengths.argmin()), 12)]
    st = bench.rows_parity(out, lse, q, k, v, pairs, [0], klen=lengths.tolist())
    assert _within_baseline(st) and st["lse_abs_max"] <= 3e-2, st
    # and the general kernel agrees with the split-K one on the whole batch
    general, _ = ops.sdpa_forward(q, k, v, key_lengths=lengths.to(cuda), kernel="mma")
    assert (out.float() - general.float()).abs().max() <= 2e-2


def test_sdxl_cross_attention_at_full_size(cuda):
    # C4 cross: 4096 queries against 77 keys, the last 20 dropped by a bool key-padding mask.
    q = bench.seeded([(2, 10, 4096, 64)], 80, cuda)[0]
    k, v = bench.seeded([(2, 10, 77, 64)] * 2, 81, cuda)
    keep = torch.ones(2, 1, 1, 77, dtype=torch.bool, device=cuda)
    keep[..., 57:] = False
    for kernel in ("flash", "mma"):
        out, _ = ops.sdpa_forward(q, k, v, mask=keep, kernel=kernel)
        ruler = ao.ruler_dense(q.cpu(), k.cpu(), v.cpu(), mask=keep.cpu())
        assert rel(out, ruler) <= FWD_BOUND, kernel
        assert _within_baseline(bench.stats_of(out, ruler)), kernel


def test_headline_forward_backward_at_full_size(cuda):
    # C2 with gradients: B 1, 14 / 2 heads, S 2048, D 64, causal; one whole GQA group against
    # float64 autograd (dk / dv sum seven query heads).
    q, k, v, do = bench.seeded([(1, 14, 2048, 64), (1, 2, 2048, 64), (1, 2, 2048, 64), (1, 14, 2048, 64)], 50, cuda)
    out, lse = ops.sdpa_forward(q, k, v, causal=True)
    ruler, dq, dk, dv = ao.grads_dense(q[:, 7:].cpu(), k[:, 1:].cpu(), v[:, 1:].cpu(), do[:, 7:].cpu(), causal=True)
    assert rel(out[:, 7:], ruler) <= FWD_BOUND
    for kernel in ("flash", "mma"):
        gq, gk, gv = ops.sdpa_backward(do, q, k, v, out, lse, causal=True, kernel=kernel)
        for name, got, want in (("dq", gq[:, 7:], dq), ("dk", gk[:, 1:], dk), ("dv", gv[:, 1:], dv)):
            assert rel(got, want) <= GRAD_BOUND, (kernel, name)
    torch.cuda.synchronize()
    _lib.device_status()


def test_packed_config_at_full_size(cuda):
    # C5: 65,536 tokens, 16 heads, D 128, lengths U[64, 4096] (seed 0), causal, forward and
    # backward; the shortest, the longest and the last sequence whole, two heads, float64.
    lens = bench.packed_lengths()
    assert sum(lens) == 65536 and min(lens) >= 64
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=cuda)
    q, k, v, do = (bench.device_randn((65536, 16, 128), 400 + j, cuda) for j in range(4))
    out, lse = ops.varlen_forward(q, k, v, cu, cu, max(lens), max(lens), causal=True)
    grads = ops.varlen_backward(do, q, k, v, out, lse, cu, cu, max(lens), max(lens), causal=True)
    torch.cuda.synchronize()
    _lib.device_status()
    st = bench.packed_parity(out, q, k, v, do, lens, grads)
    assert _within_baseline(st["out"]), st
    # gradient magnitudes grow with the sequence length: the reference's own bound is rel RMS
    starts = [0]
    for n in lens:
        starts.append(starts[-1] + n)
    i = max(range(len(lens)), key=lambda j: lens[j])
    sl = slice(starts[i], starts[i + 1])
    c = [0, lens[i]]
    hs = [0, 15]
    ruler, dq, dk, dv = ao.ruler_varlen(q[sl][:, hs].cpu(), k[sl][:, hs].cpu(), v[sl][:, hs].cpu(), c, c, causal=True,
                                        dout=do[sl][:, hs].cpu())
    assert rel(out[sl][:, hs], ruler) <= FWD_BOUND
    for name, got, want in (("dq", grads[0], dq), ("dk", grads[1], dk), ("dv", grads[2], dv)):
        assert rel(got[sl][:, hs], want) <= VARLEN_GRAD_BOUND, name
