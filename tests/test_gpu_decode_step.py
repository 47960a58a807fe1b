"""The fused decode step (rotary + cache append + attention in one launch) against the
three-op sequence the reference's models run: ktt.rotary (csrc/aten/nn/aten_fused.cpp:30-43),
StaticCache's index_copy_, sdpa with key_lengths."""

import pytest
import torch

import kohaku_tt_b200 as ktt
from kohaku_tt_b200 import ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, rel

pytestmark = pytest.mark.gpu


def _case(b, h, hk, smax, d, lengths, seed):
    q, k_new, v_new, kc, vc = ao.make_inputs(
        [(b, h, 1, d), (b, hk, 1, d), (b, hk, 1, d), (b, hk, smax, d), (b, hk, smax, d)], seed)
    pos = torch.arange(smax, dtype=torch.float32)[:, None]
    inv = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    ang = torch.cat([pos * inv, pos * inv], dim=-1)
    table_cos, table_sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    return q, k_new, v_new, kc, vc, table_cos, table_sin, lengths


# (b, h, hk, smax, d, lengths): positions on tile and warp boundaries, an empty cache, the
# last slot, one and several CTAs per pair.
CASES = [
    (4, 8, 2, 512, 128, [100, 0, 511, 383]),
    (2, 16, 2, 4096, 128, [4095, 2048]),
    (3, 14, 2, 300, 64, [63, 64, 15]),
    (5, 4, 4, 200, 64, [16, 127, 128, 199, 1]),
    (64, 16, 2, 1024, 128, None),
]


@pytest.mark.parametrize("b,h,hk,smax,d,lengths", CASES)
@pytest.mark.parametrize("by_position", [True, False])
def test_decode_step_equals_the_three_ops(cuda, b, h, hk, smax, d, lengths, by_position):
    if lengths is None:
        lengths = torch.randint(0, smax, (b,), generator=torch.Generator().manual_seed(b)).tolist()
    q, k_new, v_new, kc, vc, tcos, tsin, lengths = _case(b, h, hk, smax, d, lengths, b + h + smax + d)
    rows_cos, rows_sin = tcos[lengths], tsin[lengths]
    ruler, k_want, v_want = ao.decode_step(q, k_new, v_new, kc, vc, lengths, rows_cos, rows_sin)

    kc_d, vc_d = kc.to(cuda), vc.to(cuda)
    n_d = torch.tensor(lengths, dtype=torch.int32, device=cuda)
    n_out = torch.zeros_like(n_d)
    cos_d, sin_d = (tcos.to(cuda), tsin.to(cuda)) if by_position else (rows_cos.to(cuda), rows_sin.to(cuda))
    before = ktt.counters()
    out = ktt.decode_step(q.to(cuda), k_new.to(cuda), v_new.to(cuda), kc_d, vc_d, n_d, cos_d, sin_d,
                          lengths_out=n_out)
    assert ktt.counters()["attention_decode"] - before["attention_decode"] == 1
    # The cache holds exactly what rotary + index_copy_ put there, and nothing else moved.
    assert torch.equal(kc_d.cpu(), k_want)
    assert torch.equal(vc_d.cpu(), v_want)
    assert n_out.tolist() == [n + 1 for n in lengths]
    assert n_d.tolist() == lengths
    assert rel(out, ruler) <= FWD_BOUND
    # Bit for bit the unfused route: rotary on the host tensors, then the decode kernel on
    # the updated cache.
    q_rot = ao.rotary_composite(q, rows_cos[:, None, None, :], rows_sin[:, None, None, :])
    again, _ = ops.decode(q_rot.to(cuda), k_want.to(cuda), v_want.to(cuda), key_lengths=n_out)
    assert torch.equal(out, again)


def test_decode_step_refusals(cuda):
    q, k_new, v_new, kc, vc, tcos, tsin, _ = _case(2, 8, 2, 128, 64, [1, 2], 0)
    n = torch.tensor([1, 2], dtype=torch.int32, device=cuda)
    args = [t.to(cuda) for t in (q, k_new, v_new, kc, vc)]
    with pytest.raises(ValueError):   # fp32 rotary rows
        ktt.decode_step(*args, n, tcos.float().to(cuda), tsin.float().to(cuda))
    with pytest.raises(ValueError):   # table shorter than the cache
        ktt.decode_step(*args, n, tcos[:64].to(cuda), tsin[:64].to(cuda))
    with pytest.raises(ValueError):   # two query tokens
        ktt.decode_step(torch.cat([args[0]] * 2, dim=2), *args[1:], n, tcos.to(cuda), tsin.to(cuda))
    with pytest.raises(ValueError):   # lengths_out aliasing is caught at the C ABI
        ktt.decode_step(*args, n, tcos.to(cuda), tsin.to(cuda), lengths_out=n)
