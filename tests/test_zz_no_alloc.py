"""The allocation-free decode entry point (ktt_b200_decode_static), called through the C ABI.

It serves callers that may not allocate device memory while running; its split-K partials
live in a fixed array inside the library. The test checks it against the regular entry
point (same kernels, caller-provided scratch) on two calls in a row, with different
inputs, so that whatever the first call left in the shared array cannot leak into the
second. The file name sorts last on purpose: if this test fails under `pytest -x`, every
other test has already run.
"""

import ctypes

import pytest
import torch

from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, qkv, rel

pytestmark = pytest.mark.gpu


def _args(q, k, v, out, lengths, scale=None):
    a = _lib.DecodeArgs()
    b, h, sq, d = q.shape
    a.batch, a.heads, a.kv_heads, a.sq, a.sk, a.d, a.dv = b, h, k.shape[1], sq, k.shape[2], d, d
    a.scale = float(scale) if scale is not None else d ** -0.5
    a.q, a.k, a.v, a.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    for name, t in (("q_strides", q), ("k_strides", k), ("v_strides", v), ("out_strides", out)):
        for i in range(3):
            getattr(a, name)[i] = t.stride(i)
    a.key_lengths = lengths.data_ptr()
    return a


def _both(cuda, seed, b, h, hk, d, cap, splits=0):
    """(static result, regular result, float64 ruler) for one seeded decode problem."""
    q, k, v = qkv(b, h, hk, 1, cap, d, seed)
    g = torch.Generator().manual_seed(seed)
    lengths = torch.randint(1, cap + 1, (b,), generator=g, dtype=torch.int32)
    qc, kc, vc, ln = q.to(cuda), k.to(cuda), v.to(cuda), lengths.to(cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    static_out = torch.empty_like(qc)
    args = _args(qc, kc, vc, static_out, ln)
    args.splits = splits
    # The property the entry point exists for: the call itself allocates nothing. Everything
    # it touches exists already, so neither torch's allocator nor the driver's free-memory
    # count moves across it.
    torch.cuda.synchronize()
    free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
    _lib.check(_lib.lib().ktt_b200_decode_static(ctypes.byref(args), stream), "decode_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == held_before
    if _both.warm:   # the first call on a device takes the array's address and sets kernel attributes
        assert torch.cuda.mem_get_info()[0] == free_before
    _both.warm = True
    regular_out, _ = ops.decode(qc, kc, vc, key_lengths=ln, splits=splits)
    torch.cuda.synchronize()
    return static_out, regular_out, ao.ruler_lengths(q, k, v, lengths)


_both.warm = False


def test_static_decode_matches_the_regular_entry_point_twice(cuda):
    # Calls in a row on the one shared array: large then small (stale partials of the first
    # sit there while the second runs), then small to large again and another split count
    # (the tickets must be back at zero, and slots laid out for an earlier call must not
    # alias live partials).
    cases = ((1, (16, 16, 2, 128, 1024), 0), (2, (5, 8, 8, 64, 300), 0), (3, (16, 16, 2, 128, 1024), 2),
             (4, (24, 16, 2, 128, 700), 0))
    for seed, shape, splits in cases:
        static_out, regular_out, ruler = _both(cuda, seed, *shape, splits=splits)
        # Same kernels, same split: the two entry points agree bit for bit, and both sit
        # inside the forward bound against the float64 ruler.
        assert torch.equal(static_out, regular_out), seed
        assert rel(static_out, ruler) <= FWD_BOUND, seed


def test_static_decode_refuses_what_does_not_fit(cuda):
    # 300 (batch, kv head) pairs at head dim 128 need more than the built-in 4 MiB.
    b, h, hk, d, cap = 150, 16, 2, 128, 64
    q = torch.zeros(b, h, 1, d, dtype=torch.bfloat16, device=cuda)
    k = torch.zeros(b, hk, cap, d, dtype=torch.bfloat16, device=cuda)
    out = torch.empty_like(q)
    ln = torch.full((b,), cap, dtype=torch.int32, device=cuda)
    args = _args(q, k, k, out, ln)
    rc = _lib.lib().ktt_b200_decode_static(ctypes.byref(args), None)
    assert rc == _lib.ERR_UNSUPPORTED
    assert "built-in array holds" in _lib.last_error()
    with pytest.raises(_lib.UnsupportedAttention):
        _lib.check(rc, "decode_static")
