"""The operator surface end to end on CUDA tensors: F.scaled_dot_product_attention and
autograd land on these kernels, torch's varlen_attn does too, scopes and counters work
(tests/hardware/ops/test_attention.py, test_sdpa_kernel.py)."""

import pytest
import torch
import torch.nn.functional as F

import kohaku_tt_b200 as ktt
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, GRAD_BOUND, cu, cumulative, packed, qkv, rel

pytestmark = pytest.mark.gpu


def _delta(before):
    after = ktt.counters()
    return {k: after[k] - before[k] for k in after if after[k] != before[k]}


def test_sdpa_dispatches_here_forward_and_backward(cuda):
    q, k, v, do = qkv(2, 8, 8, 256, 256, 64, 0, extra=1)  # benchmark config 1
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
    qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
    before = ktt.counters()
    out = F.scaled_dot_product_attention(qc, kc, vc, is_causal=True)
    out.backward(do.to(cuda))
    d = _delta(before)
    assert d.get("attention_backward") == 1
    assert d.get("attention_flash", 0) + d.get("attention_mma", 0) == 1
    assert rel(out, ruler) <= FWD_BOUND
    for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
        assert rel(got, want) <= GRAD_BOUND
    # The tolerance BASELINE states for this config, beside the CPU bf16 result.
    cpu = ao.ruler_dense(q, k, v, causal=True, dtype=torch.bfloat16)
    ours, theirs = ktt.diff_stats(out, ruler), ktt.diff_stats(cpu, ruler)
    assert ours["rel_median"] <= 1e-2 and ours["abs_max"] <= 2e-2
    assert ours["abs_max"] <= 2 * theirs["abs_max"] + 1e-3


def test_gqa_masks_and_fp32_route_here(cuda):
    q, k, v = qkv(1, 14, 2, 300, 300, 64, 2)
    before = ktt.counters()
    out = F.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), is_causal=True, enable_gqa=True)
    assert sum(_delta(before).values()) >= 1
    assert rel(out, ao.ruler_dense(q, k, v, causal=True)) <= FWD_BOUND
    # SDXL cross-attention shape: 77 keys, last 20 masked by a bool key-padding mask.
    q, k, v = qkv(2, 10, 10, 512, 77, 64, 3)
    keep = torch.ones(2, 1, 1, 77, dtype=torch.bool)
    keep[..., 57:] = False
    before = ktt.counters()
    out = F.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda), attn_mask=keep.to(cuda))
    assert sum(_delta(before).values()) >= 1
    assert rel(out, ao.ruler_dense(q, k, v, mask=keep)) <= FWD_BOUND
    # fp32 inputs without gradients are cast at entry (test_flash_fp32_causal.py).
    q, k, v = ao.make_inputs([(1, 4, 128, 64)] * 3, 4, dtype=torch.float32)
    before = ktt.counters()
    out = F.scaled_dot_product_attention(q.to(cuda), k.to(cuda), v.to(cuda))
    assert out.dtype == torch.float32 and sum(_delta(before).values()) >= 1
    assert rel(out, ao.ruler_dense(q, k, v)) <= 1.2e-2


def test_overrideable_pair_and_choice_op(cuda):
    q, k, v, do = qkv(1, 2, 2, 77, 77, 64, 5, extra=1)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    assert torch.ops.aten._fused_sdp_choice(qc, kc, vc, None, 0.0, True) == 4
    assert torch.ops.aten._fused_sdp_choice(qc, kc, vc, None, 0.1, False) == 0
    res = torch.ops.aten._scaled_dot_product_fused_attention_overrideable(qc, kc, vc, None, 0.0, True)
    out, lse = res[0], res[1]
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
    assert rel(out, ruler) <= FWD_BOUND and lse.shape == (1, 2, 77)
    grads = torch.ops.aten._scaled_dot_product_fused_attention_overrideable_backward(
        do.to(cuda), qc, kc, vc, torch.empty(0, device=cuda), [True, True, True, False], out, lse,
        res[2], res[3], res[4], res[5], 0.0, True, res[6], res[7])
    for got, want in zip(grads[:3], (dq, dk, dv)):
        assert rel(got, want) <= GRAD_BOUND


def test_dropout_is_refused_not_rerouted(cuda):
    q, k, v = (t.to(cuda) for t in qkv(1, 2, 2, 64, 64, 64, 1))
    with pytest.raises(NotImplementedError):
        torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.1, False)


def test_torch_varlen_attn_runs_here(cuda):
    from torch.nn.attention.varlen import varlen_attn

    lengths = [40, 7, 90]
    c = cumulative(lengths)
    q, k, v, do = packed(lengths, lengths, 4, 4, 64, 8, extra=1)
    ruler, dq, dk, dv = ao.ruler_varlen(q, k, v, c, c, causal=True, dout=do)
    qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
    before = ktt.counters()
    out = varlen_attn(qc, kc, vc, cu(lengths, cuda), cu(lengths, cuda), 90, 90, window_size=(-1, 0))
    out.backward(do.to(cuda))
    d = _delta(before)
    assert d.get("attention_backward") == 1
    assert rel(out, ruler) <= FWD_BOUND
    for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
        assert rel(got, want) <= 2.5e-2
    # The package's own entry point gives the same result.
    again = ktt.sdpa_varlen(q.to(cuda), k.to(cuda), v.to(cuda), c, is_causal=True)
    assert torch.equal(again, out.detach())


def test_scope_selects_the_kernel(cuda):
    q, k, v = (t.to(cuda) for t in qkv(1, 4, 4, 128, 128, 64, 1))
    with ktt.sdpa_kernel("mma"):
        before = ktt.counters()
        F.scaled_dot_product_attention(q, k, v)
        assert _delta(before) == {"attention_mma": 1}
    q96 = q[..., :32].contiguous()
    with ktt.sdpa_kernel("flash"):
        with pytest.raises(NotImplementedError):  # head dim 32 is not a tcgen05 shape
            F.scaled_dot_product_attention(q96, q96, q96)


def test_merge_partials_equals_attention_over_the_union(cuda):
    from kohaku_tt_b200 import ops

    q, k, v = qkv(1, 4, 4, 200, 300, 64, 4)
    qc, kc, vc = q.to(cuda), k.to(cuda), v.to(cuda)
    o1, l1 = ops.sdpa_forward(qc, kc[:, :, :130].contiguous(), vc[:, :, :130].contiguous())
    o2, l2 = ops.sdpa_forward(qc, kc[:, :, 130:].contiguous(), vc[:, :, 130:].contiguous())
    # Three operand forms give the same merge: fp32 with fp32, fp32 with the kernel's bf16
    # output, bf16 with bf16; odd widths take the scalar path.
    acc, la = o1.float().contiguous(), l1.clone()
    ops.merge_partials(acc, la, o2.float().contiguous(), l2)
    assert rel(acc, ao.ruler_dense(q, k, v)) <= FWD_BOUND
    assert (la.cpu().double() - ao.ruler_lse(q, k, v)).abs().max() <= 3e-2
    mixed, lm = o1.float().contiguous(), l1.clone()
    ops.merge_partials(mixed, lm, o2, l2)
    assert torch.equal(mixed, acc) and torch.equal(lm, la)
    both, lb = o1.clone(), l1.clone()
    ops.merge_partials(both, lb, o2, l2)
    assert rel(both, acc) <= 4e-3 and torch.equal(lb, la)
    narrow, ln = o1[..., :63].float().contiguous(), l1.clone()
    ops.merge_partials(narrow, ln, o2[..., :63].contiguous(), l2)
    assert torch.allclose(narrow, acc[..., :63], rtol=1e-5, atol=1e-6)  # scalar path: same formula, other rounding of the multiply-adds
    # Operands that start at an odd element (views with a storage offset) are contiguous but
    # not 16-byte aligned: the scalar path takes them instead of a misaligned vector access.
    pad_a = torch.zeros(o1.numel() + 1, dtype=torch.float32, device=cuda)
    pad_b = torch.zeros(o2.numel() + 1, dtype=torch.bfloat16, device=cuda)
    off_a, off_b = pad_a[1:].view(o1.shape), pad_b[1:].view(o2.shape)
    off_a.copy_(o1.float())
    off_b.copy_(o2)
    lo = l1.clone()
    ops.merge_partials(off_a, lo, off_b, l2)
    assert torch.allclose(off_a, acc, rtol=1e-5, atol=1e-6) and torch.equal(lo, la)


# ---- torch.compile (tests/hardware/ops/test_sdpa_kernel.py:215-224) ----------------------

def test_scope_reaches_compiled_code(cuda):
    """The kernel scope is read when the compiled function runs, not when it was traced."""
    q, k, v = (t.to(cuda) for t in qkv(1, 4, 4, 128, 128, 64, 10))
    fn = torch.compile(lambda a, b, c: F.scaled_dot_product_attention(a, b, c),
                       backend="aot_eager", fullgraph=True)
    want = F.scaled_dot_product_attention(q, k, v)
    before = ktt.counters()
    with ktt.sdpa_kernel("mma"):
        first = fn(q, k, v)
    second = fn(q, k, v)
    assert _delta(before) == {"attention_mma": 1, "attention_flash": 1}
    assert torch.equal(second, want)
    assert rel(first, want.float()) <= 4e-3


def test_compiled_training_step_uses_these_kernels(cuda):
    q, k, v, do = qkv(2, 4, 2, 256, 256, 64, 12, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
    qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))

    def step(a, b, c):
        return F.scaled_dot_product_attention(a, b, c, is_causal=True, enable_gqa=True)

    fn = torch.compile(step, backend="aot_eager", fullgraph=True)
    before = ktt.counters()
    out = fn(qc, kc, vc)
    out.backward(do.to(cuda))
    d = _delta(before)
    assert d.get("attention_backward") == 1
    assert d.get("attention_flash", 0) + d.get("attention_mma", 0) == 1
    assert rel(out, ruler) <= FWD_BOUND
    for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
        assert rel(got, want) <= GRAD_BOUND


def test_key_lengths_op_compiles_whole(cuda):
    """The custom ops carry fake kernels: decode and the training route trace without a
    graph break and match eager bit for bit."""
    q, k, v = (t.to(cuda) for t in qkv(4, 8, 2, 1, 512, 128, 14))
    lengths = torch.tensor([100, 512, 1, 383], dtype=torch.int32, device=cuda)
    fn = torch.compile(lambda a, b, c, n: ktt.sdpa(a, b, c, key_lengths=n), backend="aot_eager", fullgraph=True)
    before = ktt.counters()
    got = fn(q, k, v, lengths)
    assert _delta(before) == {"attention_decode": 1}
    assert torch.equal(got, ktt.sdpa(q, k, v, key_lengths=lengths))

    q2, k2, v2, do = qkv(2, 4, 2, 96, 96, 64, 15, extra=1)
    n2 = torch.tensor([96, 40], dtype=torch.int32, device=cuda)
    a, b, c = (t.to(cuda).requires_grad_(True) for t in (q2, k2, v2))
    fn2 = torch.compile(lambda x, y, z, n: ktt.sdpa(x, y, z, key_lengths=n, is_causal=True),
                        backend="aot_eager", fullgraph=True)
    out = fn2(a, b, c, n2)
    out.backward(do.to(cuda))
    a2, b2, c2 = (t.to(cuda).requires_grad_(True) for t in (q2, k2, v2))
    eager = ktt.sdpa(a2, b2, c2, key_lengths=n2, is_causal=True)
    eager.backward(do.to(cuda))
    assert torch.equal(out, eager)
    for got_g, want_g in ((a.grad, a2.grad), (b.grad, b2.grad), (c.grad, c2.grad)):
        assert torch.equal(got_g, want_g)
    assert torch.count_nonzero(b.grad[1, :, 40:]) == 0


def test_sdxl_style_block_compiled_equals_eager(cuda):
    """tests/hardware/compile/test_pitched_attention_graphs.py:12-27: B 2, T 128, TK 77, 20
    heads of 64: linears, head views, self- and cross-attention with a key-padding mask."""
    torch.manual_seed(0)
    b, t, tk, h, d = 2, 128, 77, 20, 64
    c = h * d

    class Block(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.qkv = torch.nn.Linear(c, 3 * c, bias=False)
            self.q2 = torch.nn.Linear(c, c, bias=False)
            self.kv2 = torch.nn.Linear(c, 2 * c, bias=False)
            self.out = torch.nn.Linear(c, c, bias=False)

        def forward(self, x, ctx, keep):
            q, k, v = (z.view(b, t, h, d).transpose(1, 2) for z in self.qkv(x).chunk(3, dim=-1))
            y = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(b, t, c)
            q = self.q2(y).view(b, t, h, d).transpose(1, 2)
            k, v = (z.view(b, tk, h, d).transpose(1, 2) for z in self.kv2(ctx).chunk(2, dim=-1))
            y = F.scaled_dot_product_attention(q, k, v, attn_mask=keep).transpose(1, 2).reshape(b, t, c)
            return self.out(y)

    block = Block()
    x, ctx = torch.randn(b, t, c) / 8, torch.randn(b, tk, c) / 8
    keep = torch.ones(b, 1, 1, tk, dtype=torch.bool)
    keep[..., 57:] = False
    want = block.double()(x.double(), ctx.double(), keep)   # float64 on the CPU
    block = block.float().to(cuda).to(torch.bfloat16)
    xc, cc, kc = x.to(cuda).to(torch.bfloat16), ctx.to(cuda).to(torch.bfloat16), keep.to(cuda)
    before = ktt.counters()
    with torch.no_grad():
        eager = block(xc, cc, kc)
        d1 = _delta(before)
        compiled = torch.compile(block, backend="aot_eager", fullgraph=True)(xc, cc, kc)
    assert d1.get("attention_flash", 0) + d1.get("attention_mma", 0) == 2   # both attentions ran here
    assert torch.equal(compiled, eager)
    assert rel(eager, want) <= 3e-2   # bf16 linears around the attention


def test_sdpa_kernel_math_selects_math(cuda):
    # tests/hardware/ops/test_attention.py:63-67: torch's own switch wins over the shapes.
    from torch.nn.attention import SDPBackend, sdpa_kernel

    q, k, v = (t.to(cuda) for t in qkv(1, 2, 2, 64, 64, 64, 1))
    assert torch.ops.aten._fused_sdp_choice(q, k, v, None, 0.0, False) == 4
    with sdpa_kernel(SDPBackend.MATH):
        assert torch.ops.aten._fused_sdp_choice(q, k, v, None, 0.0, False) == 0
        # ... and PyTorch's math composite then runs the call: none of the kernels here does.
        before = ktt.counters()
        out = F.scaled_dot_product_attention(q, k, v, dropout_p=0.0)
        assert _delta(before) == {}
    assert rel(out, ao.ruler_dense(q.cpu(), k.cpu(), v.cpu())) <= FWD_BOUND
    assert torch.ops.aten._fused_sdp_choice(q, k, v, None, 0.0, False) == 4


@pytest.mark.parametrize("bias_shape", [(2, 1, 96, 96), (1, 4, 1, 96)])
def test_bias_gradient_matches_float64_autograd(cuda, bias_shape):
    # aten_attention.cpp:781-811: dS summed over the dims the bias broadcasts.
    b, h, s, d = 2, 4, 96, 64
    q, k, v, do = qkv(b, h, h, s, s, d, 21, extra=1)
    bias = torch.randn(bias_shape, generator=torch.Generator().manual_seed(22)).to(torch.bfloat16)
    qd, kd, vd, bd = (t.double().requires_grad_(True) for t in (q, k, v, bias))
    ruler = F.scaled_dot_product_attention(qd, kd, vd, attn_mask=bd)
    ruler.backward(do.double())
    qc, kc, vc, bc = (t.to(cuda).requires_grad_(True) for t in (q, k, v, bias))
    before = ktt.counters()
    out = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=bc)
    out.backward(do.to(cuda))
    assert _delta(before).get("attention_backward") == 1
    assert rel(out, ruler.detach()) <= FWD_BOUND
    assert bc.grad is not None and bc.grad.shape == bias.shape
    assert rel(bc.grad, bd.grad) <= GRAD_BOUND
    for got, want in ((qc.grad, qd.grad), (kc.grad, kd.grad), (vc.grad, vd.grad)):
        assert rel(got, want) <= GRAD_BOUND


def test_inductor_compiles_forward_backward_and_key_lengths(cuda):
    """tests/hardware/ops/test_sdpa_kernel.py:215-224 compiles with the product's real
    backend; here that is inductor, which trusts the strides the meta kernels promise."""
    q, k, v, do = qkv(2, 4, 2, 256, 256, 64, 12, extra=1)
    ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
    qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
    fn = torch.compile(lambda a, b, c: F.scaled_dot_product_attention(a, b, c, is_causal=True, enable_gqa=True) * 2.0,
                       backend="inductor", fullgraph=True)
    before = ktt.counters()
    out = fn(qc, kc, vc)
    out.backward(do.to(cuda))
    d = _delta(before)
    assert d.get("attention_backward") == 1 and d.get("attention_flash", 0) + d.get("attention_mma", 0) == 1
    assert rel(out, 2.0 * ruler) <= FWD_BOUND
    for got, want in ((qc.grad, dq), (kc.grad, dk), (vc.grad, dv)):
        assert rel(got, 2.0 * want) <= GRAD_BOUND

    # A masked call with contiguous q takes the efficient overload, whose output is laid out
    # [B, Sq, H, Dv]: the compiled graph must index it the way its meta kernel says.
    keep = torch.ones(2, 1, 1, 256, dtype=torch.bool, device=cuda)
    keep[..., 200:] = False
    masked = torch.compile(lambda a, b, c, m: F.scaled_dot_product_attention(a, b, c, attn_mask=m, enable_gqa=True) + 1.0,
                           backend="inductor", fullgraph=True)
    with torch.no_grad():
        got = masked(qc, kc, vc, keep)
        want = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=keep, enable_gqa=True) + 1.0
    assert torch.equal(got, want)
    assert rel(got - 1.0, ao.ruler_dense(q, k, v, mask=keep.cpu())) <= 2e-2   # the + 1 costs bf16 bits

    # ktt.sdpa(key_lengths=) on a head view: the fake kernel promises the real op's layout.
    x = ao.make_inputs([(2, 96, 3 * 4 * 64)], 16)[0].to(cuda).view(2, 96, 3, 4, 64)
    qh, kh, vh = (x[:, :, i].transpose(1, 2) for i in range(3))
    n = torch.tensor([96, 40], dtype=torch.int32, device=cuda)
    lengths_fn = torch.compile(lambda a, b, c, m: ktt.sdpa(a, b, c, key_lengths=m) * 1.0, backend="inductor", fullgraph=True)
    with torch.no_grad():
        assert torch.equal(lengths_fn(qh, kh, vh, n), ktt.sdpa(qh, kh, vh, key_lengths=n))


def test_refused_calls_say_how_to_reach_the_math_route_and_uninstall_restores_torch(cuda):
    from torch.nn.attention import SDPBackend, sdpa_kernel

    q, k, v = (t.to(cuda) for t in qkv(1, 2, 2, 64, 64, 64, 1))
    with pytest.raises(NotImplementedError, match="sdpa_kernel"):
        torch.ops.aten._scaled_dot_product_flash_attention(q, k, v, 0.1, False)
    # The route the message names: dropout under the math backend runs PyTorch's composite.
    with sdpa_kernel(SDPBackend.MATH):
        assert F.scaled_dot_product_attention(q, k, v, dropout_p=0.1).shape == q.shape
    ktt.uninstall()
    try:
        before = ktt.counters()
        out = F.scaled_dot_product_attention(q, k, v)   # PyTorch's own CUDA kernel again
        assert _delta(before) == {}
        assert rel(out, ao.ruler_dense(q.cpu(), k.cpu(), v.cpu())) <= FWD_BOUND
    finally:
        ktt.install()
    before = ktt.counters()
    F.scaled_dot_product_attention(q, k, v)
    assert sum(_delta(before).values()) == 1


def test_packed_rows_without_keys_are_defined(cuda):
    """Device offsets are not checked on the torch_attn route: a causal sequence with more
    queries than keys gives its first Lq - Lk rows no key. Those rows come back as zeros
    with lse = -inf, and their gradients are zero."""
    from kohaku_tt_b200 import ops

    lq, lk = [40, 7], [25, 7]
    q, k, v, do = packed(lq, lk, 2, 2, 64, 31, extra=1)
    out, lse = ops.varlen_forward(q.to(cuda), k.to(cuda), v.to(cuda), cu(lq, cuda), cu(lk, cuda), 40, 25, causal=True)
    assert torch.count_nonzero(out[:15]) == 0 and torch.isinf(lse[:, :15]).all() and (lse[:, :15] < 0).all()
    assert torch.isfinite(out).all() and torch.isfinite(lse[:, 15:]).all()
    gq, gk, gv = ops.varlen_backward(do.to(cuda), q.to(cuda), k.to(cuda), v.to(cuda), out, lse,
                                     cu(lq, cuda), cu(lk, cuda), 40, 25, causal=True)
    assert torch.count_nonzero(gq[:15]) == 0
    assert all(torch.isfinite(g).all() for g in (gq, gk, gv))


def test_cpp_and_python_registrations_agree(cuda):
    """The overloads are registered from C++ (csrc/torch_shim) by default; the Python
    registration is the stand-in. Same kernels, same layouts, same bits; the kernel scope
    reaches both."""
    from kohaku_tt_b200 import aten

    assert aten.using_cpp_registration()
    q, k, v, do = qkv(2, 4, 2, 200, 200, 64, 41, extra=1)
    keep = torch.ones(2, 1, 1, 200, dtype=torch.bool)
    keep[..., 150:] = False

    def run():
        qc, kc, vc = (t.to(cuda).requires_grad_(True) for t in (q, k, v))
        out = F.scaled_dot_product_attention(qc, kc, vc, is_causal=True, enable_gqa=True)
        out.backward(do.to(cuda))
        with torch.no_grad():
            masked = F.scaled_dot_product_attention(qc, kc, vc, attn_mask=keep.to(cuda), enable_gqa=True)
        before = ktt.counters()
        with ktt.sdpa_kernel("mma"), torch.no_grad():
            F.scaled_dot_product_attention(qc, kc, vc, enable_gqa=True)
        return out.detach(), qc.grad, kc.grad, vc.grad, masked, masked.stride(), _delta(before)

    cpp = run()
    ktt.uninstall()
    try:
        ktt.install(python=True)
        assert not aten.using_cpp_registration()
        py = run()
    finally:
        ktt.uninstall()
        ktt.install()
    assert aten.using_cpp_registration()
    for a, b in zip(cpp[:5], py[:5]):
        assert torch.equal(a, b)
    assert cpp[5] == py[5]
    assert cpp[6] == py[6] == {"attention_mma": 1}
