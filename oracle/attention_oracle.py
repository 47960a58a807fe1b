"""TEST INFRASTRUCTURE ONLY: the float64 ruler and the same-precision CPU result.

The reference judges its flash kernels against F.scaled_dot_product_attention on
float64 CPU tensors and reports torch's CPU SDPA on the bf16 tensors beside it
(tests/hardware/ops/test_flash.py:57-63, src/kohakutt/bench/ops.py:533-581,
src/kohakutt/tools/kernel_audit.py:20-41). Those two are restated here, per surface:

  ruler_dense      test_flash.py:57-63 (GQA by repeat_interleave), masks :86-117
  ruler_lengths    kohakutt/torch_backend/lengths.py:79-89 (bool mask key < length)
  ruler_varlen     tests/hardware/ops/test_flash_varlen.py:62-73 (per-sequence loop,
                   causal mask arange(m) < arange(n) + 1 + m - n)
  ruler_lse        test_flash.py:307-317 (logsumexp of the float64 scores)
  ruler_rows       the same definition evaluated for sampled query rows of one pair
  grads_*          float64 autograd of the rulers (test_flash.py:197-215)
  cpu_*            the same calls on the bf16 CPU tensors (the reference's CPU path)

Pinning: tests/test_oracle.py checks these against the plain-C restatement in
attention_ref.c, against outputs of the reference's own Python
(kohakutt.torch_backend.lengths.masked, kohakutt.core.stats.diff_stats) stored under
tests/golden/, and the packed-sequence visibility rule against the reference's own
varlen_plan.hpp compiled into oracle/_ref. The reference ships no bit-level golden
vectors for attention (its tests/hardware/golden/*.pt are generated on a card and are
not in the tree), so at the bit level parity is unpinned; at the level of the
reference's own statistical bounds it is pinned by those tests.
"""

import ctypes
import math
import os

import torch
import torch.nn.functional as F

_HERE = os.path.dirname(os.path.abspath(__file__))


def make_inputs(shapes, seed, dtype=torch.bfloat16):
    """Seeded N(0,1) tensors drawn in order on CPU in fp32, then cast: the generator of
    the reference's tests (test_flash.py:48-53)."""
    g = torch.Generator().manual_seed(seed)
    return tuple(torch.randn(*s, generator=g).to(dtype) for s in shapes)


def _rep(q, k, v, dtype):
    rep = q.shape[1] // k.shape[1]
    return (q.to(dtype), k.to(dtype).repeat_interleave(rep, 1), v.to(dtype).repeat_interleave(rep, 1))


def _top_left(sq, sk):
    return torch.arange(sk)[None, :] <= torch.arange(sq)[:, None]


def ruler_dense(q, k, v, mask=None, causal=False, scale=None, dtype=torch.float64):
    """F.scaled_dot_product_attention on `dtype` copies; causal is top-left for any
    Sq, Sk (torch's is_causal is top-left as well; the explicit mask keeps Sq > Sk
    rows defined the same way)."""
    qd, kd, vd = _rep(q, k, v, dtype)
    m = mask
    if m is not None and m.dtype != torch.bool:
        m = m.to(dtype)
    if causal:
        m = _top_left(q.shape[2], k.shape[2])
    return F.scaled_dot_product_attention(qd, kd, vd, attn_mask=m, scale=scale)


def length_mask(lengths, sq, sk, causal):
    """The bool mask [B, 1, Sq, Sk] of kohakutt.torch_backend.lengths.masked
    (lengths.py:79-89)."""
    keys = torch.arange(sk, dtype=torch.int32)
    keep = (keys[None, :] < lengths.to(torch.int32)[:, None])[:, None, None, :]
    if causal:
        rows = torch.arange(sq, dtype=torch.int32)
        keep = keep & (keys[None, :] <= rows[:, None])[None, None]
    return keep.expand(lengths.numel(), 1, sq, sk)


def ruler_lengths(q, k, v, lengths, causal=False, scale=None, dtype=torch.float64):
    qd, kd, vd = _rep(q, k, v, dtype)
    keep = length_mask(torch.as_tensor(lengths), q.shape[2], k.shape[2], causal)
    return F.scaled_dot_product_attention(qd, kd, vd, attn_mask=keep, scale=scale)


def ruler_lse(q, k, v, mask=None, causal=False, scale=None, lengths=None):
    """logsumexp over keys of the float64 logits, [B, H, Sq]."""
    qd, kd, _ = _rep(q, k, v, torch.float64)
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = qd @ kd.transpose(-1, -2) * sc
    if mask is not None:
        s = s.masked_fill(~mask, -math.inf) if mask.dtype == torch.bool else s + mask.double()
    if causal:
        s = s.masked_fill(~_top_left(q.shape[2], k.shape[2]), -math.inf)
    if lengths is not None:
        keep = length_mask(torch.as_tensor(lengths), q.shape[2], k.shape[2], False)
        s = s.masked_fill(~keep, -math.inf)
    return torch.logsumexp(s, dim=-1)


def ruler_rows(q, k, v, rows, shift=0, causal=False, scale=None, klen=None):
    """float64 attention of a few query rows of ONE (batch, head): q [Sq, D] (or the rows
    already picked, [len(rows), D]), k [Sk, D], v [Sk, Dv] -> (out [len(rows), Dv], lse).
    Row i sees keys j <= i + shift when causal (shift = Lk - Lq is the bottom-right
    alignment of varlen_plan.hpp:69-70, 0 the top-left one) and j < klen. For the sizes
    whose full float64 score matrix does not fit (S 4096 and up, the 131,072-token ring):
    each sampled row costs one [Sk, D] product."""
    rows = torch.as_tensor(rows, dtype=torch.long)
    qr = q if q.shape[0] == rows.numel() and q.shape[0] != k.shape[0] else q[rows]
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = qr.double() @ k.double().T * sc
    keys = torch.arange(k.shape[0])
    if causal:
        s = s.masked_fill(keys[None, :] > rows[:, None] + shift, -math.inf)
    if klen is not None:
        s = s.masked_fill(keys[None, :] >= klen, -math.inf)
    return torch.softmax(s, dim=-1) @ v.double(), torch.logsumexp(s, dim=-1)


def grads_dense(q, k, v, dout, mask=None, causal=False, scale=None, lengths=None, dtype=torch.float64):
    """(out, dq, dk, dv) by `dtype` autograd; dk / dv come back summed over each group
    because the repeat_interleave is inside the graph."""
    qd = q.to(dtype).requires_grad_(True)
    kd = k.to(dtype).requires_grad_(True)
    vd = v.to(dtype).requires_grad_(True)
    rep = q.shape[1] // k.shape[1]
    m = mask
    if m is not None and m.dtype != torch.bool:
        m = m.to(dtype)
    if causal:
        m = _top_left(q.shape[2], k.shape[2])
    if lengths is not None:
        m = length_mask(torch.as_tensor(lengths), q.shape[2], k.shape[2], causal)
    out = F.scaled_dot_product_attention(
        qd, kd.repeat_interleave(rep, 1), vd.repeat_interleave(rep, 1), attn_mask=m, scale=scale)
    out.backward(dout.to(dtype))
    return out.detach(), qd.grad, kd.grad, vd.grad


def rotary_composite(x, cos, sin):
    """ktt.rotary's composite (csrc/aten/nn/aten_fused.cpp:30-43): x * cos + cat(-x2, x1) *
    sin over the last dim with every product and the sum rounded in fp32, result in x's
    dtype. cos / sin broadcast against x (rows already chosen by the caller)."""
    xf = x.float()
    x1, x2 = xf.chunk(2, -1)
    rotated = torch.cat([-x2, x1], -1)
    return (xf * cos.float() + rotated * sin.float()).to(x.dtype)


def decode_step(q, k_new, v_new, k_cache, v_cache, lengths, cos_rows, sin_rows, scale=None):
    """One decode token the way the reference's model code runs it: rotary on q and k_new
    (rows cos_rows / sin_rows [B, D], one per batch entry), StaticCache `index_copy_` of the
    new key / value at position lengths[b] (docs/reference/results.md:296), attention over
    the lengths[b] + 1 keys in float64. Returns (out float64 [B, H, 1, D], updated k cache,
    updated v cache); the inputs are not modified."""
    c, s_ = cos_rows[:, None, None, :], sin_rows[:, None, None, :]
    q_rot = rotary_composite(q, c, s_)
    k_rot = rotary_composite(k_new, c, s_)
    k2, v2 = k_cache.clone(), v_cache.clone()
    for b, n in enumerate(lengths):
        k2[b, :, n] = k_rot[b, :, 0]
        v2[b, :, n] = v_new[b, :, 0]
    out = ruler_lengths(q_rot, k2, v2, [n + 1 for n in lengths], causal=False, scale=scale)
    return out, k2, v2


def _bottom_right(lq, lk):
    """Query r sees its first min(Lk, r + 1 + Lk - Lq) keys (varlen_plan.hpp:69-70)."""
    return torch.arange(lk)[None, :] < (torch.arange(lq)[:, None] + 1 + lk - lq)


def ruler_varlen(q, k, v, cu_q, cu_k, causal=False, scale=None, key_mask=None, dtype=torch.float64,
                 dout=None):
    """Per-sequence loop over packed q [Tq, H, D], k [Tk, Hk, D], v [Tk, Hk, Dv]
    (test_flash_varlen.py:62-73,201-220). Returns out [Tq, H, Dv], or with `dout`
    (out, dq, dk, dv)."""
    qd = q.to(dtype).requires_grad_(dout is not None)
    kd = k.to(dtype).requires_grad_(dout is not None)
    vd = v.to(dtype).requires_grad_(dout is not None)
    rep = q.shape[1] // k.shape[1]
    outs = []
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if q1 == q0:
            continue
        qs = qd[q0:q1].transpose(0, 1)[None]
        ks = kd[k0:k1].transpose(0, 1).repeat_interleave(rep, 0)[None]
        vs = vd[k0:k1].transpose(0, 1).repeat_interleave(rep, 0)[None]
        m = None
        if causal:
            m = _bottom_right(q1 - q0, k1 - k0)
        if key_mask is not None:
            km = key_mask[k0:k1]
            if km.dtype == torch.bool:
                km = km[None, :].expand(q1 - q0, -1)
                m = km if m is None else (m & km)
            else:
                add = km.to(dtype)[None, :].expand(q1 - q0, -1)
                if m is not None:
                    add = add.masked_fill(~m, -math.inf)
                m = add
        o = F.scaled_dot_product_attention(qs, ks, vs, attn_mask=m, scale=scale)
        outs.append(o[0].transpose(0, 1))
    out = torch.cat(outs, 0) if outs else qd.new_zeros((0, q.shape[1], v.shape[2]))
    if dout is None:
        return out.detach()
    out.backward(dout.to(dtype))
    zero = lambda t, ref: t.grad if t.grad is not None else torch.zeros_like(ref, dtype=dtype)
    return out.detach(), zero(qd, q), zero(kd, k), zero(vd, v)


def lse_varlen(q, k, v, cu_q, cu_k, causal=False, scale=None):
    """[H, Tq] float64 logsumexp per packed query (test_flash_varlen.py:314-341)."""
    rep = q.shape[1] // k.shape[1]
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    cols = []
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if q1 == q0:
            continue
        qs = q[q0:q1].double().transpose(0, 1)
        ks = k[k0:k1].double().transpose(0, 1).repeat_interleave(rep, 0)
        s = qs @ ks.transpose(-1, -2) * sc
        if causal:
            s = s.masked_fill(~_bottom_right(q1 - q0, k1 - k0), -math.inf)
        cols.append(torch.logsumexp(s, -1))
    return torch.cat(cols, -1)


# ---- the reference's CPU path: the same calls on the bf16 tensors -------------------

def cpu_dense(q, k, v, mask=None, causal=False, scale=None):
    """torch CPU SDPA on the bf16 tensors (bench/ops.py:542)."""
    gqa = q.shape[1] != k.shape[1]
    if causal and q.shape[2] != k.shape[2]:
        mask, causal = _top_left(q.shape[2], k.shape[2]), False
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=causal, scale=scale,
                                          enable_gqa=gqa)


def cpu_lengths(q, k, v, lengths, causal=False, scale=None):
    """kohakutt.torch_backend.lengths.masked on CPU tensors (lengths.py:79-89)."""
    keep = length_mask(torch.as_tensor(lengths), q.shape[2], k.shape[2], causal)
    return F.scaled_dot_product_attention(q, k, v, attn_mask=keep, scale=scale,
                                          enable_gqa=q.shape[1] != k.shape[1])


def cpu_varlen(q, k, v, cu_q, cu_k, causal=False, scale=None):
    return ruler_varlen(q, k, v, cu_q, cu_k, causal=causal, scale=scale, dtype=q.dtype)


# ---- the plain-C restatement (attention_ref.c) --------------------------------------

_C = None


def c_library(build=True):
    """libattention_ref.so, built by `make -C oracle` (gcc) on first use."""
    global _C
    if _C is not None:
        return _C
    path = os.path.join(_HERE, "_build", "libattention_ref.so")
    src = os.path.join(_HERE, "attention_ref.c")
    if build and (not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src)):
        import subprocess

        os.makedirs(os.path.dirname(path), exist_ok=True)
        subprocess.run(["gcc", "-O2", "-std=c11", "-shared", "-fPIC", "-o", path, src, "-lm"], check=True)
    lib = ctypes.CDLL(path)
    dp, ip, i, d = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_double
    lib.attn_ref_forward.argtypes = [dp, dp, dp, dp, ip, i, i, i, i, i, i, i, i, d, dp, dp]
    lib.attn_ref_backward.argtypes = [dp, dp, dp, dp, ip, dp, i, i, i, i, i, i, i, i, d, dp, dp, dp]
    _C = lib
    return lib


def _additive(mask, shape):
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        m = torch.zeros(mask.shape, dtype=torch.float64).masked_fill(~mask, -5e5)
    else:
        m = mask.double()
    while m.dim() < 4:
        m = m.unsqueeze(0)
    return m.expand(shape).contiguous()


def c_forward(q, k, v, mask=None, lengths=None, causal=0, scale=None):
    """(out, lse) in float64 from attention_ref.c; causal 0 none, 1 top-left, 2
    bottom-right."""
    lib = c_library()
    b, h, sq, d = q.shape
    hk, sk, dv = k.shape[1], k.shape[2], v.shape[3]
    qd, kd, vd = (t.double().contiguous() for t in (q, k, v))
    m = _additive(mask, (b, h, sq, sk))
    ln = None if lengths is None else torch.as_tensor(lengths, dtype=torch.int32).contiguous()
    out = torch.empty((b, h, sq, dv), dtype=torch.float64)
    lse = torch.empty((b, h, sq), dtype=torch.float64)
    sc = scale if scale is not None else 1.0 / math.sqrt(d)
    rc = lib.attn_ref_forward(
        qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), m.data_ptr() if m is not None else None,
        ln.data_ptr() if ln is not None else None, b, h, hk, sq, sk, d, dv, int(causal), sc,
        out.data_ptr(), lse.data_ptr())
    if rc:
        raise RuntimeError(f"attn_ref_forward failed ({rc})")
    return out, lse


def c_backward(q, k, v, dout, mask=None, lengths=None, causal=0, scale=None):
    """(dq, dk, dv) in float64 from attention_ref.c."""
    lib = c_library()
    b, h, sq, d = q.shape
    hk, sk, dv = k.shape[1], k.shape[2], v.shape[3]
    qd, kd, vd, dod = (t.double().contiguous() for t in (q, k, v, dout))
    m = _additive(mask, (b, h, sq, sk))
    ln = None if lengths is None else torch.as_tensor(lengths, dtype=torch.int32).contiguous()
    dq, dk, dvv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
    sc = scale if scale is not None else 1.0 / math.sqrt(d)
    rc = lib.attn_ref_backward(
        qd.data_ptr(), kd.data_ptr(), vd.data_ptr(), m.data_ptr() if m is not None else None,
        ln.data_ptr() if ln is not None else None, dod.data_ptr(), b, h, hk, sq, sk, d, dv,
        int(causal), sc, dq.data_ptr(), dk.data_ptr(), dvv.data_ptr())
    if rc:
        raise RuntimeError(f"attn_ref_backward failed ({rc})")
    return dq, dk, dvv
