"""Attention entry points beyond torch's own: `sdpa(..., key_lengths=)` and
`sdpa_varlen`, with the argument meaning and error behaviour of kohakutt.sdpa and
kohakutt.sdpa_varlen (src/kohakutt/attention.py:10-76)."""

import torch
import torch.nn.functional as F

from . import aten, ops

# The logit of a key a bool mask leaves out, and the floor of an additive mask
# (kohakutt/torch_backend/varlen.py:163-165).
MASKED_LOGIT = -5e5


def device_lengths(key_lengths, batch, keys, device):
    """`key_lengths` as an int32 [batch] tensor on `device`. A list or a CPU tensor is
    checked (1 <= length <= keys) and uploaded; a device tensor is used as it is (no
    download: the kernel clamps its values to [1, keys]). Same checks and messages as
    kohakutt/torch_backend/lengths.py:10-29."""
    if isinstance(key_lengths, torch.Tensor) and key_lengths.device.type != "cpu":
        lengths = key_lengths.to(torch.int32)
    else:
        lengths = torch.as_tensor(key_lengths, dtype=torch.int32)
        if lengths.numel() and (lengths.min() < 1 or lengths.max() > keys):
            raise ValueError(
                f"kohaku_tt_b200.sdpa: key_lengths must lie in [1, {keys}], "
                f"got {lengths.tolist()}"
            )
        lengths = lengths.to(device)
    if lengths.dim() != 1 or lengths.size(0) != batch:
        raise ValueError(
            f"kohaku_tt_b200.sdpa: key_lengths must hold one length per batch ({batch}), "
            f"got shape {tuple(lengths.shape)}"
        )
    return lengths


class _Lengths(torch.autograd.Function):
    """The kernel route with gradients: output and dq, dk, dv; the lengths get none
    (lengths.py:52-68)."""

    @staticmethod
    def forward(ctx, q, k, v, lengths, causal, scale):
        out, lse = torch.ops.ktt_b200._sdpa_lengths(q, k, v, lengths, causal, scale, True)
        ctx.save_for_backward(q, k, v, lengths, out, lse)
        ctx.args = (causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, lengths, out, lse = ctx.saved_tensors
        causal, scale = ctx.args
        dq, dk, dv = torch.ops.ktt_b200._sdpa_lengths_backward(
            grad.contiguous(), out, lse, q, k, v, lengths, causal, scale
        )
        return dq, dk, dv, None, None, None


def sdpa(q, k, v, key_lengths=None, is_causal=False, scale=None):
    """F.scaled_dot_product_attention of q [B, H, Sq, D], k / v [B, Hk, Sk, D / Dv] with
    the key mask key < key_lengths[b] (B ints in [1, Sk]: list, CPU or CUDA tensor),
    built nowhere: the kernel skips and masks those keys. Query rows past a length see
    the real keys. With few query rows and no gradients this is the split-K decode
    kernel over a static KV cache."""
    gqa = q.size(1) != k.size(1)
    if key_lengths is None:
        return F.scaled_dot_product_attention(
            q, k, v, is_causal=is_causal, scale=scale, enable_gqa=gqa
        )
    lengths = device_lengths(key_lengths, q.size(0), k.size(-2), q.device)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v)):
        return _Lengths.apply(q, k, v, lengths, bool(is_causal), scale)
    out, _ = torch.ops.ktt_b200._sdpa_lengths(q, k, v, lengths, bool(is_causal), scale, False)
    return out


def decode_step(q, k_new, v_new, k_cache, v_cache, lengths, cos, sin, scale=None, lengths_out=None):
    """One decode token in one kernel: rotate-half rotary on q [B, H, 1, D] and k_new
    [B, Hk, 1, D], the static cache's row lengths[b] <- (rotated key, v_new), attention over
    the lengths[b] + 1 keys. In the reference these are three ops (ktt.rotary twice,
    StaticCache's index_copy_, sdpa with key_lengths), the cache write alone a fifth of a
    decode token. lengths: int32 [B] on the device, keys already cached; cos / sin: bf16
    [B, D] rows for this step, or a [positions, D] table looked up at lengths[b]. No
    gradients. Returns out [B, H, 1, D]; k_cache / v_cache are updated in place and
    lengths_out (optional, another buffer) receives lengths + 1."""
    from . import ops

    with torch.no_grad():
        return ops.decode_append(q, k_new, v_new, k_cache, v_cache, lengths, cos, sin,
                                 scale=scale, lengths_out=lengths_out)


def offsets(cu_seq):
    """Cumulative sequence offsets as a tuple of ints (a list or an int tensor; a device
    tensor is downloaded) (varlen.py:23-28)."""
    if isinstance(cu_seq, torch.Tensor):
        return tuple(int(x) for x in cu_seq.detach().cpu().tolist())
    return tuple(int(x) for x in cu_seq)


def check_offsets(cu_q, cu_k, tokens_q, tokens_k, causal):
    """The host checks of varlen::intervals (ktt_flash/varlen_plan.hpp:43-82) and of the
    packed op (aten_varlen.cpp:165-231) on offsets known on the host."""
    if len(cu_q) < 2 or len(cu_q) != len(cu_k) or cu_q[0] != 0 or cu_k[0] != 0:
        raise RuntimeError(
            "kohaku_tt_b200: sdpa_varlen needs cumulative offsets [0, ..., total] of "
            "equal count for queries and keys"
        )
    if cu_q[-1] != tokens_q or cu_k[-1] != tokens_k:
        raise RuntimeError(
            "kohaku_tt_b200: sdpa_varlen offsets must end at the token count "
            f"({tokens_q} queries, {tokens_k} keys), got {cu_q[-1]} and {cu_k[-1]}"
        )
    for b in range(len(cu_q) - 1):
        lq, lk = cu_q[b + 1] - cu_q[b], cu_k[b + 1] - cu_k[b]
        if lq < 0 or lk < 0 or (lq > 0 and lk == 0):
            raise RuntimeError(
                "kohaku_tt_b200: sdpa_varlen offsets must not decrease, and a sequence "
                "with queries needs keys"
            )
        if causal and lq > lk:
            raise RuntimeError(
                "kohaku_tt_b200: causal sdpa_varlen with more queries than keys in a "
                "sequence leaves queries without keys"
            )


class _Masked(torch.autograd.Function):
    """Packed attention with a key mask: the forward and its dq, dk, dv; the mask gets no
    gradient (varlen.py:187-235)."""

    @staticmethod
    def forward(ctx, q, k, v, mask, cu_q, cu_k, max_q, max_k, causal, scale):
        out, lse = ops.varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, causal=causal,
                                      scale=scale, key_mask=mask)
        ctx.save_for_backward(q, k, v, mask, cu_q, cu_k, out, lse)
        ctx.args = (max_q, max_k, causal, scale)
        return out

    @staticmethod
    def backward(ctx, grad):
        q, k, v, mask, cu_q, cu_k, out, lse = ctx.saved_tensors
        max_q, max_k, causal, scale = ctx.args
        dq, dk, dv = ops.varlen_backward(grad, q, k, v, out, lse, cu_q, cu_k, max_q, max_k,
                                         causal=causal, scale=scale, key_mask=mask)
        return dq, dk, dv, None, None, None, None, None, None, None


def sdpa_varlen(q, k, v, cu_seq_q, cu_seq_k=None, max_q=None, max_k=None, is_causal=False,
                scale=None, attn_mask=None):
    """Scaled dot-product attention over packed variable-length sequences.

    q [Tq, H, D], k [Tk, Hkv, D] and v [Tk, Hkv, Dv] (bf16, H a multiple of Hkv) hold the
    tokens of every sequence back to back; nothing is padded. cu_seq_q / cu_seq_k are the
    cumulative sequence offsets [0, ..., total] (a list or an int tensor; cu_seq_k
    defaults to cu_seq_q). Each query attends to the keys of its own sequence; with
    is_causal query r of a sequence sees its first min(Lk, r + 1 + Lk - Lq) keys.
    Returns [Tq, H, Dv].

    attn_mask: a key mask [Tk], one value per packed key, for every query of the key's
    sequence and every head. Bool: True keeps the key. Float: added to the key's scores
    (clamped at -5e5). It gets no gradient. Other mask shapes are not taken.

    Offsets given on the host are checked there; the kernels read them on the device.
    """
    cu_q = offsets(cu_seq_q)
    cu_k = cu_q if cu_seq_k is None else offsets(cu_seq_k)
    check_offsets(cu_q, cu_k, q.size(0), k.size(0), bool(is_causal))
    lengths_q = [b - a for a, b in zip(cu_q, cu_q[1:])]
    lengths_k = [b - a for a, b in zip(cu_k, cu_k[1:])]
    max_q = max(lengths_q, default=0) if max_q is None else max_q
    max_k = max(lengths_k, default=0) if max_k is None else max_k
    dev_q = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
    dev_k = dev_q if cu_k == cu_q else torch.tensor(cu_k, dtype=torch.int32, device=q.device)
    if attn_mask is not None:
        if attn_mask.dim() != 1 or attn_mask.size(0) != k.size(0):
            raise ValueError(
                f"kohaku_tt_b200.sdpa_varlen: attn_mask must be [{k.size(0)}] "
                f"(one value per packed key), got {tuple(attn_mask.shape)}"
            )
        mask = attn_mask.to(q.device)
        return _Masked.apply(q, k, v, mask, dev_q, dev_k, max_q, max_k, bool(is_causal), scale)
    aten.install()
    out, _, _ = torch.ops.torch_attn._varlen_attn(
        q, k, v, dev_q, dev_k, max_q, max_k, bool(is_causal), scale,
        [-1, 0] if is_causal else [-1, -1],
    )
    return out
