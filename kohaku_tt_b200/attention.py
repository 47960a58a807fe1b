"""Attention entry points beyond torch's own: `sdpa(..., key_lengths=)` and
`sdpa_varlen`, with the argument meaning and error behaviour of kohakutt.sdpa and
kohakutt.sdpa_varlen (src/kohakutt/attention.py:10-76)."""

import torch
import torch.nn.functional as F

from . import aten, ops

# The logit of a key a bool mask leaves out, and the floor of an additive mask
# (kohakutt/torch_backend/varlen.py:163-165).
MASKED_LOGIT = -5e5


def _lengths_error(what):
    return ValueError(f"kohaku_tt_b200.sdpa: key_lengths must {what}")


def device_lengths(key_lengths, batch, keys, device):
    """One int32 length per batch row, resident on `device`.

    Host values (a sequence or a CPU tensor) are validated here, every one in [1, keys],
    and then copied over. Values already on a device cannot be inspected without a
    round trip, so they are only converted; the kernels clamp what they read to that
    range. The shape rule (rank 1, `batch` entries) holds for both. Messages and
    exception type follow kohakutt/torch_backend/lengths.py:10-29, which the callers'
    tests pin."""
    on_host = not (isinstance(key_lengths, torch.Tensor) and key_lengths.device.type != "cpu")
    values = torch.as_tensor(key_lengths, dtype=torch.int32) if on_host else key_lengths.to(torch.int32)
    if on_host and values.numel() > 0:
        low, high = int(values.min()), int(values.max())
        if low < 1 or high > keys:
            raise _lengths_error(f"lie in [1, {keys}], got {values.tolist()}")
    if values.dim() != 1 or values.size(0) != batch:
        raise _lengths_error(
            f"hold one length per batch ({batch}), got shape {tuple(values.shape)}"
        )
    return values.to(device) if on_host else values


class _Lengths(torch.autograd.Function):
    """Autograd node of the key-lengths route. The forward op hands back the row
    statistics with the output; they, the inputs and the lengths are what the backward
    op needs to produce dq, dk and dv. Nothing flows back to the lengths or the flags
    (the role of kohakutt/torch_backend/lengths.py:52-68, which recomputes the
    statistics instead of saving them)."""

    @staticmethod
    def forward(ctx, q, k, v, lengths, causal, scale):
        out, lse = torch.ops.ktt_b200._sdpa_lengths(q, k, v, lengths, causal, scale, True)
        ctx.causal, ctx.scale = causal, scale
        ctx.save_for_backward(out, lse, q, k, v, lengths)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        out, lse, q, k, v, lengths = ctx.saved_tensors
        grads = torch.ops.ktt_b200._sdpa_lengths_backward(
            grad_out.contiguous(), out, lse, q, k, v, lengths, ctx.causal, ctx.scale
        )
        return (*grads, None, None, None)


def sdpa(q, k, v, key_lengths=None, is_causal=False, scale=None):
    """Attention of q [B, H, Sq, D] over k [B, Hk, Sk, D] and v [B, Hk, Sk, Dv] in which
    batch row b may only look at its first key_lengths[b] keys.

    key_lengths holds B integers, each from 1 to Sk, as a list, a CPU tensor or a tensor
    on the device. No mask tensor is ever materialised: whole key blocks past a length are
    not visited and the block that straddles it is cut inside the kernel. The rule is
    about keys only; a query row whose index lies beyond the length still attends to the
    real keys. Without key_lengths this is F.scaled_dot_product_attention (grouped heads
    enabled when H != Hk). A call with a handful of query rows per key head and no
    gradient recording is served by the split-K decode kernel over a static KV cache.
    Same arguments and meaning as kohakutt.sdpa (src/kohakutt/attention.py:10-23)."""
    if key_lengths is None:
        return F.scaled_dot_product_attention(q, k, v, is_causal=is_causal, scale=scale,
                                              enable_gqa=q.size(1) != k.size(1))
    lengths = device_lengths(key_lengths, q.size(0), k.size(-2), q.device)
    causal = bool(is_causal)
    wants_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if wants_grad:
        return _Lengths.apply(q, k, v, lengths, causal, scale)
    return torch.ops.ktt_b200._sdpa_lengths(q, k, v, lengths, causal, scale, False)[0]


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
    """Host copy of a cumulative-offset vector as plain ints. Accepts any iterable of
    integers or an integer tensor; one that lives on a device costs a download (the role
    of kohakutt/torch_backend/varlen.py:23-28)."""
    host = cu_seq.detach().to("cpu").tolist() if isinstance(cu_seq, torch.Tensor) else list(cu_seq)
    return tuple(map(int, host))


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
    """Attention inside each sequence of a packed batch; the argument list of
    kohakutt.sdpa_varlen (src/kohakutt/attention.py:26-76).

    Layout: token-major bf16 tensors without padding, q [Tq, H, D], k [Tk, Hkv, D],
    v [Tk, Hkv, Dv], H divisible by Hkv. Sequence i owns query rows
    cu_seq_q[i]:cu_seq_q[i + 1] and key rows cu_seq_k[i]:cu_seq_k[i + 1]; both vectors
    start at 0 and end at the token count, and the key vector may be omitted when it
    equals the query one. They may be lists or integer tensors. A query never sees
    another sequence's keys. Under is_causal the diagonal is aligned to the end of the
    sequence: query r of a sequence with Lq queries and Lk keys sees keys
    0 .. r + Lk - Lq. The result is [Tq, H, Dv].

    attn_mask, when given, is a vector over the packed keys [Tk] shared by all heads and
    all queries of the key's sequence: booleans select keys (True = visible), floats are
    added to the logits and floored at -5e5. Masks of any other shape are rejected, and
    the mask receives no gradient.

    max_q / max_k default to the longest sequence found in the offsets. Offsets are
    validated on the host before anything is launched; the kernels then read their
    device copy."""
    causal = bool(is_causal)
    cu_q = offsets(cu_seq_q)
    cu_k = offsets(cu_seq_k) if cu_seq_k is not None else cu_q
    check_offsets(cu_q, cu_k, q.size(0), k.size(0), causal)

    def longest(cu):
        return max((hi - lo for lo, hi in zip(cu[:-1], cu[1:])), default=0)

    max_q = longest(cu_q) if max_q is None else max_q
    max_k = longest(cu_k) if max_k is None else max_k
    dev_q = torch.tensor(cu_q, dtype=torch.int32, device=q.device)
    dev_k = dev_q if cu_k == cu_q else torch.tensor(cu_k, dtype=torch.int32, device=q.device)
    if attn_mask is None:
        aten.install()
        window = [-1, 0] if causal else [-1, -1]
        return torch.ops.torch_attn._varlen_attn(q, k, v, dev_q, dev_k, max_q, max_k, causal,
                                                 scale, window)[0]
    if attn_mask.dim() != 1 or attn_mask.size(0) != k.size(0):
        raise ValueError(
            f"kohaku_tt_b200.sdpa_varlen: attn_mask must be [{k.size(0)}] "
            f"(one value per packed key), got {tuple(attn_mask.shape)}"
        )
    return _Masked.apply(q, k, v, attn_mask.to(q.device), dev_q, dev_k, max_q, max_k, causal, scale)
