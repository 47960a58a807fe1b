"""The operator surface: aten fused-SDPA overloads on the CUDA key, torch's packed
varlen ops, and this package's own key-lengths ops.

The reference registers `_fused_sdp_choice` and the `_scaled_dot_product_fused_attention_
overrideable` pair for its device (aten_attention.cpp:959-974). For CUDA tensors PyTorch's
SDPA composite asks its own backend chooser and then calls one of three fused overloads
(flash, efficient, cuDNN); all three, their backwards, and the overrideable pair are
pointed at the kernels of this package, so `F.scaled_dot_product_attention` lands here
whatever the chooser picks. Nothing is registered until install() is called.
"""

import math

import torch

from . import _lib, ops
from .numerics import current_kernels

SDP_MATH, SDP_FLASH, SDP_EFFICIENT, SDP_CUDNN, SDP_OVERRIDEABLE = 0, 1, 2, 3, 4

_ATEN = None
_INSTALLED = False


def fused_refusal(q, k, v, mask, dropout_p, is_causal, scale):
    """None when the fused kernels take the call, else the first condition it fails.
    The rules of fused_refusal (aten_attention.cpp:62-127), minus the ones that only
    describe Tensix limits (grouped heads with gradients are taken here)."""
    grads = torch.is_grad_enabled() and any(t.requires_grad for t in (q, k, v))
    for t in (q, k, v):
        ok_dtype = t.dtype == torch.bfloat16 or (t.dtype == torch.float32 and not grads)
        if t.dim() != 4 or t.numel() == 0 or not ok_dtype or t.dtype != q.dtype:
            return "q, k and v must be non-empty 4-D bf16 (fp32 without gradients)"
    if dropout_p != 0.0:
        return "dropout"
    if k.size(3) != q.size(3):
        return "q and k need one head dim"
    if (k.size(0) != q.size(0) or v.size(0) != q.size(0) or v.size(1) != k.size(1)
            or q.size(1) % k.size(1) != 0 or v.size(2) != k.size(2)):
        return "q, k and v shapes do not match (K / V heads must divide Q heads)"
    if max(q.size(3), v.size(3)) > 256:
        return "head dims above 256 are not taken"
    if is_causal and mask is not None:
        return "causal takes no mask"
    if mask is not None:
        if mask.dim() > 4:
            return "the mask must broadcast to [B, H, Sq, Sk]"
        full = (q.size(0), q.size(1), q.size(2), k.size(2))
        for i in range(mask.dim()):
            s = mask.size(mask.dim() - 1 - i)
            if s != 1 and s != full[3 - i]:
                return "the mask must broadcast to [B, H, Sq, Sk]"
    return None


def _describe(t):
    return f"{list(t.shape)} {str(t.dtype).replace('torch.', '')}"


def refuse_attention(q, k, v, mask, is_causal, kernels, why):
    """Raises the scope refusal, worded like refuse_attention
    (aten_attention.cpp:157-192)."""
    m = "none"
    if mask is not None:
        m = ("bool " if mask.dtype == torch.bool else "additive ") + _describe(mask)
    names = ", ".join(repr(k_) for k_ in kernels)
    raise RuntimeError(
        f"kohaku_tt_b200.sdpa_kernel({names}): no allowed kernel takes attention q "
        f"{_describe(q)}, k {_describe(k)}, v {_describe(v)}, mask {m}"
        f"{', causal' if is_causal else ''}: {why}"
    )


def fused_backends_enabled():
    """True unless torch's own switch (`torch.nn.attention.sdpa_kernel`, the
    `torch.backends.cuda.enable_*_sdp` flags) has turned off every fused backend whose
    overload lands in this package: flash, efficient, cuDNN and overrideable. The
    reference asks the one switch its overload sits behind
    (`userEnabledOverrideableSDP`, aten_attention.cpp:204-207)."""
    c = torch._C
    return bool(c._get_flash_sdp_enabled() or c._get_mem_efficient_sdp_enabled()
                or c._get_cudnn_sdp_enabled() or c._get_overrideable_sdp_enabled())


def fused_sdp_choice(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False, *,
                     scale=None, enable_gqa=False):
    """aten::_fused_sdp_choice: SDP_OVERRIDEABLE (4) when the fused kernels take the
    call, SDP_MATH (0) when they refuse it or when torch's `sdpa_kernel` context has the
    fused backends off (tt_fused_sdp_choice, aten_attention.cpp:194-219;
    tests/hardware/ops/test_attention.py:63-67)."""
    if not fused_backends_enabled():
        return SDP_MATH
    why = fused_refusal(q, k, v, attn_mask, dropout_p, is_causal, scale)
    if why is None:
        return SDP_OVERRIDEABLE
    return SDP_MATH


def _checked(q, k, v, mask, dropout_p, is_causal, scale):
    why = fused_refusal(q, k, v, mask, dropout_p, is_causal, scale)
    if why is not None:
        kernels = current_kernels()
        if tuple(kernels) != ("flash", "mma"):
            refuse_attention(q, k, v, mask, is_causal, kernels, why)
        raise _lib.UnsupportedAttention(
            f"kohaku_tt_b200: fused attention refused: {why}. On CUDA PyTorch picks the fused "
            "overload itself, so a refused call cannot fall back to the math composite from "
            "here: wrap it in torch.nn.attention.sdpa_kernel(SDPBackend.MATH), or call "
            "kohaku_tt_b200.uninstall()")


def _as_bf16(q, k, v):
    """fp32 inputs without gradients are cast at entry and the output cast back
    (aten_attention.cpp:400-415)."""
    if q.dtype == torch.float32:
        return q.to(torch.bfloat16), k.to(torch.bfloat16), v.to(torch.bfloat16), True
    return q, k, v, False


def _out_like(q, dv):
    """Output laid out the way torch's meta kernels of the flash, cuDNN and overrideable
    overloads promise (`empty_like(query)`: the query's stride order), so compiled graphs
    that trust the meta strides index it correctly."""
    if dv == q.size(3):
        return torch.empty_like(q)
    order = sorted(range(4), key=lambda i: (q.stride(i), -i), reverse=True)   # slowest dim first
    shape = (q.size(0), q.size(1), q.size(2), dv)
    out = torch.empty([shape[i] for i in order], dtype=q.dtype, device=q.device)
    return out.permute([order.index(i) for i in range(4)])


def _out_efficient(q, dv):
    """The efficient overload's meta promises [B, Sq, H, Dv] storage seen as [B, H, Sq, Dv]."""
    return torch.empty((q.size(0), q.size(2), q.size(1), dv), dtype=q.dtype, device=q.device).transpose(1, 2)


def _bias_or_none(attn_bias):
    """Autograd hands a backward an undefined or empty tensor when the forward had no
    bias."""
    if attn_bias is None or attn_bias.numel() == 0:
        return None
    return attn_bias


def _empty(device, dtype=torch.int64):
    return torch.empty((0,), dtype=dtype, device=device)


def _rng(device):
    # Dropout is refused, so nobody reads the generator state: left unwritten (a zero fill
    # would be one more kernel launch on every attention call).
    return torch.empty((2,), dtype=torch.uint64, device=device), torch.empty((), dtype=torch.uint64, device=device)


def _seed_pair(device):
    """Philox seed and offset outputs of the fused ops: unwritten, for the same reason."""
    return torch.empty((), dtype=torch.int64, device=device), torch.empty((), dtype=torch.int64, device=device)


# ---- aten::_scaled_dot_product_flash_attention (+ backward) ------------------------

def _flash_forward(q, k, v, dropout_p=0.0, is_causal=False, return_debug_mask=False, *, scale=None):
    _checked(q, k, v, None, dropout_p, is_causal, scale)
    qb, kb, vb, cast = _as_bf16(q, k, v)
    out, lse = ops.sdpa_forward(qb, kb, vb, causal=is_causal, scale=scale, out=_out_like(qb, vb.size(3)))
    if cast:
        out = out.to(torch.float32)
    seed, offset = _rng(q.device)
    return (out, lse, _empty(q.device), _empty(q.device), q.size(2), k.size(2), seed, offset,
            _empty(q.device, q.dtype))


def _flash_backward(grad_out, q, k, v, out, logsumexp, cum_seq_q, cum_seq_k, max_q, max_k,
                    dropout_p, is_causal, philox_seed, philox_offset, *, scale=None):
    _checked(q, k, v, None, dropout_p, is_causal, scale)
    return ops.sdpa_backward(grad_out, q, k, v, out, logsumexp, causal=is_causal, scale=scale)


# ---- aten::_scaled_dot_product_efficient_attention (+ backward) --------------------

def _efficient_forward(q, k, v, attn_bias, compute_log_sumexp, dropout_p=0.0, is_causal=False, *, scale=None):
    _checked(q, k, v, attn_bias, dropout_p, is_causal, scale)
    qb, kb, vb, cast = _as_bf16(q, k, v)
    rows = (q.size(2) + 31) // 32 * 32
    out, lse = ops.sdpa_forward(qb, kb, vb, mask=attn_bias, causal=is_causal, scale=scale,
                                need_lse=bool(compute_log_sumexp), lse_rows=rows,
                                out=_out_efficient(qb, vb.size(3)))
    if lse is None:
        lse = torch.empty((q.size(0), q.size(1), 0), dtype=torch.float32, device=q.device)
    if cast:
        out = out.to(torch.float32)
    seed, offset = _seed_pair(q.device)
    return out, lse, seed, offset


def _bias_gradient(grad_out, q, k, v, attn_bias, logsumexp, is_causal, scale):
    """Gradient of an additive bias: dS summed over the dims the bias broadcasts,
    recomputed with separate matmul / softmax steps as the reference's masked backward
    does (aten_attention.cpp:781-811)."""
    rep = q.size(1) // k.size(1)
    kf = k.float().repeat_interleave(rep, 1)
    vf = v.float().repeat_interleave(rep, 1)
    sc = scale if scale is not None else 1.0 / math.sqrt(q.size(3))
    s = torch.matmul(q.float(), kf.transpose(-1, -2)) * sc + attn_bias.float().clamp_min(-5e5)
    p = torch.softmax(s, dim=-1)
    dp = torch.matmul(grad_out.float(), vf.transpose(-1, -2))
    ds = p * (dp - (dp * p).sum(-1, keepdim=True))
    bias = attn_bias
    while bias.dim() < 4:
        bias = bias.unsqueeze(0)
    dims = [i for i in range(4) if bias.size(i) == 1 and ds.size(i) != 1]
    if dims:
        ds = ds.sum(dims, keepdim=True)
    return ds.reshape(attn_bias.shape).to(attn_bias.dtype)


def _efficient_backward(grad_out, q, k, v, attn_bias, out, logsumexp, philox_seed, philox_offset,
                        dropout_p, grad_input_mask, is_causal=False, *, scale=None):
    attn_bias = _bias_or_none(attn_bias)
    _checked(q, k, v, attn_bias, dropout_p, is_causal, scale)
    dq, dk, dv = ops.sdpa_backward(grad_out, q, k, v, out, logsumexp, mask=attn_bias,
                                   causal=is_causal, scale=scale)
    dbias = None
    if attn_bias is not None and len(grad_input_mask) > 3 and grad_input_mask[3]:
        dbias = _bias_gradient(grad_out, q, k, v, attn_bias, logsumexp, is_causal, scale)
    return dq, dk, dv, dbias


# ---- aten::_scaled_dot_product_cudnn_attention (+ backward) ------------------------

def _cudnn_forward(q, k, v, attn_bias, compute_log_sumexp, dropout_p=0.0, is_causal=False,
                   return_debug_mask=False, *, scale=None):
    _checked(q, k, v, attn_bias, dropout_p, is_causal, scale)
    qb, kb, vb, cast = _as_bf16(q, k, v)
    out, lse = ops.sdpa_forward(qb, kb, vb, mask=attn_bias, causal=is_causal, scale=scale,
                                need_lse=True, out=_out_like(qb, vb.size(3)))
    if cast:
        out = out.to(torch.float32)
    seed, offset = _seed_pair(q.device)
    return (out, lse.unsqueeze(-1), _empty(q.device), _empty(q.device), q.size(2), k.size(2),
            seed, offset, _empty(q.device, q.dtype))


def _cudnn_backward(grad_out, q, k, v, out, logsumexp, philox_seed, philox_offset, attn_bias,
                    cum_seq_q, cum_seq_k, max_q, max_k, dropout_p, is_causal, *, scale=None):
    attn_bias = _bias_or_none(attn_bias)
    _checked(q, k, v, attn_bias, dropout_p, is_causal, scale)
    lse = logsumexp.squeeze(-1) if logsumexp.dim() == 4 else logsumexp
    return ops.sdpa_backward(grad_out, q, k, v, out, lse.contiguous(), mask=attn_bias,
                             causal=is_causal, scale=scale)


# ---- aten::_scaled_dot_product_fused_attention_overrideable (+ backward) -----------
# The reference's own surface (tt_sdpa_overrideable, aten_attention.cpp:389-713, and its
# backward, :715-812).

def _overrideable_forward(q, k, v, attn_bias=None, dropout_p=0.0, is_causal=False,
                          return_debug_mask=False, *, scale=None):
    _checked(q, k, v, attn_bias, dropout_p, is_causal, scale)
    qb, kb, vb, cast = _as_bf16(q, k, v)
    out, lse = ops.sdpa_forward(qb, kb, vb, mask=attn_bias, causal=is_causal, scale=scale,
                                out=_out_like(qb, vb.size(3)))
    if cast:
        out = out.to(torch.float32)
    seed, offset = _seed_pair(q.device)
    return (out, lse, _empty(q.device), _empty(q.device), q.size(2), k.size(2), seed, offset,
            _empty(q.device, q.dtype))


def _overrideable_backward(grad_out, q, k, v, attn_bias, grad_input_mask, out, logsumexp, cum_seq_q,
                           cum_seq_k, max_q, max_k, dropout_p, is_causal, philox_seed, philox_offset,
                           *, scale=None):
    bias = _bias_or_none(attn_bias)
    _checked(q, k, v, bias, dropout_p, is_causal, scale)
    dq, dk, dv = ops.sdpa_backward(grad_out, q, k, v, out, logsumexp, mask=bias,
                                   causal=is_causal, scale=scale)
    dbias = None
    if bias is not None and len(grad_input_mask) > 3 and grad_input_mask[3]:
        dbias = _bias_gradient(grad_out, q, k, v, bias, logsumexp, is_causal, scale)
    if dbias is None:
        dbias = _empty(q.device, q.dtype)
    return dq, dk, dv, dbias


# ---- key-lengths ops (ktt::_sdpa_lengths*, aten_lengths.cpp:69-149,175-196) ----------

@torch.library.custom_op("ktt_b200::_sdpa_lengths", mutates_args=(), device_types="cuda")
def _sdpa_lengths(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, lengths: torch.Tensor,
                  is_causal: bool, scale: float | None, stats: bool) -> tuple[torch.Tensor, torch.Tensor]:
    if not stats and not is_causal and ops.decode_takes(q, k, v):
        # lse always has its full shape, so that the fake kernel below (which cannot ask
        # about pointers) describes every route.
        return ops.decode(q, k, v, key_lengths=lengths, scale=scale, need_lse=True)
    out, lse = ops.sdpa_forward(q, k, v, key_lengths=lengths, causal=is_causal, scale=scale,
                                need_lse=True)
    return out, lse


@_sdpa_lengths.register_fake
def _(q, k, v, lengths, is_causal, scale, stats):
    # The same layout rule as the real op: [B, S, H, Dv] storage for head views of a
    # [B, S, H * D] tensor on the prefill route, contiguous otherwise (ops._out_like_query).
    b, h, s, d = q.shape
    decode_route = not stats and not is_causal and (h // max(k.size(1), 1)) * s <= 16 and d in (64, 128) and v.size(3) == d
    if not decode_route and ops.is_head_view(q):
        out = q.new_empty((b, s, h, v.size(3))).transpose(1, 2)
    else:
        out = q.new_empty((b, h, s, v.size(3)))
    return out, q.new_empty((b, h, s), dtype=torch.float32)


@torch.library.custom_op("ktt_b200::_sdpa_lengths_backward", mutates_args=(), device_types="cuda")
def _sdpa_lengths_backward(grad: torch.Tensor, out: torch.Tensor, lse: torch.Tensor, q: torch.Tensor,
                           k: torch.Tensor, v: torch.Tensor, lengths: torch.Tensor, is_causal: bool,
                           scale: float | None) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    return ops.sdpa_backward(grad, q, k, v, out, lse, key_lengths=lengths, causal=is_causal, scale=scale)


@_sdpa_lengths_backward.register_fake
def _(grad, out, lse, q, k, v, lengths, is_causal, scale):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


# ---- packed varlen ops (torch_attn::_varlen_attn*, kohakutt/torch_backend/varlen.py) ----

_FULL_WINDOW, _CAUSAL_WINDOW = (-1, -1), (-1, 0)


def _causal(is_causal, window_size):
    """Folds torch's (left, right) attention window into the causal flag. Only the two
    windows that mean "everything" and "everything up to the diagonal" exist here; a
    sliding window is refused rather than silently widened (the contract of
    kohakutt/torch_backend/varlen.py:107-114)."""
    window = _FULL_WINDOW if window_size is None else tuple(window_size)
    if window == _CAUSAL_WINDOW:
        return True
    if window != _FULL_WINDOW:
        raise NotImplementedError(
            "kohaku_tt_b200: varlen attention takes window_size (-1, -1) or (-1, 0)"
        )
    return bool(is_causal)


def _unsupported(**given):
    """Refuses optional arguments of torch's packed op that have no kernel behind them
    (paged caches, per-sequence used lengths): any that was actually passed is named."""
    passed = sorted(name for name in given if given[name] is not None)
    if passed:
        raise NotImplementedError(
            "kohaku_tt_b200: varlen attention does not support " + ", ".join(passed)
        )


def _varlen_forward(query, key, value, cu_seq_q, cu_seq_k, max_q, max_k, is_causal=False,
                    scale=None, window_size=None, enable_gqa=False, seqused_k=None,
                    block_table=None, num_splits=None, backend=1):
    """torch_attn::_varlen_attn on CUDA: (output [Tq, H, Dv], log-sum-exp [H, Tq], rng
    state) (varlen.py:62-104)."""
    _unsupported(seqused_k=seqused_k, block_table=block_table)
    causal = _causal(is_causal, window_size)
    cu_q = cu_seq_q.to(device=query.device, dtype=torch.int32).contiguous()
    cu_k = cu_q if cu_seq_k is None else cu_seq_k.to(device=query.device, dtype=torch.int32).contiguous()
    out, lse = ops.varlen_forward(query, key, value, cu_q, cu_k, max_q, max_k, causal=causal, scale=scale)
    return out, lse, torch.empty((2,), dtype=torch.uint64, device=query.device)


def _varlen_backward(grad_out, query, key, value, out, lse, cu_seq_q, cu_seq_k, max_q, max_k,
                     is_causal, rng_state, scale=None, window_size=None, backend=1):
    """torch_attn::_varlen_attn_backward on CUDA: (dq, dk, dv) packed as query, key,
    value (varlen.py:117-160)."""
    causal = _causal(is_causal, window_size)
    cu_q = cu_seq_q.to(device=query.device, dtype=torch.int32).contiguous()
    cu_k = cu_q if cu_seq_k is None else cu_seq_k.to(device=query.device, dtype=torch.int32).contiguous()
    return ops.varlen_backward(grad_out, query, key, value, out, lse, cu_q, cu_k, max_q, max_k,
                               causal=causal, scale=scale)


_VARLEN_DONE = False
_USING_SHIM = False


def using_cpp_registration():
    """True when the aten overloads are registered from C++ (csrc/torch_shim), False when
    the Python registration below stands in."""
    return _INSTALLED and _USING_SHIM


def install(python=None):
    """Points the CUDA kernels of the aten fused-SDPA overloads, `_fused_sdp_choice` and
    torch's packed varlen ops at this package. Idempotent. Raises when the library is
    missing: a silent PyTorch route would defeat the point of installing.

    The overloads are registered from C++ (a TORCH_LIBRARY-style block in
    csrc/torch_shim/aten_shim.cpp, as the reference registers its own,
    aten_attention.cpp:959-974) when that shim has been built; `python=True` (or the
    environment variable KTT_B200_PYTHON_ATEN=1) asks for the Python registration below,
    which is also the stand-in when the shim is missing."""
    global _ATEN, _INSTALLED, _VARLEN_DONE, _USING_SHIM
    if _INSTALLED:
        return
    _lib.lib()
    import os
    import warnings

    if python is None:
        python = os.environ.get("KTT_B200_PYTHON_ATEN", "0") == "1"
    handle = None if python else _lib.shim()
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")  # "overriding a previously registered kernel"
        if handle is not None:
            if handle.ktt_b200_aten_install() != 0:
                raise RuntimeError("kohaku_tt_b200: the C++ registration of the aten overloads failed")
            _USING_SHIM = True
            from .numerics import _tell_shim

            _tell_shim()
        else:
            _USING_SHIM = False
            _register_python()
        if not _VARLEN_DONE:
            from torch.nn.attention import varlen

            varlen._varlen_attn.register_kernel("cuda")(_varlen_forward)
            varlen._varlen_attn_backward.register_kernel("cuda")(_varlen_backward)
            _VARLEN_DONE = True
    _INSTALLED = True


def _register_python():
    """The same overloads registered from Python (torch.library)."""
    global _ATEN
    _ATEN = torch.library.Library("aten", "IMPL")
    if True:
        table = {
            "_scaled_dot_product_flash_attention": _flash_forward,
            "_scaled_dot_product_flash_attention_backward": _flash_backward,
            "_scaled_dot_product_efficient_attention": _efficient_forward,
            "_scaled_dot_product_efficient_attention_backward": _efficient_backward,
            "_scaled_dot_product_cudnn_attention": _cudnn_forward,
            "_scaled_dot_product_cudnn_attention_backward": _cudnn_backward,
            "_scaled_dot_product_fused_attention_overrideable": _overrideable_forward,
            "_scaled_dot_product_fused_attention_overrideable_backward": _overrideable_backward,
            "_fused_sdp_choice": fused_sdp_choice,
        }
        for name, fn in table.items():
            _ATEN.impl(name, fn, "CUDA")


def uninstall():
    """Takes the aten overloads of install() back out: PyTorch's own CUDA kernels answer
    again. (The packed varlen ops of torch.nn.attention.varlen keep this package's kernels:
    custom-op kernels cannot be unregistered.)"""
    global _ATEN, _INSTALLED, _USING_SHIM
    if _ATEN is not None:
        _ATEN._destroy()
        _ATEN = None
    if _USING_SHIM:
        _lib.shim().ktt_b200_aten_uninstall()
        _USING_SHIM = False
    _INSTALLED = False


class installed_for:
    """`with installed_for(): ...` installs the overloads for the block and takes them out
    again if they were not installed before it."""

    def __enter__(self):
        self.was = _INSTALLED
        install()
        return self

    def __exit__(self, *exc):
        if not self.was:
            uninstall()
        return False


def installed():
    return _INSTALLED
