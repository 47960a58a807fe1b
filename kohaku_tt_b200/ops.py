"""Tensor-level entry points over the C ABI: forward, backward, packed and decode calls.

Torch is plumbing here: it owns device memory and the current stream, and hands raw
pointers, sizes and element strides to libktt_b200.so. Every function fails loudly when
the library is missing or refuses the call; nothing falls back to PyTorch math.
"""

import ctypes
import math

import torch

from . import _lib
from .numerics import current_kernels

_MASK_DTYPES = {
    torch.bool: _lib.MASK_BOOL,
    torch.uint8: _lib.MASK_BOOL,
    torch.bfloat16: _lib.MASK_BF16,
    torch.float32: _lib.MASK_F32,
    torch.float16: _lib.MASK_F16,
}

# 'flash' = the TMA + tcgen05 kernels, 'flash_wide' = the head-dim-128 tcgen05 forward's design also
# at head dim 64 (where 'flash' runs the two-stream kernel), 'mma' = warp MMA.
_KERNELS = {"auto": _lib.KERNEL_AUTO, "mma": _lib.KERNEL_MMA, "flash": _lib.KERNEL_TC5,
            "flash_wide": _lib.KERNEL_TC5_WIDE}


def _kernel_code(kernel):
    """`kernel` ('auto', 'flash' = TMA + tcgen05, 'mma' = warp MMA) narrowed by the
    enclosing sdpa_kernel scope."""
    allowed = current_kernels()
    if kernel == "auto":
        if set(allowed) >= {"flash", "mma"}:
            return _lib.KERNEL_AUTO
        if "flash" in allowed:
            return _lib.KERNEL_TC5
        if "mma" in allowed:
            return _lib.KERNEL_MMA
        raise RuntimeError(
            f"kohaku_tt_b200.sdpa_kernel({allowed!r}): no device kernel is allowed and "
            "there is no math fallback"
        )
    if kernel not in _KERNELS:
        raise ValueError(f"kohaku_tt_b200: unknown kernel {kernel!r}")
    return _KERNELS[kernel]


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "kohaku_tt_b200: attention runs on CUDA tensors only "
                f"(got a {t.device.type} tensor); there is no CPU fallback"
            )


def _rows_contiguous(t):
    """`t` with a unit innermost stride (head views pass through untouched)."""
    return t if t.stride(-1) == 1 else t.contiguous()


def _bhs_strides(t):
    """(batch, head, row) element strides of a [B, H, S, D] tensor."""
    return (t.stride(0), t.stride(1), t.stride(2))


def _ths_strides(t):
    """(batch = 0, head, row) element strides of a packed [T, H, D] tensor."""
    return (0, t.stride(1), t.stride(0))


def _set3(field, values):
    for i, v in enumerate(values):
        field[i] = int(v)


def is_head_view(q):
    """True when q [B, H, S, D] is a head view of a [B, S, H*D] (or fused qkv) storage."""
    b, h, s, d = q.shape
    return h > 1 and s > 1 and q.stride(1) == d and q.stride(2) >= h * d


def _out_like_query(q, dv):
    """Output [B, H, Sq, Dv]: laid out [B, Sq, H, Dv] when q is a head view of a
    [B, S, H*D] storage (the reference's pitched route, aten_attention.cpp:605-628),
    else contiguous."""
    b, h, s, d = q.shape
    if is_head_view(q):
        return torch.empty((b, s, h, dv), dtype=q.dtype, device=q.device).transpose(1, 2)
    return torch.empty((b, h, s, dv), dtype=q.dtype, device=q.device)


def _mask_operand(args, mask, b, h, sq, sk):
    """Fills the mask fields from a mask broadcastable to [b, h, sq, sk]."""
    if mask is None:
        args.mask = None
        args.mask_dtype = _lib.MASK_NONE
        return None
    if mask.dim() > 4:
        raise _lib.UnsupportedAttention(
            "kohaku_tt_b200: the mask must broadcast to [B, H, Sq, Sk]"
        )
    if mask.dtype not in _MASK_DTYPES:
        mask = mask.to(torch.float32)
    m = mask
    while m.dim() < 4:
        m = m.unsqueeze(0)
    full = (b, h, sq, sk)
    for have, want in zip(m.shape, full):
        if have != 1 and have != want:
            raise _lib.UnsupportedAttention(
                "kohaku_tt_b200: the mask must broadcast to [B, H, Sq, Sk]"
            )
    m = m.expand(full)
    args.mask = m.data_ptr()
    args.mask_dtype = _MASK_DTYPES[m.dtype]
    for i in range(4):
        args.mask_strides[i] = m.stride(i)
    return m  # keeps the expanded view (and its storage) alive over the call


# The persistent forward kernel can draw its work items from a counter instead of a fixed
# deal (a zeroed int32 passed as the call's workspace: one small fill per call). On an
# undisturbed GPU the fixed deal measured as fast or faster (headline batch 8, packed
# 65,536 tokens), so it is off unless asked for: `dynamic_work(True)` for code whose
# attention kernels share the SMs with other kernels.
_DYNAMIC = {"on": False, "min_items_per_sm": 6}


def dynamic_work(on=True, min_items_per_sm=6):
    """Switches counter-driven work distribution of the tcgen05 forward on or off for work
    lists of at least `min_items_per_sm` items per SM. Returns the previous setting."""
    old = dict(_DYNAMIC)
    _DYNAMIC["on"], _DYNAMIC["min_items_per_sm"] = bool(on), int(min_items_per_sm)
    return old


_FORWARD_WORKSPACE = {}


def forward_workspace(args, device):
    """The head-dim-64 forward kernel's workspace (the counter its CTAs draw their tiles
    from): one zero-filled buffer per (device, stream); the kernel leaves it zero, so it is
    filled once. Returns the buffer or None when the kernel that will run uses none."""
    need = _lib.lib().ktt_b200_sdpa_forward_workspace(ctypes.byref(args))
    if need <= 0:
        return None
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    buf = _FORWARD_WORKSPACE.get(key)
    if buf is None or buf.numel() < need:
        buf = torch.zeros((need,), dtype=torch.uint8, device=device)
        _FORWARD_WORKSPACE[key] = buf
    args.workspace, args.workspace_bytes = buf.data_ptr(), buf.numel()
    return buf


def drop_forward_workspaces():
    """Forgets the cached forward workspaces (after a device-wait error their counters may
    be left non-zero)."""
    _FORWARD_WORKSPACE.clear()


def _work_counter(args, device, dynamic=None):
    """Sets args.workspace: the head-dim-64 kernel's cached workspace, or (head dim 128) a
    zeroed counter when dynamic work distribution applies (`dynamic`: this call's own
    choice, None = the module setting; False also keeps the head-dim-64 kernel on its fixed
    deal of whole tiles)."""
    if dynamic is not False:
        buf = forward_workspace(args, device)
        if buf is not None:
            return buf
    if args.d == 64 and args.kernel != _lib.KERNEL_TC5_WIDE:
        return None
    if not (_DYNAMIC["on"] if dynamic is None else dynamic):
        return None
    tiles = (args.sq + 127) // 128
    if dynamic is None and args.heads * args.batch * tiles < _DYNAMIC["min_items_per_sm"] * _sm_count(device):
        return None
    counter = torch.zeros((4,), dtype=torch.int32, device=device)
    args.workspace, args.workspace_bytes = counter.data_ptr(), 16
    return counter


_SMS = {}


def _sm_count(device):
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index not in _SMS:
        _SMS[index] = torch.cuda.get_device_properties(index).multi_processor_count
    return _SMS[index]


def _stream(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _dense_args(q, k, v, mask, key_lengths, causal, scale, kernel):
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        raise _lib.UnsupportedAttention("kohaku_tt_b200: q, k and v must be 4-D [B, H, S, D]")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise _lib.UnsupportedAttention("kohaku_tt_b200: q, k and v must be bf16")
    b, h, sq, d = q.shape
    if k.shape[0] != b or v.shape[0] != b or k.shape[1] != v.shape[1] or k.shape[2] != v.shape[2]:
        raise _lib.UnsupportedAttention(
            "kohaku_tt_b200: q, k and v shapes do not match (K / V heads must divide Q heads)"
        )
    if k.shape[3] != d:
        raise _lib.UnsupportedAttention("kohaku_tt_b200: q and k need one head dim")
    args = _lib.AttnArgs()
    args.batch, args.heads, args.kv_heads = b, h, k.shape[1]
    args.sq, args.sk, args.d, args.dv = sq, k.shape[2], d, v.shape[3]
    # True is PyTorch's top-left alignment; "bottom_right" puts the diagonal at the last
    # query and key (what a ring step over the tail of a longer sequence needs).
    if causal == "bottom_right":
        args.causal = _lib.CAUSAL_BOTTOM_RIGHT
    else:
        args.causal = _lib.CAUSAL_TOP_LEFT if causal else _lib.CAUSAL_NONE
    args.scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    args.kernel = _kernel_code(kernel)
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    _set3(args.q_strides, _bhs_strides(q))
    _set3(args.k_strides, _bhs_strides(k))
    _set3(args.v_strides, _bhs_strides(v))
    keep = [_mask_operand(args, mask, b, h, sq, k.shape[2])]
    if key_lengths is not None:
        if key_lengths.dtype != torch.int32 or key_lengths.dim() != 1 or key_lengths.numel() != b:
            raise ValueError("kohaku_tt_b200: key_lengths must be int32 [B]")
        key_lengths = key_lengths.contiguous()
        args.key_lengths = key_lengths.data_ptr()
        keep.append(key_lengths)
    return args, keep


def sdpa_forward(q, k, v, mask=None, key_lengths=None, causal=False, scale=None,
                 need_lse=True, kernel="auto", lse_rows=None, dynamic=None, out=None):
    """Dense attention forward: out [B, H, Sq, Dv] bf16 and, with need_lse, the row
    log-sum-exp [B, H, lse_rows or Sq] fp32 (natural log).

    q [B, H, Sq, D], k / v [B, Hk, Sk, D / Dv] bf16 with any batch / head / row strides;
    mask bool (True keeps) or additive, broadcastable to [B, H, Sq, Sk]; key_lengths
    int32 [B] on the device; causal is top-left aligned.
    Stands where bridge::sdpa / sdpa_train / sdpa_lengths stand in the reference
    (device_attention.cpp:265-497,607-679,836-907)."""
    _require_cuda(q, k, v, mask, key_lengths)
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    args, keep = _dense_args(q, k, v, mask, key_lengths, causal, scale, kernel)
    with torch.cuda.device(q.device):
        if out is None:
            out = _out_like_query(q, v.shape[3])
        elif out.shape != (q.shape[0], q.shape[1], q.shape[2], v.shape[3]) or out.dtype != q.dtype or out.stride(3) != 1:
            raise ValueError("kohaku_tt_b200.sdpa_forward: `out` must be [B, H, Sq, Dv] in q's dtype with a unit last stride")
        args.out = out.data_ptr()
        _set3(args.out_strides, _bhs_strides(out))
        lse = None
        if need_lse:
            rows = q.shape[2] if lse_rows is None else int(lse_rows)
            lse = torch.empty((q.shape[0], q.shape[1], rows), dtype=torch.float32, device=q.device)
            args.lse = lse.data_ptr()
            _set3(args.lse_strides, (lse.stride(0), lse.stride(1), 1))
        counter = _work_counter(args, q.device, dynamic)
        _lib.check(_lib.lib().ktt_b200_sdpa_forward(ctypes.byref(args), _stream(q.device)), "sdpa_forward")
        del counter
    del keep
    return out, lse


def sdpa_backward(dout, q, k, v, out, lse, mask=None, key_lengths=None, causal=False,
                  scale=None, kernel="auto"):
    """dq, dk, dv of sdpa_forward from its output and log-sum-exp; dk / dv are summed
    over each GQA group. Stands where bridge::sdpa_train_backward and
    sdpa_lengths_backward stand (device_attention.cpp:909-959,1208-1281)."""
    _require_cuda(dout, q, k, v, out, lse, mask, key_lengths)
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    dout, out = _rows_contiguous(dout), _rows_contiguous(out)
    args, keep = _dense_args(q, k, v, mask, key_lengths, causal, scale, kernel)
    if lse.dtype != torch.float32 or lse.dim() != 3 or lse.stride(2) != 1:
        raise ValueError("kohaku_tt_b200: lse must be fp32 [B, H, rows] with unit row stride")
    with torch.cuda.device(q.device):
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        args.out, args.lse, args.dout = out.data_ptr(), lse.data_ptr(), dout.data_ptr()
        args.dq, args.dk, args.dv_out = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        _set3(args.out_strides, _bhs_strides(out))
        _set3(args.lse_strides, (lse.stride(0), lse.stride(1), 1))
        _set3(args.dout_strides, _bhs_strides(dout))
        _set3(args.dq_strides, _bhs_strides(dq))
        _set3(args.dk_strides, _bhs_strides(dk))
        _set3(args.dv_strides, _bhs_strides(dv))
        handle = _lib.lib()
        nbytes = handle.ktt_b200_sdpa_backward_workspace(ctypes.byref(args))
        if nbytes <= 0:
            _lib.check(_lib.ERR_UNSUPPORTED, "sdpa_backward")
        work = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
        args.workspace, args.workspace_bytes = work.data_ptr(), nbytes
        _lib.check(handle.ktt_b200_sdpa_backward(ctypes.byref(args), _stream(q.device)), "sdpa_backward")
    del keep
    return dq, dk, dv


def _packed_args(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, key_mask, kernel):
    if q.dim() != 3 or k.dim() != 3 or v.dim() != 3:
        raise _lib.UnsupportedAttention("kohaku_tt_b200: packed q, k and v must be 3-D [T, H, D]")
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        raise _lib.UnsupportedAttention("kohaku_tt_b200: q, k and v must be bf16")
    if k.shape[0] != v.shape[0] or k.shape[1] != v.shape[1] or k.shape[2] != q.shape[2]:
        raise _lib.UnsupportedAttention("kohaku_tt_b200: packed q, k and v shapes do not match")
    for cu in (cu_q, cu_k):
        if cu.dtype != torch.int32 or cu.dim() != 1 or not cu.is_contiguous():
            raise ValueError("kohaku_tt_b200: cu_seqlens must be contiguous int32 [n + 1]")
    if cu_q.numel() != cu_k.numel() or cu_q.numel() < 2:
        raise ValueError("kohaku_tt_b200: cu_seq_q and cu_seq_k need equal counts >= 2")
    args = _lib.AttnArgs()
    args.batch = cu_q.numel() - 1
    args.heads, args.kv_heads = q.shape[1], k.shape[1]
    args.sq, args.sk = max(int(max_q), 1), max(int(max_k), 1)
    args.total_q, args.total_k = q.shape[0], k.shape[0]
    args.d, args.dv = q.shape[2], v.shape[2]
    args.causal = _lib.CAUSAL_BOTTOM_RIGHT if causal else _lib.CAUSAL_NONE
    args.scale = float(scale) if scale is not None else 1.0 / math.sqrt(q.shape[2])
    args.kernel = _kernel_code(kernel)
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    _set3(args.q_strides, _ths_strides(q))
    _set3(args.k_strides, _ths_strides(k))
    _set3(args.v_strides, _ths_strides(v))
    args.cu_seqlens_q, args.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    keep = []
    if key_mask is not None:
        if key_mask.dim() != 1 or key_mask.shape[0] != k.shape[0]:
            raise ValueError(
                f"kohaku_tt_b200.sdpa_varlen: attn_mask must be [{k.shape[0]}] "
                f"(one value per packed key), got {tuple(key_mask.shape)}"
            )
        if key_mask.dtype not in _MASK_DTYPES:
            key_mask = key_mask.to(torch.float32)
        key_mask = key_mask.contiguous()
        args.mask = key_mask.data_ptr()
        args.mask_dtype = _MASK_DTYPES[key_mask.dtype]
        args.mask_strides[0] = args.mask_strides[1] = args.mask_strides[2] = 0
        args.mask_strides[3] = 1
        keep.append(key_mask)
    return args, keep


def varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, causal=False, scale=None,
                   key_mask=None, kernel="auto"):
    """Packed attention forward: out [Tq, H, Dv] bf16, lse [H, Tq] fp32.

    q [Tq, H, D], k [Tk, Hk, D], v [Tk, Hk, Dv]; cu_q / cu_k int32 [n + 1] on the
    device; causal is bottom-right aligned; key_mask [Tk] bool or additive.
    Stands where bridge::sdpa_varlen stands (device_attention.cpp:681-761); the offsets
    are consumed on the device, so there is no host plan to build or cache
    (kohakutt/torch_backend/varlen.py:31-46)."""
    _require_cuda(q, k, v, cu_q, cu_k, key_mask)
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    args, keep = _packed_args(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, key_mask, kernel)
    with torch.cuda.device(q.device):
        out = torch.empty((q.shape[0], q.shape[1], v.shape[2]), dtype=q.dtype, device=q.device)
        lse = torch.empty((q.shape[1], q.shape[0]), dtype=torch.float32, device=q.device)
        args.out, args.lse = out.data_ptr(), lse.data_ptr()
        _set3(args.out_strides, _ths_strides(out))
        _set3(args.lse_strides, (0, lse.stride(0), 1))
        counter = _work_counter(args, q.device)
        _lib.check(_lib.lib().ktt_b200_sdpa_forward(ctypes.byref(args), _stream(q.device)), "varlen_forward")
        del counter
    del keep
    return out, lse


def varlen_backward(dout, q, k, v, out, lse, cu_q, cu_k, max_q, max_k, causal=False,
                    scale=None, key_mask=None, kernel="auto"):
    """dq, dk, dv of varlen_forward, packed like q, k, v (bridge::sdpa_varlen_backward,
    device_attention.cpp:763-834)."""
    _require_cuda(dout, q, k, v, out, lse, cu_q, cu_k, key_mask)
    q, k, v = _rows_contiguous(q), _rows_contiguous(k), _rows_contiguous(v)
    dout, out = _rows_contiguous(dout), _rows_contiguous(out)
    args, keep = _packed_args(q, k, v, cu_q, cu_k, max_q, max_k, causal, scale, key_mask, kernel)
    if lse.dtype != torch.float32 or tuple(lse.shape) != (q.shape[1], q.shape[0]) or lse.stride(1) != 1:
        raise ValueError("kohaku_tt_b200: packed lse must be fp32 [H, Tq]")
    with torch.cuda.device(q.device):
        # No clearing: every row inside a sequence is written by the CTA that owns it (zeros
        # where nothing reaches it) and the library zeroes the rows no sequence covers.
        dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
        dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
        dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
        args.out, args.lse, args.dout = out.data_ptr(), lse.data_ptr(), dout.data_ptr()
        args.dq, args.dk, args.dv_out = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
        _set3(args.out_strides, _ths_strides(out))
        _set3(args.lse_strides, (0, lse.stride(0), 1))
        _set3(args.dout_strides, _ths_strides(dout))
        _set3(args.dq_strides, _ths_strides(dq))
        _set3(args.dk_strides, _ths_strides(dk))
        _set3(args.dv_strides, _ths_strides(dv))
        handle = _lib.lib()
        nbytes = handle.ktt_b200_sdpa_backward_workspace(ctypes.byref(args))
        if nbytes <= 0:
            _lib.check(_lib.ERR_UNSUPPORTED, "varlen_backward")
        work = torch.empty((nbytes,), dtype=torch.uint8, device=q.device)
        args.workspace, args.workspace_bytes = work.data_ptr(), nbytes
        _lib.check(handle.ktt_b200_sdpa_backward(ctypes.byref(args), _stream(q.device)), "varlen_backward")
    del keep
    return dq, dk, dv


def decode_takes(q, k, v):
    """True when the split-K decode kernel takes the shapes (bf16, D == Dv in {64, 128},
    at most 16 query rows per K / V head, 16-byte aligned cache rows)."""
    if q.dim() != 4 or k.dim() != 4 or v.dim() != 4:
        return False
    if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
        return False
    b, h, sq, d = q.shape
    hk = k.shape[1]
    if hk == 0 or h % hk or v.shape[3] != d or d not in (64, 128) or (h // hk) * sq > 16 or b > 512:
        return False
    if any(t.stride(-1) != 1 for t in (q, k, v)):
        return False
    if any(s % 8 for t in (k, v) for s in t.stride()[:3]) or any(s % 2 for s in q.stride()[:3]):
        return False
    return k.data_ptr() % 16 == 0 and v.data_ptr() % 16 == 0 and q.data_ptr() % 4 == 0


_DECODE_SCRATCH = {}


def decode_scratch(args, device):
    """A cached per-device scratch buffer large enough for `args` (split-K partials)."""
    need = _lib.lib().ktt_b200_decode_scratch_bytes(ctypes.byref(args))
    if need <= 0:
        _lib.check(_lib.ERR_UNSUPPORTED, "decode")
    # One buffer per device: concurrent decode calls on several streams of one device must
    # pass their own `scratch` (calls sharing a buffer must not overlap on the GPU).
    key = device.index
    buf = _DECODE_SCRATCH.get(key)
    if buf is None or buf.numel() < need:
        # Zero-filled: the kernel's ticket counters must start at zero (it leaves them so).
        buf = torch.zeros((need,), dtype=torch.uint8, device=device)
        _DECODE_SCRATCH[key] = buf
    return buf, need


def decode(q, k, v, key_lengths=None, scale=None, need_lse=False, splits=0, scratch=None):
    """Decode attention of q [B, H, Sq, D] (H / Hk * Sq <= 16) against a static cache
    k / v [B, Hk, Smax, D]; key_lengths int32 [B] on the device (clamped to [1, Smax]).
    `scratch`, when given, must have been zero-filled once before its first use.
    Returns (out [B, H, Sq, D] bf16, lse or None). The decode route of
    ktt::_sdpa_lengths (aten_lengths.cpp:69-99, aten_attention.cpp:578-604)."""
    _require_cuda(q, k, v, key_lengths)
    if not decode_takes(q, k, v):
        raise _lib.UnsupportedAttention("kohaku_tt_b200.decode: shapes or strides not taken")
    b, h, sq, d = q.shape
    args = _lib.DecodeArgs()
    args.batch, args.heads, args.kv_heads = b, h, k.shape[1]
    args.sq, args.sk, args.d, args.dv = sq, k.shape[2], d, d
    args.scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    args.q, args.k, args.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    _set3(args.q_strides, _bhs_strides(q))
    _set3(args.k_strides, _bhs_strides(k))
    _set3(args.v_strides, _bhs_strides(v))
    args.splits = int(splits)
    if key_lengths is not None:
        if key_lengths.dtype != torch.int32 or key_lengths.dim() != 1 or key_lengths.numel() != b:
            raise ValueError("kohaku_tt_b200: key_lengths must be int32 [B]")
        key_lengths = key_lengths.contiguous()
        args.key_lengths = key_lengths.data_ptr()
    with torch.cuda.device(q.device):
        out = torch.empty((b, h, sq, d), dtype=q.dtype, device=q.device)
        args.out = out.data_ptr()
        _set3(args.out_strides, _bhs_strides(out))
        lse = None
        if need_lse:
            lse = torch.empty((b, h, sq), dtype=torch.float32, device=q.device)
            args.lse = lse.data_ptr()
        if scratch is None:
            scratch, need = decode_scratch(args, q.device)
        else:
            need = scratch.numel() * scratch.element_size()
        args.scratch, args.scratch_bytes = scratch.data_ptr(), need
        _lib.check(_lib.lib().ktt_b200_decode(ctypes.byref(args), _stream(q.device)), "decode")
    return out, lse


def decode_append(q, k_new, v_new, k_cache, v_cache, lengths, cos, sin, by_position=None,
                  scale=None, lengths_out=None, scratch=None):
    """One decode step in one launch: rotate-half rotary of q [B, H, 1, D] and k_new
    [B, Hk, 1, D] (ktt.rotary, aten_fused.cpp:30-43), k_cache / v_cache [B, Hk, Smax, D]
    row lengths[b] <- (rotated key, v_new) (the StaticCache `index_copy_`), attention over
    the lengths[b] + 1 keys. lengths int32 [B] on the device = keys already cached (< Smax);
    they are not changed, lengths_out (another int32 [B]) receives lengths + 1 when given.
    cos / sin bf16: [B, D] rows per batch, or a [positions, D] table indexed by lengths[b]
    (`by_position`; default: a table when the row count differs from B). Returns out
    [B, H, 1, D]; the caches are updated in place."""
    _require_cuda(q, k_cache, v_cache, lengths)
    b, h, sq, d = q.shape
    if sq != 1 or k_new.shape != (b, k_cache.shape[1], 1, d) or v_new.shape != k_new.shape:
        raise ValueError("kohaku_tt_b200.decode_append: q [B, H, 1, D], k_new / v_new [B, Hk, 1, D]")
    if not decode_takes(q, k_cache, v_cache):
        raise _lib.UnsupportedAttention("kohaku_tt_b200.decode_append: shapes or strides not taken")
    if lengths.dtype != torch.int32 or lengths.dim() != 1 or lengths.numel() != b:
        raise ValueError("kohaku_tt_b200: lengths must be int32 [B]")
    cos2, sin2 = cos.reshape(-1, d), sin.reshape(-1, d)
    if cos2.dtype != torch.bfloat16 or sin2.dtype != torch.bfloat16 or cos2.shape != sin2.shape:
        raise ValueError("kohaku_tt_b200.decode_append: cos / sin must be bf16 rows of D values, same shape")
    if cos2.stride(-1) != 1 or sin2.stride(-1) != 1 or cos2.stride(0) != sin2.stride(0):
        cos2, sin2 = cos2.contiguous(), sin2.contiguous()
    if by_position is None:
        by_position = cos2.shape[0] != b
    if by_position and cos2.shape[0] < k_cache.shape[2]:
        raise ValueError("kohaku_tt_b200.decode_append: the rotary table must cover every cache position")
    if not by_position and cos2.shape[0] != b:
        raise ValueError("kohaku_tt_b200.decode_append: one rotary row per batch entry")
    if k_new.stride(-1) != 1 or v_new.stride(-1) != 1:
        k_new, v_new = k_new.contiguous(), v_new.contiguous()
    app = _lib.DecodeAppendArgs()
    args = app.base
    args.batch, args.heads, args.kv_heads = b, h, k_cache.shape[1]
    args.sq, args.sk, args.d, args.dv = 1, k_cache.shape[2], d, d
    args.scale = float(scale) if scale is not None else 1.0 / math.sqrt(d)
    args.q, args.k, args.v = q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
    _set3(args.q_strides, _bhs_strides(q))
    _set3(args.k_strides, _bhs_strides(k_cache))
    _set3(args.v_strides, _bhs_strides(v_cache))
    lengths = lengths.contiguous()
    args.key_lengths = lengths.data_ptr()
    app.k_new, app.v_new = k_new.data_ptr(), v_new.data_ptr()
    app.k_new_strides[0], app.k_new_strides[1] = k_new.stride(0), k_new.stride(1)
    app.v_new_strides[0], app.v_new_strides[1] = v_new.stride(0), v_new.stride(1)
    app.cos, app.sin = cos2.data_ptr(), sin2.data_ptr()
    app.rope_row_stride = cos2.stride(0)
    app.rope_by_position = 1 if by_position else 0
    if lengths_out is not None:
        if lengths_out.dtype != torch.int32 or lengths_out.shape != lengths.shape or not lengths_out.is_contiguous():
            raise ValueError("kohaku_tt_b200: lengths_out must be a contiguous int32 [B]")
        app.lengths_out = lengths_out.data_ptr()
    with torch.cuda.device(q.device):
        out = torch.empty((b, h, 1, d), dtype=q.dtype, device=q.device)
        args.out = out.data_ptr()
        _set3(args.out_strides, _bhs_strides(out))
        if scratch is None:
            scratch, need = decode_scratch(args, q.device)
        else:
            need = scratch.numel() * scratch.element_size()
        args.scratch, args.scratch_bytes = scratch.data_ptr(), need
        _lib.check(_lib.lib().ktt_b200_decode_append(ctypes.byref(app), _stream(q.device)), "decode_append")
    return out


def merge_partials(out, lse, out2, lse2):
    """In place: (out, lse) <- merge with (out2, lse2), two attention results of the
    same queries over disjoint key sets. out [..., Dv] bf16 or fp32 (out2 the same, or bf16
    into an fp32 out), lse [...] fp32."""
    _require_cuda(out, lse, out2, lse2)
    if not (out.is_contiguous() and out2.is_contiguous() and lse.is_contiguous() and lse2.is_contiguous()):
        raise ValueError("kohaku_tt_b200.merge_partials: operands must be contiguous")
    mixed = out.dtype == torch.float32 and out2.dtype == torch.bfloat16
    if out.shape != out2.shape or lse.shape != lse2.shape or (out.dtype != out2.dtype and not mixed):
        raise ValueError("kohaku_tt_b200.merge_partials: operand shapes or dtypes differ")
    dv = out.shape[-1]
    rows = out.numel() // dv
    if lse.numel() != rows or lse.dtype != torch.float32 or lse2.dtype != torch.float32:
        raise ValueError("kohaku_tt_b200.merge_partials: lse must be fp32 with one value per row")
    if out.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError("kohaku_tt_b200.merge_partials: out must be bf16 or fp32")
    with torch.cuda.device(out.device):
        _lib.check(
            _lib.lib().ktt_b200_merge_partials(
                out.data_ptr(), lse.data_ptr(), out2.data_ptr(), lse2.data_ptr(),
                rows, dv, 2 if mixed else int(out.dtype == torch.float32), _stream(out.device)),
            "merge_partials")
    return out, lse
