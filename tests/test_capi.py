"""The C-ABI library loads, exports every symbol include/ktt_b200.h declares, and its
host-side checks answer without a GPU (no kernel is launched in this file)."""

import ctypes
import os
import re

import pytest

from kohaku_tt_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "ktt_b200.h")).read()
    return re.findall(r"KTT_B200_API\s+[\w\s\*]+?\b(ktt_b200_\w+)\s*\(", text)


def test_every_declared_symbol_is_exported(built_lib):
    names = _declared()
    assert len(names) >= 12
    raw = ctypes.CDLL(_lib.LIB_PATH)
    for name in names:
        assert hasattr(raw, name), name
    assert set(names) >= set(_lib.EXPORTS)


def test_abi_version_and_counters(built_lib):
    assert built_lib.ktt_b200_abi_version() == 1
    _lib.reset_counters()
    assert all(v == 0 for v in _lib.counters().values())


def test_struct_layout_matches_the_header(built_lib):
    # Natural alignment on both sides: spot-check sizes that would shift on a mismatch.
    assert ctypes.sizeof(_lib.AttnArgs) % 8 == 0
    assert _lib.AttnArgs.total_q.offset == 24
    assert _lib.AttnArgs.q.offset == 64
    assert _lib.DecodeArgs.q.offset == 32


def _args(**kw):
    a = _lib.AttnArgs()
    a.batch, a.heads, a.kv_heads, a.sq, a.sk, a.d, a.dv = 2, 4, 2, 64, 64, 64, 64
    a.scale = 0.125
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_supported_and_refusals_answer_on_the_host(built_lib):
    assert built_lib.ktt_b200_sdpa_supported(ctypes.byref(_args())) == 1
    assert built_lib.ktt_b200_sdpa_backward_supported(ctypes.byref(_args())) == 1
    for kw, text in [
        (dict(kv_heads=3), "K / V heads must divide Q heads"),
        (dict(d=512), "head dims above 256"),
        (dict(sq=0), "non-empty"),
        (dict(causal=1, mask_dtype=_lib.MASK_BOOL, mask=1), "causal takes no mask"),
        (dict(scale=0.0), "scale must be positive"),
        (dict(mask_dtype=_lib.MASK_BOOL), "mask pointer and mask dtype disagree"),
    ]:
        assert built_lib.ktt_b200_sdpa_supported(ctypes.byref(_args(**kw))) == 0
        assert text in _lib.last_error()


def test_null_pointers_are_rejected_before_any_launch(built_lib):
    rc = built_lib.ktt_b200_sdpa_forward(ctypes.byref(_args()), None)
    assert rc == _lib.ERR_BAD_ARGUMENT
    assert "null tensor pointer" in _lib.last_error()
    with pytest.raises(ValueError):
        _lib.check(rc, "sdpa_forward")
    rc = built_lib.ktt_b200_sdpa_backward(ctypes.byref(_args()), None)
    assert rc == _lib.ERR_BAD_ARGUMENT
    assert built_lib.ktt_b200_merge_partials(None, None, None, None, 4, 64, 0, None) == _lib.ERR_BAD_ARGUMENT


def test_dump_request_checks_its_arguments(built_lib):
    # Setting and clearing the request is host state only; nothing is launched.
    fake = ctypes.c_void_p(4096)
    assert built_lib.ktt_b200_set_dump(fake, -1, 0, 0, 4) == _lib.ERR_BAD_ARGUMENT
    assert built_lib.ktt_b200_set_dump(fake, 0, 0, 0, 0) == _lib.ERR_BAD_ARGUMENT
    assert built_lib.ktt_b200_set_dump(None, 0, 0, 0, 0) == 0


def test_backward_workspace_size(built_lib):
    # One fp32 per (batch, head, query row), rows padded to 64 ...
    delta = 2 * 4 * 128 * 4
    assert built_lib.ktt_b200_sdpa_backward_workspace(ctypes.byref(_args(sq=100, kv_heads=4))) == delta
    # ... plus, for grouped heads on a small grid, fp32 dV / dK partials of each part the
    # group is split into (2 tensors x batch 2 x kv heads 2 x 2 parts x 64 keys x 64 dims)
    # and one ticket counter per (batch, kv head, key block), padded to 256 bytes.
    assert built_lib.ktt_b200_sdpa_backward_workspace(ctypes.byref(_args(sq=100))) == delta + 2 * 2 * 2 * 2 * 64 * 64 * 4 + 256


def test_decode_refusals(built_lib):
    d = _lib.DecodeArgs()
    d.batch, d.heads, d.kv_heads, d.sq, d.sk, d.d, d.dv = 4, 16, 2, 1, 4096, 128, 128
    for name in ("q_strides", "k_strides", "v_strides", "out_strides"):
        for i, s in enumerate((16 * 128, 128, 128)):
            getattr(d, name)[i] = s
    d.scale = 0.1
    # Scratch size needs the SM count only when a device is present; the refusal rules do not.
    d.heads = 64
    assert built_lib.ktt_b200_decode_scratch_bytes(ctypes.byref(d)) == 0
    assert "at most 16 query rows" in _lib.last_error()
    d.heads, d.d = 16, 96
    assert built_lib.ktt_b200_decode(ctypes.byref(d), None) == _lib.ERR_UNSUPPORTED
    assert "head dim 64 or 128" in _lib.last_error()
