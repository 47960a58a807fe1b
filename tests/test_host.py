"""Host-side logic of the operator surface: refusal rules, scopes, argument checks and the
loud failure without CUDA. No GPU needed."""

import json
import os

import pytest
import torch

import kohaku_tt_b200 as ktt
from kohaku_tt_b200 import aten, attention, ops

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _qkv(b=1, h=2, hk=2, sq=77, sk=77, d=64, dtype=torch.bfloat16):
    return (torch.zeros(b, h, sq, d, dtype=dtype), torch.zeros(b, hk, sk, d, dtype=dtype),
            torch.zeros(b, hk, sk, d, dtype=dtype))


def test_choice_is_overrideable_for_fused_shapes():
    # tests/hardware/ops/test_attention.py:21-67.
    q, k, v = _qkv()
    assert aten.fused_sdp_choice(q, k, v, is_causal=True) == aten.SDP_OVERRIDEABLE
    assert aten.fused_sdp_choice(q, k, v, dropout_p=0.1) == aten.SDP_MATH
    q32, k32, v32 = _qkv(dtype=torch.float32)
    assert aten.fused_sdp_choice(q32, k32, v32) == aten.SDP_OVERRIDEABLE
    q32.requires_grad_(True)
    assert aten.fused_sdp_choice(q32, k32, v32) == aten.SDP_MATH


@pytest.mark.parametrize("kw,why", [
    (dict(dropout_p=0.1), "dropout"),
    (dict(is_causal=True, mask=torch.ones(77, 77, dtype=torch.bool)), "causal takes no mask"),
    (dict(mask=torch.ones(3, 77, dtype=torch.bool)), "the mask must broadcast"),
    (dict(mask=torch.ones(1, 1, 1, 1, 77)), "the mask must broadcast"),
])
def test_refusal_reasons(kw, why):
    q, k, v = _qkv()
    got = aten.fused_refusal(q, k, v, kw.get("mask"), kw.get("dropout_p", 0.0), kw.get("is_causal", False), None)
    assert got is not None and why in got


def test_refusal_shapes():
    q, k, v = _qkv(h=4, hk=3)
    assert "K / V heads must divide Q heads" in aten.fused_refusal(q, k, v, None, 0.0, False, None)
    q, k, v = _qkv()
    assert "4-D bf16" in aten.fused_refusal(q[0], k[0], v[0], None, 0.0, False, None)
    assert "4-D bf16" in aten.fused_refusal(q.half(), k.half(), v.half(), None, 0.0, False, None)


def test_scope_refusal_names_shapes_and_reason():
    # tests/hardware/ops/test_sdpa_kernel.py:114-133.
    q, k, v = _qkv()
    with ktt.sdpa_kernel("flash"):
        with pytest.raises(RuntimeError) as e:
            aten._checked(q, k, v, None, 0.1, True, None)
    text = str(e.value)
    assert "sdpa_kernel('flash')" in text and "[1, 2, 77, 64] bfloat16" in text
    assert "causal" in text and "dropout" in text
    with pytest.raises(ktt.UnsupportedAttention):
        aten._checked(q, k, v, None, 0.1, True, None)


def test_sdpa_kernel_scope_validates_names():
    with pytest.raises(ValueError):
        ktt.sdpa_kernel("ttnn")
    with pytest.raises(ValueError):
        ktt.sdpa_kernel()
    with ktt.sdpa_kernel("mma") as ks:
        assert ks == ("mma",)
        with ktt.sdpa_kernel(["flash", "mma"]) as inner:
            assert inner == ("flash", "mma")
    from kohaku_tt_b200.numerics import current_kernels

    assert current_kernels() == ktt.KERNELS


def test_device_lengths_matches_the_references_checks():
    with open(os.path.join(GOLDEN, "device_lengths.json")) as f:
        cases = json.load(f)
    for c in cases:
        if "ok" in c:
            t = attention.device_lengths(c["arg"], c["batch"], c["keys"], torch.device("cpu"))
            assert t.tolist() == c["ok"] and str(t.dtype) == c["dtype"]
        else:
            with pytest.raises(ValueError) as e:
                attention.device_lengths(c["arg"], c["batch"], c["keys"], torch.device("cpu"))
            assert str(e.value) == c["error"].replace("kohakutt.sdpa", "kohaku_tt_b200.sdpa")


def test_offset_checks():
    # tests/hardware/ops/test_flash_varlen.py:525-534 and varlen_plan.hpp:43-82.
    attention.check_offsets((0, 4, 9), (0, 4, 9), 9, 9, True)
    with pytest.raises(RuntimeError):
        attention.check_offsets((0, 4, 8), (0, 4, 8), 9, 9, False)
    with pytest.raises(RuntimeError):
        attention.check_offsets((0, 4), (0, 4, 9), 4, 9, False)
    with pytest.raises(RuntimeError):
        attention.check_offsets((0, 4, 9), (0, 4, 4), 9, 4, False)
    with pytest.raises(RuntimeError):
        attention.check_offsets((0, 4, 9), (0, 2, 9), 9, 9, True)


def test_varlen_mask_shape_is_checked_before_anything_runs():
    q = torch.zeros(9, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError) as e:
        ktt.sdpa_varlen(q, q, q, [0, 4, 9], attn_mask=torch.ones(2, 9))
    assert "one value per packed key" in str(e.value)


def test_cpu_tensors_fail_loudly(built_lib):
    q, k, v = _qkv()
    with pytest.raises(RuntimeError) as e:
        ops.sdpa_forward(q, k, v)
    assert "no CPU fallback" in str(e.value)
    with pytest.raises(RuntimeError):
        ops.decode(q, k, v)
    with pytest.raises(RuntimeError):
        ops.varlen_forward(q[0].transpose(0, 1), k[0].transpose(0, 1), v[0].transpose(0, 1),
                           torch.tensor([0, 77], dtype=torch.int32),
                           torch.tensor([0, 77], dtype=torch.int32), 77, 77)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from kohaku_tt_b200 import _lib

    monkeypatch.setattr(_lib, "_LIB", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libktt_b200.so"))
    with pytest.raises(RuntimeError) as e:
        _lib.lib()
    assert "no CPU or PyTorch fallback" in str(e.value)


def test_window_and_paging_arguments_are_refused():
    with pytest.raises(NotImplementedError):
        aten._causal(False, [128, 0])
    assert aten._causal(False, [-1, 0]) is True and aten._causal(False, None) is False
    with pytest.raises(NotImplementedError):
        aten._unsupported(seqused_k=torch.zeros(1), block_table=None)


def test_decode_takes_rules():
    q = torch.zeros(4, 16, 1, 128, dtype=torch.bfloat16)
    k = torch.zeros(4, 2, 512, 128, dtype=torch.bfloat16)
    assert ops.decode_takes(q, k, k)
    assert not ops.decode_takes(q.float(), k.float(), k.float())
    assert not ops.decode_takes(torch.zeros(4, 64, 1, 128, dtype=torch.bfloat16), k, k)
    assert not ops.decode_takes(q[..., :96], k[..., :96], k[..., :96])
