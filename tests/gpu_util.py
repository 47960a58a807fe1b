"""Helpers shared by the GPU parity tests: seeded inputs and the reference's bounds."""

import torch

from kohaku_tt_b200 import stats
from oracle import attention_oracle as ao

FWD_BOUND = 8e-3    # rel RMS of the forward vs float64 (tests/hardware/ops/test_flash.py:15)
GRAD_BOUND = 2e-2   # rel RMS of dense gradients (test_flash.py:225)
VARLEN_GRAD_BOUND = 2.5e-2  # packed gradients (test_flash_varlen.py:188-248)
LSE_RMS = 6e-3      # RMS of lse vs float64 logsumexp (test_flash.py:229)


def qkv(b, h, hk, sq, sk, d, seed, dv=None, extra=0):
    """q, k, v (+ `extra` tensors shaped like the output) drawn in that order."""
    dv = d if dv is None else dv
    shapes = [(b, h, sq, d), (b, hk, sk, d), (b, hk, sk, dv)] + [(b, h, sq, dv)] * extra
    return ao.make_inputs(shapes, seed)


def packed(lq, lk, h, hk, d, seed, dv=None, extra=0):
    dv = d if dv is None else dv
    tq, tk = sum(lq), sum(lk)
    shapes = [(tq, h, d), (tk, hk, d), (tk, hk, dv)] + [(tq, h, dv)] * extra
    return ao.make_inputs(shapes, seed)


def cumulative(lengths):
    out = [0]
    for n in lengths:
        out.append(out[-1] + n)
    return out


def cu(lengths, device):
    return torch.tensor(cumulative(lengths), dtype=torch.int32, device=device)


def rel(y, ref):
    return stats.rel_rms(y, ref)


def rms(y, ref):
    return (y.detach().double().cpu() - ref.double()).pow(2).mean().sqrt().item()
