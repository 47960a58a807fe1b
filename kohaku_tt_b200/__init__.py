"""B200-native flash attention behind Kohaku-TT's operator surface.

    import kohaku_tt_b200 as ktt
    ktt.install()                      # F.scaled_dot_product_attention on CUDA -> these kernels
    y = ktt.sdpa(q, k, v, key_lengths=lengths)
    y = ktt.sdpa_varlen(q, k, v, cu_seqlens)
    with ktt.sdpa_kernel("flash"): ...

Everything runs on hand-written sm_100a CUDA in lib/libktt_b200.so (C ABI in
include/ktt_b200.h); there is no CPU or PyTorch-math fallback.
"""

from ._lib import UnsupportedAttention, counters, reset_counters
from ._lib import build as _build_library
from ._lib import build_shim as _build_shim
from .aten import fused_sdp_choice, install, installed, installed_for, uninstall
from .attention import decode_step, sdpa, sdpa_varlen
from .numerics import KERNELS, sdpa_kernel
from .stats import diff_stats, format_stats, rel_rms
from .trace import debug_flash_dump

AVAILABLE = True


def build(force=False, verbose=False):
    """Compiles libktt_b200.so (nvcc, sm_100a) and the C++ registration shim of the aten
    overloads (g++ against the installed torch) when they are stale."""
    path = _build_library(force=force, verbose=verbose)
    _build_shim(force=force)
    return path

__all__ = [
    "AVAILABLE",
    "KERNELS",
    "UnsupportedAttention",
    "build",
    "counters",
    "decode_step",
    "diff_stats",
    "format_stats",
    "fused_sdp_choice",
    "install",
    "installed",
    "installed_for",
    "rel_rms",
    "reset_counters",
    "sdpa",
    "sdpa_kernel",
    "debug_flash_dump",
    "sdpa_varlen",
    "uninstall",
]
