"""Kernel-selection scope: `sdpa_kernel("flash")` / `sdpa_kernel("mma")`.

Mirrors kohakutt.sdpa_kernel (src/kohakutt/core/numerics.py:156-166): attention calls
made inside the scope run only on the named kernels, forward and backward, and a call
none of them takes raises with each kernel's reason. The reference's other names ('own',
'ttnn', 'math') select vendor or composite routes that do not exist here; they are
rejected. The fidelity / approx knobs of kohakutt.numerics are Tensix-specific and are
not carried over.
"""

import contextlib
import threading

KERNELS = ("flash", "mma")

_LOCAL = threading.local()


def _stack():
    if not hasattr(_LOCAL, "stack"):
        _LOCAL.stack = []
    return _LOCAL.stack


def current_kernels():
    """The kernel names the calling thread's innermost scope allows."""
    stack = _stack()
    return stack[-1] if stack else KERNELS


class sdpa_kernel(contextlib.ContextDecorator):
    """A scope (context manager or decorator) that runs the attention calls made in it
    on `kernels` only: 'flash' (TMA + tcgen05) and / or 'mma' (warp MMA), given as
    arguments or one list."""

    def __init__(self, *kernels):
        names = []
        for k in kernels:
            names.extend([k] if isinstance(k, str) else k)
        for name in names:
            if name not in KERNELS:
                raise ValueError(
                    f"kohaku_tt_b200.sdpa_kernel: unknown kernel {name!r}; "
                    f"this build has {KERNELS}"
                )
        if not names:
            raise ValueError("kohaku_tt_b200.sdpa_kernel: name at least one kernel")
        self.kernels = tuple(dict.fromkeys(names))

    def __enter__(self):
        _stack().append(self.kernels)
        _tell_shim()
        return self.kernels

    def __exit__(self, *exc):
        _stack().pop()
        _tell_shim()
        return False


def _tell_shim():
    """The C++ registration of the aten overloads keeps its own copy of the calling thread's
    scope (it cannot call back into Python per attention call)."""
    from . import _lib

    handle = _lib._SHIM
    if handle is None:
        return
    stack = _stack()
    if not stack:
        handle.ktt_b200_aten_set_scope(_lib.KERNEL_AUTO, b"")
        return
    allowed = stack[-1]
    if set(allowed) >= {"flash", "mma"}:
        code = _lib.KERNEL_AUTO
    elif "flash" in allowed:
        code = _lib.KERNEL_TC5
    elif "mma" in allowed:
        code = _lib.KERNEL_MMA
    else:
        code = -1
    handle.ktt_b200_aten_set_scope(code, ", ".join(repr(k) for k in allowed).encode())
