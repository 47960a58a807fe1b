"""Build and ctypes binding of libktt_b200.so (the C ABI of include/ktt_b200.h).

The library is compiled in-tree by nvcc for sm_100a only. There is no fallback: when it
is missing or cannot be loaded every operator of this package raises.
"""

import ctypes
import os
import shutil
import subprocess

_HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(_HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(_HERE), "include")
LIB_DIR = os.path.join(_HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libktt_b200.so")
# Extra nvcc flags for experiments (for example -DKTT_ROW_POLY_PAIRS=3); empty in normal use.
EXTRA_NVCC_FLAGS = os.environ.get("KTT_B200_NVCC_FLAGS", "").split()

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--shared",
    "-Xcompiler",
    "-fPIC,-fvisibility=hidden",
]

OK = 0
ERR_UNSUPPORTED = -1
ERR_BAD_ARGUMENT = -2
ERR_LAUNCH = -3
ERR_DEVICE_WAIT = -4

MASK_NONE, MASK_BOOL, MASK_BF16, MASK_F32, MASK_F16 = range(5)
CAUSAL_NONE, CAUSAL_TOP_LEFT, CAUSAL_BOTTOM_RIGHT = range(3)
KERNEL_AUTO, KERNEL_MMA, KERNEL_TC5, KERNEL_TC5_WIDE = range(4)

EXPORTS = (
    "ktt_b200_abi_version",
    "ktt_b200_last_error",
    "ktt_b200_counters",
    "ktt_b200_reset_counters",
    "ktt_b200_device_status",
    "ktt_b200_selftest_wait_timeout",
    "ktt_b200_probe_read",
    "ktt_b200_set_trace",
    "ktt_b200_set_dump",
    "ktt_b200_sdpa_supported",
    "ktt_b200_sdpa_backward_supported",
    "ktt_b200_sdpa_forward",
    "ktt_b200_sdpa_forward_workspace",
    "ktt_b200_forward_streams_per_sm",
    "ktt_b200_sdpa_backward_workspace",
    "ktt_b200_sdpa_backward",
    "ktt_b200_decode_scratch_bytes",
    "ktt_b200_decode",
    "ktt_b200_decode_static",
    "ktt_b200_decode_append",
    "ktt_b200_merge_partials",
)

_i32, _i64, _f32, _ptr = ctypes.c_int32, ctypes.c_int64, ctypes.c_float, ctypes.c_void_p


class AttnArgs(ctypes.Structure):
    """struct ktt_b200_attn_args."""

    _fields_ = [
        ("batch", _i32),
        ("heads", _i32),
        ("kv_heads", _i32),
        ("sq", _i32),
        ("sk", _i32),
        ("total_q", _i64),
        ("total_k", _i64),
        ("d", _i32),
        ("dv", _i32),
        ("causal", _i32),
        ("scale", _f32),
        ("kernel", _i32),
        ("q", _ptr),
        ("k", _ptr),
        ("v", _ptr),
        ("out", _ptr),
        ("lse", _ptr),
        ("q_strides", _i64 * 3),
        ("k_strides", _i64 * 3),
        ("v_strides", _i64 * 3),
        ("out_strides", _i64 * 3),
        ("lse_strides", _i64 * 3),
        ("mask", _ptr),
        ("mask_dtype", _i32),
        ("mask_strides", _i64 * 4),
        ("key_lengths", _ptr),
        ("cu_seqlens_q", _ptr),
        ("cu_seqlens_k", _ptr),
        ("dout", _ptr),
        ("dq", _ptr),
        ("dk", _ptr),
        ("dv_out", _ptr),
        ("dout_strides", _i64 * 3),
        ("dq_strides", _i64 * 3),
        ("dk_strides", _i64 * 3),
        ("dv_strides", _i64 * 3),
        ("workspace", _ptr),
        ("workspace_bytes", _i64),
    ]


class DecodeArgs(ctypes.Structure):
    """struct ktt_b200_decode_args."""

    _fields_ = [
        ("batch", _i32),
        ("heads", _i32),
        ("kv_heads", _i32),
        ("sq", _i32),
        ("sk", _i32),
        ("d", _i32),
        ("dv", _i32),
        ("scale", _f32),
        ("q", _ptr),
        ("k", _ptr),
        ("v", _ptr),
        ("out", _ptr),
        ("lse", _ptr),
        ("q_strides", _i64 * 3),
        ("k_strides", _i64 * 3),
        ("v_strides", _i64 * 3),
        ("out_strides", _i64 * 3),
        ("key_lengths", _ptr),
        ("splits", _i32),
        ("scratch", _ptr),
        ("scratch_bytes", _i64),
    ]


class DecodeAppendArgs(ctypes.Structure):
    """struct ktt_b200_decode_append_args."""

    _fields_ = [
        ("base", DecodeArgs),
        ("k_new", _ptr),
        ("v_new", _ptr),
        ("k_new_strides", _i64 * 2),
        ("v_new_strides", _i64 * 2),
        ("cos", _ptr),
        ("sin", _ptr),
        ("rope_row_stride", _i64),
        ("rope_by_position", _i32),
        ("lengths_out", _ptr),
    ]


def sources():
    return sorted(
        os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu")
    )


def _stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC, f) for f in os.listdir(CSRC)]
    deps.append(os.path.join(INCLUDE, "ktt_b200.h"))
    return any(os.path.getmtime(d) > built for d in deps)


def build(force=False, verbose=False):
    """Compiles every .cu under csrc/ into lib/libktt_b200.so for sm_100a (nvcc
    cross-compiles without a GPU). Returns the library path."""
    if not force and not _stale():
        return LIB_PATH
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("kohaku_tt_b200: nvcc not found; cannot build libktt_b200.so")
    os.makedirs(LIB_DIR, exist_ok=True)
    tmp = LIB_PATH + ".tmp"
    cmd = [nvcc, *NVCC_FLAGS, *EXTRA_NVCC_FLAGS, "-I", INCLUDE, "-o", tmp, *sources()]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(
            "kohaku_tt_b200: nvcc failed\n" + proc.stdout[-4000:] + proc.stderr[-8000:]
        )
    os.replace(tmp, LIB_PATH)
    if verbose:
        print(proc.stderr)
    return LIB_PATH


SHIM_SRC = os.path.join(CSRC, "torch_shim", "aten_shim.cpp")
SHIM_PATH = os.path.join(LIB_DIR, "libktt_b200_aten.so")


def build_shim(force=False):
    """Compiles the C++ registration of the aten overloads (csrc/torch_shim/aten_shim.cpp)
    against the installed torch and libktt_b200.so. Returns its path."""
    import torch
    from torch.utils import cpp_extension

    deps = [SHIM_SRC, os.path.join(INCLUDE, "ktt_b200.h")]
    if not force and os.path.exists(SHIM_PATH) and all(os.path.getmtime(d) <= os.path.getmtime(SHIM_PATH) for d in deps):
        return SHIM_PATH
    build()
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    tmp = SHIM_PATH + ".tmp"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
           f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    for inc in cpp_extension.include_paths():
        cmd += ["-I", inc]
    cmd += ["-I", os.path.join(cuda_home, "include"), SHIM_SRC, "-o", tmp,
            "-L", torch_lib, "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-lc10", "-lc10_cuda",
            "-L", LIB_DIR, "-lktt_b200", "-Wl,-rpath,$ORIGIN", f"-Wl,-rpath,{torch_lib}"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("kohaku_tt_b200: g++ failed on the aten shim\n" + proc.stderr[-8000:])
    os.replace(tmp, SHIM_PATH)
    return SHIM_PATH


_SHIM = None


def shim():
    """The loaded C++ registration shim, or None when it has not been built (the Python
    registration of aten.py then stands in)."""
    global _SHIM
    if _SHIM is None and os.path.exists(SHIM_PATH):
        lib()
        import torch  # noqa: F401  (its libraries must be loaded first)

        handle = ctypes.CDLL(SHIM_PATH)
        handle.ktt_b200_aten_set_scope.argtypes = [ctypes.c_int, ctypes.c_char_p]
        handle.ktt_b200_aten_set_scope.restype = None
        _SHIM = handle
    return _SHIM


_LIB = None


def lib():
    """The loaded library. Raises when it has not been built: there is no other path."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"kohaku_tt_b200: {LIB_PATH} is missing. Build it with "
            "`python -c 'import __graft_entry__ as g; g.build()'` (needs nvcc); "
            "there is no CPU or PyTorch fallback."
        )
    handle = ctypes.CDLL(LIB_PATH)
    for name in EXPORTS:
        if not hasattr(handle, name):
            raise RuntimeError(f"kohaku_tt_b200: {LIB_PATH} does not export {name}")
    handle.ktt_b200_abi_version.restype = ctypes.c_int
    handle.ktt_b200_last_error.restype = ctypes.c_char_p
    handle.ktt_b200_counters.argtypes = [ctypes.POINTER(_i64)]
    handle.ktt_b200_sdpa_supported.argtypes = [ctypes.POINTER(AttnArgs)]
    handle.ktt_b200_sdpa_backward_supported.argtypes = [ctypes.POINTER(AttnArgs)]
    handle.ktt_b200_sdpa_forward.argtypes = [ctypes.POINTER(AttnArgs), _ptr]
    handle.ktt_b200_sdpa_forward_workspace.argtypes = [ctypes.POINTER(AttnArgs)]
    handle.ktt_b200_sdpa_forward_workspace.restype = _i64
    handle.ktt_b200_forward_streams_per_sm.restype = ctypes.c_int
    handle.ktt_b200_sdpa_backward_workspace.argtypes = [ctypes.POINTER(AttnArgs)]
    handle.ktt_b200_sdpa_backward_workspace.restype = _i64
    handle.ktt_b200_sdpa_backward.argtypes = [ctypes.POINTER(AttnArgs), _ptr]
    handle.ktt_b200_decode_scratch_bytes.argtypes = [ctypes.POINTER(DecodeArgs)]
    handle.ktt_b200_decode_scratch_bytes.restype = _i64
    handle.ktt_b200_decode.argtypes = [ctypes.POINTER(DecodeArgs), _ptr]
    handle.ktt_b200_decode_static.argtypes = [ctypes.POINTER(DecodeArgs), _ptr]
    handle.ktt_b200_decode_append.argtypes = [ctypes.POINTER(DecodeAppendArgs), _ptr]
    handle.ktt_b200_set_trace.argtypes = [_ptr]
    handle.ktt_b200_set_dump.argtypes = [_ptr, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_int32]
    handle.ktt_b200_set_dump.restype = ctypes.c_int
    handle.ktt_b200_selftest_wait_timeout.argtypes = [_ptr]
    handle.ktt_b200_probe_read.argtypes = [_ptr, ctypes.c_int64, _ptr, _ptr]
    handle.ktt_b200_merge_partials.argtypes = [_ptr, _ptr, _ptr, _ptr, _i64, _i32, _i32, _ptr]
    if handle.ktt_b200_abi_version() != 1:
        raise RuntimeError("kohaku_tt_b200: libktt_b200.so has another ABI version")
    _LIB = handle
    return handle


def last_error():
    return lib().ktt_b200_last_error().decode("utf-8", "replace")


class UnsupportedAttention(NotImplementedError):
    """The kernels do not take the call (the reference raises
    KohakuTTUnsupportedOperator, a NotImplementedError: kohakutt/fallback.py:6-8)."""


def check(status, what):
    """Maps a status of the C ABI to the exception class the reference raises."""
    if status == OK:
        return
    msg = f"kohaku_tt_b200.{what}: {last_error()}"
    if status == ERR_UNSUPPORTED:
        raise UnsupportedAttention(msg)
    if status == ERR_BAD_ARGUMENT:
        raise ValueError(msg)
    raise RuntimeError(msg)


COUNTER_NAMES = (
    "attention_flash",
    "attention_mma",
    "attention_backward",
    "attention_decode",
    "attention_refused",
    "device_wait_timeouts",
    "attention_backward_flash",
)


def counters():
    """Calls per kernel family since the last reset (kohakutt.counters()'s attention_*
    entries, tt_bridge.hpp:112-136)."""
    buf = (_i64 * 8)()
    check(lib().ktt_b200_counters(buf), "counters")
    return {name: int(buf[i]) for i, name in enumerate(COUNTER_NAMES)}


def device_status():
    """Raises when a tcgen05 kernel gave up a bounded wait since the last check (call
    after a synchronize)."""
    code = ctypes.c_int(0)
    check(lib().ktt_b200_device_status(ctypes.byref(code)), "device_status")


def reset_counters():
    check(lib().ktt_b200_reset_counters(), "reset_counters")
