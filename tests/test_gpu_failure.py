"""The device-side failure report end to end, without faulting anything: a bounded wait
that runs out is recorded in the host-visible status word, surfaces as an exception at the
next call, is counted, and leaves the GPU and the library usable
(the counterpart of the reference stream's deferred first-failure report,
csrc/core/device/stream.hpp:11-47)."""

import ctypes

import pytest
import torch

import kohaku_tt_b200 as ktt
from kohaku_tt_b200 import _lib, ops
from oracle import attention_oracle as ao
from tests.gpu_util import FWD_BOUND, qkv, rel

pytestmark = pytest.mark.gpu


def test_a_wait_that_runs_out_is_reported_counted_and_survivable(cuda):
    torch.cuda.synchronize()
    _lib.device_status()   # clean slate
    before = ktt.counters()["device_wait_timeouts"]
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    # One warp waits ~1e5 cycles on a barrier nobody arrives at, gives up and returns.
    _lib.check(_lib.lib().ktt_b200_selftest_wait_timeout(stream), "selftest")
    torch.cuda.synchronize()   # the kernel ended by itself
    q, k, v = (t.to(cuda) for t in qkv(1, 2, 2, 256, 256, 64, 3))
    # The next tcgen05 launch refuses to run on top of an unreported failure ...
    with pytest.raises(RuntimeError, match="gave up waiting .code 999"):
        ops.sdpa_forward(q, k, v, kernel="flash")
    assert ktt.counters()["device_wait_timeouts"] == before + 1
    ops.drop_forward_workspaces()
    # ... and with the report delivered everything works again.
    _lib.device_status()
    out, _ = ops.sdpa_forward(q, k, v, kernel="flash")
    assert rel(out, ao.ruler_dense(q.cpu(), k.cpu(), v.cpu())) <= FWD_BOUND
    # The explicit query reports the same way.
    _lib.check(_lib.lib().ktt_b200_selftest_wait_timeout(stream), "selftest")
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="code 999"):
        _lib.device_status()
    _lib.device_status()
    assert ktt.counters()["device_wait_timeouts"] == before + 2


def test_profiling_stamp_readers_run(cuda, capsys):
    # kohaku_tt_b200.trace: one traced launch of each kernel family at the benchmark shapes.
    from kohaku_tt_b200 import trace

    trace.forward(cuda)
    trace.backward(cuda)
    trace.decode(cuda)
    text = capsys.readouterr().out
    assert "key block" in text and "dK/dV CTAs" in text and "stream end" in text
    _lib.device_status()   # nothing gave up waiting while traced


def test_plain_read_probe_checks_its_arguments(cuda):
    import ctypes

    handle = _lib.lib()
    buf = torch.zeros(1 << 20, dtype=torch.uint8, device=cuda)
    sink = torch.zeros(1, dtype=torch.int32, device=cuda)
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda).cuda_stream)
    assert handle.ktt_b200_probe_read(ctypes.c_void_p(buf.data_ptr()), 1 << 20, ctypes.c_void_p(sink.data_ptr()), stream) == 0
    torch.cuda.synchronize()
    assert int(sink.item()) in (0, 1)
    for ptr, nbytes in ((buf.data_ptr() + 8, 1 << 10), (buf.data_ptr(), (1 << 10) + 4), (0, 1 << 10)):
        assert handle.ktt_b200_probe_read(ctypes.c_void_p(ptr), nbytes, ctypes.c_void_p(sink.data_ptr()), stream) == _lib.ERR_BAD_ARGUMENT
