"""Multi-rank host logic on CPU: ownership helpers, and ring attention over gloo ranks with
the block computation done by the float64 oracle, so that only the schedule, the messages
and the merge rule are under test (world sizes 2 and 4)."""

import math
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from kohaku_tt_b200 import parallel
from oracle import attention_oracle as ao


def test_shard_range_and_pairs():
    assert [parallel.shard_range(10, 4, r) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    pairs = parallel.shard_pairs(2, 10, 8)          # SDXL: 20 (batch, head) pairs over 8 GPUs
    assert sorted(p for r in pairs for p in r) == [(b, h) for b in range(2) for h in range(10)]
    assert max(map(len, pairs)) - min(map(len, pairs)) <= 1
    assert parallel.shard_pairs(64, 2, 8)[3] == [(b, h) for b in range(24, 32) for h in range(2)]


def test_shard_sequences_balances_work_and_keeps_sequences_whole():
    g = torch.Generator().manual_seed(0)
    lengths = [int(x) for x in torch.randint(64, 4097, (31,), generator=g)]
    for world in (1, 2, 4, 8):
        bounds = parallel.shard_sequences(lengths, world)
        assert bounds[0][0] == 0 and bounds[-1][1] == len(lengths)
        assert all(a[1] == b[0] for a, b in zip(bounds, bounds[1:]))
        work = [sum(n * n for n in lengths[a:b]) for a, b in bounds]
        assert all(w > 0 for w in work)
        assert max(work) <= 2.2 * sum(work) / world
    cu = [0]
    for n in lengths:
        cu.append(cu[-1] + n)
    rebased, (lo, hi) = parallel.rebase_cu_seqlens(cu, 3, 7)
    assert rebased[0] == 0 and rebased[-1] == hi - lo == sum(lengths[3:7])


def test_zigzag_roundtrip_and_balance():
    x = torch.arange(2 * 16 * 3).reshape(2, 16, 3)
    shards = parallel.zigzag_split(x, 4, dim=1)
    assert torch.equal(parallel.zigzag_merge(shards, dim=1), x)
    # Every rank does the same number of block products per step, and over all steps every
    # (query chunk, key chunk) pair with key <= query is visited exactly once.
    for world in (2, 4, 8):
        seen = set()
        for rank in range(world):
            mine = parallel.zigzag_chunks(world, rank)
            for step in range(world):
                j = (rank - step) % world
                theirs = parallel.zigzag_chunks(world, j)
                parts = parallel._visible_parts(world, rank, step)
                assert sum(len(kh) for _, kh, _ in parts) == 2 if step else True
                for half, key_halves, causal in parts:
                    for kh in key_halves:
                        pair = (mine[half], theirs[kh])
                        assert pair[1] <= pair[0] and pair not in seen
                        assert (causal is not False) == (pair[0] == pair[1]) or causal == "bottom_right"
                        seen.add(pair)
        chunks = 2 * world
        assert seen == {(a, b) for a in range(chunks) for b in range(a + 1)}


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cpu_attend(q, k, v, causal, scale):
    """Block attention in float64 with the oracle's rules (top-left or bottom-right)."""
    if causal == "bottom_right":
        out, lse = ao.c_forward(q, k, v, causal=2, scale=scale)
    else:
        out, lse = ao.c_forward(q, k, v, causal=1 if causal else 0, scale=scale)
    return out, lse.float()


def _cpu_attend_backward(dout, q, k, v, out, lse, causal, scale):
    """Block gradients against the *global* statistics: P = exp(S - lse), delta from the
    final output, exactly what the CUDA backward computes per block."""
    qd, kd, vd, dod, od = (t.double() for t in (q, k, v, dout, out))
    rep = q.shape[1] // k.shape[1]
    kr, vr = kd.repeat_interleave(rep, 1), vd.repeat_interleave(rep, 1)
    sc = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    s = qd @ kr.transpose(-1, -2) * sc
    lq, lk = q.shape[2], k.shape[2]
    if causal:
        shift = lk - lq if causal == "bottom_right" else 0
        keep = torch.arange(lk)[None, :] <= torch.arange(lq)[:, None] + shift
        s = s.masked_fill(~keep, -math.inf)
    p = torch.exp(s - lse.double()[..., None])
    delta = (dod * od).sum(-1, keepdim=True)
    ds = p * (dod @ vr.transpose(-1, -2) - delta)
    dq = ds @ kr * sc
    dk = (ds.transpose(-1, -2) @ qd * sc).reshape(k.shape[0], k.shape[1], rep, lk, -1).sum(2)
    dv = (p.transpose(-1, -2) @ dod).reshape(v.shape[0], v.shape[1], rep, lk, -1).sum(2)
    return dq, dk, dv


def _cpu_merge(acc_out, acc_lse, out, lse):
    m = torch.maximum(acc_lse, lse)
    wa, wb = torch.exp(acc_lse - m), torch.exp(lse - m)
    acc_out.copy_((acc_out * wa[..., None] + out.float() * wb[..., None]) / (wa + wb)[..., None])
    acc_lse.copy_(m + torch.log(wa + wb))


def _ring_worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        b, h, hk, chunk, d = 1, 4, 2, 24, 32
        seq = 2 * world * chunk
        q, k, v, do = ao.make_inputs([(b, h, seq, d), (b, hk, seq, d), (b, hk, seq, d), (b, h, seq, d)], 5,
                                     dtype=torch.float32)
        ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
        mine = lambda t: parallel.zigzag_split(t, world, dim=2)[rank]
        out, lse = parallel.ring_forward(mine(q), mine(k), mine(v), attend=_cpu_attend, merge=_cpu_merge)
        assert (out.double() - mine(ruler)).abs().max() < 1e-5
        assert (lse.double() - mine(ao.ruler_lse(q, k, v, causal=True))).abs().max() < 1e-5
        gq, gk, gv = parallel.ring_backward(mine(do), mine(q), mine(k), mine(v), mine(ruler).float(), lse,
                                            attend_backward=_cpu_attend_backward)
        for got, want in ((gq, dq), (gk, dk), (gv, dv)):
            assert (got.double() - mine(want)).abs().max() < 1e-4
        result[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_over_gloo_ranks(world):
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        result = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_ring_worker, args=(r, world, port, result)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(180)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(result) == {r: "ok" for r in range(world)}


def _silent_rank_worker(rank, world, port, result):
    """Failure detection on the host: rank 1 never posts its ring send; rank 0's receive
    runs into the process-group timeout and raises instead of hanging."""
    import datetime

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 0:
            q, k, v = ao.make_inputs([(1, 2, 16, 32)] * 3, 1, dtype=torch.float32)
            try:
                parallel.ring_forward(q, k, v, attend=_cpu_attend, merge=_cpu_merge)
                result[rank] = "no error"
            except Exception as e:  # gloo reports a timeout / closed connection
                result[rank] = "raised"
        else:
            result[rank] = "silent"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_silent_rank_is_detected_on_the_host():
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        result = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_silent_rank_worker, args=(r, 2, port, result)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(120)
        for p in procs:
            if p.is_alive():
                p.kill()
        assert result.get(0) == "raised" and result.get(1) == "silent"
