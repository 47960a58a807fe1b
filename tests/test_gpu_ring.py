"""Ring attention on real GPUs (needs two): K/V blocks pulled out of the previous rank's
memory by device-to-device copies (the default on GPUs) and sent by NCCL send/recv (the
fallback), the CUDA kernels per block, merge by log-sum-exp; against the float64 ruler of the
whole sequence, and the two exchanges against each other bit for bit."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, result):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import kohaku_tt_b200 as ktt
        from kohaku_tt_b200 import parallel
        from oracle import attention_oracle as ao

        b, h, hk, chunk, d = 1, 4, 2, 256, 64
        seq = 2 * world * chunk
        q, k, v, do = ao.make_inputs([(b, h, seq, d), (b, hk, seq, d), (b, hk, seq, d), (b, h, seq, d)], 9)
        ruler, dq, dk, dv = ao.grads_dense(q, k, v, do, causal=True)
        mine = lambda t: parallel.zigzag_split(t, world, dim=2)[rank]
        qc, kc, vc, doc = (mine(t).to(dev) for t in (q, k, v, do))
        out, lse = parallel.ring_forward(qc, kc, vc)
        assert ktt.rel_rms(out, mine(ruler)) <= 8e-3
        assert (lse.cpu().double() - mine(ao.ruler_lse(q, k, v, causal=True))).abs().max() <= 3e-2
        gq, gk, gv = parallel.ring_backward(doc, qc, kc, vc, out, lse)
        for got, want in ((gq, dq), (gk, dk), (gv, dv)):
            assert ktt.rel_rms(got, mine(want)) <= 2e-2
        # The same through the process group's send / recv: the exchange moves bytes, the
        # arithmetic is the same, twice over (a second call reuses the shared slots).
        for _ in range(2):
            out2, lse2 = parallel.ring_forward(qc, kc, vc, exchange="p2p")
            again, again_lse = parallel.ring_forward(qc, kc, vc, exchange="peer")
            assert torch.equal(out, out2) and torch.equal(lse, lse2)
            assert torch.equal(out, again) and torch.equal(lse, again_lse)
            grads2 = parallel.ring_backward(doc, qc, kc, vc, out, lse, exchange="p2p")
            grads3 = parallel.ring_backward(doc, qc, kc, vc, out, lse, exchange="peer")
            assert all(torch.equal(a, b_) for a, b_ in zip((gq, gk, gv), grads2))
            assert all(torch.equal(a, b_) for a, b_ in zip((gq, gk, gv), grads3))
        torch.cuda.synchronize()
        parallel._PeerRing.release_all()
        result[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_ring_attention_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    with ctx.Manager() as manager:
        result = manager.dict()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, result)) for r in range(2)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(300)
        assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
        assert dict(result) == {0: "ok", 1: "ok"}
