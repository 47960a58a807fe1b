"""Splitting attention work over the GPUs of one node.

Every attention configuration but one shards with no communication: (batch, head) pairs
are independent, as are packed sequences. That is the reference's own mesh rule (batch and
heads pass through, `aten_attention.cpp:500-527`) and what its tests pin ("no mixing across
pairs", `tests/hardware/ops/test_flash.py:580-590`). The helpers below only decide who
owns what.

The exception is one causal sequence too long for a GPU. The reference has no sequence
parallelism; its semantics there are simply "the same causal attention". `ring_forward`
and `ring_backward` compute exactly that with the sequence cut into 2 x W chunks, rank r
owning chunks r and 2W-1-r (zigzag, so every rank has the same causal work), K/V blocks
passed around a ring into local memory, and per-step partial results merged by their
log-sum-exp. On GPUs a rank pulls the previous rank's block with a device-to-device copy out
of CUDA-IPC-shared memory (`_PeerRing`: copy engines over NVLink, which need no SM, so the
copy runs beside the persistent attention kernels; a one-element all-reduce per step is the
only collective); point-to-point sends (NCCL, or gloo in the CPU tests) are the fallback.
No attention kernel reads another GPU's memory.
"""

import torch
import torch.distributed as dist


# ---- ownership ------------------------------------------------------------------------

def shard_range(n, world, rank):
    """[start, stop) of `n` items for `rank` of `world`, sizes differing by at most one."""
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def shard_pairs(batch, kv_heads, world):
    """The (batch, kv head) pairs of each rank, as evenly as possible; a pair is a whole GQA
    group, so K/V heads are never split from their query heads."""
    pairs = [(b, h) for b in range(batch) for h in range(kv_heads)]
    out = []
    for rank in range(world):
        lo, hi = shard_range(len(pairs), world, rank)
        out.append(pairs[lo:hi])
    return out


def shard_sequences(lengths, world, causal=True):
    """Contiguous ranges [first, last) of whole packed sequences per rank, balanced by
    attention work (sum of L^2 when causal or dense; the longest remaining prefix goes to
    the rank that keeps the maximum lowest)."""
    cost = [float(n) * float(n) for n in lengths]
    total = sum(cost)
    bounds, acc, start = [], 0.0, 0
    for rank in range(world):
        remaining_ranks = world - rank
        target = (total - acc) / remaining_ranks
        stop, got = start, 0.0
        # Leave at least one sequence for each later rank when there are enough.
        limit = len(lengths) - (remaining_ranks - 1) if len(lengths) >= world else len(lengths)
        while stop < limit and (got == 0.0 or got + cost[stop] / 2 <= target):
            got += cost[stop]
            stop += 1
        if rank == world - 1:
            stop = len(lengths)
            got = total - acc
        bounds.append((start, stop))
        acc += got
        start = stop
    return bounds


def rebase_cu_seqlens(cu_seqlens, first, last):
    """Offsets of sequences [first, last) rebased to start at 0, and the token range they
    cover in the packed tensors."""
    lo, hi = cu_seqlens[first], cu_seqlens[last]
    return [c - lo for c in cu_seqlens[first:last + 1]], (lo, hi)


# ---- ring attention ---------------------------------------------------------------------

def zigzag_chunks(world, rank):
    """The two sequence chunks (of 2 x world) that `rank` owns."""
    return rank, 2 * world - 1 - rank


def zigzag_split(x, world, dim):
    """Splits a full-sequence tensor along `dim` into the per-rank zigzag shards."""
    chunks = x.chunk(2 * world, dim=dim)
    return [torch.cat([chunks[r], chunks[2 * world - 1 - r]], dim=dim).contiguous() for r in range(world)]


def zigzag_merge(shards, dim):
    """Inverse of zigzag_split."""
    world = len(shards)
    chunks = [None] * (2 * world)
    for r, s in enumerate(shards):
        a, b = s.chunk(2, dim=dim)
        chunks[r], chunks[2 * world - 1 - r] = a, b
    return torch.cat(chunks, dim=dim)


def _default_attend(q, k, v, causal, scale):
    from . import ops

    # The K/V exchange runs beside these kernels and takes SMs from them for a while: the
    # CTAs draw their work from a counter, so the ones that start late just draw less.
    return ops.sdpa_forward(q, k, v, causal=causal, scale=scale, need_lse=True, dynamic=True)


def _default_attend_backward(dout, q, k, v, out, lse, causal, scale):
    from . import ops

    return ops.sdpa_backward(dout, q, k, v, out, lse, causal=causal, scale=scale)


def _default_merge(acc_out, acc_lse, out, lse):
    from . import ops

    ops.merge_partials(acc_out, acc_lse, out.contiguous(), lse.contiguous())


def _exchange(send, recv_like, group, rank, world):
    """Starts sending `send` (a list of tensors) to the next rank and receiving the same
    shapes from the previous one; returns (received tensors, requests)."""
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    recv = [torch.empty_like(t) for t in recv_like]
    ops_ = []
    for t in send:
        ops_.append(dist.P2POp(dist.isend, t, dist.get_global_rank(group, nxt) if group is not None else nxt, group))
    for t in recv:
        ops_.append(dist.P2POp(dist.irecv, t, dist.get_global_rank(group, prv) if group is not None else prv, group))
    return recv, dist.batch_isend_irecv(ops_)


class _PeerRing:
    """Two slots per rank for a travelling block (a flat buffer per slot) in memory the
    next rank can read: at step s a rank computes on slot s % 2 while a copy engine
    pulls the previous rank's slot s % 2 into its own slot (s + 1) % 2.

    Measured on 4 and 8 B200s with the 134 MB K/V block of the long-context workload: NCCL
    send/recv moved it at 161 GB/s per direction and, needing SMs that the persistent
    attention kernels hold, mostly ran after a step's compute instead of beside it (ring
    forward 5.97 ms on 4 GPUs for 4.28 ms of compute)."""

    _cache = {}

    def __init__(self, numel, dtype, device, group):
        from torch.multiprocessing.reductions import reduce_tensor

        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.flat = torch.empty((2, numel), dtype=dtype, device=device)
        self.flag = torch.zeros((1,), dtype=torch.int32, device=device)
        self.copy_stream = torch.cuda.Stream(device=device)
        self.prev_flat = None
        # Every rank takes part in both collectives below whatever happens to it, and all
        # ranks reach the same verdict: a ring that one rank could not set up is used by none.
        try:
            mine = reduce_tensor(self.flat)
        except Exception:   # no CUDA IPC for this memory in this environment
            mine = None
        handles = [None] * self.world
        dist.all_gather_object(handles, mine, group=group)
        good = torch.ones((1,), dtype=torch.int32, device=device)
        if any(h is None for h in handles):
            good.zero_()
        else:
            try:
                rebuild, args = handles[(self.rank - 1) % self.world]
                self.prev_flat = rebuild(*args)   # the previous rank's two slots, mapped into this process
            except Exception:
                good.zero_()
        dist.all_reduce(good, op=dist.ReduceOp.MIN, group=group)
        self.usable = bool(good.item())

    @classmethod
    def get(cls, numel, dtype, device, group):
        """The ring of this size for this group, or None where the ranks cannot read each
        other's memory (the callers then use the process group's send / recv)."""
        key = (numel, dtype, device, id(group) if group is not None else None)
        if key not in cls._cache:
            cls._cache[key] = cls(numel, dtype, device, group)
        ring = cls._cache[key]
        return ring if ring.usable else None

    @classmethod
    def release_all(cls):
        """Drops every ring: first the mappings of the previous ranks' slots, then, when every
        rank has done so, the slots themselves (a collective; call it on every rank before
        the process group goes)."""
        rings = list(cls._cache.values())
        cls._cache.clear()
        for ring in rings:
            torch.cuda.synchronize(ring.flat.device)
            ring.prev_flat = None
        for ring in rings:
            dist.barrier(group=ring.group)
            ring.flat = None

    def barrier(self):
        """Every rank's stream has reached this point (its kernels and the copies it waited for
        are done) before any rank's stream goes on."""
        dist.all_reduce(self.flag, group=self.group)

    def pull(self, step):
        """Starts copying the previous rank's slot step % 2 into this rank's other slot, on
        the copy stream, once the current stream has got here; returns the event to wait for."""
        here = torch.cuda.Event()
        here.record(torch.cuda.current_stream(self.flat.device))
        self.copy_stream.wait_event(here)
        with torch.cuda.stream(self.copy_stream):
            self.flat[(step + 1) % 2].copy_(self.prev_flat[step % 2], non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        return done

    def pull_into(self, dst, slot):
        """The same for the previous rank's slot `slot` into a local tensor `dst` (flat)."""
        here = torch.cuda.Event()
        here.record(torch.cuda.current_stream(self.flat.device))
        self.copy_stream.wait_event(here)
        with torch.cuda.stream(self.copy_stream):
            dst.copy_(self.prev_flat[slot], non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        return done


def _visible_parts(world, rank, step):
    """What the local queries see of the K/V block that arrives at `step` (the block of rank
    j = rank - step): a list of (query half, key halves, causal mode).

    Chunk order is global: rank r holds chunks r (half 0) and 2W-1-r (half 1).
      step 0, own block : half 0 x own half 0 on the diagonal; half 1 x both key halves,
                          diagonal at the end (bottom-right).
      j < r             : both query halves see the block's early chunk whole, and nothing
                          of its late chunk.
      j > r             : only query half 1 sees the block, both chunks whole.
    Every step costs the same number of (query, key) pairs: that is the zigzag's point."""
    j = (rank - step) % world
    if step == 0:
        return [(0, (0,), True), (1, (0, 1), "bottom_right")]
    if j < rank:
        return [(0, (0,), False), (1, (0,), False)]
    return [(1, (0, 1), False)]


def ring_forward(q, k, v, group=None, scale=None, attend=None, merge=None, exchange="auto"):
    """Causal attention of one sequence sharded zigzag over the ranks of `group`.

    q [B, H, 2C, D], k / v [B, Hk, 2C, D / Dv]: this rank's two chunks back to back. Returns
    (out [B, H, 2C, Dv] in q's dtype, lse [B, H, 2C] fp32). `attend(q, k, v, causal, scale)
    -> (out, lse)` and `merge(acc_out, acc_lse, out, lse)` default to this package's CUDA
    kernels; the CPU tests pass their own. `exchange`: "peer" (copies out of the previous
    rank's memory, CUDA only), "p2p" (send / recv of the process group) or "auto"."""
    attend = attend or _default_attend
    merge = merge or _default_merge
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    c = q.shape[2] // 2
    qh = [q[:, :, :c].contiguous(), q[:, :, c:].contiguous()]
    acc_out = [None, None]
    acc_lse = [None, None]
    peer = None
    if world > 1 and (exchange == "peer" or (exchange == "auto" and q.is_cuda and k.dtype == v.dtype)):
        # One flat buffer per slot: K then V.
        peer = _PeerRing.get(k.numel() + v.numel(), k.dtype, k.device, group)
        if peer is None and exchange == "peer":
            raise RuntimeError("ring_forward: the ranks cannot read each other's memory (CUDA IPC)")
    if peer is not None:
        peer.flat[0, :k.numel()].view(k.shape).copy_(k)
        peer.flat[0, k.numel():].view(v.shape).copy_(v)
        peer.barrier()   # every rank's slot 0 is filled, and nobody still works on an earlier call
    block = [k.contiguous(), v.contiguous()]
    for step in range(world):
        pending = None
        if step + 1 < world:
            if peer is not None:
                pulled = peer.pull(step)
            else:
                nxt, pending = _exchange(block, block, group, rank, world)
        if peer is not None:
            slot = peer.flat[step % 2]
            block = [slot[:k.numel()].view(k.shape), slot[k.numel():].view(v.shape)]
        kb, vb = block
        for half, key_halves, causal in _visible_parts(world, rank, step):
            # The early chunk is a view: the kernels read it through its strides.
            ks = kb if key_halves == (0, 1) else kb[:, :, :c]
            vs = vb if key_halves == (0, 1) else vb[:, :, :c]
            out, lse = attend(qh[half], ks, vs, causal, scale)
            if acc_out[half] is None:
                acc_out[half], acc_lse[half] = out.float().contiguous(), lse.contiguous().clone()
            else:
                merge(acc_out[half], acc_lse[half], out, lse)
        if pending is not None:
            for req in pending:
                req.wait()
            block = nxt
        if peer is not None and step + 1 < world:
            # The next step starts (and the slot just worked on may be overwritten, here and by
            # the next rank's pull) when every rank has finished this step's kernels and copy.
            torch.cuda.current_stream(k.device).wait_event(pulled)
            peer.barrier()
    out = torch.cat(acc_out, dim=2).to(q.dtype)
    return out, torch.cat(acc_lse, dim=2)


def _ring_backward_peer(dout, q, k, v, out, lse, group, scale, attend_backward, rings):
    """ring_backward with the blocks and the accumulators pulled out of the previous rank's
    memory (`_PeerRing`). Slot s % 2 of the accumulator ring holds, after step s, the sum of
    the contributions of every rank that has held the block this rank holds at step s; the
    next rank pulls it during step s + 1 and adds its own. After the last step the previous
    rank's slot is this rank's own block's gradient."""
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    dev = q.device
    c = q.shape[2] // 2
    halves = lambda t: [t[:, :, :c].contiguous(), t[:, :, c:].contiguous()]
    qh, doh, oh = halves(q), halves(dout), halves(out)
    lh = [lse[:, :, :c].contiguous(), lse[:, :, c:].contiguous()]
    dq = [torch.zeros(qh[0].shape, dtype=torch.float32, device=dev) for _ in range(2)]
    nk, nv = k.numel(), v.numel()
    blocks, sums = rings
    arrived = torch.empty((nk + nv,), dtype=torch.float32, device=dev)   # the previous rank's sums for the block in hand
    blocks.flat[0, :nk].view(k.shape).copy_(k)
    blocks.flat[0, nk:].view(v.shape).copy_(v)
    blocks.barrier()
    main = torch.cuda.current_stream(dev)
    for step in range(world):
        kv_pulled = blocks.pull(step) if step + 1 < world else None
        sums_pulled = sums.pull_into(arrived, (step - 1) % 2) if step > 0 else None
        slot = blocks.flat[step % 2]
        kb, vb = slot[:nk].view(k.shape), slot[nk:].view(v.shape)
        mine = sums.flat[step % 2]
        gk_sum, gv_sum = mine[:nk].view(k.shape), mine[nk:].view(v.shape)
        mine.zero_()
        for half, key_halves, causal in _visible_parts(world, rank, step):
            both = key_halves == (0, 1)
            ks = kb if both else kb[:, :, :c]
            vs = vb if both else vb[:, :, :c]
            gq, gk, gv = attend_backward(doh[half], qh[half], ks, vs, oh[half], lh[half], causal, scale)
            dq[half] += gq.float()
            span = slice(None) if both else slice(0, c)
            gk_sum[:, :, span] += gk.float()
            gv_sum[:, :, span] += gv.float()
        if sums_pulled is not None:
            main.wait_event(sums_pulled)
            mine += arrived
        if kv_pulled is not None:
            main.wait_event(kv_pulled)
        blocks.barrier()   # every rank's sums of this step are complete and its pulls are done
    main.wait_event(sums.pull_into(arrived, (world - 1) % 2))
    dk, dv = arrived[:nk].view(k.shape).to(k.dtype), arrived[nk:].view(v.shape).to(v.dtype)
    blocks.barrier()       # nobody overwrites a slot (a later call) that a neighbour still reads
    return torch.cat(dq, dim=2).to(q.dtype), dk, dv


def ring_backward(dout, q, k, v, out, lse, group=None, scale=None, attend_backward=None, exchange="auto"):
    """dq, dk, dv of ring_forward for this rank's shard. K/V blocks travel the ring again,
    each followed by an fp32 accumulator for its dk / dv that collects every rank's
    contribution and is handed back to the block's owner after the last step.

    The accumulators run one hop behind the blocks: a rank computes its contribution to the
    block it holds while that block's accumulator is still on its way from the previous
    rank, adds the two when it lands and sends the sum on while the next block is being
    worked on. Neither exchange waits for the other's compute. `exchange` as in
    ring_forward (on GPUs the default pulls both out of the previous rank's memory)."""
    attend_backward = attend_backward or _default_attend_backward
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world > 1 and (exchange == "peer" or (exchange == "auto" and q.is_cuda and k.dtype == v.dtype)):
        n = k.numel() + v.numel()
        rings = (_PeerRing.get(n, k.dtype, q.device, group), _PeerRing.get(n, torch.float32, q.device, group))
        if rings[0] is not None and rings[1] is not None:
            return _ring_backward_peer(dout, q, k, v, out, lse, group, scale, attend_backward, rings)
        if exchange == "peer":
            raise RuntimeError("ring_backward: the ranks cannot read each other's memory (CUDA IPC)")
    c = q.shape[2] // 2
    halves = lambda t: [t[:, :, :c].contiguous(), t[:, :, c:].contiguous()]
    qh, doh, oh = halves(q), halves(dout), halves(out)
    lh = [lse[:, :, :c].contiguous(), lse[:, :, c:].contiguous()]
    dq = [torch.zeros(qh[0].shape, dtype=torch.float32, device=q.device) for _ in range(2)]
    kv = [k.contiguous(), v.contiguous()]
    acc_in, acc_reqs, acc_sent = None, None, None   # the block in hand's accumulators on their way here (and the sums on their way out)
    for step in range(world):
        kb, vb = kv
        pending_kv = None
        if step + 1 < world:
            nxt_kv, pending_kv = _exchange(kv, kv, group, rank, world)
        # This rank's contribution to the block in hand.
        gk_sum = torch.zeros(kb.shape, dtype=torch.float32, device=kb.device)
        gv_sum = torch.zeros(vb.shape, dtype=torch.float32, device=vb.device)
        for half, key_halves, causal in _visible_parts(world, rank, step):
            both = key_halves == (0, 1)
            ks = kb if both else kb[:, :, :c]
            vs = vb if both else vb[:, :, :c]
            gq, gk, gv = attend_backward(doh[half], qh[half], ks, vs, oh[half], lh[half], causal, scale)
            dq[half] += gq.float()
            span = slice(None) if both else slice(0, c)
            gk_sum[:, :, span] += gk.float()
            gv_sum[:, :, span] += gv.float()
        if acc_reqs is not None:        # what the ranks before this one have added for the block
            for req in acc_reqs:        # (one exchange: the previous sums have left by then too)
                req.wait()
            gk_sum += acc_in[0]
            gv_sum += acc_in[1]
        # Send the sums on (after the last step: home to the block's owner) and start receiving
        # the accumulators of the next block in hand.
        acc_sent = [gk_sum, gv_sum]
        acc_in, acc_reqs = _exchange(acc_sent, acc_sent, group, rank, world)
        if pending_kv is not None:
            for req in pending_kv:
                req.wait()
            kv = nxt_kv
    for req in acc_reqs:
        req.wait()
    del acc_sent
    # After `world` hops the accumulators of this rank's own block are back.
    return (torch.cat(dq, dim=2).to(q.dtype), acc_in[0].to(k.dtype), acc_in[1].to(v.dtype))
