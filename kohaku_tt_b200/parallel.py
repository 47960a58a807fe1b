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
passed around a ring with point-to-point sends (NCCL over NVLink on GPUs, gloo in the CPU
tests) into local memory, and per-step partial results merged by their log-sum-exp.
No kernel reads another GPU's memory.
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


def ring_forward(q, k, v, group=None, scale=None, attend=None, merge=None):
    """Causal attention of one sequence sharded zigzag over the ranks of `group`.

    q [B, H, 2C, D], k / v [B, Hk, 2C, D / Dv]: this rank's two chunks back to back. Returns
    (out [B, H, 2C, Dv] in q's dtype, lse [B, H, 2C] fp32). `attend(q, k, v, causal, scale)
    -> (out, lse)` and `merge(acc_out, acc_lse, out, lse)` default to this package's CUDA
    kernels; the CPU tests pass their own."""
    attend = attend or _default_attend
    merge = merge or _default_merge
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    c = q.shape[2] // 2
    qh = [q[:, :, :c].contiguous(), q[:, :, c:].contiguous()]
    acc_out = [None, None]
    acc_lse = [None, None]
    block = [k.contiguous(), v.contiguous()]
    for step in range(world):
        pending = None
        if step + 1 < world:
            nxt, pending = _exchange(block, block, group, rank, world)
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
    out = torch.cat(acc_out, dim=2).to(q.dtype)
    return out, torch.cat(acc_lse, dim=2)


def ring_backward(dout, q, k, v, out, lse, group=None, scale=None, attend_backward=None):
    """dq, dk, dv of ring_forward for this rank's shard. K/V blocks travel the ring again,
    each followed by an fp32 accumulator for its dk / dv that collects every rank's
    contribution and is handed back to the block's owner after the last step.

    The accumulators run one hop behind the blocks: a rank computes its contribution to the
    block it holds while that block's accumulator is still on its way from the previous
    rank, adds the two when it lands and sends the sum on while the next block is being
    worked on. Neither exchange waits for the other's compute."""
    attend_backward = attend_backward or _default_attend_backward
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
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
