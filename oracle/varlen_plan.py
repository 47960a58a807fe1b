"""TEST INFRASTRUCTURE ONLY: the packed-sequence visibility rule and tile-row plan.

Restates varlen::intervals and varlen::plan (ktt_flash/varlen_plan.hpp:43-82,88-143):
per packed query the half-open range [lo, hi) of packed key indices it sees, and per row
of 32 query tokens the key tiles [kfirst, klast] its tokens touch, of which the first `a`
and last `b` are partial (need an element mask). The CUDA kernels derive the same facts
on the device from cu_seqlens; tests compare them through this file.

Pinned against the reference's own header compiled into oracle/_ref/varlen_plan (where
the reference tree is mounted) and against tests/golden/varlen_plan.json generated from
it.
"""


class PlanError(ValueError):
    pass


def intervals(cu_q, cu_k, causal):
    """(lo, hi) lists, one entry per packed query token."""
    if len(cu_q) < 2 or len(cu_q) != len(cu_k) or cu_q[0] != 0 or cu_k[0] != 0:
        raise PlanError("offsets must be [0, ..., total] of equal count for queries and keys")
    lo, hi = [], []
    for b in range(len(cu_q) - 1):
        lq, lk = cu_q[b + 1] - cu_q[b], cu_k[b + 1] - cu_k[b]
        if lq < 0 or lk < 0 or (lq > 0 and lk == 0):
            raise PlanError("offsets must not decrease, and a sequence with queries needs keys")
        for r in range(lq):
            seen = min(lk, r + 1 + lk - lq) if causal else lk
            if seen <= 0:
                raise PlanError("causal with more queries than keys leaves queries without keys")
            lo.append(cu_k[b])
            hi.append(cu_k[b] + seen)
    return lo, hi


def plan(cu_q, cu_k, causal, tile=32):
    """Rows (kfirst, klast, a, b, u0) per `tile` packed queries, and the mask-tile count."""
    lo, hi = intervals(cu_q, cu_k, causal)
    rows, tiles = [], 0
    for i in range(0, len(lo), tile):
        idx = [min(i + r, len(lo) - 1) for r in range(tile)]
        rlo, rhi = [lo[t] for t in idx], [hi[t] for t in idx]
        kfirst, klast = min(rlo) // tile, (max(rhi) - 1) // tile
        nk = klast - kfirst + 1
        clear0 = max(kfirst, (max(rlo) + tile - 1) // tile)
        clear1 = min(klast + 1, min(rhi) // tile)
        if clear0 < clear1:
            a, b = clear0 - kfirst, klast + 1 - clear1
        else:
            a, b = nk, 0
        rows.append((kfirst, klast, a, b, tiles))
        tiles += a + b
    return rows, tiles
