"""Readers of the kernels' profiling stamps (`ktt_b200_set_trace`), the counterpart of the
reference's FLASH_PROFILE device zones (ktt_flash/compute.cpp:25-30, program.hpp:56-65).

    python -m kohaku_tt_b200.trace forward     # head-dim-64 forward, headline shape
    python -m kohaku_tt_b200.trace backward    # tcgen05 backward, headline shape
    python -m kohaku_tt_b200.trace decode      # split-K decode, B 64, lengths U[512, 4096]

Each runs the workload a few times untraced, once with a trace buffer set, and prints where
the time of that launch went. The stamps are SM clocks (forward, per key block) or the
global nanosecond timer (per CTA).

`debug_flash_dump(q, k, v, is_causal, row)` is the counterpart of the reference's
`torch.ops.ktt._debug_flash_dump` (aten_attention.cpp:814-831): the intermediate values of
one query tile of the head-dim-64 forward, read out of the kernel's own registers."""

import collections
import statistics
import sys

import torch

from . import _lib, ops

ROWS = 64 + 1024   # 64 key-block rows of CTA 0, then one row per CTA
HEADLINE = dict(heads=14, kv_heads=2, seq=2048, dim=64)


def _randn(shape, gen, dev):
    return torch.randn(shape, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)


def _traced(dev, fn, warm=3):
    """Rows of the trace buffer [ROWS, 8] of one call of `fn` after `warm` untraced ones."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    buf = torch.zeros(ROWS * 8, dtype=torch.int64, device=dev)
    handle = _lib.lib()
    handle.ktt_b200_set_trace(buf.data_ptr())
    try:
        fn()
        torch.cuda.synchronize()
    finally:
        handle.ktt_b200_set_trace(None)
    _lib.device_status()
    return buf.cpu().view(ROWS, 8)


def _cta_rows(table, limit=1024):
    rows = table[64:64 + limit]
    return rows[rows[:, 0] > 0]


def _by_sm(rows):
    t0 = int(rows[:, 0].min())
    per_sm = collections.defaultdict(list)
    for r in rows:
        per_sm[int(r[2])].append((int(r[0]) - t0, int(r[1]) - t0, int(r[3])))
    return t0, per_sm


def forward(dev):
    """Key-block timeline of CTA 0 / stream 0 and the per-SM spread of the forward launch."""
    c = HEADLINE
    gen = torch.Generator(device=dev).manual_seed(0)
    q = _randn((1, c["heads"], c["seq"], c["dim"]), gen, dev)
    k = _randn((1, c["kv_heads"], c["seq"], c["dim"]), gen, dev)
    v = _randn((1, c["kv_heads"], c["seq"], c["dim"]), gen, dev)
    table = _traced(dev, lambda: ops.sdpa_forward(q, k, v, causal=True, kernel="flash"))
    base = int(table[0, 0])
    print("key block: S ready | maximum known | exponentials done | P published | first chunk loaded | "
          "its exponentials done | previous P V done | second chunk loaded   (clk after the first S)")
    for j in range(64):
        if int(table[j, 0]) == 0:
            break
        order = (0, 1, 2, 3, 4, 5, 6, 7)
        print(f"  {j:2d}: " + " | ".join(f"{int(table[j, s]) - base:6d}" if int(table[j, s]) else "     -" for s in order))
    epi = table[60]
    if int(epi[0]):
        other = ", other stream's half in %d, read %d, merged %d" % tuple(int(epi[i]) - base for i in (3, 4, 5)) if int(epi[3]) else ""
        print("epilogue: last P V done %d, row sums exchanged %d%s, written %d (clk after the first S)"
              % (int(epi[0]) - base, int(epi[2]) - base, other, int(epi[1]) - base))
    rows = _cta_rows(table)
    _, per_sm = _by_sm(rows)
    ends = sorted(max(e for _, e, _ in v_) for v_ in per_sm.values())
    blocks = sorted(sum(n for _, _, n in v_) for v_ in per_sm.values())
    print(f"streams {len(rows)} on {len(per_sm)} SMs; SM end ns min / median / max {ends[0]} / {ends[len(ends) // 2]} / {ends[-1]}; "
          f"key blocks per SM min / median / max {blocks[0]} / {blocks[len(blocks) // 2]} / {blocks[-1]}")


def backward(dev):
    """Per-CTA durations of the tcgen05 backward by kind and length, and the phases of a CTA."""
    c = HEADLINE
    gen = torch.Generator(device=dev).manual_seed(0)
    q = _randn((1, c["heads"], c["seq"], c["dim"]), gen, dev)
    do = _randn((1, c["heads"], c["seq"], c["dim"]), gen, dev)
    k = _randn((1, c["kv_heads"], c["seq"], c["dim"]), gen, dev)
    v = _randn((1, c["kv_heads"], c["seq"], c["dim"]), gen, dev)
    out, lse = ops.sdpa_forward(q, k, v, causal=True)
    table = _traced(dev, lambda: ops.sdpa_backward(do, q, k, v, out, lse, causal=True))
    rows = _cta_rows(table, 512)   # rows past 512 hold the per-warp item-loop clocks of the first CTAs
    t0, per_sm = _by_sm(rows)
    print(f"CTAs {len(rows)} on {len(per_sm)} SMs, first start to last end {(int(rows[:, 1].max()) - t0) / 1e3:.1f} us")
    group = c["heads"] // c["kv_heads"]
    blocks = c["seq"] // 128
    n_dkv = c["heads"] * blocks   # kv heads x head parts (the group is split over its heads here) x key blocks
    recs = []
    for r in rows:
        cid, dur = int(r[3]), int(r[1]) - int(r[0])
        local = cid if cid < n_dkv else cid - n_dkv
        items = blocks - (local // c["heads"]) % blocks
        recs.append((dur, "dK/dV" if cid < n_dkv else "dQ", items, r))
    for kind in ("dK/dV", "dQ"):
        for items in (blocks, blocks // 2, 1):
            d = sorted(x[0] for x in recs if x[1] == kind and x[2] == items)
            if d:
                print(f"  {kind} CTAs of {items:2d} items: {len(d)} CTAs, ns min / median / max {d[0]} / {d[len(d) // 2]} / {d[-1]}")
        ph = []
        for dur, kd, items, r in recs:
            if kd == kind and int(r[4]) and int(r[5]) and int(r[6]):
                stored = int(r[7]) if int(r[7]) else int(r[6])
                ph.append((int(r[4]) - int(r[0]), int(r[5]) - int(r[4]), int(r[6]) - int(r[5]), stored - int(r[6]), int(r[1]) - stored))
        if ph:
            med = [statistics.median(x[i] for x in ph) for i in range(5)]
            print(f"  {kind} median CTA ns: set-up {med[0]:.0f} | to first scores {med[1]:.0f} | item loop {med[2]:.0f} | "
                  f"results stored {med[3]:.0f} | ticket, sum of the parts, teardown {med[4]:.0f}")
    del group
    # Where the item loop of a dK/dV CTA spends its clocks, per score warp (first 56 CTAs).
    names = ["meeting + next fetch", "wait for S", "phase 1 (P)", "wait for dP", "phase 2 (dS)"]
    per_warp = []
    for w in range(8):
        rws = torch.stack([table[64 + 512 + c * 8 + w] for c in range(56)])
        rws = rws[rws[:, 5] >= 8]
        if len(rws):
            n = rws[:, 5].double()
            per_warp.append([float((rws[:, i].double() / n).median()) for i in range(5)])
    if per_warp:
        med = [statistics.median(x[i] for x in per_warp) for i in range(5)]
        print("  dK/dV item loop, clk per item (median over score warps): "
              + " | ".join(f"{nm} {v:.0f}" for nm, v in zip(names, med)) + f" | sum {sum(med):.0f}")
    # The same for the first dQ CTAs (the longest: all key blocks).
    names = ["mask row", "wait for S", "phase 1 (P)", "wait for dP", "phase 2 (dS)"]
    per_warp = []
    for w in range(8):
        rws = torch.stack([table[64 + 512 + 448 + c * 8 + w] for c in range(8)])
        rws = rws[rws[:, 5] >= 8]
        if len(rws):
            n = rws[:, 5].double()
            per_warp.append([float((rws[:, i].double() / n).median()) for i in range(5)])
    if per_warp:
        med = [statistics.median(x[i] for x in per_warp) for i in range(5)]
        print("  dQ item loop, clk per item (median over score warps): "
              + " | ".join(f"{nm} {v:.0f}" for nm, v in zip(names, med)) + f" | sum {sum(med):.0f}")


def decode(dev):
    """Phase stamps of the decode kernel's CTAs on the benchmark's decode workload."""
    g = torch.Generator().manual_seed(0)
    lengths = torch.randint(512, 4097, (64,), generator=g, dtype=torch.int32)
    gen = torch.Generator(device=dev).manual_seed(0)
    caches = [(_randn((64, 2, 4096, 128), gen, dev), _randn((64, 2, 4096, 128), gen, dev)) for _ in range(2)]
    q = _randn((64, 16, 1, 128), gen, dev)
    ln = lengths.to(dev)
    turn = [0]

    def call():
        turn[0] += 1
        ops.decode(q, *caches[turn[0] % 2], key_lengths=ln)

    table = _traced(dev, call, warm=4)
    rows = _cta_rows(table)
    t0 = int(rows[:, 0].min())
    names = ["start", "dependency met", "lengths scanned", "first tile landed", "stream end", "end"]
    for i, name in enumerate(names):
        col = sorted(int(x) - t0 for x in rows[:, i] if int(x))
        if col:
            print(f"  {name:18s} ns min / median / max {col[0]} / {col[len(col) // 2]} / {col[-1]}")


def debug_flash_dump(q, k, v, is_causal, row, scale=None):
    """Runs the head-dim-64 tcgen05 forward on (q, k, v) [B, H, S, 64] and returns what the
    kernel held for query tile `row` (index over B x H x query tiles of 128 rows, as in the
    reference's op): a dict with, per key block of the tile, `x` [blocks, 128, 128] (the
    exponents: scaled logit minus the reference maximum, -inf where the key is hidden), `p`
    (2^x as the bf16 values fed to P V) and `m` [blocks, 2, 128] (the reference maximum of
    each half row during the block); and `o` [128, 64] (unnormalised accumulator), `m_row`,
    `l_row` [128] at the end of the tile, plus the launch's `out` and `lse`. Blocks the tile
    does not have (causal) stay NaN."""
    if q.shape[-1] != 64 or q.dim() != 4:
        raise _lib.UnsupportedAttention("debug_flash_dump: the head-dim-64 forward only ([B, H, S, 64])")
    b, h, s, _ = q.shape
    tiles = (s + 127) // 128
    blocks = (k.shape[2] + 127) // 128
    bi, hi, ti = row // (h * tiles), (row // tiles) % h, row % tiles
    if not 0 <= bi < b:
        raise ValueError("debug_flash_dump: row %d of %d" % (row, b * h * tiles))
    block_floats, tail_floats = 2 * 128 * 128 + 2 * 128, 128 * 64 + 2 * 128
    buf = torch.full((blocks * block_floats + tail_floats,), float("nan"), dtype=torch.float32, device=q.device)
    handle = _lib.lib()
    if handle.ktt_b200_set_dump(buf.data_ptr(), bi, hi, ti, blocks) != 0:
        raise RuntimeError(_lib.last_error())
    try:
        out, lse = ops.sdpa_forward(q, k, v, causal=is_causal, scale=scale, kernel="flash")
        torch.cuda.synchronize(q.device)
    finally:
        handle.ktt_b200_set_dump(None, 0, 0, 0, 0)
    _lib.device_status()
    per_block = buf[:blocks * block_floats].view(blocks, block_floats)
    tail = buf[blocks * block_floats:]
    return {
        "batch": bi, "head": hi, "q_tile": ti,
        "x": per_block[:, :128 * 128].reshape(blocks, 128, 128),
        "p": per_block[:, 128 * 128:2 * 128 * 128].reshape(blocks, 128, 128),
        "m": per_block[:, 2 * 128 * 128:].reshape(blocks, 2, 128),
        "o": tail[:128 * 64].view(128, 64),
        "m_row": tail[128 * 64:128 * 64 + 128],
        "l_row": tail[128 * 64 + 128:],
        "out": out, "lse": lse,
    }


def main(argv):
    import kohaku_tt_b200 as ktt

    ktt.build()
    dev = torch.device("cuda", 0)
    what = argv[1] if len(argv) > 1 else "forward"
    {"forward": forward, "backward": backward, "decode": decode}[what](dev)


if __name__ == "__main__":
    main(sys.argv)
