"""Regenerates the golden fixtures in this folder from the reference itself.

Run where the reference tree is mounted (it cannot travel to a GPU box):

    make -C oracle ref REFERENCE=<reference>
    PYTHONPATH=<reference>/src python tests/golden/make_goldens.py

Sources of truth used, all the reference's own code:
  kohakutt.core.stats.diff_stats                       -> diff_stats.json
  kohakutt.torch_backend.lengths.masked (CPU tensors)  -> lengths_masked.pt
  kohakutt.torch_backend.lengths.device_lengths        -> device_lengths.json
  kohakutt.torch_backend.varlen.key_mask               -> key_mask.pt
  ktt_flash/varlen_plan.hpp via oracle/_ref/varlen_plan -> varlen_plan.json
  ktt.rotary's composite (csrc/aten/nn/aten_fused.cpp:30-43), a sequence of aten ops:
  the same aten calls issued one by one on CPU tensors  -> rotary.pt

Inputs are seeded exactly as the reference's tests seed theirs
(tests/hardware/ops/test_flash.py:48-53): torch.Generator().manual_seed(seed), randn in
fp32 on CPU, cast to bf16.
"""

import hashlib
import json
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))

# Key-length cases of tests/hardware/ops/test_attention_lengths.py:16-35.
LENGTH_CASES = [
    (4, 2, 2, 33, 32, [1, 32, 33, 17], False),
    (4, 2, 2, 33, 32, [1, 32, 33, 17], True),
    (2, 4, 2, 197, 64, [197, 64], False),
    (4, 4, 2, 70, 64, [1, 33, 70, 64], True),
    (3, 2, 2, 128, 64, [96, 1, 128], False),
]

# Packed length sets of tests/hardware/ops/test_flash_varlen.py:18-43,188-248 and
# test_flash_varlen_gaps.py:120-308: (lengths_q, lengths_k or None, causal).
PLAN_CASES = [
    ([32], None, False),
    ([40], None, False),
    ([1, 31, 33, 5, 64, 100], None, False),
    ([1, 31, 33, 5, 64, 100], None, True),
    ([3] * 50, None, True),
    ([32, 64, 96], None, True),
    ([201] * 8, None, False),
    ([700, 13, 1500], None, True),
    ([40, 7, 90], [25, 70, 33], False),
    ([40, 0, 90], [25, 70, 33], False),
    ([40, 7, 90], [50, 20, 100], True),
    ([4100, 100], None, True),
    ([5, 40, 3, 33, 70, 1, 31], None, True),
    ([40, 7, 90], [25, 70, 33], True),   # rejected: causal with Lq > Lk
    ([10, 5], [10, 0], False),           # rejected: queries without keys
]


def seeded(shapes, seed, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(*s, generator=g).to(dtype) for s in shapes]


def cumulative(lengths):
    out = [0]
    for n in lengths:
        out.append(out[-1] + n)
    return out


# Rotary cases: (x shape [B, H, S, D], rows of the cos / sin table, seed). The table has
# more rows than S so that the composite's narrow(-2, 0, S) does something.
ROTARY_CASES = [((2, 4, 7, 64), 16, 300), ((1, 2, 1, 128), 1, 301), ((3, 2, 33, 32), 40, 302)]


def aten_rotary(x, cos, sin):
    """The aten calls of rotary_composite (csrc/aten/nn/aten_fused.cpp:30-43), one per
    line and in its order, on CPU tensors."""
    s = x.size(-2)
    xf = torch.ops.aten.to.dtype(x, torch.float32)
    halves = torch.ops.aten.chunk.default(xf, 2, -1)
    rotated = torch.ops.aten.cat.default([torch.ops.aten.neg.default(halves[1]), halves[0]], -1)
    c = torch.ops.aten.to.dtype(torch.ops.aten.narrow.default(cos, -2, 0, s), torch.float32)
    n = torch.ops.aten.to.dtype(torch.ops.aten.narrow.default(sin, -2, 0, s), torch.float32)
    total = torch.ops.aten.add.Tensor(torch.ops.aten.mul.Tensor(xf, c), torch.ops.aten.mul.Tensor(rotated, n))
    return torch.ops.aten.to.dtype(total, x.dtype)


def rotary_fixture():
    out = {}
    for idx, (shape, rows, seed) in enumerate(ROTARY_CASES):
        (x,) = seeded([shape], seed)
        ang = seeded([(rows, shape[-1])], seed + 50, torch.float32)[0]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        out[f"case{idx}"] = {"x": x, "cos": cos, "sin": sin, "y": aten_rotary(x, cos, sin)}
    torch.save(out, os.path.join(HERE, "rotary.pt"))


def main():
    rotary_fixture()
    import kohakutt  # noqa: F401  (the reference package; AVAILABLE is False without a card)
    from kohakutt.core.stats import diff_stats
    from kohakutt.torch_backend import lengths as ref_lengths
    from kohakutt.torch_backend import varlen as ref_varlen

    # 1. diff_stats on seeded pairs, including zeros and non-finite entries.
    stats = []
    for seed, n in [(0, 1000), (1, 4096), (2, 17)]:
        a, b = seeded([(n,), (n,)], seed, torch.float32)
        r = (b + 0.01 * a).to(torch.bfloat16)
        ref = b.double().clone()
        if n > 20:
            ref[3] = 0.0
            r[5] = float("inf")
            ref[7] = float("nan")
        stats.append({"seed": seed, "n": n, "stats": diff_stats(r, ref)})
    with open(os.path.join(HERE, "diff_stats.json"), "w") as f:
        json.dump(stats, f, indent=1)

    # 2. lengths.masked on CPU bf16 tensors.
    masked = {}
    for idx, (b, h, hk, s, d, lens, causal) in enumerate(LENGTH_CASES):
        q, k, v = seeded([(b, h, s, d), (b, hk, s, d), (b, hk, s, d)], 100 + idx)
        out = ref_lengths.masked(q, k, v, torch.tensor(lens, dtype=torch.int32), causal, None)
        masked[f"case{idx}"] = out
    torch.save(masked, os.path.join(HERE, "lengths_masked.pt"))

    # 3. device_lengths: accepted values and the error messages.
    dl = []
    for arg, batch, keys in [([1, 5], 2, 5), ([0, 5], 2, 5), ([1, 6], 2, 5), ([1, 2, 3], 2, 5)]:
        try:
            t = ref_lengths.device_lengths(arg, batch, keys, torch.device("cpu"))
            dl.append({"arg": arg, "batch": batch, "keys": keys, "ok": t.tolist(), "dtype": str(t.dtype)})
        except ValueError as e:
            dl.append({"arg": arg, "batch": batch, "keys": keys, "error": str(e)})
    with open(os.path.join(HERE, "device_lengths.json"), "w") as f:
        json.dump(dl, f, indent=1)

    # 4. varlen.key_mask conversions (bool and additive, clamp at -5e5, divided by scale).
    g = torch.Generator().manual_seed(5)
    keep = torch.rand(64, generator=g) > 0.3
    add = torch.randn(64, generator=g) * 3
    add[::7] = float("-inf")
    km = {
        "keep": keep,
        "add": add,
        "bool_scale_0.125": ref_varlen.key_mask(keep, 0.125, 64, torch.device("cpu")),
        "add_scale_0.125": ref_varlen.key_mask(add, 0.125, 64, torch.device("cpu")),
    }
    torch.save(km, os.path.join(HERE, "key_mask.pt"))

    # 5. The packed-sequence planner, through the reference's own header.
    exe = os.path.join(ROOT, "oracle", "_ref", "varlen_plan")
    if not os.path.exists(exe):
        sys.exit("build oracle/_ref first: make -C oracle ref REFERENCE=<reference>")
    plans = []
    for lq, lk, causal in PLAN_CASES:
        cu_q, cu_k = cumulative(lq), cumulative(lk if lk is not None else lq)
        entry = {"cu_q": cu_q, "cu_k": cu_k, "causal": causal}
        for key_side in (0, 1):
            text = subprocess.run(
                [exe, str(int(causal)), str(key_side), str(len(cu_q) - 1), *map(str, cu_q), *map(str, cu_k)],
                capture_output=True, text=True, check=True).stdout.split("\n")
            if text[0].startswith("error"):
                entry["error"] = text[0][6:]
                break
            n = int(text[0].split()[1])
            iv = [tuple(map(int, line.split())) for line in text[1:1 + n]]
            head = text[1 + n].split()
            nrows, tiles = int(head[1]), int(head[2])
            rows = [list(map(int, line.split())) for line in text[2 + n:2 + n + nrows]]
            if key_side == 0:
                entry["queries"] = n
                entry["intervals_sha256"] = hashlib.sha256(json.dumps(iv).encode()).hexdigest()
                entry["intervals_head"] = iv[:4]
                entry["intervals_tail"] = iv[-4:]
                entry["rows"] = rows
                entry["tiles"] = tiles
            else:
                entry["key_rows"] = rows
                entry["key_tiles"] = tiles
        plans.append(entry)
    with open(os.path.join(HERE, "varlen_plan.json"), "w") as f:
        json.dump(plans, f)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
