"""Error statistics of a result against a ruler (typically CPU float64).

Same quantities and keys as kohakutt.diff_stats (src/kohakutt/core/stats.py:9-40), so
numbers here read side by side with the reference's: statistics are reported, not
judged.
"""

import torch


def _triple(t):
    if t.numel() == 0:
        return 0.0, 0.0, 0.0
    return t.max().item(), t.median().item(), t.mean().item()


def diff_stats(result, reference):
    """abs / rel error max, median, mean (rel over positions where the ruler is
    nonzero), cosine similarity and the count of non-finite results, all in float64
    over the positions where both sides are finite."""
    got = result.detach().to("cpu", torch.float64).reshape(-1)
    want = reference.detach().to("cpu", torch.float64).reshape(-1)
    both = torch.isfinite(got) & torch.isfinite(want)
    delta = (got - want).abs()
    usable = both & (want != 0)
    abs_max, abs_median, abs_mean = _triple(delta[both])
    rel_max, rel_median, rel_mean = _triple(delta[usable] / want[usable].abs())
    g, w = got[both], want[both]
    scale = g.norm() * w.norm()
    return {
        "abs_max": abs_max,
        "abs_median": abs_median,
        "abs_mean": abs_mean,
        "rel_max": rel_max,
        "rel_median": rel_median,
        "rel_mean": rel_mean,
        "cosine": (torch.dot(g, w) / scale).item() if scale > 0 else 1.0,
        "nonfinite": int((~torch.isfinite(got)).sum()),
    }


def format_stats(stats):
    """One line with every statistic of diff_stats."""
    return (
        "abs max {abs_max:.3e} med {abs_median:.3e} mean {abs_mean:.3e} | "
        "rel max {rel_max:.3e} med {rel_median:.3e} mean {rel_mean:.3e} | "
        "cos {cosine:.6f} | nonfinite {nonfinite}"
    ).format(**stats)


def rel_rms(result, reference):
    """||result - reference|| / ||reference|| in float64: the metric of the reference's
    attention tests (tests/hardware/ops/test_flash.py:44-45)."""
    want = reference.detach().to("cpu", torch.float64)
    return ((result.detach().to("cpu", torch.float64) - want).norm() / want.norm()).item()
