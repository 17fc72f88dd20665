"""Helpers shared by the parity tests."""
import torch


def band_check(scores: torch.Tensor, k: int, got, want, band: float, what="") -> int:
    """Two index lists for "the k largest of ``scores``" must be equal as sets, or differ only on positions whose
    score lies within ``band`` of the k-th largest score (positions that close to the threshold are interchangeable
    between two correct implementations that sum in a different order).  ``got`` / ``want`` may carry extra entries
    that are not part of the top-k (the appended window positions): those must agree exactly.  Returns the number of
    positions that differ."""
    got, want = [int(i) for i in got], [int(i) for i in want]
    assert len(got) == len(want), (what, len(got), len(want))
    diff = set(got) ^ set(want)
    if not diff:
        return 0
    s = scores.detach().float().cpu()
    kth = torch.sort(s, descending=True).values[min(k, s.numel()) - 1].item()
    bad = [i for i in diff if not (0 <= i < s.numel()) or abs(s[i].item() - kth) > band]
    assert not bad, (what, f"{len(bad)} of {len(diff)} differing positions lie outside the {band} band", bad[:8])
    return len(diff)
