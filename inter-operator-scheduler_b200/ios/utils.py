from typing import Sequence


def seqeq(seq1: Sequence, seq2: Sequence):
    """True when the two sequences agree on their common prefix."""
    return all(a == b for a, b in zip(seq1, seq2))


def iter_subset(s: int, include_emtpy_set=False):
    """
    Yield the non-empty sub-masks of bitmask ``s`` in decreasing numeric order (then 0 if asked):
    the standard ``sub = (sub - 1) & s`` walk (reference ``python/ios/utils.py:14-24``).
    """
    sub = s
    while sub:
        yield sub
        sub = (sub - 1) & s
    if include_emtpy_set:
        yield 0
