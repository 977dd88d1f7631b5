"""Stop sequences over generated token ids, and what may be shown while generating.

The reference matches stop strings against the decoded text of the tokens generated so far
(src/app/cli/runtime/streaming.zig:11-40).  This engine takes and returns token ids, so a stop
sequence here is a sequence of token ids and the same rules apply to ids instead of bytes:
generation ends when the generated ids end with a stop sequence, which is not part of the
response; while streaming, a tail that may still grow into a stop sequence is held back."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence


@dataclass(frozen=True)
class StopAnalysis:
    printable_len: int     # ids that can be shown now
    stop_hit: bool
    response_len: int      # ids of the response (without the stop sequence that ended it)


def analyze_generated(ids: Sequence[int], stop_sequences: Sequence[Sequence[int]]) -> StopAnalysis:
    """streaming.zig:11-40 on ids: the first stop sequence (in the order given) that the ids end
    with ends the response; otherwise the longest tail that is a proper prefix of a stop sequence
    is not printable yet.  Empty stop sequences are ignored."""
    n = len(ids)
    max_overlap = 0
    for stop in stop_sequences or ():
        m = len(stop)
        if m == 0:
            continue
        if n >= m and list(ids[n - m:]) == list(stop):
            return StopAnalysis(n - m, True, n - m)
        for overlap in range(min(n, m - 1), 0, -1):
            if list(ids[n - overlap:]) == list(stop[:overlap]):
                max_overlap = max(max_overlap, overlap)
                break
    return StopAnalysis(n - max_overlap, False, n)


def stop_hit_at(ids: Sequence[int], end: int, stop_sequences: Sequence[Sequence[int]]) -> int:
    """Length of the first stop sequence that ``ids[:end]`` ends with, or 0 (the check the
    scheduler makes after every token, without copying the output)."""
    for stop in stop_sequences or ():
        m = len(stop)
        if 0 < m <= end and all(ids[end - m + j] == stop[j] for j in range(m)):
            return m
    return 0
