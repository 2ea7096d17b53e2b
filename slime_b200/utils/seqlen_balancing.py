"""Bin packing and k-way balanced partitioning of sequence lengths.

Parity: slime/utils/seqlen_balancing.py (karmarkar_karp :20, greedy :126,
get_seqlen_balanced_partitions :146, first_fit_pack :180,
expand_bins_by_splitting :218, get_reverse_idx :232).
"""

from __future__ import annotations

import heapq


def karmarkar_karp(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Largest-differencing method generalised to k parts.

    State = a k-tuple of (sum, members) sorted by sum; repeatedly merge the two
    states with the largest spread, pairing the heaviest part of one with the
    lightest of the other. With ``equal_size`` items are first grouped k at a
    time (sorted by weight) so every part receives the same item count.
    """
    n, k = len(seqlen_list), k_partitions
    order = sorted(range(n), key=lambda i: (seqlen_list[i], i))

    def make_state(items):
        parts = [(seqlen_list[i], [i]) for i in items]
        parts += [(0, [])] * (k - len(parts))
        parts.sort(key=lambda p: p[0])
        return parts

    states = []
    if equal_size:
        assert n % k == 0, f"{n} items cannot be split into {k} equal-size parts"
        for off in range(0, n, k):
            states.append(make_state(order[off : off + k]))
    else:
        states = [make_state([i]) for i in order]

    heap = []
    for uid, st in enumerate(states):
        heapq.heappush(heap, (-(st[-1][0] - st[0][0]), uid, st))
    uid = len(states)
    while len(heap) > 1:
        _, _, a = heapq.heappop(heap)
        _, _, b = heapq.heappop(heap)
        merged = [(a[i][0] + b[k - 1 - i][0], a[i][1] + b[k - 1 - i][1]) for i in range(k)]
        merged.sort(key=lambda p: p[0])
        heapq.heappush(heap, (-(merged[-1][0] - merged[0][0]), uid, merged))
        uid += 1
    final = heap[0][2] if heap else [(0, [])] * k
    parts = [sorted(p[1]) for p in final]
    if equal_size:
        for p in parts:
            assert len(p) * k == n
    return parts


def greedy_partition(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Longest-processing-time greedy; ``equal_size`` biases by item count."""
    bias = sum(seqlen_list) + 1 if equal_size else 0
    loads = [0] * k_partitions
    parts: list[list[int]] = [[] for _ in range(k_partitions)]
    for i in sorted(range(len(seqlen_list)), key=lambda j: -seqlen_list[j]):
        tgt = min(range(k_partitions), key=lambda p: loads[p])
        parts[tgt].append(i)
        loads[tgt] += seqlen_list[i] + bias
    return [sorted(p) for p in parts]


def get_seqlen_balanced_partitions(seqlen_list: list[int], k_partitions: int, equal_size: bool) -> list[list[int]]:
    """Partition indices into ``k_partitions`` lists with near-equal weight sums.

    Every index appears exactly once; no part is empty; parts come heaviest first (ties: more items first, then the
    smaller first index), each part's indices ascending: the same sample-to-rank assignment as the reference's
    partitioner (slime/utils/seqlen_balancing.py:20-110), so a run can be compared rank by rank.
    """
    assert len(seqlen_list) >= k_partitions, f"{len(seqlen_list)} items < {k_partitions} partitions"
    parts = karmarkar_karp(seqlen_list, k_partitions, equal_size)
    if any(len(p) == 0 for p in parts):  # degenerate weights (e.g. zeros): fall back
        parts = greedy_partition(seqlen_list, k_partitions, equal_size)
    seen = sorted(i for p in parts for i in p)
    assert seen == list(range(len(seqlen_list)))
    assert all(parts), "empty partition"
    parts = [sorted(p) for p in parts]
    return sorted(parts, key=lambda p: (-sum(seqlen_list[i] for i in p), -len(p), p[0]))


def first_fit_pack(total_lengths, max_tokens_per_bin: int) -> list[list[int]]:
    """First-fit in arrival order. A sample above the cap gets a bin of its own."""
    bins: list[list[int]] = []
    room: list[int] = []
    for i, n in enumerate(total_lengths):
        placed = False
        if n <= max_tokens_per_bin:
            for b in range(len(bins)):
                if room[b] >= n:
                    bins[b].append(i)
                    room[b] -= n
                    placed = True
                    break
        if not placed:
            bins.append([i])
            room.append(max(0, max_tokens_per_bin - n) if n <= max_tokens_per_bin else 0)
    return bins


def _split_bin_by_tokens(bin_indices: list[int], lengths) -> list[list[int]]:
    """Split one bin into two halves of near-equal token count (LPT over two sides)."""
    a, b, sa, sb = [], [], 0, 0
    for i in sorted(bin_indices, key=lambda j: -lengths[j]):
        if sa <= sb:
            a.append(i)
            sa += lengths[i]
        else:
            b.append(i)
            sb += lengths[i]
    return [sorted(a), sorted(b)]


def expand_bins_by_splitting(bins: list[list[int]], target_count: int, lengths) -> None:
    """Grow ``bins`` in place to ``target_count`` by halving the heaviest multi-sample bin."""
    while len(bins) < target_count:
        cands = [k for k, b in enumerate(bins) if len(b) > 1]
        if not cands:
            return
        k = max(cands, key=lambda j: sum(lengths[i] for i in bins[j]))
        left, right = _split_bin_by_tokens(bins[k], lengths)
        bins[k] = left
        bins.append(right)


def get_reverse_idx(idx_map):
    rev = [0] * len(idx_map)
    for new, old in enumerate(idx_map):
        rev[old] = new
    return rev
