"""Debug mode for data-dependent indices (``SLIME_B200_CHECKS=1``).

A kernel fault on a shared GPU is expensive (the context is lost, and the device may be too), and the tools that would
localise it are not always available. The indices that can actually go out of range at run time are the data-dependent
ones: token ids, cache slots, block-table pages, positions, routed-expert destinations, segment tables. With the switch
on, every op that takes such an index tensor validates it on the host BEFORE the launch and raises ``IndexCheckError``
naming the op, the argument, the offending value and where it sits; nothing is launched with a bad index. The checks
synchronise (they read the tensors), so the mode is for debugging runs and for tests, not for timing.
"""

from __future__ import annotations

import os

import torch


class IndexCheckError(IndexError):
    pass


def enabled() -> bool:
    return os.environ.get("SLIME_B200_CHECKS", "0") == "1"


def index_range(op: str, arg: str, idx: torch.Tensor | None, upper: int, lower: int = 0) -> None:
    """Every element of ``idx`` lies in ``[lower, upper)``."""
    if idx is None or not enabled() or idx.numel() == 0:
        return
    flat = idx.reshape(-1)
    bad = (flat < lower) | (flat >= upper)
    if bool(bad.any()):
        where = int(torch.nonzero(bad)[0])
        raise IndexCheckError(f"{op}: {arg}[{where}] = {int(flat[where])} is outside [{lower}, {upper}) "
                              f"({int(bad.sum())} of {flat.numel()} entries are)")  # fmt: skip


def segments(op: str, seg: torch.Tensor, tq: int, tk: int) -> None:
    """A flash-attention segment table ``[n, 4] = (q_off, q_len, k_off, k_len)`` stays inside its tensors."""
    if not enabled() or seg.numel() == 0:
        return
    s = seg.long().cpu()
    for name, off, ln, total in (("query", s[:, 0], s[:, 1], tq), ("key", s[:, 2], s[:, 3], tk)):
        bad = (off < 0) | (ln < 0) | (off + ln > total)
        if bool(bad.any()):
            i = int(torch.nonzero(bad)[0])
            raise IndexCheckError(f"{op}: segment {i} covers {name} rows [{int(off[i])}, {int(off[i] + ln[i])}) of {total}")


def paged(op: str, block_table: torch.Tensor, seq_lens: torch.Tensor, page_size: int, num_slots: int) -> None:
    """The pages a decode step will read exist: lengths fit the table, and the used entries point inside the cache."""
    if not enabled() or seq_lens.numel() == 0:
        return
    lens = seq_lens.long().cpu()
    cap = block_table.shape[1] * page_size
    if bool((lens < 0).any()) or bool((lens > cap).any()):
        i = int(torch.nonzero((lens < 0) | (lens > cap))[0])
        raise IndexCheckError(f"{op}: seq_lens[{i}] = {int(lens[i])} does not fit a block table of {cap} tokens")
    bt = block_table.long().cpu()
    pages = num_slots // page_size
    for b in range(bt.shape[0]):
        used = -(-int(lens[b]) // page_size)
        row = bt[b, :used]
        if used and (bool((row < 0).any()) or bool((row >= pages).any())):
            j = int(torch.nonzero((row < 0) | (row >= pages))[0])
            raise IndexCheckError(f"{op}: block_table[{b}, {j}] = {int(row[j])} is not one of the cache's {pages} pages")
