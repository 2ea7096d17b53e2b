"""Device-side weight movement for the trainer -> engine sync.

``copy_tensors`` moves any number of (source, destination) tensor pairs of equal byte size in ONE kernel launch
(``sb_multi_copy``: a table of pointers and sizes, CTAs spread over the bytes), instead of one ``copy_`` launch per
parameter: a 36-layer dense model syncs ~400 tensors per step. Destinations may be peer-mapped memory of another GPU
on the same NVLink domain (plain stores), which is how shards reach an engine that lives on other GPUs.
CPU tensors fall back to ``copy_``.
"""

from __future__ import annotations

import torch


def copy_tensors(pairs) -> int:
    """Copy ``src -> dst`` for every pair (same dtype and number of elements, both contiguous). Returns bytes moved."""
    pairs = [(s, d) for s, d in pairs if s.numel() > 0]
    if not pairs:
        return 0
    total = 0
    if not pairs[0][0].is_cuda:
        for s, d in pairs:
            d.copy_(s.view_as(d))
            total += s.numel() * s.element_size()
        return total
    from slime_b200.ops import _lib

    n = len(pairs)
    table = torch.empty(3, n, dtype=torch.int64)
    for i, (s, d) in enumerate(pairs):
        assert s.is_contiguous() and d.is_contiguous() and s.dtype == d.dtype and s.numel() == d.numel(), "copy pairs must match"
        nbytes = s.numel() * s.element_size()
        table[0, i], table[1, i], table[2, i] = s.data_ptr(), d.data_ptr(), nbytes
        total += nbytes
    dev = pairs[0][0].device
    tdev = table.pin_memory().to(dev, non_blocking=True)
    fn = _lib.bind("sb_multi_copy", [_lib.c_void_p, _lib.c_void_p, _lib.c_void_p, _lib.c_int, _lib.c_long, _lib.c_int, _lib.c_void_p])
    _lib.check(fn(tdev[0].data_ptr(), tdev[1].data_ptr(), tdev[2].data_ptr(), n, total, _lib.sm_count(dev), _lib.stream()),
               "sb_multi_copy")
    # the table must outlive the launch: the caching allocator keeps the block bound to this stream until it is reused
    # by later work on the same stream, which is ordered after the kernel
    return total
