"""Paged KV cache with hash-based prefix sharing.

Pages hold ``page_size`` tokens; the per-layer K and V tensors are
``[num_pages * page_size, Hkv, D]`` (slot = page * page_size + offset). A page whose
tokens form a complete, committed prefix block is indexed by the hash chain of its
token ids, so requests that share a prompt prefix (the ``n_samples_per_prompt`` siblings
of a GRPO group, multi-turn continuations) reuse the same physical pages. Only committed
KV is indexed, so an aborted / partial request never poisons the index. Unreferenced
indexed pages stay resident until evicted in LRU order; with a ``HostKVTier`` an evicted page's contents move to pinned
host memory under the same hash and come back on the next prefix match that reaches them.

The allocator hot path (free list, ref counts, hash index) is native C++ when the
``_engine_native`` extension is built; this module is the same logic in Python and the
fallback used by CPU tests.
"""

from __future__ import annotations

import collections
import hashlib
import struct

import torch


class OutOfPages(RuntimeError):
    pass


def _hash_block(parent: bytes, tokens) -> bytes:
    h = hashlib.blake2b(parent, digest_size=16)
    h.update(struct.pack(f"<{len(tokens)}i", *tokens))
    return h.digest()


class PageAllocator:
    def __init__(self, num_pages: int, page_size: int, enable_prefix_cache: bool = True):
        self.num_pages, self.page_size = num_pages, page_size
        self.enable_prefix_cache = enable_prefix_cache
        self.free = collections.deque(range(num_pages))
        self.refcnt = [0] * num_pages
        self.page_hash: list[bytes | None] = [None] * num_pages
        self.index: dict[bytes, int] = {}
        self.lru: collections.OrderedDict[int, None] = collections.OrderedDict()  # refcnt==0 indexed pages
        self.hits = self.queries = 0
        self.host_tier = None  # HostKVTier: where evicted pages go and where a broken chain is looked up again

    # ---- capacity --------------------------------------------------------------------
    def available(self) -> int:
        return len(self.free) + len(self.lru)

    def _take_page(self) -> int:
        if self.free:
            return self.free.popleft()
        if self.lru:
            page, _ = self.lru.popitem(last=False)
            if self.host_tier is not None and self.page_hash[page] is not None:
                self.host_tier.store(self.page_hash[page], page)
            self._unindex(page)
            return page
        raise OutOfPages("KV cache exhausted")

    def _unindex(self, page: int):
        h = self.page_hash[page]
        if h is not None and self.index.get(h) == page:
            del self.index[h]
        self.page_hash[page] = None

    def alloc(self, n: int) -> list[int]:
        if n > self.available():
            raise OutOfPages(f"need {n} pages, {self.available()} available")
        out = []
        for _ in range(n):
            p = self._take_page()
            self.refcnt[p] = 1
            out.append(p)
        return out

    def retain(self, page: int):
        if self.refcnt[page] == 0:
            self.lru.pop(page, None)
        self.refcnt[page] += 1

    def release(self, pages):
        for p in pages:
            self.refcnt[p] -= 1
            assert self.refcnt[p] >= 0, f"page {p} released too often"
            if self.refcnt[p] == 0:
                if self.page_hash[p] is not None:
                    self.lru[p] = None
                else:
                    self.free.append(p)

    # ---- prefix index -------------------------------------------------------------------
    def match_prefix(self, tokens: list[int]) -> tuple[list[int], bytes]:
        """Longest chain of indexed full pages matching ``tokens``; pages are retained for the caller.
        At least one token is always left uncached so the request still produces logits."""
        pages, parent = [], b""
        if not self.enable_prefix_cache:
            return pages, parent
        ps = self.page_size
        full = (len(tokens) - 1) // ps
        self.queries += full
        for i in range(full):
            h = _hash_block(parent, tokens[i * ps : (i + 1) * ps])
            p = self.index.get(h)
            if p is None:
                p = self._from_host(h)
                if p is None:
                    break
            else:
                self.retain(p)
            pages.append(p)
            parent = h
        self.hits += len(pages)
        return pages, parent

    def _from_host(self, h: bytes) -> int | None:
        """Bring a block that was evicted to the host tier back into a device page (retained for the caller)."""
        tier = self.host_tier
        if tier is None or not tier.touch(h) or self.available() == 0:
            return None
        page = self.alloc(1)[0]  # may push another unreferenced page out to the host tier
        if not tier.fetch(h, page):
            self.release([page])
            return None
        self.index[h] = page
        self.page_hash[page] = h
        return page

    def commit(self, page: int, parent: bytes, tokens: list[int]) -> bytes:
        """Index a full page whose KV has been written. Returns its chain hash."""
        h = _hash_block(parent, tokens)
        if self.enable_prefix_cache and h not in self.index and self.page_hash[page] is None:
            self.index[h] = page
            self.page_hash[page] = h
        return h

    def flush(self):
        """Drop the prefix index (weights changed: cached KV is stale)."""
        for p in list(self.lru):
            self.free.append(p)
        self.lru.clear()
        self.index.clear()
        self.page_hash = [None] * self.num_pages
        if self.host_tier is not None:
            self.host_tier.flush()

    def stats(self):
        out = {"free": len(self.free), "cached": len(self.lru), "hit_rate": self.hits / max(self.queries, 1)}
        if self.host_tier is not None:
            out.update(host_cached=len(self.host_tier.index), host_hits=self.host_tier.hits, host_stores=self.host_tier.stores)
        return out


class PagedKVCache:
    """Device tensors + allocator. Memory tag ``kv_cache``: released / re-created as a whole."""

    def __init__(self, num_layers, num_kv_heads, head_dim, num_pages, page_size, dtype, device, enable_prefix_cache=True,
                 v_head_dim: int | None = None):  # fmt: skip
        """``v_head_dim``: width of the value slab when it differs from the key slab's (0 for latent attention, whose
        single cached vector per token serves as key and value)."""
        self.num_layers, self.hkv, self.d = num_layers, num_kv_heads, head_dim
        self.dv = head_dim if v_head_dim is None else v_head_dim
        self.page_size, self.num_pages, self.dtype, self.device = page_size, num_pages, dtype, device
        self.allocator = PageAllocator(num_pages, page_size, enable_prefix_cache)
        self.k: list[torch.Tensor] = []
        self.v: list[torch.Tensor] = []
        self.allocate()

    def allocate(self):
        if self.k:
            return
        slots = self.num_pages * self.page_size
        # one slab per kind so a layer's cache is a contiguous view
        self._k_slab = torch.zeros(self.num_layers, slots, self.hkv, self.d, dtype=self.dtype, device=self.device)
        self._v_slab = torch.zeros(self.num_layers, slots, self.hkv, self.dv, dtype=self.dtype, device=self.device)
        self.k = [self._k_slab[i] for i in range(self.num_layers)]
        self.v = [self._v_slab[i] for i in range(self.num_layers)]

    def release(self):
        self.k, self.v = [], []
        self._k_slab = self._v_slab = None
        tier = self.allocator.host_tier
        self.allocator = PageAllocator(self.num_pages, self.page_size, self.allocator.enable_prefix_cache)
        if tier is not None:  # the device pages are gone; what the host holds stays valid until the weights change
            self.allocator.host_tier = tier
        if torch.cuda.is_available():
            torch.cuda.empty_cache()

    @staticmethod
    def bytes_per_page(num_layers, num_kv_heads, head_dim, page_size, dtype=torch.bfloat16, v_head_dim: int | None = None) -> int:
        width = head_dim + (head_dim if v_head_dim is None else v_head_dim)
        return num_layers * page_size * num_kv_heads * width * torch.empty(0, dtype=dtype).element_size()


class HostKVTier:
    """Second tier of the prefix cache: pinned host memory for pages the device tier evicted.

    ``store`` copies one page of every layer to a host slot (evicting the least recently used host page when full),
    ``fetch`` copies it back into a freshly allocated device page. Both copies run on the current stream, so they are
    ordered against the kernels that wrote the page before and the ones that overwrite it after. Same role as the
    engine's hierarchical cache behind ``--sglang-enable-hierarchical-cache`` / ``--sglang-hicache-ratio`` and the
    ``--release-hicache`` switch that frees the host pool when the KV cache is released
    (docker/patch/latest/sglang-release_hicache.patch in the reference)."""

    def __init__(self, kv: PagedKVCache, num_host_pages: int):
        self.kv, self.num_pages = kv, int(num_host_pages)
        self.index: collections.OrderedDict[bytes, int] = collections.OrderedDict()  # hash -> host slot, LRU order
        self.free = collections.deque(range(self.num_pages))
        self.hits = self.stores = 0
        self.k = self.v = None
        self.allocate()

    def allocate(self):
        if self.k is not None:
            return
        kv, pin = self.kv, self.kv.device.type == "cuda"
        self.k = torch.empty(self.num_pages, kv.num_layers, kv.page_size, kv.hkv, kv.d, dtype=kv.dtype, pin_memory=pin)
        self.v = torch.empty(self.num_pages, kv.num_layers, kv.page_size, kv.hkv, kv.dv, dtype=kv.dtype, pin_memory=pin)

    def release(self):
        """Free the host pool (``--release-hicache``)."""
        self.flush()
        self.k = self.v = None

    def flush(self):
        self.index.clear()
        self.free = collections.deque(range(self.num_pages))

    def num_bytes(self) -> int:
        return 0 if self.k is None else self.k.numel() * self.k.element_size() + self.v.numel() * self.v.element_size()

    def touch(self, h: bytes) -> bool:
        if self.k is None or h not in self.index:
            return False
        self.index.move_to_end(h)
        return True

    def _rows(self, page: int) -> slice:
        ps = self.kv.page_size
        return slice(page * ps, (page + 1) * ps)

    def store(self, h: bytes, page: int):
        if self.k is None or self.num_pages == 0 or not self.kv.k:
            return
        if h in self.index:
            self.index.move_to_end(h)
            return
        slot = self.free.popleft() if self.free else self.index.popitem(last=False)[1]
        rows = self._rows(page)
        self.k[slot].copy_(self.kv._k_slab[:, rows], non_blocking=True)
        self.v[slot].copy_(self.kv._v_slab[:, rows], non_blocking=True)
        self.index[h] = slot
        self.stores += 1

    def fetch(self, h: bytes, page: int) -> bool:
        slot = self.index.get(h)
        if slot is None or self.k is None or not self.kv.k:
            return False
        rows = self._rows(page)
        self.kv._k_slab[:, rows].copy_(self.k[slot], non_blocking=True)
        self.kv._v_slab[:, rows].copy_(self.v[slot], non_blocking=True)
        self.hits += 1
        return True
