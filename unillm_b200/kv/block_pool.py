"""Paged KV allocation (the L2 / PagedAttention tier) and the radix prefix tree (L1), as Python
front ends of the C++ core in ``csrc/kv/kv_core.cpp``.

``BlockPool`` is the reference-counted page pool the engine uses.  ``PagedKvAllocator`` keeps the
reference's sequence-level API (``crates/kv/src/lib.rs:207-403``: ``allocate_sequence(max_length) ->
(seq_id, pages)``, ``extend_sequence``, ``free_sequence``, ``get_sequence``, ``get_stats``, ``defragment``)
on top of it and additionally exports block tables.  ``KvPage`` / ``KvBlock`` / ``KvSequence`` mirror
``lib.rs:37-204``.
"""
from __future__ import annotations

import ctypes as C
from array import array
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

from ..ops import _native as N
from ..types import MemoryError_, InvalidInput


def _lib():
    lib = N.host_lib()
    if not getattr(lib, "_ubkv_ready", False):
        lib.ubkv_pool_create.restype = C.c_void_p
        lib.ubkv_pool_create.argtypes = [C.c_int]
        lib.ubkv_pool_destroy.argtypes = [C.c_void_p]
        lib.ubkv_pool_alloc.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_int)]
        lib.ubkv_pool_incref.argtypes = [C.c_void_p, C.c_int]
        lib.ubkv_pool_decref.argtypes = [C.c_void_p, C.c_int]
        lib.ubkv_pool_num_free.argtypes = [C.c_void_p]
        lib.ubkv_pool_refcount.argtypes = [C.c_void_p, C.c_int]
        lib.ubkv_pool_stats.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
        lib.ubkv_radix_create.restype = C.c_void_p
        lib.ubkv_radix_create.argtypes = [C.c_int, C.c_void_p]
        lib.ubkv_radix_destroy.argtypes = [C.c_void_p]
        lib.ubkv_radix_match.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_int), C.c_int,
                                         C.POINTER(C.c_int)]
        lib.ubkv_radix_acquire.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_int), C.c_int,
                                           C.POINTER(C.c_int)]
        lib.ubkv_radix_insert.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.POINTER(C.c_int),
                                          C.POINTER(C.c_int)]
        lib.ubkv_radix_lock.argtypes = [C.c_void_p, C.c_int, C.c_int]
        lib.ubkv_radix_evict.argtypes = [C.c_void_p, C.c_int]
        lib.ubkv_radix_evictable.argtypes = [C.c_void_p]
        lib.ubkv_radix_stats.argtypes = [C.c_void_p, C.POINTER(C.c_uint64)]
        lib._ubkv_ready = True
    return lib


class BlockPool:
    """Fixed set of KV blocks with reference counts; a block returns to the free list at count 0."""

    def __init__(self, num_blocks: int, block_size: int = 16):
        if num_blocks <= 0 or block_size <= 0:
            raise InvalidInput("num_blocks and block_size must be positive")
        self.num_blocks, self.block_size = num_blocks, block_size
        self._lib = _lib()
        self._h = self._lib.ubkv_pool_create(num_blocks)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ubkv_pool_destroy(h)

    def allocate(self, n: int) -> List[int]:
        if n <= 0:
            return []
        buf = (C.c_int * n)()
        if self._lib.ubkv_pool_alloc(self._h, n, buf) != 0:
            raise MemoryError_(f"Not enough free pages: want {n}, have {self.num_free()}")
        return list(buf)

    def try_allocate(self, n: int) -> Optional[List[int]]:
        if n <= 0:
            return []
        buf = (C.c_int * n)()
        return list(buf) if self._lib.ubkv_pool_alloc(self._h, n, buf) == 0 else None

    def incref(self, block: int) -> int:
        r = self._lib.ubkv_pool_incref(self._h, block)
        if r < 0:
            raise InvalidInput(f"incref of free or invalid block {block}")
        return r

    def free(self, block: int) -> int:
        """Drops one reference; returns the remaining count."""
        r = self._lib.ubkv_pool_decref(self._h, block)
        if r < 0:
            raise InvalidInput(f"double free or invalid block {block}")
        return r

    def free_many(self, blocks: Sequence[int]) -> None:
        for b in blocks:
            self.free(b)

    def num_free(self) -> int:
        return self._lib.ubkv_pool_num_free(self._h)

    def refcount(self, block: int) -> int:
        return self._lib.ubkv_pool_refcount(self._h, block)

    def stats(self) -> Dict[str, int]:
        out = (C.c_uint64 * 4)()
        self._lib.ubkv_pool_stats(self._h, out)
        return {"allocated_total": out[0], "freed_total": out[1], "failed_allocations": out[2],
                "free_blocks": out[3], "total_blocks": self.num_blocks, "used_blocks": self.num_blocks - out[3]}


class RadixTree:
    """Path-compressed prefix tree over whole token blocks (RadixAttention)."""

    def __init__(self, pool: BlockPool):
        self.pool = pool
        self.block_size = pool.block_size
        self._lib = _lib()
        self._h = self._lib.ubkv_radix_create(pool.block_size, pool._h)

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h:
            self._lib.ubkv_radix_destroy(h)

    @staticmethod
    def _arr(tokens: Sequence[int]):
        # array('i') builds at C speed; the ctypes view shares its buffer (no per-element Python calls)
        a = array("i", tokens)
        return (C.c_int32 * len(a)).from_buffer(a)

    def match_prefix(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        """Longest cached prefix in whole blocks -> (block ids, node handle to lock)."""
        n = len(tokens)
        nb = n // self.block_size
        if nb == 0:
            return [], 0
        out = (C.c_int * nb)()
        node = C.c_int(0)
        m = self._lib.ubkv_radix_match(self._h, self._arr(tokens[: nb * self.block_size]), nb * self.block_size, out,
                                       nb, C.byref(node))
        return list(out[:m]), node.value

    def acquire_prefix(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        """``match_prefix`` that also locks the matched path and takes one pool reference per matched block, as one
        step with respect to eviction (for callers on several threads).  Undo with ``unlock(node)`` and one
        ``BlockPool.free`` per block."""
        n = len(tokens)
        nb = n // self.block_size
        if nb == 0:
            return [], 0
        out = (C.c_int * nb)()
        node = C.c_int(0)
        m = self._lib.ubkv_radix_acquire(self._h, self._arr(tokens[: nb * self.block_size]), nb * self.block_size, out,
                                         nb, C.byref(node))
        return list(out[:m]), node.value

    def insert(self, tokens: Sequence[int], blocks: Sequence[int]) -> Tuple[int, int]:
        """Caches the whole-block prefix of ``tokens`` backed by ``blocks`` (the tree takes its own
        reference on newly adopted blocks).  Returns (number of new blocks adopted, node handle)."""
        nb = min(len(tokens) // self.block_size, len(blocks))
        if nb == 0:
            return 0, 0
        node = C.c_int(0)
        barr = (C.c_int * nb)(*blocks[:nb])
        a = self._lib.ubkv_radix_insert(self._h, self._arr(tokens[: nb * self.block_size]), nb * self.block_size,
                                        barr, C.byref(node))
        return a, node.value

    def lock(self, node: int) -> None:
        if node > 0:
            self._lib.ubkv_radix_lock(self._h, node, 1)

    def unlock(self, node: int) -> None:
        if node > 0:
            self._lib.ubkv_radix_lock(self._h, node, -1)

    def evict(self, num_blocks: int) -> int:
        return self._lib.ubkv_radix_evict(self._h, num_blocks)

    def clear(self) -> int:
        """Drops every cache entry that no live sequence has locked (all of them once the sequences are released)."""
        n = 0
        while True:
            k = self.evict(1 << 30)
            if k <= 0:
                return n
            n += k

    def evictable_blocks(self) -> int:
        return self._lib.ubkv_radix_evictable(self._h)

    def stats(self) -> Dict[str, int]:
        o = (C.c_uint64 * 8)()
        self._lib.ubkv_radix_stats(self._h, o)
        return {"hits": o[0], "misses": o[1], "hit_tokens": o[2], "query_tokens": o[3], "evictions": o[4],
                "inserted_blocks": o[5], "cached_blocks": o[6], "nodes": o[7]}


# ------------------------------------------------------------------------------------------------
# Reference-shaped sequence allocator
# ------------------------------------------------------------------------------------------------
@dataclass
class KvPage:
    id: int
    device_ptr: int = 0
    is_allocated: bool = False
    sequence_id: Optional[int] = None
    last_access: float = 0.0

    def allocate(self, seq_id: int) -> None:
        self.is_allocated, self.sequence_id, self.last_access = True, seq_id, time.time()

    def free(self) -> None:
        self.is_allocated, self.sequence_id = False, None


@dataclass
class KvBlock:
    """A group of ``page_count`` consecutive pages (``lib.rs:79-142``)."""

    id: int
    page_count: int
    base_device_ptr: int
    page_size: int
    pages: List[KvPage] = field(default_factory=list)

    def __post_init__(self):
        if not self.pages:
            self.pages = [KvPage(self.id * self.page_count + i, self.base_device_ptr + i * self.page_size)
                          for i in range(self.page_count)]

    def allocate_page(self, seq_id: int) -> Optional[int]:
        for p in self.pages:
            if not p.is_allocated:
                p.allocate(seq_id)
                return p.id
        return None

    def free_page(self, page_id: int) -> bool:
        for p in self.pages:
            if p.id == page_id and p.is_allocated:
                p.free()
                return True
        return False


@dataclass
class KvSequence:
    seq_id: int
    max_length: int
    pages: List[int] = field(default_factory=list)
    current_length: int = 0
    created_at: float = field(default_factory=time.time)

    def add_page(self, page_id: int) -> None:
        self.pages.append(page_id)

    def remove_page(self, page_id: int) -> bool:
        if page_id in self.pages:
            self.pages.remove(page_id)
            return True
        return False

    def needs_more_pages(self, page_size: int) -> bool:
        return self.current_length > len(self.pages) * page_size

    def pages_needed(self, page_size: int) -> int:
        return (self.max_length + page_size - 1) // page_size


@dataclass
class KvAllocatorStats:
    total_pages: int
    allocated_pages: int
    free_pages: int
    active_sequences: int
    utilization_percent: float


class PagedKvAllocator:
    def __init__(self, total_pages: int, page_size_tokens: int = 16, pages_per_block: int = 16, base_ptr: int = 0,
                 bytes_per_page: int = 0):
        self.total_pages, self.page_size, self.pages_per_block = total_pages, page_size_tokens, pages_per_block
        self.base_ptr, self.bytes_per_page = base_ptr, bytes_per_page
        self.pool = BlockPool(total_pages, page_size_tokens)
        self.sequences: Dict[int, KvSequence] = {}
        self._next = 1

    def allocate_sequence(self, max_length: int) -> Tuple[int, List[int]]:
        need = (max_length + self.page_size - 1) // self.page_size
        pages = self.pool.allocate(need)
        sid = self._next
        self._next += 1
        seq = KvSequence(sid, max_length, pages)
        self.sequences[sid] = seq
        return sid, list(pages)

    def extend_sequence(self, seq_id: int, additional_length: int) -> List[int]:
        seq = self.sequences.get(seq_id)
        if seq is None:
            raise InvalidInput(f"Sequence {seq_id} not found")
        new_max = seq.max_length + additional_length
        need = (new_max + self.page_size - 1) // self.page_size - len(seq.pages)
        new = self.pool.allocate(need) if need > 0 else []
        seq.pages.extend(new)
        seq.max_length = new_max
        return new

    def free_sequence(self, seq_id: int) -> None:
        seq = self.sequences.pop(seq_id, None)
        if seq is None:
            raise InvalidInput(f"Sequence {seq_id} not found")
        self.pool.free_many(seq.pages)

    def get_sequence(self, seq_id: int) -> Optional[KvSequence]:
        return self.sequences.get(seq_id)

    def get_active_sequences(self) -> List[KvSequence]:
        return list(self.sequences.values())

    def block_table(self, seq_id: int) -> List[int]:
        return list(self.sequences[seq_id].pages)

    def page_device_ptr(self, page_id: int) -> int:
        return self.base_ptr + page_id * self.bytes_per_page

    def get_stats(self) -> KvAllocatorStats:
        free = self.pool.num_free()
        used = self.total_pages - free
        return KvAllocatorStats(self.total_pages, used, free, len(self.sequences), 100.0 * used / self.total_pages)

    def defragment(self) -> int:
        """Pages are position-independent behind block tables, so there is nothing to compact; returns 0."""
        return 0
