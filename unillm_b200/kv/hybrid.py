"""Hybrid KV cache (radix tier over paged tier), its tiering policy, device memory backends and pool,
and the GPU-integrated façade.

Parity with ``crates/kv/src``: ``CacheHandle`` / ``CacheTier`` / ``KVTensorPair`` (``hybrid_cache.rs:28-64``),
``RadixCache`` with ``find_longest_prefix`` / ``insert_sequence`` / stats (``:137-338``), ``AdaptiveCachePolicy`` /
``CachePolicy`` with the 0.6 / 0.2 prefix-sharing thresholds and promote / demote thresholds (``:342-462``),
``HybridKVCache`` (``:485-682``) and ``analyze_request`` (``:716-732``); ``GpuMemoryBackend`` with CUDA and mock
implementations, ``GpuAwareMemoryPool`` (``gpu_memory.rs:110-476, 508-589``); ``GpuIntegratedCache(+Builder)``
(``gpu_integrated_cache.rs:18-406``).

What is different: everything that the reference leaves as a stub or a leak works here -- sequences
can be freed, lookups return the cached blocks, radix leaves are unpinned when their user finishes
and eviction terminates, ``analyze_request`` inspects the real tree, the CUDA backend calls the real
C entry points (``csrc/kv/cuda_memory_backend.cu``), async copies really copy, and ``defragment``
releases pooled blocks back to the device instead of dropping them.  HIP is out of scope.
"""
from __future__ import annotations

import ctypes as C
import enum
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Sequence, Tuple

from ..types import DeviceError, InvalidInput, MemoryError_
from .block_pool import BlockPool, PagedKvAllocator, RadixTree


class CacheTier(enum.Enum):
    L1Radix = "l1_radix"
    L2Paged = "l2_paged"
    L3Extended = "l3_extended"


@dataclass(frozen=True)
class CacheHandle:
    tier: CacheTier
    id: int


@dataclass
class KVTensorPair:
    key_ptr: int
    value_ptr: int
    token_count: int
    head_dim: int
    num_heads: int
    size_bytes: int = 0

    @staticmethod
    def new(key_ptr: int, value_ptr: int, token_count: int, head_dim: int, num_heads: int) -> "KVTensorPair":
        return KVTensorPair(key_ptr, value_ptr, token_count, head_dim, num_heads, token_count * head_dim * num_heads * 2 * 2)


@dataclass
class RadixCacheStats:
    total_nodes: int = 0
    cache_hits: int = 0
    cache_misses: int = 0
    evictions: int = 0
    cached_blocks: int = 0
    hit_tokens: int = 0


class RadixCache:
    """Reference-shaped front of :class:`RadixTree`: token sequences in, (node, matched length) out."""

    def __init__(self, max_nodes: int = 10000, block_size: int = 16, pool: Optional[BlockPool] = None):
        self.max_blocks = max_nodes
        self.pool = pool or BlockPool(max(max_nodes, 1), block_size)
        self.tree = RadixTree(self.pool)
        self.block_size = block_size
        self.kv: Dict[int, KVTensorPair] = {}

    def find_longest_prefix(self, tokens: Sequence[int]) -> Tuple[Optional[int], int]:
        blocks, node = self.tree.match_prefix(list(tokens))
        return (node if blocks else None), len(blocks) * self.block_size

    def lookup_blocks(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        return self.tree.match_prefix(list(tokens))

    def insert_sequence(self, tokens: Sequence[int], kv_data: Optional[KVTensorPair] = None,
                        blocks: Optional[Sequence[int]] = None) -> int:
        """Caches the whole-block prefix of ``tokens``.  Without ``blocks`` fresh pool blocks back it."""
        nb = len(tokens) // self.block_size
        if nb == 0:
            return 0
        own = blocks is None
        if own:
            cached = self.tree.stats()["cached_blocks"]
            if cached + nb > self.max_blocks:
                self.tree.evict(cached + nb - self.max_blocks)
            got = self.pool.try_allocate(nb)
            if got is None:
                self.tree.evict(nb - self.pool.num_free())
                got = self.pool.allocate(nb)
            blocks = got
        _, node = self.tree.insert(list(tokens), list(blocks))
        if own:
            for b in blocks:            # the tree holds its own reference on what it adopted
                self.pool.free(b)
        if kv_data is not None:
            self.kv[node] = kv_data
        return node

    def pin(self, node: int) -> None:
        self.tree.lock(node)

    def unpin(self, node: int) -> None:
        self.tree.unlock(node)

    def evict(self, num_blocks: int) -> int:
        return self.tree.evict(num_blocks)

    def get_stats(self) -> RadixCacheStats:
        s = self.tree.stats()
        return RadixCacheStats(s["nodes"], s["hits"], s["misses"], s["evictions"], s["cached_blocks"], s["hit_tokens"])


class CachePolicy(enum.Enum):
    RadixPreferred = "radix_preferred"
    PagedPreferred = "paged_preferred"
    Balanced = "balanced"
    WorkloadAdaptive = "workload_adaptive"


@dataclass
class AccessPattern:
    sequence_id: int
    token_count: int
    shared_prefix_length: int
    timestamp: float = field(default_factory=time.monotonic)


@dataclass
class SequenceInfo:
    token_count: int
    has_common_prefix: bool
    expected_reuse: float = 0.0
    max_length: int = 0


class AdaptiveCachePolicy:
    RADIX_THRESHOLD, PAGED_THRESHOLD = 0.6, 0.2
    PROMOTE_FREQ, DEMOTE_FREQ, EVICT_FREQ = 0.7, 0.3, 0.1

    def __init__(self, policy: CachePolicy = CachePolicy.Balanced):
        self.current_policy = policy
        self.prefix_sharing_ratio = 0.0

    @staticmethod
    def new() -> "AdaptiveCachePolicy":
        return AdaptiveCachePolicy()

    def analyze_workload(self, patterns: Sequence[AccessPattern]) -> None:
        if not patterns:
            return
        shared = sum(1 for p in patterns if p.shared_prefix_length > 0)
        self.prefix_sharing_ratio = shared / len(patterns)
        if self.prefix_sharing_ratio > self.RADIX_THRESHOLD:
            self.current_policy = CachePolicy.RadixPreferred
        elif self.prefix_sharing_ratio < self.PAGED_THRESHOLD:
            self.current_policy = CachePolicy.PagedPreferred
        else:
            self.current_policy = CachePolicy.Balanced

    def select_tier(self, info: SequenceInfo) -> CacheTier:
        p = self.current_policy
        if p == CachePolicy.RadixPreferred:
            return CacheTier.L1Radix
        if p == CachePolicy.PagedPreferred:
            return CacheTier.L2Paged
        return CacheTier.L1Radix if (info.has_common_prefix or info.expected_reuse > 0.5) else CacheTier.L2Paged

    def should_promote(self, handle: CacheHandle, access_frequency: float) -> Optional[CacheTier]:
        if handle.tier == CacheTier.L2Paged and access_frequency > self.PROMOTE_FREQ:
            return CacheTier.L1Radix
        if handle.tier == CacheTier.L3Extended and access_frequency > self.DEMOTE_FREQ:
            return CacheTier.L2Paged
        return None

    def should_demote(self, handle: CacheHandle, access_frequency: float) -> Optional[CacheTier]:
        if handle.tier == CacheTier.L1Radix and access_frequency < self.DEMOTE_FREQ:
            return CacheTier.L2Paged
        if handle.tier == CacheTier.L2Paged and access_frequency < self.EVICT_FREQ:
            return CacheTier.L3Extended
        return None


@dataclass
class CacheAnalysis:
    cache_hit_potential: float
    estimated_cache_savings: int          # tokens that need no prefill
    recommended_tier: CacheTier


@dataclass
class HybridCacheStats:
    l1_stats: RadixCacheStats
    l2_total_pages: int
    l2_free_pages: int
    l2_active_sequences: int
    l3_entries: int
    total_sequences: int
    promotions: int
    demotions: int
    policy: str


class HybridKVCache:
    """L1 radix tree and L2 paged allocator over ONE block pool, plus an L3 host spill map."""

    def __init__(self, l1_max_nodes: int = 10000, l2_total_pages: int = 100000, l2_page_size: int = 16,
                 l2_pages_per_block: int = 16, base_ptr: int = 0, bytes_per_page: int = 0):
        self.l2 = PagedKvAllocator(l2_total_pages, l2_page_size, l2_pages_per_block, base_ptr, bytes_per_page)
        self.l1 = RadixCache(l1_max_nodes, l2_page_size, pool=self.l2.pool)
        self.l3: Dict[int, bytes] = {}
        self.policy = AdaptiveCachePolicy()
        self.page_size = l2_page_size
        self.handles: Dict[CacheHandle, dict] = {}
        self.patterns: Deque[AccessPattern] = deque(maxlen=1000)
        self._accesses = 0
        self._next_l1 = 1
        self.promotions = self.demotions = 0

    def allocate_sequence(self, tokens: Sequence[int], max_length: int) -> CacheHandle:
        tokens = list(tokens)
        blocks, node = self.l1.lookup_blocks(tokens)
        shared = len(blocks) * self.page_size
        tier = self.policy.select_tier(SequenceInfo(len(tokens), shared > 0, max_length=max_length))
        if tier == CacheTier.L1Radix and len(tokens) >= self.page_size:
            try:
                node = self.l1.insert_sequence(tokens)
                self.l1.pin(node)
                h = CacheHandle(CacheTier.L1Radix, self._next_l1)
                self._next_l1 += 1
                self.handles[h] = {"node": node, "tokens": len(tokens), "shared": shared}
                self.record_access(h, tokens, shared)
                return h
            except MemoryError_:
                pass
        sid, pages = self.l2.allocate_sequence(max(max_length, len(tokens)))
        h = CacheHandle(CacheTier.L2Paged, sid)
        self.handles[h] = {"pages": pages, "tokens": len(tokens), "shared": shared}
        self.record_access(h, tokens, shared)
        return h

    def free_sequence(self, handle: CacheHandle) -> None:
        info = self.handles.pop(handle, None)
        if info is None:
            raise InvalidInput(f"unknown cache handle {handle}")
        if handle.tier == CacheTier.L1Radix:
            self.l1.unpin(info["node"])
        elif handle.tier == CacheTier.L2Paged:
            self.l2.free_sequence(handle.id)
        else:
            self.l3.pop(handle.id, None)

    def lookup(self, tokens: Sequence[int]) -> Tuple[List[int], int]:
        """Cached blocks for the longest whole-block prefix and the number of tokens they cover."""
        blocks, _ = self.l1.lookup_blocks(list(tokens))
        return blocks, len(blocks) * self.page_size

    def block_table(self, handle: CacheHandle) -> List[int]:
        if handle.tier == CacheTier.L2Paged:
            return self.l2.block_table(handle.id)
        raise InvalidInput("only paged handles own a block table")

    def record_access(self, handle: CacheHandle, tokens: Sequence[int], shared_prefix: int = 0) -> None:
        self.patterns.append(AccessPattern(handle.id, len(tokens), shared_prefix))
        self._accesses += 1
        if self._accesses % 100 == 0:
            self.policy.analyze_workload(list(self.patterns))

    def migrate(self, handle: CacheHandle, tokens: Sequence[int], to: CacheTier) -> CacheHandle:
        """Tier migration: re-home a sequence (promotion L2 -> L1 publishes it to the radix tree)."""
        if handle.tier == to:
            return handle
        info = self.handles.get(handle)
        if info is None:
            raise InvalidInput(f"unknown cache handle {handle}")
        if handle.tier == CacheTier.L2Paged and to == CacheTier.L1Radix:
            pages = info["pages"]
            _, node = self.l1.tree.insert(list(tokens), pages)
            self.l1.pin(node)
            self.l2.free_sequence(handle.id)           # the tree keeps its own references on the adopted pages
            self.handles.pop(handle)
            h = CacheHandle(CacheTier.L1Radix, self._next_l1)
            self._next_l1 += 1
            self.handles[h] = {"node": node, "tokens": len(tokens), "shared": info["shared"]}
            self.promotions += 1
            return h
        if handle.tier == CacheTier.L1Radix and to == CacheTier.L2Paged:
            self.l1.unpin(info["node"])
            self.handles.pop(handle)
            sid, pages = self.l2.allocate_sequence(len(tokens))
            h = CacheHandle(CacheTier.L2Paged, sid)
            self.handles[h] = {"pages": pages, "tokens": len(tokens), "shared": info["shared"]}
            self.demotions += 1
            return h
        raise InvalidInput(f"migration {handle.tier} -> {to} is not supported")

    def analyze_request(self, prompt_tokens: Sequence[int], max_tokens: int = 0) -> CacheAnalysis:
        toks = list(prompt_tokens)
        _, cached = self.lookup(toks)
        pot = cached / len(toks) if toks else 0.0
        tier = self.policy.select_tier(SequenceInfo(len(toks), cached > 0, max_length=len(toks) + max_tokens))
        return CacheAnalysis(pot, cached, tier)

    def get_stats(self) -> HybridCacheStats:
        s = self.l2.get_stats()
        return HybridCacheStats(self.l1.get_stats(), s.total_pages, s.free_pages, s.active_sequences, len(self.l3),
                                len(self.handles), self.promotions, self.demotions, self.policy.current_policy.value)


# ------------------------------------------------------------------------------------------------
# device memory backends
# ------------------------------------------------------------------------------------------------
class GpuMemoryError(DeviceError):
    prefix = "GPU memory error"


@dataclass(frozen=True)
class GpuDevicePtr:
    ptr: int
    size: int
    alignment: int = 256
    device_id: int = 0

    def is_aligned(self) -> bool:
        return self.ptr % self.alignment == 0

    def offset(self, nbytes: int) -> "GpuDevicePtr":
        if nbytes > self.size:
            raise GpuMemoryError(f"offset {nbytes} beyond allocation of {self.size} bytes")
        return GpuDevicePtr(self.ptr + nbytes, self.size - nbytes, self.alignment, self.device_id)


@dataclass
class GpuDeviceProperties:
    name: str
    total_memory: int
    multiprocessor_count: int
    compute_capability: Tuple[int, int]
    max_shared_memory_per_block: int
    l2_cache_size: int
    memory_bus_width: int = 0


class GpuMemoryBackend:
    def allocate_device(self, size: int, alignment: int = 256) -> GpuDevicePtr: raise NotImplementedError
    def free_device(self, p: GpuDevicePtr) -> None: raise NotImplementedError
    def allocate_pinned(self, size: int) -> int: raise NotImplementedError
    def free_pinned(self, host_ptr: int) -> None: raise NotImplementedError
    def copy_h2d_async(self, dst: GpuDevicePtr, host_ptr: int, size: int, stream: int = 0) -> None: raise NotImplementedError
    def copy_d2h_async(self, host_ptr: int, src: GpuDevicePtr, size: int, stream: int = 0) -> None: raise NotImplementedError
    def synchronize(self, stream: int = 0) -> None: raise NotImplementedError
    def memory_info(self) -> Tuple[int, int]: raise NotImplementedError
    def device_properties(self) -> GpuDeviceProperties: raise NotImplementedError


class CudaMemoryBackend(GpuMemoryBackend):
    """Calls the C entry points ``ub_cuda_*`` of the kernel library (one ``cudaMemcpyAsync`` per copy)."""

    def __init__(self, device_id: int = 0):
        from ..ops import _native as N

        self.lib = N.cuda_lib()
        self.device_id = device_id
        self.lib.ub_cuda_device_count.restype = C.c_int
        if self.lib.ub_cuda_device_count() <= device_id:
            raise GpuMemoryError(f"CUDA device {device_id} not available")
        for name, args in (("ub_cuda_malloc_aligned", [C.POINTER(C.c_void_p), C.c_ulonglong, C.c_ulonglong]),
                           ("ub_cuda_free", [C.c_void_p]), ("ub_cuda_malloc_host", [C.POINTER(C.c_void_p), C.c_ulonglong]),
                           ("ub_cuda_free_host", [C.c_void_p]),
                           ("ub_cuda_memcpy_h2d_async", [C.c_void_p, C.c_void_p, C.c_ulonglong, C.c_void_p]),
                           ("ub_cuda_memcpy_d2h_async", [C.c_void_p, C.c_void_p, C.c_ulonglong, C.c_void_p]),
                           ("ub_cuda_stream_synchronize", [C.c_void_p]), ("ub_cuda_set_device", [C.c_int]),
                           ("ub_cuda_mem_info", [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong)])):
            f = getattr(self.lib, name)
            f.restype, f.argtypes = C.c_int, args
        self._check(self.lib.ub_cuda_set_device(device_id), "set device")

    def _check(self, rc: int, what: str) -> None:
        if rc != 0:
            raise GpuMemoryError(f"{what} failed: {self.lib.ub_cuda_error_string(rc).decode()}")

    def allocate_device(self, size, alignment=256):
        p = C.c_void_p()
        self._check(self.lib.ub_cuda_malloc_aligned(C.byref(p), size, alignment), f"device allocation of {size} bytes")
        return GpuDevicePtr(p.value, size, alignment, self.device_id)

    def free_device(self, p):
        self._check(self.lib.ub_cuda_free(p.ptr), "device free")

    def allocate_pinned(self, size):
        p = C.c_void_p()
        self._check(self.lib.ub_cuda_malloc_host(C.byref(p), size), f"pinned allocation of {size} bytes")
        return p.value

    def free_pinned(self, host_ptr):
        self._check(self.lib.ub_cuda_free_host(host_ptr), "pinned free")

    def copy_h2d_async(self, dst, host_ptr, size, stream=0):
        self._check(self.lib.ub_cuda_memcpy_h2d_async(dst.ptr, host_ptr, size, stream), "H2D copy")

    def copy_d2h_async(self, host_ptr, src, size, stream=0):
        self._check(self.lib.ub_cuda_memcpy_d2h_async(host_ptr, src.ptr, size, stream), "D2H copy")

    def synchronize(self, stream=0):
        self._check(self.lib.ub_cuda_stream_synchronize(stream), "stream synchronize")

    def memory_info(self):
        f, t = C.c_ulonglong(), C.c_ulonglong()
        self._check(self.lib.ub_cuda_mem_info(C.byref(f), C.byref(t)), "mem info")
        return f.value, t.value

    def device_properties(self):
        from ..ops import _native as N

        pr = N.UbDeviceProps()
        self.lib.ub_cuda_device_props.restype = C.c_int
        self.lib.ub_cuda_device_props.argtypes = [C.c_int, C.c_void_p]
        self._check(self.lib.ub_cuda_device_props(self.device_id, C.byref(pr)), "device properties")
        return GpuDeviceProperties(pr.name.decode(), pr.total_mem, pr.sm_count, (pr.cc_major, pr.cc_minor),
                                   pr.max_smem_per_block, pr.l2_bytes, pr.mem_bus_bits)


class MockGpuBackend(GpuMemoryBackend):
    """Bump allocator over fake addresses starting at 0x1000_0000 with a host shadow of every allocation
    (so copies can be checked) -- the CPU test double (``gpu_memory.rs:508-589``)."""

    def __init__(self, total_memory: int = 1 << 30, device_id: int = 0):
        self.total, self.used, self.next = total_memory, 0, 0x1000_0000
        self.device_id = device_id
        self.allocs: Dict[int, bytearray] = {}
        self.pinned: Dict[int, bytearray] = {}
        self._next_pinned = 0x7000_0000
        self.copies = {"h2d": 0, "d2h": 0}

    def allocate_device(self, size, alignment=256):
        if self.used + size > self.total:
            raise GpuMemoryError(f"out of memory: {size} requested, {self.total - self.used} free")
        self.next = (self.next + alignment - 1) // alignment * alignment
        p = GpuDevicePtr(self.next, size, alignment, self.device_id)
        self.allocs[p.ptr] = bytearray(size)
        self.next += size
        self.used += size
        return p

    def free_device(self, p):
        b = self.allocs.pop(p.ptr, None)
        if b is None:
            raise GpuMemoryError(f"free of unknown device pointer {p.ptr:#x}")
        self.used -= len(b)

    def allocate_pinned(self, size):
        p = self._next_pinned
        self._next_pinned += (size + 4095) // 4096 * 4096
        self.pinned[p] = bytearray(size)
        return p

    def free_pinned(self, host_ptr):
        if self.pinned.pop(host_ptr, None) is None:
            raise GpuMemoryError("free of unknown pinned pointer")

    def _dev(self, p: GpuDevicePtr, size: int) -> Tuple[bytearray, int]:
        for base, buf in self.allocs.items():
            if base <= p.ptr and p.ptr + size <= base + len(buf):
                return buf, p.ptr - base
        raise GpuMemoryError(f"device range {p.ptr:#x}+{size} is not inside an allocation")

    def copy_h2d_async(self, dst, host_ptr, size, stream=0):
        buf, off = self._dev(dst, size)
        buf[off:off + size] = self.pinned[host_ptr][:size]
        self.copies["h2d"] += 1

    def copy_d2h_async(self, host_ptr, src, size, stream=0):
        buf, off = self._dev(src, size)
        self.pinned[host_ptr][:size] = buf[off:off + size]
        self.copies["d2h"] += 1

    def synchronize(self, stream=0):
        return None

    def memory_info(self):
        return self.total - self.used, self.total

    def device_properties(self):
        return GpuDeviceProperties("MockGPU", self.total, 148, (10, 0), 227 * 1024, 126 << 20, 8192)


@dataclass
class GpuMemoryPoolStats:
    total_allocated: int
    total_pooled: int
    allocation_count: int
    pool_hits: int
    pool_misses: int
    device_free: int
    device_total: int


class GpuAwareMemoryPool:
    """Size-bucketed free lists over a backend, 256-byte alignment, power-of-two buckets."""

    ALIGN = 256

    def __init__(self, backend: GpuMemoryBackend):
        self.backend = backend
        self.buckets: Dict[int, List[GpuDevicePtr]] = {}
        self.live: Dict[int, GpuDevicePtr] = {}
        self.hits = self.misses = 0

    @staticmethod
    def new_cuda(device_id: int = 0) -> "GpuAwareMemoryPool":
        return GpuAwareMemoryPool(CudaMemoryBackend(device_id))

    @staticmethod
    def new_mock(total_memory: int = 1 << 30) -> "GpuAwareMemoryPool":
        return GpuAwareMemoryPool(MockGpuBackend(total_memory))

    @staticmethod
    def _bucket(size: int) -> int:
        b = GpuAwareMemoryPool.ALIGN
        while b < size:
            b <<= 1
        return b

    def allocate_aligned(self, size: int, alignment: int = 256) -> GpuDevicePtr:
        if size <= 0:
            raise InvalidInput("allocation size must be positive")
        b = self._bucket(size)
        lst = self.buckets.get(b)
        if lst:
            p = lst.pop()
            self.hits += 1
        else:
            p = self.backend.allocate_device(b, max(alignment, self.ALIGN))
            self.misses += 1
        self.live[p.ptr] = p
        return p

    def allocate_kv_cache(self, token_count: int, head_dim: int, num_heads: int, dtype_bytes: int = 2) -> KVTensorPair:
        half = token_count * head_dim * num_heads * dtype_bytes
        half_al = (half + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        p = self.allocate_aligned(2 * half_al)
        return KVTensorPair(p.ptr, p.ptr + half_al, token_count, head_dim, num_heads, 2 * half)

    def free_to_pool(self, p: GpuDevicePtr) -> None:
        q = self.live.pop(p.ptr, None)
        if q is None:
            raise GpuMemoryError(f"free of unknown pointer {p.ptr:#x}")
        self.buckets.setdefault(q.size, []).append(q)

    def get_memory_stats(self) -> GpuMemoryPoolStats:
        f, t = self.backend.memory_info()
        return GpuMemoryPoolStats(sum(p.size for p in self.live.values()),
                                  sum(p.size for l in self.buckets.values() for p in l), len(self.live), self.hits,
                                  self.misses, f, t)

    def defragment(self) -> int:
        """Returns half of every bucket's cached blocks to the device; returns the bytes released."""
        released = 0
        for lst in self.buckets.values():
            for _ in range(len(lst) // 2 + (len(lst) % 2 if len(lst) > 1 else 0)):
                p = lst.pop()
                self.backend.free_device(p)
                released += p.size
        return released

    def release_all(self) -> None:
        for lst in self.buckets.values():
            while lst:
                self.backend.free_device(lst.pop())


@dataclass
class GpuIntegratedCacheStats:
    hybrid: HybridCacheStats
    memory: GpuMemoryPoolStats
    h2d_transfers: int
    d2h_transfers: int
    promotions: int
    demotions: int
    active_allocations: int


class GpuBackendType(enum.Enum):
    Cuda = "cuda"
    Mock = "mock"


class GpuIntegratedCache:
    def __init__(self, hybrid: HybridKVCache, pool: GpuAwareMemoryPool):
        self.hybrid, self.pool = hybrid, pool
        self.device_ptrs: Dict[CacheHandle, KVTensorPair] = {}
        self.tokens: Dict[CacheHandle, List[int]] = {}
        self.h2d = self.d2h = 0

    @staticmethod
    def new_cuda(device_id: int = 0, **kw) -> "GpuIntegratedCache":
        return GpuIntegratedCacheBuilder(device_id, GpuBackendType.Cuda).build(**kw)

    def allocate_sequence(self, tokens: Sequence[int], max_length: int, head_dim: int, num_heads: int) -> CacheHandle:
        h = self.hybrid.allocate_sequence(tokens, max_length)
        try:
            self.device_ptrs[h] = self.pool.allocate_kv_cache(max(max_length, len(tokens)), head_dim, num_heads)
        except Exception:
            self.hybrid.free_sequence(h)
            raise
        self.tokens[h] = list(tokens)
        return h

    def free_sequence(self, handle: CacheHandle) -> None:
        kv = self.device_ptrs.pop(handle, None)
        if kv is None:
            raise GpuMemoryError(f"unknown cache handle {handle}")
        self.pool.free_to_pool(self.pool.live[kv.key_ptr])
        self.tokens.pop(handle, None)
        self.hybrid.free_sequence(handle)

    def device_pointers(self, handle: CacheHandle) -> KVTensorPair:
        return self.device_ptrs[handle]

    def copy_h2d_async(self, handle: CacheHandle, host_ptr: int, size: int, stream: int = 0) -> None:
        kv = self.device_ptrs[handle]
        if size > kv.size_bytes + 2 * GpuAwareMemoryPool.ALIGN:
            raise GpuMemoryError(f"copy of {size} bytes exceeds the sequence's {kv.size_bytes}-byte allocation")
        self.pool.backend.copy_h2d_async(self.pool.live[kv.key_ptr], host_ptr, size, stream)
        self.h2d += 1

    def copy_d2h_async(self, handle: CacheHandle, host_ptr: int, size: int, stream: int = 0) -> None:
        kv = self.device_ptrs[handle]
        self.pool.backend.copy_d2h_async(host_ptr, self.pool.live[kv.key_ptr], size, stream)
        self.d2h += 1

    def synchronize(self, stream: int = 0) -> None:
        self.pool.backend.synchronize(stream)

    def _rehome(self, handle: CacheHandle, to: CacheTier) -> CacheHandle:
        new = self.hybrid.migrate(handle, self.tokens.get(handle, []), to)
        if new != handle:
            self.device_ptrs[new] = self.device_ptrs.pop(handle)
            self.tokens[new] = self.tokens.pop(handle, [])
        return new

    def promote_to_l1(self, handle: CacheHandle) -> CacheHandle:
        return self._rehome(handle, CacheTier.L1Radix)

    def demote_from_l1(self, handle: CacheHandle) -> CacheHandle:
        return self._rehome(handle, CacheTier.L2Paged)

    def optimize_layout(self) -> int:
        return self.pool.defragment()

    def prefetch_sequences(self, handles: Sequence[CacheHandle]) -> int:
        """Touches the handles so the policy sees them as hot; returns how many were known."""
        n = 0
        for h in handles:
            if h in self.device_ptrs:
                self.hybrid.record_access(h, self.tokens.get(h, []))
                n += 1
        return n

    def get_device_properties(self) -> GpuDeviceProperties:
        return self.pool.backend.device_properties()

    def get_stats(self) -> GpuIntegratedCacheStats:
        return GpuIntegratedCacheStats(self.hybrid.get_stats(), self.pool.get_memory_stats(), self.h2d, self.d2h,
                                       self.hybrid.promotions, self.hybrid.demotions, len(self.device_ptrs))


class GpuIntegratedCacheBuilder:
    def __init__(self, device_id: int = 0, backend_type: GpuBackendType = GpuBackendType.Cuda):
        self.device_id, self.backend_type = device_id, backend_type
        self.l1_max_nodes, self.l2_total_pages, self.l2_page_size, self.pages_per_block = 10000, 100000, 16, 16
        self.mock_memory = 1 << 30

    def with_l1_capacity(self, max_nodes: int) -> "GpuIntegratedCacheBuilder":
        self.l1_max_nodes = max_nodes
        return self

    def with_l2_capacity(self, total_pages: int, page_size: int) -> "GpuIntegratedCacheBuilder":
        self.l2_total_pages, self.l2_page_size = total_pages, page_size
        return self

    def with_block_size(self, pages_per_block: int) -> "GpuIntegratedCacheBuilder":
        self.pages_per_block = pages_per_block
        return self

    def with_mock_memory(self, nbytes: int) -> "GpuIntegratedCacheBuilder":
        self.mock_memory = nbytes
        return self

    def build(self) -> GpuIntegratedCache:
        pool = GpuAwareMemoryPool.new_cuda(self.device_id) if self.backend_type == GpuBackendType.Cuda else \
            GpuAwareMemoryPool.new_mock(self.mock_memory)
        return GpuIntegratedCache(HybridKVCache(self.l1_max_nodes, self.l2_total_pages, self.l2_page_size,
                                                self.pages_per_block), pool)
