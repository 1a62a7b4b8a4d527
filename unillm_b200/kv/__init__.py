"""Hybrid KV cache: paged block pool (L2), radix prefix tree (L1), tiering policy, device memory pool."""
from .block_pool import BlockPool, KvAllocatorStats, KvBlock, KvPage, KvSequence, PagedKvAllocator, RadixTree
from .hybrid import (AccessPattern, AdaptiveCachePolicy, CacheAnalysis, CacheHandle, CachePolicy, CacheTier,
                     CudaMemoryBackend, GpuAwareMemoryPool, GpuBackendType, GpuDevicePtr, GpuDeviceProperties,
                     GpuIntegratedCache, GpuIntegratedCacheBuilder, GpuIntegratedCacheStats, GpuMemoryBackend,
                     GpuMemoryError, HybridCacheStats, HybridKVCache, KVTensorPair, MockGpuBackend, RadixCache,
                     RadixCacheStats, SequenceInfo)
