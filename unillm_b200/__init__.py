"""unillm_b200: an LLM inference framework written for NVIDIA B200 (sm_100a).

Layers (lowest first): ``ops`` (CUDA kernels behind a C ABI, plus the ``TensorOps`` reference layer in
``tensor_core``), ``models`` (47 architectures behind ``Model`` / ``ModelRegistry``), ``kv`` (block pool, radix
tree, hybrid cache), ``engine`` (continuous-batching engine and GPU runner), ``dist`` (tensor / expert parallel
runtime with fused compute+collective kernels), ``scheduler``, ``inference`` (async serving API), ``weights``
(SafeTensors / PyTorch / GGUF), ``pipeline`` + ``cli`` + ``benchmark``.

Attribute access is lazy so that ``import unillm_b200`` stays cheap; ``unillm_b200.LLMEngine`` and the other names
listed in ``_EXPORTS`` resolve on first use.
"""
from __future__ import annotations

import importlib

__version__ = "0.1.0"

_EXPORTS = {
    # core types and configs
    "ModelError": "types", "DataType": "types", "Device": "types", "ModelFeature": "types",
    "Tensor": "tensor", "Runtime": "tensor",
    "Tracer": "utils", "span": "utils", "ReplicaRouter": "engine.replica",
    "GenerationConfig": "config", "EngineConfig": "config", "model_config": "config", "ModelConfig": "config",
    "Model": "model_core", "ModelInputs": "model_core", "ModelOutputs": "model_core", "ModelWeights": "model_core",
    "ModelRegistry": "model_core", "ModelFactory": "model_core", "registry": "model_core",
    "TensorOps": "tensor_core", "ops_fn": "tensor_core",
    "Sampler": "sampling", "GreedySampler": "sampling", "SamplingParams": "sampling",
    "Tokenizer": "tokenizer", "BatchTokenizer": "tokenizer",
    "KVCache": "kv_cache", "LayerKVCache": "kv_cache",
    "RoPECache": "precompute", "CausalMaskCache": "precompute", "SlidingWindowMaskCache": "precompute",
    # pipeline, registry, observability
    "InferencePipeline": "pipeline", "InferencePipelineBuilder": "pipeline", "InferenceMetrics": "pipeline",
    "OllamaRegistry": "ollama", "ModelInfo": "ollama",
    "METRICS": "inference.metrics", "SimpleMetrics": "inference.metrics",
    # engine and serving
    "LLMEngine": "engine.llm_engine", "GpuModelRunner": "engine.runner", "CpuModelRunner": "engine.cpu_runner",
    "UniLLMInferenceEngine": "inference", "InferenceRequest": "inference", "InferenceResponse": "inference",
    "InferenceEngine": "inference", "RequestBuilder": "inference", "ChatMessage": "inference",
    "ResponseStream": "inference", "StreamSender": "inference", "ResponseChunk": "inference",
    "FinishReason": "inference", "BatchProcessor": "inference", "BatchOptimizer": "inference",
    "BatchingStrategy": "inference", "PerformanceCollector": "inference", "EngineHealth": "inference",
    "HealthStatus": "inference",
    # KV bookkeeping
    "PagedKvAllocator": "kv", "RadixCache": "kv", "HybridKVCache": "kv", "AdaptiveCachePolicy": "kv",
    "CacheHandle": "kv", "CacheTier": "kv", "GpuIntegratedCache": "kv", "GpuIntegratedCacheBuilder": "kv",
    # host-side scheduling policies
    "ContinuousBatchingScheduler": "scheduler", "IntelligentScheduler": "scheduler", "SchedulingPolicy": "scheduler",
    "ChunkedPrefillManager": "scheduler", "ChunkedPrefillConfig": "scheduler", "StreamOverlapManager": "scheduler",
    "CacheAwareAnalyzer": "scheduler", "GpuMemoryTracker": "scheduler", "AdaptivePolicyEngine": "scheduler",
    "AdmissionController": "scheduler", "Request": "scheduler", "RequestBatch": "scheduler",
    "RequestPriority": "scheduler", "RequestState": "scheduler",
    # weights
    "ModelLoader": "weights", "UnifiedWeightLoader": "weights", "ConfigLoader": "weights",
    # benchmark
    "BenchmarkRunner": "benchmark.harness", "BenchmarkConfig": "benchmark.harness", "InferenceBackend": "benchmark.harness",
}

__all__ = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module 'unillm_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(f".{mod}", __name__), name)
    globals()[name] = value
    return value
