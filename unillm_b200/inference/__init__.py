"""Asynchronous serving engine and its API types (exports follow ``crates/inference/src/lib.rs:14-38``)."""
from .engine import (Batch, BatchingStrategy, BatchOptimizer, BatchProcessor, EngineConfig, InferenceEngine,
                     ServingModelConfig, UniLLMInferenceEngine)
from .metrics import METRICS, HealthMonitor, InferenceMetrics, PerformanceCollector, RequestTimer, SimpleMetrics
from .types import (AttentionMechanism, ChatMessage, EngineHealth, FinishReason, GenerationStats, HealthStatus,
                    InferenceError, InferenceRequest, InferenceResponse, RequestBuilder, RequestMetadata,
                    ResponseBuilder, ResponseChunk, ResponseStream, StreamSender, TokenInfo)
from ..sampling import SamplingParams
