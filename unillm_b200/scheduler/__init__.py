"""Scheduling: batch formation, chunked prefill, stream planning, policies, memory tracking, admission.
(Exports follow ``crates/scheduler/src/lib.rs:20-32``.)"""
from .core import (ChunkedPrefillConfig, ChunkedPrefillManager, ContinuousBatchingScheduler, OperationData, PrefillChunk,
                   PrefillStats, Request, RequestBatch, RequestPriority, RequestState, SchedulerStats, StreamOperation,
                   StreamOverlapManager, StreamOverlapStats, StreamPriority, StreamType, create_compute_operation,
                   create_d2h_operation, create_decode_operation, create_h2d_operation, create_prefill_operation)
from .policies import (AdaptivePolicyEngine, AdmissionController, AdmissionDecision, AllocationEvent,
                       AllocationRecommendation, BatchAnalysis, CacheAwareAnalyzer, CacheAwareBatchOptimizer,
                       GpuMemoryStats, GpuMemoryTracker, IntelligentScheduler, IntelligentSchedulerStats, KvShape,
                       MemoryFeasibility, OptimalBatchSize, OptimizationResult, PerformancePredictor, PolicyAction,
                       PolicyDecision, PrefixSharingGroup, RequestAnalysis, ResourceLimits, ResourceUsage, ScheduleInfo,
                       SchedulerMetrics, SchedulingPolicy, WatermarkStatus, WorkloadAnalyzer, WorkloadType, engine_policy)
