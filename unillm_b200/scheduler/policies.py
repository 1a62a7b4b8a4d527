"""Scheduling policies and the analysers around them: ``SchedulingPolicy`` (5 variants),
``CacheAwareBatchOptimizer``, ``IntelligentScheduler``, ``CacheAwareAnalyzer``, ``GpuMemoryTracker``,
``AdaptivePolicyEngine`` and ``AdmissionController``.

Parity with ``crates/scheduler/src``: ``intelligent_scheduler.rs`` (policies ``:18-29``, request analysis
``:62-108``, ``optimize_batch`` ``:111-224``, latency prior 128->10 ms ... 8192->300 ms ``:331-334``,
``IntelligentScheduler`` ``:362-603``, ``schedule_request`` ``:709-716``), ``cache_analyzer.rs`` (prefix groups
with a 32-token minimum ``:119-177``, hit-rate priors ``:180-212``, 50 us/token prefill model ``:252``),
``gpu_memory_tracker.rs`` (feasibility ``:51-102``, batch-size search ``:105-138``, pressure curve),
``adaptive_policy.rs`` (workload classes, switch thresholds ``:56-110``) and the orphan
``admission_control.rs`` (limits ``:9-32``, decisions ``:66-73``).

Where the reference has constant stubs, this module computes from real state: cache-hit potential
comes from a radix-tree lookup of the actual prompt, KV bytes from the model's shape, memory totals
from the block pool, fragmentation / OOM risk / watermarks from the allocation history.
The policy callables returned by :func:`engine_policy` plug into ``LLMEngine(policy=...)``.
"""
from __future__ import annotations

import bisect
import enum
import math
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional, Sequence, Tuple

from ..types import InvalidInput
from .core import Request, RequestBatch, RequestPriority, RequestState


class SchedulingPolicy(enum.Enum):
    FCFS = "fcfs"
    LongestPrefixMatch = "longest_prefix_match"
    CacheAware = "cache_aware"
    GpuMemoryOptimized = "gpu_memory_optimized"
    AdaptiveML = "adaptive"


@dataclass
class KvShape:
    """What one cached token costs: 2 (K,V) * layers * kv_heads * head_dim * bytes."""

    num_layers: int = 32
    num_kv_heads: int = 32
    head_dim: int = 128
    dtype_bytes: int = 2
    tp: int = 1

    def bytes_per_token(self) -> int:
        return 2 * self.num_layers * max(1, self.num_kv_heads // self.tp) * self.head_dim * self.dtype_bytes


@dataclass
class RequestAnalysis:
    request_id: int
    cache_hit_potential: float        # fraction of the prompt found in the prefix cache
    prefix_match_score: float
    cached_tokens: int
    memory_requirement: int           # KV bytes this request will need beyond the cached prefix
    predicted_latency: float          # seconds
    priority_weight: float


_LATENCY_TABLE = ((128, 0.010), (512, 0.025), (2048, 0.080), (8192, 0.300))


class PerformancePredictor:
    """Piece-wise linear prior over sequence length, scaled by the uncached fraction; refined online by
    an exponential moving average of observed step times per token."""

    def __init__(self):
        self.table = list(_LATENCY_TABLE)
        self.scale = 1.0

    def base_latency(self, seq_len: int) -> float:
        xs = [x for x, _ in self.table]
        i = bisect.bisect_left(xs, seq_len)
        if i == 0:
            return self.table[0][1] * seq_len / xs[0]
        if i >= len(xs):
            return self.table[-1][1] * seq_len / xs[-1]
        (x0, y0), (x1, y1) = self.table[i - 1], self.table[i]
        return y0 + (y1 - y0) * (seq_len - x0) / (x1 - x0)

    def predict_latency(self, request: Request, cache_hit_potential: float, memory_requirement: int = 0) -> float:
        return self.scale * self.base_latency(request.total_length()) * (1.0 - 0.8 * cache_hit_potential)

    def observe(self, predicted: float, actual: float) -> None:
        if predicted > 0 and actual > 0:
            self.scale = 0.9 * self.scale + 0.1 * self.scale * actual / predicted


class CacheAwareBatchOptimizer:
    def __init__(self, prefix_lookup: Optional[Callable[[Sequence[int]], int]] = None,
                 policy: SchedulingPolicy = SchedulingPolicy.CacheAware, kv: Optional[KvShape] = None):
        self.prefix_lookup = prefix_lookup or (lambda toks: 0)
        self.policy = policy
        self.kv = kv or KvShape()
        self.predictor = PerformancePredictor()

    def analyze_request(self, r: Request) -> RequestAnalysis:
        n = len(r.prompt_tokens)
        cached = min(n, max(0, int(self.prefix_lookup(r.prompt_tokens))))
        hit = cached / n if n else 0.0
        prefix_score = min(1.0, math.log10(max(n, 1)) / 4.0) * (0.5 + 0.5 * hit)
        mem = (r.total_length() - cached) * self.kv.bytes_per_token()
        lat = self.predictor.predict_latency(r, hit, mem)
        return RequestAnalysis(r.id, hit, prefix_score, cached, mem, lat, 1.0 + 0.5 * int(r.priority))

    def optimize_batch(self, requests: Sequence[Request], max_batch_size: int, max_memory: int) -> List[int]:
        an = {r.id: self.analyze_request(r) for r in requests}
        order = list(requests)
        p = self.policy
        if p == SchedulingPolicy.LongestPrefixMatch:
            order.sort(key=lambda r: (-an[r.id].cached_tokens, r.created_at))
        elif p == SchedulingPolicy.CacheAware:
            order.sort(key=lambda r: (-(an[r.id].cache_hit_potential * an[r.id].priority_weight), r.created_at))
        elif p == SchedulingPolicy.GpuMemoryOptimized:
            order.sort(key=lambda r: (an[r.id].memory_requirement, r.created_at))
        elif p == SchedulingPolicy.AdaptiveML:
            order.sort(key=lambda r: (-(0.5 * an[r.id].cache_hit_potential + 0.3 * an[r.id].priority_weight / 2.5
                                        - 0.2 * min(1.0, an[r.id].predicted_latency / 0.3)), r.created_at))
        else:
            order.sort(key=lambda r: (-int(r.priority), r.created_at))
        out, mem = [], 0
        for r in order:
            if len(out) >= max_batch_size:
                break
            if mem + an[r.id].memory_requirement > max_memory and out:
                continue
            out.append(r.id)
            mem += an[r.id].memory_requirement
        return out


@dataclass
class WorkloadCharacteristics:
    average_cache_hit_potential: float = 0.0
    average_prompt_length: float = 0.0
    average_memory_requirement: float = 0.0
    request_count: int = 0


class WorkloadAnalyzer:
    def __init__(self, window: int = 1000):
        self.history: Deque[RequestAnalysis] = deque(maxlen=window)
        self.lengths: Deque[int] = deque(maxlen=window)

    def analyze_request(self, a: RequestAnalysis, prompt_len: int = 0) -> None:
        self.history.append(a)
        self.lengths.append(prompt_len)

    def get_workload_characteristics(self) -> WorkloadCharacteristics:
        n = len(self.history)
        if n == 0:
            return WorkloadCharacteristics()
        return WorkloadCharacteristics(sum(a.cache_hit_potential for a in self.history) / n,
                                       sum(self.lengths) / n, sum(a.memory_requirement for a in self.history) / n, n)


@dataclass
class IntelligentSchedulerStats:
    total_requests: int = 0
    total_batches: int = 0
    completed_requests: int = 0
    policy: str = "cache_aware"
    policy_switches: int = 0
    average_cache_hit_potential: float = 0.0
    average_batch_size: float = 0.0


@dataclass
class ScheduleInfo:
    gpu_id: int
    memory_pressure: float
    estimated_latency: float
    cached_tokens: int = 0


class IntelligentScheduler:
    def __init__(self, max_batch_size: int = 32, max_memory: int = 8 << 30,
                 policy: SchedulingPolicy = SchedulingPolicy.CacheAware,
                 prefix_lookup: Optional[Callable[[Sequence[int]], int]] = None, kv: Optional[KvShape] = None,
                 memory_tracker: Optional["GpuMemoryTracker"] = None, num_gpus: int = 1,
                 policy_eval_interval_s: float = 30.0):
        self.max_batch_size, self.max_memory = max_batch_size, max_memory
        self.optimizer = CacheAwareBatchOptimizer(prefix_lookup, policy, kv)
        self.workload = WorkloadAnalyzer()
        self.adaptive = AdaptivePolicyEngine(policy)
        self.memory_tracker = memory_tracker
        self.pending: List[Request] = []
        self.active: Dict[int, Request] = {}
        self.num_gpus = num_gpus
        self.gpu_load = [0] * num_gpus
        self._next_id, self._next_batch = 1, 1
        self.stats = IntelligentSchedulerStats(policy=policy.value)
        self.last_policy_eval = time.monotonic()
        self.policy_eval_interval = policy_eval_interval_s
        self.last_batch_time = time.monotonic()

    @staticmethod
    def new_minimal(prefix_lookup: Optional[Callable[[Sequence[int]], int]] = None) -> "IntelligentScheduler":
        return IntelligentScheduler(prefix_lookup=prefix_lookup)

    @property
    def policy(self) -> SchedulingPolicy:
        return self.optimizer.policy

    def add_request(self, prompt_tokens: Sequence[int], max_output_length: int,
                    priority: RequestPriority = RequestPriority.Normal) -> int:
        rid = self._next_id
        self._next_id += 1
        r = Request.new(rid, prompt_tokens, max_output_length, priority)
        self.pending.append(r)
        a = self.optimizer.analyze_request(r)
        self.workload.analyze_request(a, len(prompt_tokens))
        self.stats.total_requests += 1
        n = self.stats.total_requests
        self.stats.average_cache_hit_potential += (a.cache_hit_potential - self.stats.average_cache_hit_potential) / n
        return rid

    def create_optimal_batch(self) -> Optional[RequestBatch]:
        if not self.pending:
            return None
        limit = self.max_batch_size
        if self.memory_tracker is not None:
            limit = max(1, min(limit, self.memory_tracker.suggest_batch_size(self.pending).recommended))
        ids = set(self.optimizer.optimize_batch(self.pending, limit, self.max_memory))
        if not ids:
            return None
        chosen = [r for r in self.pending if r.id in ids]
        self.pending = [r for r in self.pending if r.id not in ids]       # nothing is dropped
        now = time.monotonic()
        for r in chosen:
            r.state, r.started_at = RequestState.Prefilling, now
            self.active[r.id] = r
        b = RequestBatch.new(self._next_batch, chosen)
        self._next_batch += 1
        st = self.stats
        st.total_batches += 1
        st.average_batch_size += (len(chosen) - st.average_batch_size) / st.total_batches
        self.last_batch_time = now
        return b

    def evaluate_and_adapt_policy(self, metrics: Optional["SchedulerMetrics"] = None, force: bool = False) -> bool:
        now = time.monotonic()
        if not force and now - self.last_policy_eval < self.policy_eval_interval:
            return False
        self.last_policy_eval = now
        wc = self.workload.get_workload_characteristics()
        m = metrics or SchedulerMetrics(cache_hit_rate=wc.average_cache_hit_potential,
                                        memory_pressure=self.memory_tracker.memory_pressure() if self.memory_tracker else 0.0,
                                        queue_length=len(self.pending), policy=self.policy)
        d = self.adaptive.analyze_and_adapt(m)
        if d.action == PolicyAction.Switch and d.new_policy != self.policy:
            self.optimizer.policy = d.new_policy
            self.stats.policy, self.stats.policy_switches = d.new_policy.value, self.stats.policy_switches + 1
            return True
        return False

    def schedule_request(self, prompt_tokens: Sequence[int], max_tokens: int = 0) -> ScheduleInfo:
        """Placement of one request: least-loaded replica, current memory pressure, predicted latency."""
        r = Request.new(0, prompt_tokens, max_tokens)
        a = self.optimizer.analyze_request(r)
        gpu = min(range(self.num_gpus), key=lambda g: self.gpu_load[g])
        self.gpu_load[gpu] += 1
        pressure = self.memory_tracker.memory_pressure() if self.memory_tracker else 0.0
        return ScheduleInfo(gpu, pressure, a.predicted_latency, a.cached_tokens)

    def release_gpu(self, gpu_id: int) -> None:
        self.gpu_load[gpu_id] = max(0, self.gpu_load[gpu_id] - 1)

    def get_comprehensive_stats(self) -> IntelligentSchedulerStats:
        return self.stats

    def should_create_batch(self, window_s: float = 0.010) -> bool:
        return bool(self.pending) and (len(self.pending) >= self.max_batch_size or
                                       time.monotonic() - self.last_batch_time >= window_s)

    def pending_count(self) -> int:
        return len(self.pending)

    def active_count(self) -> int:
        return len(self.active)

    def complete_request(self, request_id: int) -> None:
        r = self.active.pop(request_id, None)
        if r is None:
            raise InvalidInput(f"Request {request_id} not active")
        r.state, r.completed_at = RequestState.Completed, time.monotonic()
        self.stats.completed_requests += 1


def engine_policy(policy: SchedulingPolicy, prefix_lookup: Callable[[Sequence[int]], int]):
    """Ordering function for ``LLMEngine(policy=...)``: takes the waiting sequences, returns them in
    admission order."""
    def order(seqs):
        if policy == SchedulingPolicy.FCFS:
            return sorted(seqs, key=lambda s: (-s.priority, s.arrival))
        cached = {id(s): prefix_lookup(s.prompt_ids) for s in seqs}
        if policy == SchedulingPolicy.LongestPrefixMatch:
            return sorted(seqs, key=lambda s: (-cached[id(s)], s.arrival))
        if policy == SchedulingPolicy.GpuMemoryOptimized:
            return sorted(seqs, key=lambda s: (len(s.prompt_ids) + s.params.max_tokens - cached[id(s)], s.arrival))
        return sorted(seqs, key=lambda s: (-(cached[id(s)] / max(1, len(s.prompt_ids))) * (1 + 0.5 * s.priority), s.arrival))
    return order


# ------------------------------------------------------------------------------------------------
# cache-aware batch analysis
# ------------------------------------------------------------------------------------------------
@dataclass
class PrefixSharingGroup:
    request_ids: List[int]
    shared_prefix_length: int
    estimated_savings_tokens: int


@dataclass
class BatchAnalysis:
    prefix_groups: List[PrefixSharingGroup]
    predicted_hit_rates: Dict[int, float]
    total_memory_bytes: int
    shared_memory_savings_bytes: int
    predicted_prefill_time: float
    total_prompt_tokens: int


@dataclass
class OptimizationResult:
    reordered: bool
    groups: int
    estimated_speedup: float


class CacheAwareAnalyzer:
    MIN_SHARED_PREFIX = 32

    def __init__(self, prefix_lookup: Optional[Callable[[Sequence[int]], int]] = None, kv: Optional[KvShape] = None,
                 us_per_prefill_token: float = 50.0):
        self.prefix_lookup = prefix_lookup
        self.kv = kv or KvShape()
        self.us_per_token = us_per_prefill_token

    @staticmethod
    def _common_prefix(a: Sequence[int], b: Sequence[int]) -> int:
        n = min(len(a), len(b))
        i = 0
        while i < n and a[i] == b[i]:
            i += 1
        return i

    def _groups(self, requests: Sequence[Request]) -> List[PrefixSharingGroup]:
        """Sort by token sequence so neighbours share the longest prefixes (O(n log n) instead of pairwise)."""
        order = sorted(requests, key=lambda r: r.prompt_tokens)
        groups: List[PrefixSharingGroup] = []
        cur: List[Request] = []
        cur_len = 0
        for r in order:
            if cur:
                c = self._common_prefix(cur[0].prompt_tokens, r.prompt_tokens)
                c = min(c, cur_len) if len(cur) > 1 else c
                if c >= self.MIN_SHARED_PREFIX:
                    cur.append(r)
                    cur_len = c
                    continue
                if len(cur) > 1:
                    groups.append(PrefixSharingGroup([x.id for x in cur], cur_len, cur_len * (len(cur) - 1)))
            cur, cur_len = [r], len(r.prompt_tokens)
        if len(cur) > 1:
            groups.append(PrefixSharingGroup([x.id for x in cur], cur_len, cur_len * (len(cur) - 1)))
        return groups

    def analyze_request_batch(self, requests: Sequence[Request]) -> BatchAnalysis:
        groups = self._groups(requests)
        hit: Dict[int, float] = {}
        for r in requests:
            n = len(r.prompt_tokens)
            if self.prefix_lookup is not None:
                hit[r.id] = min(1.0, self.prefix_lookup(r.prompt_tokens) / max(1, n))
            else:
                hit[r.id] = 0.7 if n > 1024 else 0.5 if n > 256 else 0.3
        in_group = {rid: g for g in groups for rid in g.request_ids}
        for rid, g in in_group.items():
            n = len(next(r for r in requests if r.id == rid).prompt_tokens)
            hit[rid] = max(hit[rid], g.shared_prefix_length / max(1, n) * (len(g.request_ids) - 1) / len(g.request_ids))
        bpt = self.kv.bytes_per_token()
        total_tokens = sum(len(r.prompt_tokens) for r in requests)
        saved = sum(g.estimated_savings_tokens for g in groups)
        return BatchAnalysis(groups, hit, sum(r.total_length() for r in requests) * bpt, saved * bpt,
                             (total_tokens - saved) * self.us_per_token * 1e-6, total_tokens)

    def optimize_batch_composition(self, requests: List[Request]) -> OptimizationResult:
        """Reorders in place so that members of a prefix group are adjacent, group leader first."""
        groups = self._groups(requests)
        if not groups:
            return OptimizationResult(False, 0, 1.0)
        pos = {r.id: i for i, r in enumerate(requests)}
        key: Dict[int, Tuple[int, int]] = {}
        for g in groups:
            first = min(pos[i] for i in g.request_ids)
            for i in g.request_ids:
                key[i] = (first, pos[i])
        before = [r.id for r in requests]
        requests.sort(key=lambda r: key.get(r.id, (pos[r.id], pos[r.id])))
        total = sum(len(r.prompt_tokens) for r in requests)
        saved = sum(g.estimated_savings_tokens for g in groups)
        return OptimizationResult(before != [r.id for r in requests], len(groups), total / max(1, total - saved))


# ------------------------------------------------------------------------------------------------
# GPU memory tracker
# ------------------------------------------------------------------------------------------------
class AllocationRecommendation(enum.Enum):
    Proceed = "proceed"
    ProceedWithCaution = "proceed_with_caution"
    Reject = "reject"


class WatermarkStatus(enum.Enum):
    Normal = "normal"
    High = "high"
    Critical = "critical"


@dataclass
class MemoryFeasibility:
    feasible: bool
    required: int
    available: int
    recommendation: AllocationRecommendation
    pressure_after: float


@dataclass
class OptimalBatchSize:
    recommended: int
    max_feasible: int
    memory_limited: bool


@dataclass
class AllocationEvent:
    size: int
    allocation_id: int
    timestamp: float = field(default_factory=time.monotonic)
    kind: str = "alloc"


@dataclass
class GpuMemoryStats:
    total_memory: int
    available_memory: int
    used_memory: int
    peak_usage: int
    memory_pressure: float
    fragmentation_ratio: float
    oom_risk_score: float
    watermark: WatermarkStatus
    allocations: int
    deallocations: int


class GpuMemoryTracker:
    def __init__(self, total_memory: int, kv: Optional[KvShape] = None, history: int = 1000,
                 free_bytes_fn: Optional[Callable[[], int]] = None):
        self.total = int(total_memory)
        self.available = int(total_memory)
        self.kv = kv or KvShape()
        self.events: Deque[AllocationEvent] = deque(maxlen=history)
        self.live: Dict[int, int] = {}
        self.peak = 0
        self.n_alloc = self.n_free = 0
        self.free_bytes_fn = free_bytes_fn         # e.g. block pool free blocks * bytes per block

    def _avail(self) -> int:
        return int(self.free_bytes_fn()) if self.free_bytes_fn is not None else self.available

    def memory_pressure(self) -> float:
        used = 1.0 - self._avail() / self.total if self.total else 1.0
        if used < 0.7:
            return 0.2 * used / 0.7
        if used < 0.95:
            return 0.2 + 0.8 * (used - 0.7) / 0.25
        return 1.0

    def batch_memory_requirement(self, requests: Sequence[Request]) -> int:
        return sum(r.total_length() for r in requests) * self.kv.bytes_per_token()

    def can_accommodate_batch(self, requests: Sequence[Request]) -> MemoryFeasibility:
        need, avail = self.batch_memory_requirement(requests), self._avail()
        after = 1.0 - (avail - need) / self.total if self.total else 1.0
        if need > avail:
            rec = AllocationRecommendation.Reject
        elif after > 0.9:
            rec = AllocationRecommendation.ProceedWithCaution
        else:
            rec = AllocationRecommendation.Proceed
        return MemoryFeasibility(need <= avail, need, avail, rec, max(0.0, min(1.0, after)))

    def suggest_batch_size(self, requests: Sequence[Request]) -> OptimalBatchSize:
        p = self.memory_pressure()
        frac = 0.9 if p < 0.3 else 0.8 if p < 0.7 else 0.6
        budget = int(self._avail() * frac)
        sizes = [r.total_length() * self.kv.bytes_per_token() for r in requests]
        acc, n = 0, 0
        for s in sizes:                         # prefix of the queue that fits (binary search over a monotone sum)
            if acc + s > budget:
                break
            acc += s
            n += 1
        mx, acc2 = 0, 0
        for s in sizes:
            if acc2 + s > self._avail():
                break
            acc2 += s
            mx += 1
        return OptimalBatchSize(n, mx, n < len(requests))

    def record_allocation(self, event: AllocationEvent) -> None:
        self.events.append(event)
        self.live[event.allocation_id] = event.size
        self.available -= event.size
        self.peak = max(self.peak, self.total - self.available)
        self.n_alloc += 1

    def record_deallocation(self, size: int, allocation_id: int) -> None:
        self.events.append(AllocationEvent(size, allocation_id, kind="free"))
        self.available = min(self.total, self.available + self.live.pop(allocation_id, size))
        self.n_free += 1

    def fragmentation_ratio(self) -> float:
        """1 - (largest live allocation / mean live allocation normalised): spread of live block sizes."""
        if len(self.live) < 2:
            return 0.0
        v = list(self.live.values())
        mean = sum(v) / len(v)
        var = sum((x - mean) ** 2 for x in v) / len(v)
        return min(1.0, math.sqrt(var) / mean) if mean > 0 else 0.0

    def oom_risk_score(self) -> float:
        """Pressure plus the recent allocation trend (bytes/s over the last events) against what is free."""
        ev = [e for e in self.events if e.kind == "alloc"][-50:]
        trend = 0.0
        if len(ev) >= 2 and ev[-1].timestamp > ev[0].timestamp:
            rate = sum(e.size for e in ev) / (ev[-1].timestamp - ev[0].timestamp)
            trend = min(1.0, rate * 1.0 / max(1, self._avail()))       # share of free memory consumed per second
        return max(0.0, min(1.0, 0.7 * self.memory_pressure() + 0.3 * trend))

    def watermark(self) -> WatermarkStatus:
        used = 1.0 - self._avail() / self.total if self.total else 1.0
        return WatermarkStatus.Critical if used >= 0.95 else WatermarkStatus.High if used >= 0.85 else WatermarkStatus.Normal

    def get_memory_stats(self) -> GpuMemoryStats:
        a = self._avail()
        return GpuMemoryStats(self.total, a, self.total - a, self.peak, self.memory_pressure(), self.fragmentation_ratio(),
                              self.oom_risk_score(), self.watermark(), self.n_alloc, self.n_free)


# ------------------------------------------------------------------------------------------------
# adaptive policy engine
# ------------------------------------------------------------------------------------------------
class WorkloadType(enum.Enum):
    CacheHeavy = "cache_heavy"
    MemoryConstrained = "memory_constrained"
    HighThroughput = "high_throughput"
    Mixed = "mixed"
    Unknown = "unknown"


class RiskLevel(enum.IntEnum):
    Low = 0
    Medium = 1
    High = 2


class PolicyAction(enum.Enum):
    Keep = "keep"
    Switch = "switch"


@dataclass
class SchedulerMetrics:
    cache_hit_rate: float = 0.0
    memory_pressure: float = 0.0
    throughput_tokens_per_s: float = 0.0
    average_latency_ms: float = 0.0
    queue_length: int = 0
    policy: SchedulingPolicy = SchedulingPolicy.CacheAware
    timestamp: float = field(default_factory=time.monotonic)


@dataclass
class PolicyDecision:
    action: PolicyAction
    new_policy: SchedulingPolicy
    confidence: float
    expected_improvement: float
    workload: WorkloadType


@dataclass
class PolicySummary:
    policy: SchedulingPolicy
    samples: int
    average_throughput: float
    average_latency_ms: float
    average_cache_hit_rate: float
    score: float


class PolicyPerformanceMetrics:
    def __init__(self):
        self.samples = 0
        self.tput = self.lat = self.hit = 0.0

    def update_with_metrics(self, m: SchedulerMetrics) -> None:
        self.samples += 1
        k = 1.0 / self.samples
        self.tput += (m.throughput_tokens_per_s - self.tput) * k
        self.lat += (m.average_latency_ms - self.lat) * k
        self.hit += (m.cache_hit_rate - self.hit) * k

    def overall_score(self) -> float:
        t = self.tput / (self.tput + 1000.0) if self.tput > 0 else 0.0
        l = 1.0 / (1.0 + self.lat / 100.0)
        return 0.5 * t + 0.3 * l + 0.2 * self.hit


class AdaptivePolicyEngine:
    WINDOW = 100
    MIN_GAIN = 0.1
    MAX_TRANSITION_COST_S = 0.050

    def __init__(self, initial: SchedulingPolicy = SchedulingPolicy.CacheAware):
        self.current = initial
        self.window: Deque[SchedulerMetrics] = deque(maxlen=self.WINDOW)
        self.perf: Dict[SchedulingPolicy, PolicyPerformanceMetrics] = {p: PolicyPerformanceMetrics() for p in SchedulingPolicy}
        self.confidence = 0.5
        self.history: List[Tuple[float, SchedulingPolicy, SchedulingPolicy]] = []

    def classify(self) -> WorkloadType:
        if len(self.window) < 3:
            return WorkloadType.Unknown
        recent = list(self.window)[-20:]
        hit = sum(m.cache_hit_rate for m in recent) / len(recent)
        pres = sum(m.memory_pressure for m in recent) / len(recent)
        q = sum(m.queue_length for m in recent) / len(recent)
        if pres > 0.8:
            return WorkloadType.MemoryConstrained
        if hit > 0.6:
            return WorkloadType.CacheHeavy
        if q > 32 and hit < 0.2:
            return WorkloadType.HighThroughput
        return WorkloadType.Mixed

    @staticmethod
    def recommended(w: WorkloadType) -> SchedulingPolicy:
        return {WorkloadType.CacheHeavy: SchedulingPolicy.LongestPrefixMatch,
                WorkloadType.MemoryConstrained: SchedulingPolicy.GpuMemoryOptimized,
                WorkloadType.HighThroughput: SchedulingPolicy.FCFS,
                WorkloadType.Mixed: SchedulingPolicy.CacheAware}.get(w, SchedulingPolicy.CacheAware)

    def transition_cost(self, a: SchedulingPolicy, b: SchedulingPolicy) -> float:
        return 0.0 if a == b else 0.005       # re-sorting the waiting queue

    def analyze_and_adapt(self, m: SchedulerMetrics) -> PolicyDecision:
        self.window.append(m)
        self.perf[m.policy].update_with_metrics(m)
        w = self.classify()
        target = self.recommended(w)
        cur_s, tgt_s = self.perf[self.current].overall_score(), self.perf[target].overall_score()
        untried = self.perf[target].samples == 0
        gain = (0.15 if untried else tgt_s - cur_s)
        risk = RiskLevel.Low if (w != WorkloadType.Unknown and len(self.window) >= 5) else RiskLevel.Medium
        self.confidence = min(1.0, 0.3 + 0.07 * len(self.window))
        if (target != self.current and gain > self.MIN_GAIN and risk <= RiskLevel.Low
                and self.transition_cost(self.current, target) < self.MAX_TRANSITION_COST_S):
            self.history.append((time.monotonic(), self.current, target))
            self.current = target
            return PolicyDecision(PolicyAction.Switch, target, self.confidence, gain, w)
        return PolicyDecision(PolicyAction.Keep, self.current, self.confidence, max(0.0, gain), w)

    def predict_optimal_policy(self, incoming: Sequence[Request]) -> SchedulingPolicy:
        if not incoming:
            return self.current
        groups = CacheAwareAnalyzer()._groups(incoming)
        shared = sum(len(g.request_ids) for g in groups) / len(incoming)
        if shared > 0.6:
            return SchedulingPolicy.LongestPrefixMatch
        if shared < 0.2:
            return SchedulingPolicy.FCFS
        return SchedulingPolicy.CacheAware

    def current_policy_info(self) -> Tuple[SchedulingPolicy, float]:
        return self.current, self.confidence

    def get_policy_performance_summary(self) -> List[PolicySummary]:
        return [PolicySummary(p, x.samples, x.tput, x.lat, x.hit, x.overall_score()) for p, x in self.perf.items()]


# ------------------------------------------------------------------------------------------------
# admission control
# ------------------------------------------------------------------------------------------------
@dataclass
class ResourceLimits:
    max_concurrent_requests: int = 32
    max_total_tokens: int = 65536
    max_memory_bytes: int = 8 << 30
    max_utilization: float = 0.9
    max_queue_wait_s: float = 30.0


@dataclass
class ResourceUsage:
    active_requests: int = 0
    total_tokens: int = 0
    memory_bytes: int = 0

    @staticmethod
    def new() -> "ResourceUsage":
        return ResourceUsage()


@dataclass
class AdmissionDecision:
    kind: str                      # "admitted" | "queued" | "rejected"
    estimated_wait_s: float = 0.0
    reason: Optional[str] = None

    @property
    def admitted(self) -> bool:
        return self.kind == "admitted"


@dataclass
class AdmissionStats:
    admitted: int = 0
    queued: int = 0
    rejected: int = 0
    completed: int = 0


class AdmissionController:
    def __init__(self, limits: Optional[ResourceLimits] = None, kv: Optional[KvShape] = None):
        self.limits = limits or ResourceLimits()
        self.kv = kv or KvShape()
        self.usage = ResourceUsage()
        self.queue: List[Tuple[int, float, int, int, int]] = []      # (-priority, time, id, tokens, bytes)
        self.admitted: Dict[int, Tuple[int, int]] = {}
        self.stats = AdmissionStats()
        self._avg_service_s = 1.0

    def _fits(self, tokens: int, nbytes: int) -> bool:
        l, u = self.limits, self.usage
        return (u.active_requests < l.max_concurrent_requests and u.total_tokens + tokens <= l.max_total_tokens
                and u.memory_bytes + nbytes <= l.max_memory_bytes * l.max_utilization)

    def admit_request(self, request_id: int, prompt_len: int, max_new_tokens: int,
                      priority: RequestPriority = RequestPriority.Normal) -> AdmissionDecision:
        tokens = prompt_len + max_new_tokens
        nbytes = tokens * self.kv.bytes_per_token()
        l = self.limits
        if tokens > l.max_total_tokens or nbytes > l.max_memory_bytes * l.max_utilization:
            self.stats.rejected += 1
            return AdmissionDecision("rejected", reason=f"request needs {tokens} tokens / {nbytes} bytes, beyond the limits")
        if not self.queue and self._fits(tokens, nbytes):
            self._take(request_id, tokens, nbytes)
            return AdmissionDecision("admitted")
        eta = (len(self.queue) + 1) * self._avg_service_s / max(1, l.max_concurrent_requests)
        if eta > l.max_queue_wait_s:
            self.stats.rejected += 1
            return AdmissionDecision("rejected", reason=f"estimated wait {eta:.1f}s exceeds {l.max_queue_wait_s}s")
        self.queue.append((-int(priority), time.monotonic(), request_id, tokens, nbytes))
        self.queue.sort()
        self.stats.queued += 1
        return AdmissionDecision("queued", estimated_wait_s=eta)

    def _take(self, rid: int, tokens: int, nbytes: int) -> None:
        u = self.usage
        u.active_requests += 1
        u.total_tokens += tokens
        u.memory_bytes += nbytes
        self.admitted[rid] = (tokens, nbytes)
        self.stats.admitted += 1

    def complete_request(self, request_id: int, service_time_s: Optional[float] = None) -> List[int]:
        """Releases the request's resources and admits queued requests that now fit; returns their ids."""
        t = self.admitted.pop(request_id, None)
        if t is None:
            raise InvalidInput(f"request {request_id} was not admitted")
        u = self.usage
        u.active_requests -= 1
        u.total_tokens -= t[0]
        u.memory_bytes -= t[1]
        self.stats.completed += 1
        if service_time_s is not None:
            self._avg_service_s = 0.9 * self._avg_service_s + 0.1 * service_time_s
        released = []
        while self.queue and self._fits(self.queue[0][3], self.queue[0][4]):
            _, _, rid, tokens, nbytes = self.queue.pop(0)
            self._take(rid, tokens, nbytes)
            released.append(rid)
        return released

    def get_stats(self) -> AdmissionStats:
        return self.stats
