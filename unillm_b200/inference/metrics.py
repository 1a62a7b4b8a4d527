"""Serving metrics: ``PerformanceCollector`` (request timeline, latency percentiles, throughput window,
error log, Prometheus text) and the process-wide ``METRICS`` singleton.

Parity: ``crates/inference/src/metrics.rs`` (``InferenceMetrics`` sections ``:10-193``, ``PerformanceCollector``
with a 10k-event timeline and 1k latency samples -> avg/p50/p95/p99, RPS / throughput over the last
60 s, errors by type and severity, ``export_prometheus`` ``:196-729``) and
``crates/runtime/src/simple_observability.rs`` (``SimpleMetrics``: atomics for requests / in-flight / errors /
tokens / cache hits+misses, ``RequestTimer``, Prometheus exposition, ``HealthMonitor``, enable switch
``UNILLM_OBSERVABILITY_ENABLED`` ``:15-302``).  Additions: TTFT and TPOT percentile series (the benchmark
metrics), per-step engine gauges, KV-block gauges, and the resource / cache sections are filled from the
engine instead of being left at zero.
"""
from __future__ import annotations

import os
import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, List, Optional, Tuple


def _pct(sorted_vals: List[float], q: float) -> float:
    if not sorted_vals:
        return 0.0
    i = min(len(sorted_vals) - 1, max(0, int(round(q * (len(sorted_vals) - 1)))))
    return sorted_vals[i]


@dataclass
class LatencySummary:
    count: int = 0
    avg: float = 0.0
    p50: float = 0.0
    p95: float = 0.0
    p99: float = 0.0
    max: float = 0.0

    @staticmethod
    def of(vals) -> "LatencySummary":
        v = sorted(vals)
        if not v:
            return LatencySummary()
        return LatencySummary(len(v), sum(v) / len(v), _pct(v, 0.5), _pct(v, 0.95), _pct(v, 0.99), v[-1])


@dataclass
class RequestStats:
    total: int = 0
    completed: int = 0
    failed: int = 0
    in_flight: int = 0
    queued: int = 0


@dataclass
class PerformanceMetrics:
    latency_ms: LatencySummary = field(default_factory=LatencySummary)
    ttft_ms: LatencySummary = field(default_factory=LatencySummary)
    tpot_ms: LatencySummary = field(default_factory=LatencySummary)
    requests_per_second: float = 0.0
    tokens_per_second: float = 0.0


@dataclass
class ResourceMetrics:
    kv_blocks_total: int = 0
    kv_blocks_used: int = 0
    gpu_memory_used: int = 0
    gpu_memory_total: int = 0
    device_time_ms_per_step: float = 0.0
    batch_size_last: int = 0


@dataclass
class CacheMetrics:
    prefix_hit_tokens: int = 0
    prefix_query_tokens: int = 0
    evictions: int = 0
    cached_blocks: int = 0

    @property
    def hit_rate(self) -> float:
        return self.prefix_hit_tokens / self.prefix_query_tokens if self.prefix_query_tokens else 0.0


@dataclass
class ErrorMetrics:
    total: int = 0
    by_type: Dict[str, int] = field(default_factory=dict)
    by_severity: Dict[str, int] = field(default_factory=dict)
    last: Optional[str] = None


@dataclass
class QualityMetrics:
    average_output_tokens: float = 0.0
    finish_reasons: Dict[str, int] = field(default_factory=dict)


@dataclass
class InferenceMetrics:
    timestamp: float = field(default_factory=time.time)
    requests: RequestStats = field(default_factory=RequestStats)
    performance: PerformanceMetrics = field(default_factory=PerformanceMetrics)
    resources: ResourceMetrics = field(default_factory=ResourceMetrics)
    cache: CacheMetrics = field(default_factory=CacheMetrics)
    errors: ErrorMetrics = field(default_factory=ErrorMetrics)
    quality: QualityMetrics = field(default_factory=QualityMetrics)


class PerformanceCollector:
    TIMELINE, SAMPLES, WINDOW_S = 10000, 1000, 60.0

    def __init__(self):
        self._lock = threading.Lock()
        self.timeline: Deque[Tuple[float, str, str]] = deque(maxlen=self.TIMELINE)      # (time, request id, event)
        self.lat: Deque[float] = deque(maxlen=self.SAMPLES)
        self.ttft: Deque[float] = deque(maxlen=self.SAMPLES)
        self.tpot: Deque[float] = deque(maxlen=self.SAMPLES)
        self.done: Deque[Tuple[float, int]] = deque()                                   # (time, tokens) inside the window
        self.m = InferenceMetrics()
        self._out_tokens_sum = 0

    def record_request_start(self, rid: str) -> None:
        with self._lock:
            self.timeline.append((time.time(), rid, "start"))
            self.m.requests.total += 1
            self.m.requests.in_flight += 1

    def record_request_complete(self, rid: str, latency_ms: float, tokens: int, ttft_ms: Optional[float] = None,
                                tpot_ms: Optional[float] = None, finish_reason: str = "completed") -> None:
        now = time.time()
        with self._lock:
            self.timeline.append((now, rid, "complete"))
            r = self.m.requests
            r.completed += 1
            r.in_flight = max(0, r.in_flight - 1)
            self.lat.append(latency_ms)
            if ttft_ms is not None:
                self.ttft.append(ttft_ms)
            if tpot_ms is not None:
                self.tpot.append(tpot_ms)
            self.done.append((now, tokens))
            self._out_tokens_sum += tokens
            q = self.m.quality
            q.average_output_tokens = self._out_tokens_sum / r.completed
            q.finish_reasons[finish_reason] = q.finish_reasons.get(finish_reason, 0) + 1

    def record_error(self, rid: str, kind: str, severity: str = "medium", msg: str = "") -> None:
        with self._lock:
            self.timeline.append((time.time(), rid, f"error:{kind}"))
            e = self.m.errors
            e.total += 1
            e.by_type[kind] = e.by_type.get(kind, 0) + 1
            e.by_severity[severity] = e.by_severity.get(severity, 0) + 1
            e.last = msg or kind
            r = self.m.requests
            r.failed += 1
            r.in_flight = max(0, r.in_flight - 1)

    def update_engine(self, *, queued: int = 0, kv_total: int = 0, kv_used: int = 0, batch: int = 0,
                      step_ms: float = 0.0, hit_tokens: int = 0, query_tokens: int = 0, evictions: int = 0,
                      cached_blocks: int = 0, gpu_used: int = 0, gpu_total: int = 0) -> None:
        with self._lock:
            self.m.requests.queued = queued
            res, c = self.m.resources, self.m.cache
            res.kv_blocks_total, res.kv_blocks_used, res.batch_size_last = kv_total, kv_used, batch
            res.device_time_ms_per_step, res.gpu_memory_used, res.gpu_memory_total = step_ms, gpu_used, gpu_total
            c.prefix_hit_tokens, c.prefix_query_tokens, c.evictions, c.cached_blocks = hit_tokens, query_tokens, evictions, cached_blocks

    def get_metrics(self) -> InferenceMetrics:
        now = time.time()
        with self._lock:
            while self.done and now - self.done[0][0] > self.WINDOW_S:
                self.done.popleft()
            span = max(1e-6, min(self.WINDOW_S, now - self.done[0][0])) if self.done else 1.0
            p = self.m.performance
            p.latency_ms, p.ttft_ms, p.tpot_ms = LatencySummary.of(self.lat), LatencySummary.of(self.ttft), LatencySummary.of(self.tpot)
            p.requests_per_second = len(self.done) / span if len(self.done) > 1 else float(len(self.done))
            p.tokens_per_second = sum(t for _, t in self.done) / span if self.done else 0.0
            self.m.timestamp = now
            return self.m

    def error_rate(self) -> float:
        r = self.m.requests
        return r.failed / r.total if r.total else 0.0

    def export_prometheus(self) -> str:
        m = self.get_metrics()
        out = []

        def g(name, val, help_, typ="gauge"):
            out.append(f"# HELP {name} {help_}\n# TYPE {name} {typ}\n{name} {val}")

        g("unillm_requests_total", m.requests.total, "Requests received", "counter")
        g("unillm_requests_completed_total", m.requests.completed, "Requests completed", "counter")
        g("unillm_requests_failed_total", m.requests.failed, "Requests failed", "counter")
        g("unillm_requests_in_flight", m.requests.in_flight, "Requests being processed")
        g("unillm_requests_queued", m.requests.queued, "Requests waiting")
        for q, v in (("0.5", m.performance.latency_ms.p50), ("0.95", m.performance.latency_ms.p95), ("0.99", m.performance.latency_ms.p99)):
            out.append(f'unillm_request_latency_ms{{quantile="{q}"}} {v}')
        for q, v in (("0.5", m.performance.ttft_ms.p50), ("0.99", m.performance.ttft_ms.p99)):
            out.append(f'unillm_time_to_first_token_ms{{quantile="{q}"}} {v}')
        for q, v in (("0.5", m.performance.tpot_ms.p50), ("0.99", m.performance.tpot_ms.p99)):
            out.append(f'unillm_time_per_output_token_ms{{quantile="{q}"}} {v}')
        g("unillm_requests_per_second", m.performance.requests_per_second, "Completed requests per second (60 s window)")
        g("unillm_tokens_per_second", m.performance.tokens_per_second, "Output tokens per second (60 s window)")
        g("unillm_kv_blocks_used", m.resources.kv_blocks_used, "KV cache blocks in use")
        g("unillm_kv_blocks_total", m.resources.kv_blocks_total, "KV cache blocks")
        g("unillm_prefix_cache_hit_rate", m.cache.hit_rate, "Share of prompt tokens served from the radix cache")
        g("unillm_errors_total", m.errors.total, "Errors", "counter")
        for k, v in m.errors.by_type.items():
            out.append(f'unillm_errors_by_type{{type="{k}"}} {v}')
        return "\n".join(out) + "\n"


# ------------------------------------------------------------------------------------------------
# process-wide simple metrics
# ------------------------------------------------------------------------------------------------
class RequestTimer:
    def __init__(self, metrics: "SimpleMetrics", endpoint: str):
        self.m, self.endpoint, self.t0 = metrics, endpoint, time.perf_counter()
        self.done = False

    def finish(self, error: bool = False) -> float:
        if self.done:
            return 0.0
        self.done = True
        dt = time.perf_counter() - self.t0
        self.m._request_end(dt, error)
        return dt

    def __enter__(self):
        return self

    def __exit__(self, et, ev, tb):
        self.finish(error=et is not None)
        return False


class SimpleMetrics:
    def __init__(self):
        self._lock = threading.Lock()
        self.enabled = os.environ.get("UNILLM_OBSERVABILITY_ENABLED", "1").lower() not in ("0", "false", "no")
        self.requests_total = self.requests_in_flight = self.errors_total = self.tokens_generated = 0
        self.cache_hits = self.cache_misses = 0
        self.duration_sum = 0.0
        self.started = time.time()

    def initialize(self, level: Optional[str] = None) -> None:
        """Configures logging (level from ``UNILLM_LOG_LEVEL``, default info) with request-scoped fields."""
        import logging

        lvl = (level or os.environ.get("UNILLM_LOG_LEVEL", "info")).upper()
        logging.basicConfig(level=getattr(logging, lvl, logging.INFO),
                            format='{"ts":"%(asctime)s","level":"%(levelname)s","logger":"%(name)s","msg":"%(message)s"}')

    def request_start(self, endpoint: str = "generate") -> RequestTimer:
        if self.enabled:
            with self._lock:
                self.requests_total += 1
                self.requests_in_flight += 1
        return RequestTimer(self, endpoint)

    def _request_end(self, dt: float, error: bool) -> None:
        if not self.enabled:
            return
        with self._lock:
            self.requests_in_flight = max(0, self.requests_in_flight - 1)
            self.duration_sum += dt
            if error:
                self.errors_total += 1

    def token_generated(self, n: int = 1) -> None:
        if self.enabled:
            with self._lock:
                self.tokens_generated += n

    def cache_hit(self, n: int = 1) -> None:
        if self.enabled:
            with self._lock:
                self.cache_hits += n

    def cache_miss(self, n: int = 1) -> None:
        if self.enabled:
            with self._lock:
                self.cache_misses += n

    def error(self, kind: str = "error") -> None:
        if self.enabled:
            with self._lock:
                self.errors_total += 1

    def cache_hit_rate(self) -> float:
        t = self.cache_hits + self.cache_misses
        return self.cache_hits / t if t else 0.0

    def get_stats(self) -> Dict[str, float]:
        with self._lock:
            return {"requests_total": self.requests_total, "requests_in_flight": self.requests_in_flight,
                    "errors_total": self.errors_total, "tokens_generated": self.tokens_generated,
                    "cache_hits": self.cache_hits, "cache_misses": self.cache_misses,
                    "cache_hit_rate": self.cache_hit_rate(), "uptime_s": time.time() - self.started,
                    "avg_request_s": self.duration_sum / self.requests_total if self.requests_total else 0.0}

    def get_prometheus_metrics(self) -> str:
        s = self.get_stats()
        lines = []
        for k, typ in (("requests_total", "counter"), ("requests_in_flight", "gauge"), ("errors_total", "counter"),
                       ("tokens_generated", "counter"), ("cache_hits", "counter"), ("cache_misses", "counter"),
                       ("cache_hit_rate", "gauge"), ("uptime_s", "gauge")):
            lines.append(f"# TYPE unillm_{k} {typ}\nunillm_{k} {s[k]}")
        return "\n".join(lines) + "\n"

    def get_health_status(self) -> Dict[str, object]:
        s = self.get_stats()
        err_rate = s["errors_total"] / s["requests_total"] if s["requests_total"] else 0.0
        status = "healthy" if err_rate < 0.05 else "degraded" if err_rate < 0.25 else "unhealthy"
        return {"status": status, "error_rate": err_rate, **HealthMonitor.sample()}


class HealthMonitor:
    """Host CPU / memory / GPU presence snapshot (``simple_observability.rs:259-302``)."""

    @staticmethod
    def sample() -> Dict[str, object]:
        out: Dict[str, object] = {"gpu_available": os.path.exists("/dev/nvidia0") or bool(os.environ.get("CUDA_VISIBLE_DEVICES"))}
        try:
            import psutil

            vm = psutil.virtual_memory()
            out.update(cpu_percent=psutil.cpu_percent(interval=None), memory_used=vm.used, memory_total=vm.total)
        except Exception:
            pass
        return out


METRICS = SimpleMetrics()


def start_request_span(request_id: str, endpoint: str) -> Dict[str, str]:
    return {"request_id": request_id, "endpoint": endpoint, "span": "request"}


def start_inference_span(model: str, batch_size: int) -> Dict[str, object]:
    return {"model": model, "batch_size": batch_size, "span": "inference"}
