"""Spans, NVTX ranges and structured JSON logs.

The reference initialises a JSON `tracing` subscriber and defines two span helpers, `start_request_span(request_id,
endpoint)` and `start_inference_span(model, batch_size)` (``crates/runtime/src/simple_observability.rs:57-86,333-342``),
which nothing calls.  Here a span is a context manager that (a) pushes an NVTX range when CUDA is present and
``UNILLM_NVTX=1`` (visible in Nsight Systems timelines of the engine phases), (b) records wall time into the tracer's
ring buffer and (c) emits one JSON log line at DEBUG level with the span's fields.  The engine wraps schedule / launch /
fetch / process in spans; ``Tracer.summary()`` gives per-name count / mean / p50 / p99.
"""
from __future__ import annotations

import json
import logging
import os
import threading
import time
from collections import defaultdict, deque
from contextlib import contextmanager
from typing import Deque, Dict, Iterator, Optional

log = logging.getLogger("unillm_b200.trace")


def _nvtx():
    if os.environ.get("UNILLM_NVTX", "0") != "1":
        return None
    try:
        import torch

        if torch.cuda.is_available():
            return torch.cuda.nvtx
    except Exception:  # pragma: no cover
        pass
    return None


class Tracer:
    def __init__(self, capacity: int = 4096):
        self.enabled = os.environ.get("UNILLM_TRACE", "1") != "0"
        self._spans: Dict[str, Deque[float]] = defaultdict(lambda: deque(maxlen=capacity))
        self._lock = threading.Lock()
        self._nvtx = _nvtx()
        self._local = threading.local()

    @contextmanager
    def span(self, name: str, **fields) -> Iterator[dict]:
        if not self.enabled:
            yield fields
            return
        stack = getattr(self._local, "stack", None)
        if stack is None:
            stack = self._local.stack = []
        parent = stack[-1] if stack else None
        stack.append(name)
        if self._nvtx is not None:
            self._nvtx.range_push(name)
        t0 = time.perf_counter()
        try:
            yield fields
        finally:
            dt = time.perf_counter() - t0
            if self._nvtx is not None:
                self._nvtx.range_pop()
            stack.pop()
            with self._lock:
                self._spans[name].append(dt)
            if log.isEnabledFor(logging.DEBUG):
                log.debug(json.dumps({"span": name, "parent": parent, "ms": round(dt * 1e3, 3), **fields}, default=str))

    def summary(self) -> Dict[str, dict]:
        out = {}
        with self._lock:
            for name, xs in self._spans.items():
                s = sorted(xs)
                n = len(s)
                if n:
                    out[name] = {"count": n, "mean_ms": 1e3 * sum(s) / n, "p50_ms": 1e3 * s[n // 2],
                                 "p99_ms": 1e3 * s[min(n - 1, int(n * 0.99))]}
        return out

    def reset(self) -> None:
        with self._lock:
            self._spans.clear()


_TRACER: Optional[Tracer] = None


def get_tracer() -> Tracer:
    global _TRACER
    if _TRACER is None:
        _TRACER = Tracer()
    return _TRACER


def span(name: str, **fields):
    return get_tracer().span(name, **fields)


def start_request_span(request_id: str, endpoint: str = "generate"):
    return span("request", request_id=request_id, endpoint=endpoint)


def start_inference_span(model: str, batch_size: int):
    return span("inference", model=model, batch_size=batch_size)


def export_torch_profile(fn, path: str, steps: int = 3) -> str:
    """Runs ``fn`` ``steps`` times under ``torch.profiler`` and writes a Chrome trace (CPU + CUDA activities)."""
    import torch
    from torch.profiler import ProfilerActivity, profile

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    with profile(activities=acts) as prof:
        for _ in range(steps):
            fn()
        if torch.cuda.is_available():
            torch.cuda.synchronize()
    prof.export_chrome_trace(path)
    return path
