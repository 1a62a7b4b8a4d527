"""Scheduler building blocks with the reference's public surface: request / batch types, the
batch-forming ``ContinuousBatchingScheduler``, ``ChunkedPrefillManager`` and ``StreamOverlapManager``.

Parity with ``crates/scheduler/src``: ``Request`` / ``RequestBatch`` / ``RequestPriority`` / ``RequestState``
(``lib.rs:36-193``), ``ContinuousBatchingScheduler`` (``lib.rs:196-416``) and ``SchedulerStats`` (``:420-449``);
``ChunkedPrefillConfig`` / ``PrefillChunk`` / ``ChunkedPrefillManager`` / ``PrefillStats``
(``chunked_prefill.rs:8-311``); ``StreamType`` / ``StreamPriority`` / ``StreamOperation`` / ``OperationData`` /
``StreamOverlapManager`` and the ``create_*_operation`` helpers (``stream_overlap.rs:9-377``).

Behavioural differences, on purpose:
 * ``create_batch`` pushes EVERY request that did not fit back to the queue (the reference drops all but
   the first misfit, ``lib.rs:292-296``).
 * Prefill chunks do not overlap: with a KV cache, re-running 64 tokens per chunk boundary
   (``chunk_overlap``, ``chunked_prefill.rs:8-28``) would only recompute cached keys.  ``chunk_overlap`` is
   accepted and ignored unless ``recompute_overlap=True``.
 * ``StreamOverlapManager`` can be bound to real CUDA streams (``bind_cuda_streams``); without a GPU it
   is the same pure bookkeeping as the reference.
The iteration-level loop that the serving engine actually runs is ``unillm_b200.engine.llm_engine``.
"""
from __future__ import annotations

import enum
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Deque, Dict, List, Optional, Sequence, Tuple

from ..types import InvalidInput


class RequestPriority(enum.IntEnum):
    Low = 0
    Normal = 1
    High = 2
    Critical = 3


class RequestState(enum.Enum):
    Waiting = "waiting"
    Prefilling = "prefilling"
    Decoding = "decoding"
    Completed = "completed"
    Failed = "failed"


@dataclass
class Request:
    id: int
    prompt_tokens: List[int]
    max_output_length: int
    priority: RequestPriority = RequestPriority.Normal
    current_output_length: int = 0
    state: RequestState = RequestState.Waiting
    created_at: float = field(default_factory=time.monotonic)
    started_at: Optional[float] = None
    completed_at: Optional[float] = None
    kv_seq_id: Optional[int] = None
    prefill_tokens_processed: int = 0
    is_prefill: bool = True
    failure_reason: Optional[str] = None

    @staticmethod
    def new(id: int, prompt_tokens: Sequence[int], max_output_length: int,
            priority: RequestPriority = RequestPriority.Normal) -> "Request":
        return Request(id, list(prompt_tokens), max_output_length, priority)

    def total_length(self) -> int:
        return len(self.prompt_tokens) + self.max_output_length

    def remaining_output_length(self) -> int:
        return max(0, self.max_output_length - self.current_output_length)

    def is_completed(self) -> bool:
        return self.state in (RequestState.Completed, RequestState.Failed)

    def age(self) -> float:
        return time.monotonic() - self.created_at

    def processing_time(self) -> Optional[float]:
        if self.started_at is None:
            return None
        return (self.completed_at or time.monotonic()) - self.started_at


@dataclass
class RequestBatch:
    batch_id: int
    requests: List[Request]
    created_at: float = field(default_factory=time.monotonic)
    is_prefill_batch: bool = True
    max_sequence_length: int = 0
    total_tokens: int = 0

    @staticmethod
    def new(batch_id: int, requests: List[Request]) -> "RequestBatch":
        b = RequestBatch(batch_id, requests)
        b.is_prefill_batch = any(r.is_prefill for r in requests)
        b.max_sequence_length = max((r.total_length() for r in requests), default=0)
        b.total_tokens = sum(r.total_length() for r in requests)
        return b

    def size(self) -> int:
        return len(self.requests)

    def is_empty(self) -> bool:
        return not self.requests

    def age(self) -> float:
        return time.monotonic() - self.created_at


@dataclass
class SchedulerStats:
    total_requests: int = 0
    completed_requests: int = 0
    failed_requests: int = 0
    total_batches: int = 0
    average_batch_size: float = 0.0
    average_wait_time_ms: float = 0.0
    requeued_requests: int = 0


class ContinuousBatchingScheduler:
    def __init__(self, max_batch_size: int, max_sequence_length: int, batching_window_ms: int = 10):
        if max_batch_size <= 0 or max_sequence_length <= 0:
            raise InvalidInput("max_batch_size and max_sequence_length must be positive")
        self.max_batch_size = max_batch_size
        self.max_sequence_length = max_sequence_length      # used as the token budget of one batch
        self.batching_window = batching_window_ms / 1000.0
        self.pending: Deque[Request] = deque()
        self.active: Dict[int, Request] = {}
        self.completed: Dict[int, Request] = {}
        self.current_batch: Optional[RequestBatch] = None
        self.last_batch_time = time.monotonic()
        self._next_request_id = 1
        self._next_batch_id = 1
        self.stats = SchedulerStats()

    def add_request(self, prompt_tokens: Sequence[int], max_output_length: int,
                    priority: RequestPriority = RequestPriority.Normal) -> int:
        if len(prompt_tokens) + max_output_length > self.max_sequence_length:
            raise InvalidInput(f"request of {len(prompt_tokens) + max_output_length} tokens exceeds "
                               f"max_sequence_length {self.max_sequence_length}")
        rid = self._next_request_id
        self._next_request_id += 1
        self.pending.append(Request.new(rid, prompt_tokens, max_output_length, priority))
        self.stats.total_requests += 1
        return rid

    def create_batch(self) -> Optional[RequestBatch]:
        if not self.pending:
            return None
        drained = sorted(self.pending, key=lambda r: -int(r.priority))       # stable: FIFO inside a priority
        self.pending.clear()
        chosen: List[Request] = []
        tokens = 0
        rest: List[Request] = []
        for r in drained:
            if not rest and len(chosen) < self.max_batch_size and tokens + r.total_length() <= self.max_sequence_length:
                chosen.append(r)
                tokens += r.total_length()
            else:
                rest.append(r)
        for r in rest:
            self.pending.append(r)
        self.stats.requeued_requests += len(rest)
        if not chosen:
            return None
        now = time.monotonic()
        for r in chosen:
            r.state, r.started_at = RequestState.Prefilling, now
            self.active[r.id] = r
        batch = RequestBatch.new(self._next_batch_id, chosen)
        self._next_batch_id += 1
        self.current_batch = batch
        self.last_batch_time = now
        st = self.stats
        st.total_batches += 1
        st.average_batch_size += (len(chosen) - st.average_batch_size) / st.total_batches
        wait = sum(now - r.created_at for r in chosen) / len(chosen) * 1e3
        st.average_wait_time_ms += (wait - st.average_wait_time_ms) / st.total_batches
        return batch

    def should_create_batch(self) -> bool:
        return self.current_batch is None or (time.monotonic() - self.last_batch_time) >= self.batching_window

    def _finish(self, request_id: int, state: RequestState, reason: Optional[str] = None) -> None:
        r = self.active.pop(request_id, None)
        if r is None:
            raise InvalidInput(f"Request {request_id} not found in active requests")
        r.state, r.completed_at, r.failure_reason = state, time.monotonic(), reason
        self.completed[request_id] = r

    def complete_request(self, request_id: int) -> None:
        self._finish(request_id, RequestState.Completed)
        self.stats.completed_requests += 1

    def fail_request(self, request_id: int, reason: str) -> None:
        self._finish(request_id, RequestState.Failed, reason)
        self.stats.failed_requests += 1

    def get_current_batch(self) -> Optional[RequestBatch]:
        return self.current_batch

    def clear_current_batch(self) -> None:
        self.current_batch = None

    def pending_count(self) -> int:
        return len(self.pending)

    def active_count(self) -> int:
        return len(self.active)

    def get_stats(self) -> SchedulerStats:
        return self.stats

    def get_active_requests(self) -> List[Request]:
        return list(self.active.values())

    def get_completed_requests(self) -> List[Request]:
        return list(self.completed.values())

    def update_request_state(self, request_id: int, new_state: RequestState) -> None:
        r = self.active.get(request_id)
        if r is None:
            raise InvalidInput(f"Request {request_id} not found")
        r.state = new_state
        if new_state == RequestState.Decoding:
            r.is_prefill = False

    def get_request(self, request_id: int) -> Optional[Request]:
        return self.active.get(request_id) or self.completed.get(request_id) or \
            next((r for r in self.pending if r.id == request_id), None)


# ------------------------------------------------------------------------------------------------
# chunked prefill
# ------------------------------------------------------------------------------------------------
@dataclass
class ChunkedPrefillConfig:
    max_chunk_size: int = 2048
    parallel_chunks: int = 4
    chunk_overlap: int = 64
    chunking_threshold: int = 4096
    recompute_overlap: bool = False


@dataclass
class PrefillChunk:
    chunk_id: int
    request_id: int
    start_pos: int
    end_pos: int
    tokens: List[int]
    priority: int                     # lower = earlier
    is_processed: bool = False
    created_at: float = field(default_factory=time.monotonic)
    processing_time: Optional[float] = None

    def size(self) -> int:
        return self.end_pos - self.start_pos

    def mark_processed(self) -> None:
        self.is_processed = True
        self.processing_time = time.monotonic() - self.created_at


@dataclass
class PrefillStats:
    total_chunks_created: int = 0
    total_chunks_processed: int = 0
    total_requests_chunked: int = 0
    average_chunk_size: float = 0.0


class ChunkedPrefillManager:
    def __init__(self, config: Optional[ChunkedPrefillConfig] = None):
        self.config = config or ChunkedPrefillConfig()
        self.active: Dict[int, PrefillChunk] = {}
        self.completed: Dict[int, List[PrefillChunk]] = {}
        self.expected: Dict[int, int] = {}
        self._next = 1
        self.stats = PrefillStats()

    def create_chunks(self, request_id: int, prompt_tokens: Sequence[int]) -> List[int]:
        c = self.config
        n = len(prompt_tokens)
        if n == 0:
            raise InvalidInput("empty prompt")
        spans: List[Tuple[int, int]] = []
        if n <= c.chunking_threshold:
            spans.append((0, n))
        else:
            step_back = c.chunk_overlap if c.recompute_overlap else 0
            start = 0
            while start < n:
                end = min(n, start + c.max_chunk_size)
                spans.append((start, end))
                if end == n:
                    break
                start = end - step_back
            self.stats.total_requests_chunked += 1
        ids = []
        for i, (s, e) in enumerate(spans):
            cid = self._next
            self._next += 1
            self.active[cid] = PrefillChunk(cid, request_id, s, e, list(prompt_tokens[s:e]), i)
            ids.append(cid)
        self.expected[request_id] = self.expected.get(request_id, 0) + len(ids)
        st = self.stats
        for s, e in spans:
            st.total_chunks_created += 1
            st.average_chunk_size += ((e - s) - st.average_chunk_size) / st.total_chunks_created
        return ids

    def get_next_chunk(self) -> Optional[Tuple[int, PrefillChunk]]:
        """Earliest unprocessed chunk; chunks of one request are served in order."""
        best = None
        for cid, ch in self.active.items():
            if ch.is_processed:
                continue
            if best is None or (ch.priority, ch.created_at, cid) < (best[1].priority, best[1].created_at, best[0]):
                best = (cid, ch)
        return best

    def complete_chunk(self, chunk_id: int) -> None:
        ch = self.active.pop(chunk_id, None)
        if ch is None:
            raise InvalidInput(f"Chunk {chunk_id} not found")
        ch.mark_processed()
        self.completed.setdefault(ch.request_id, []).append(ch)
        self.stats.total_chunks_processed += 1

    def is_request_complete(self, request_id: int) -> bool:
        return request_id in self.expected and len(self.completed.get(request_id, [])) >= self.expected[request_id]

    def get_completed_chunks(self, request_id: int) -> Optional[List[PrefillChunk]]:
        return self.completed.get(request_id)

    def get_active_chunks(self) -> List[PrefillChunk]:
        return list(self.active.values())

    def get_stats(self) -> PrefillStats:
        return self.stats

    def clear_completed_chunks(self, request_id: int) -> None:
        self.completed.pop(request_id, None)
        self.expected.pop(request_id, None)

    def active_chunk_count(self) -> int:
        return len(self.active)

    def completed_chunk_count(self) -> int:
        return sum(len(v) for v in self.completed.values())

    def estimate_processing_time(self, prompt_length: int, us_per_token: float = 50.0) -> float:
        """Seconds; chunks run back to back on one GPU, so chunking adds only per-chunk launch overhead."""
        c = self.config
        chunks = 1 if prompt_length <= c.chunking_threshold else -(-prompt_length // c.max_chunk_size)
        return prompt_length * us_per_token * 1e-6 + chunks * 1e-3


# ------------------------------------------------------------------------------------------------
# stream overlap
# ------------------------------------------------------------------------------------------------
class StreamType(enum.Enum):
    H2D = "h2d"
    D2H = "d2h"
    Compute = "compute"
    Prefill = "prefill"
    Decode = "decode"


class StreamPriority(enum.IntEnum):
    Low = 0
    Normal = 1
    High = 2
    Critical = 3


@dataclass
class OperationData:
    kind: str                                  # "h2d" | "d2h" | "compute" | "prefill" | "decode"
    payload: Dict[str, Any] = field(default_factory=dict)


@dataclass
class StreamOperation:
    op_id: int
    stream_type: StreamType
    priority: StreamPriority
    data: OperationData
    estimated_duration: float
    dependencies: List[int] = field(default_factory=list)
    created_at: float = field(default_factory=time.monotonic)
    started_at: Optional[float] = None
    stream_id: Optional[int] = None


@dataclass
class StreamOverlapStats:
    total_operations: int = 0
    completed_operations: int = 0
    overlapped_operations: int = 0
    total_scheduled: int = 0


class StreamOverlapManager:
    def __init__(self, streams_per_type: int = 2):
        self.free_streams: Dict[StreamType, Deque[int]] = {t: deque() for t in StreamType}
        self.pending: List[StreamOperation] = []
        self.active: Dict[int, StreamOperation] = {}
        self.completed: List[int] = []
        self._next_op = 1
        self._next_stream = 0
        self.cuda_streams: Dict[int, Any] = {}
        self.stats = StreamOverlapStats()
        for t in StreamType:
            for _ in range(streams_per_type):
                self.add_stream(t, self._next_stream)
                self._next_stream += 1

    @staticmethod
    def new() -> "StreamOverlapManager":
        return StreamOverlapManager()

    def add_stream(self, stream_type: StreamType, stream_id: int) -> None:
        self.free_streams[stream_type].append(stream_id)

    def bind_cuda_streams(self, device=None) -> None:
        """Attach a real non-blocking CUDA stream to every stream id (GPU only)."""
        import torch

        for q in self.free_streams.values():
            for sid in q:
                self.cuda_streams[sid] = torch.cuda.Stream(device=device)

    def submit_operation(self, stream_type: StreamType, priority: StreamPriority, data: OperationData,
                         estimated_duration: float, dependencies: Optional[List[int]] = None) -> int:
        oid = self._next_op
        self._next_op += 1
        self.pending.append(StreamOperation(oid, stream_type, priority, data, estimated_duration, list(dependencies or [])))
        self.stats.total_operations += 1
        return oid

    def schedule_operations(self) -> List[Tuple[int, int]]:
        """Starts every pending operation whose dependencies completed and whose stream type has a free
        stream, highest priority first.  Returns (op_id, stream_id) pairs."""
        done = set(self.completed)
        started: List[Tuple[int, int]] = []
        self.pending.sort(key=lambda o: (-int(o.priority), o.created_at, o.op_id))
        keep = []
        for op in self.pending:
            if all(d in done for d in op.dependencies) and self.free_streams[op.stream_type]:
                sid = self.free_streams[op.stream_type].popleft()
                op.stream_id, op.started_at = sid, time.monotonic()
                self.active[op.op_id] = op
                started.append((op.op_id, sid))
            else:
                keep.append(op)
        self.pending = keep
        self.stats.total_scheduled += len(started)
        if len(self.active) > 1:
            self.stats.overlapped_operations += len(started)
        return started

    def complete_operation(self, op_id: int) -> None:
        op = self.active.pop(op_id, None)
        if op is None:
            raise InvalidInput(f"Operation {op_id} not found in active operations")
        self.completed.append(op_id)
        if len(self.completed) > 4096:
            self.completed = self.completed[-2048:]
        self.return_stream(op.stream_type, op.stream_id)
        self.stats.completed_operations += 1

    def return_stream(self, stream_type: StreamType, stream_id: int) -> None:
        if stream_id not in self.free_streams[stream_type]:
            self.free_streams[stream_type].append(stream_id)

    def pending_count(self) -> int:
        return len(self.pending)

    def active_count(self) -> int:
        return len(self.active)

    def get_stats(self) -> StreamOverlapStats:
        return self.stats

    def get_active_operations(self) -> List[StreamOperation]:
        return list(self.active.values())

    def estimate_overlap_efficiency(self) -> float:
        """1 - (critical path / serial time) over the active operations, grouped by stream type."""
        if not self.active:
            return 0.0
        per_type: Dict[StreamType, float] = {}
        for op in self.active.values():
            per_type[op.stream_type] = per_type.get(op.stream_type, 0.0) + op.estimated_duration
        serial = sum(per_type.values())
        return 0.0 if serial <= 0 else 1.0 - max(per_type.values()) / serial


def create_h2d_operation(src: int, dst: int, size: int) -> OperationData:
    return OperationData("h2d", {"src_ptr": src, "dst_ptr": dst, "size": size})


def create_d2h_operation(src: int, dst: int, size: int) -> OperationData:
    return OperationData("d2h", {"src_ptr": src, "dst_ptr": dst, "size": size})


def create_compute_operation(kernel_id: int, grid, block, shared_mem: int = 0, args=None) -> OperationData:
    return OperationData("compute", {"kernel_id": kernel_id, "grid": tuple(grid), "block": tuple(block),
                                     "shared_mem": shared_mem, "args": list(args or [])})


def create_prefill_operation(request_id: int, chunk_id: int, tokens: Sequence[int]) -> OperationData:
    return OperationData("prefill", {"request_id": request_id, "chunk_id": chunk_id, "tokens": list(tokens)})


def create_decode_operation(request_ids: Sequence[int], batch_size: int) -> OperationData:
    return OperationData("decode", {"request_ids": list(request_ids), "batch_size": batch_size})
