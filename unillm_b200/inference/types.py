"""Serving API types: requests, responses, streams, errors, health.

Parity with ``crates/inference/src``: ``InferenceRequest`` / ``ChatMessage`` / ``RequestMetadata`` /
``RequestBuilder`` with its 17 ``with_*`` setters, ``validate``, ``generate_cache_key``, ``estimated_complexity``,
``is_expired`` (``request.rs:7-335``); ``InferenceResponse`` / ``FinishReason`` / ``ResponseChunk`` /
``ResponseStream`` / ``StreamSender`` / ``ResponseBuilder`` (``response.rs:8-428``); ``InferenceError`` (9
variants), ``SamplingParams``, ``EngineHealth`` / ``HealthStatus``, ``ExecutionContext``, ``AttentionMechanism``,
``TokenInfo``, ``GenerationStats`` (``types.rs:10-319``).  ``SamplingParams`` is the one from
``unillm_b200.sampling`` (same fields).
"""
from __future__ import annotations

import asyncio
import enum
import hashlib
import time
import uuid
from dataclasses import dataclass, field
from typing import Any, AsyncIterator, Dict, List, Optional

from ..sampling import SamplingParams
from ..scheduler.core import RequestPriority


class InferenceError(Exception):
    kind = "inference_error"
    severity = "medium"

    def __init__(self, msg: str = ""):
        super().__init__(msg)
        self.msg = msg


def _err(name, kind, severity):
    return type(name, (InferenceError,), {"kind": kind, "severity": severity})


InvalidRequest = _err("InvalidRequest", "invalid_request", "low")
ModelNotLoaded = _err("ModelNotLoaded", "model_not_loaded", "high")
GpuError = _err("GpuError", "gpu_error", "critical")
MemoryError = _err("MemoryError", "memory_error", "high")
TimeoutError_ = _err("TimeoutError_", "timeout", "medium")
QueueFull = _err("QueueFull", "queue_full", "medium")
EngineShutdown = _err("EngineShutdown", "engine_shutdown", "high")
TokenizationError = _err("TokenizationError", "tokenization_error", "low")
InternalError = _err("InternalError", "internal_error", "critical")
INFERENCE_ERROR_VARIANTS = (InvalidRequest, ModelNotLoaded, GpuError, MemoryError, TimeoutError_, QueueFull,
                            EngineShutdown, TokenizationError, InternalError)


class AttentionMechanism(enum.Enum):
    MultiHead = "multi_head"
    GroupedQuery = "grouped_query"
    MultiQuery = "multi_query"
    FlashAttention = "flash_attention"
    PagedAttention = "paged_attention"
    RadixAttention = "radix_attention"
    HybridCacheAttention = "hybrid_cache_attention"


class HealthStatus(enum.Enum):
    Healthy = "healthy"
    Degraded = "degraded"
    Unhealthy = "unhealthy"
    Initializing = "initializing"
    Shutdown = "shutdown"


@dataclass
class EngineHealth:
    status: HealthStatus
    uptime_s: float
    active_requests: int
    queued_requests: int
    error_rate: float
    kv_cache_utilization: float
    last_error: Optional[str] = None
    device_errors: int = 0


@dataclass
class ChatMessage:
    role: str
    content: str
    name: Optional[str] = None


@dataclass
class RequestMetadata:
    client_id: Optional[str] = None
    session_id: Optional[str] = None
    priority: RequestPriority = RequestPriority.Normal
    timeout_s: Optional[float] = None
    attention_mechanism: Optional[AttentionMechanism] = None
    stream: bool = False
    logprobs: Optional[int] = None
    echo: bool = False
    tags: List[str] = field(default_factory=list)
    cache_key: Optional[str] = None


@dataclass
class ExecutionContext:
    created_at: float = field(default_factory=time.monotonic)
    started_at: Optional[float] = None
    completed_at: Optional[float] = None
    expires_at: Optional[float] = None

    def queue_time(self) -> float:
        return (self.started_at or time.monotonic()) - self.created_at

    def execution_time(self) -> Optional[float]:
        if self.started_at is None:
            return None
        return (self.completed_at or time.monotonic()) - self.started_at

    def is_expired(self) -> bool:
        return self.expires_at is not None and time.monotonic() > self.expires_at


@dataclass
class InferenceRequest:
    prompt: Optional[str] = None
    messages: Optional[List[ChatMessage]] = None
    prompt_token_ids: Optional[List[int]] = None
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    metadata: RequestMetadata = field(default_factory=RequestMetadata)
    context: ExecutionContext = field(default_factory=ExecutionContext)
    request_id: str = field(default_factory=lambda: str(uuid.uuid4()))

    @staticmethod
    def new(prompt: str) -> "InferenceRequest":
        return InferenceRequest(prompt=prompt)

    @staticmethod
    def chat(messages: List[ChatMessage]) -> "InferenceRequest":
        return InferenceRequest(messages=list(messages))

    def conversation_context(self) -> Optional[str]:
        if not self.messages:
            return None
        return "\n".join(f"{m.role}: {m.content}" for m in self.messages)

    def text(self) -> str:
        return self.prompt if self.prompt is not None else (self.conversation_context() or "")

    def estimated_complexity(self) -> float:
        n = len(self.prompt_token_ids) if self.prompt_token_ids is not None else len(self.text()) / 4.0
        return (n + self.sampling_params.max_tokens * 2.0) / 1000.0

    def is_expired(self) -> bool:
        return self.context.is_expired()

    def queue_time(self) -> float:
        return self.context.queue_time()

    def execution_time(self) -> Optional[float]:
        return self.context.execution_time()

    def mark_started(self) -> None:
        self.context.started_at = time.monotonic()

    def generate_cache_key(self) -> str:
        md = self.metadata
        if md.cache_key:
            return md.cache_key
        body = self.text() if self.prompt_token_ids is None else ",".join(map(str, self.prompt_token_ids))
        if md.session_id:
            return f"session:{md.session_id}:{len(body)}"
        return "prompt:" + hashlib.sha1(body.encode("utf-8")).hexdigest()[:16]

    def validate(self) -> None:
        if not self.prompt and not self.messages and not self.prompt_token_ids:
            raise InvalidRequest("Either prompt or messages must be provided")
        sp = self.sampling_params
        if not (0.0 <= sp.temperature <= 2.0):
            raise InvalidRequest("temperature must be between 0.0 and 2.0")
        if not (0.0 <= sp.top_p <= 1.0):
            raise InvalidRequest("top_p must be between 0.0 and 1.0")
        if not (1 <= sp.max_tokens <= 8192):
            raise InvalidRequest("max_tokens must be between 1 and 8192")
        if sp.top_k is not None and sp.top_k < 0:
            raise InvalidRequest("top_k must be non-negative")


class RequestBuilder:
    def __init__(self, prompt: Optional[str] = None, messages: Optional[List[ChatMessage]] = None):
        self.r = InferenceRequest(prompt=prompt, messages=messages)

    @staticmethod
    def new(prompt: str) -> "RequestBuilder":
        return RequestBuilder(prompt=prompt)

    @staticmethod
    def chat(messages: List[ChatMessage]) -> "RequestBuilder":
        return RequestBuilder(messages=list(messages))

    def with_sampling_params(self, p: SamplingParams): self.r.sampling_params = p; return self
    def with_temperature(self, t: float): self.r.sampling_params.temperature = t; return self
    def with_max_tokens(self, n: int): self.r.sampling_params.max_tokens = n; return self
    def with_top_p(self, p: float): self.r.sampling_params.top_p = p; return self
    def with_top_k(self, k: int): self.r.sampling_params.top_k = k; return self
    def with_stop_sequences(self, s: List[str]): self.r.sampling_params.stop_sequences = list(s); return self
    def with_seed(self, seed: int): self.r.sampling_params.seed = seed; return self
    def with_priority(self, p: RequestPriority): self.r.metadata.priority = p; return self

    def with_timeout(self, seconds: float):
        self.r.metadata.timeout_s = seconds
        self.r.context.expires_at = self.r.context.created_at + seconds
        return self

    def with_client_id(self, c: str): self.r.metadata.client_id = c; return self
    def with_session_id(self, s: str): self.r.metadata.session_id = s; return self
    def with_streaming(self): self.r.metadata.stream = True; return self
    def with_logprobs(self, n: int): self.r.metadata.logprobs = n; return self
    def with_echo(self): self.r.metadata.echo = True; return self
    def with_attention_mechanism(self, m: AttentionMechanism): self.r.metadata.attention_mechanism = m; return self
    def with_tags(self, tags: List[str]): self.r.metadata.tags = list(tags); return self
    def with_cache_key(self, k: str): self.r.metadata.cache_key = k; return self
    def with_token_ids(self, ids: List[int]): self.r.prompt_token_ids = list(ids); return self

    def build(self) -> InferenceRequest:
        return self.r


# ------------------------------------------------------------------------------------------------
# responses
# ------------------------------------------------------------------------------------------------
@dataclass
class FinishReason:
    kind: str                       # completed | length | stop | aborted | error | timeout
    detail: Optional[str] = None

    Completed = None
    Length = None

    @staticmethod
    def stop(s: str = "") -> "FinishReason": return FinishReason("stop", s)
    @staticmethod
    def error(s: str) -> "FinishReason": return FinishReason("error", s)
    @staticmethod
    def aborted() -> "FinishReason": return FinishReason("aborted")
    @staticmethod
    def timeout() -> "FinishReason": return FinishReason("timeout")


FinishReason.Completed = FinishReason("completed")
FinishReason.Length = FinishReason("length")


@dataclass
class TokenInfo:
    id: int
    text: str
    logprob: Optional[float] = None
    top_logprobs: Optional[Dict[str, float]] = None


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    completion_tokens: int = 0
    total_tokens: int = 0
    time_to_first_token_ms: float = 0.0
    total_time_ms: float = 0.0
    tokens_per_second: float = 0.0
    time_per_output_token_ms: float = 0.0
    cache_hit_tokens: int = 0
    queue_time_ms: float = 0.0


@dataclass
class CacheInfo:
    cache_hit: bool = False
    cached_tokens: int = 0
    cache_tier: Optional[str] = None


@dataclass
class ResourceUsage:
    gpu_time_ms: float = 0.0
    kv_blocks: int = 0
    preemptions: int = 0


@dataclass
class ResponseMetadata:
    model_name: str = "default"
    created: float = field(default_factory=time.time)
    index: int = 0
    cache_info: CacheInfo = field(default_factory=CacheInfo)
    resource_usage: ResourceUsage = field(default_factory=ResourceUsage)


@dataclass
class InferenceResponse:
    request_id: str
    text: str
    tokens: Optional[List[TokenInfo]] = None
    stats: GenerationStats = field(default_factory=GenerationStats)
    metadata: ResponseMetadata = field(default_factory=ResponseMetadata)
    finished: bool = True
    finish_reason: Optional[FinishReason] = None


@dataclass
class ResponseChunk:
    request_id: str
    delta: str
    token: Optional[TokenInfo] = None
    cumulative_text: str = ""
    finished: bool = False
    finish_reason: Optional[FinishReason] = None
    index: int = 0


class ResponseStream:
    """Unbounded async queue of chunks (``response.rs:232-361``)."""

    def __init__(self, request_id: str):
        self.request_id = request_id
        self._q: "asyncio.Queue[Optional[ResponseChunk]]" = asyncio.Queue()
        self._done = False

    async def next(self) -> Optional[ResponseChunk]:
        if self._done:
            return None
        c = await self._q.get()
        if c is None or c.finished:
            self._done = True
        return c

    def __aiter__(self) -> AsyncIterator[ResponseChunk]:
        return self

    async def __anext__(self) -> ResponseChunk:
        c = await self.next()
        if c is None:
            raise StopAsyncIteration
        return c

    async def collect(self) -> InferenceResponse:
        text, toks, reason = "", [], None
        async for c in self:
            text += c.delta
            if c.token is not None:
                toks.append(c.token)
            if c.finished:
                reason = c.finish_reason
        return InferenceResponse(self.request_id, text, toks or None, finished=True, finish_reason=reason)


class StreamSender:
    def __init__(self, stream: ResponseStream, loop: Optional[asyncio.AbstractEventLoop] = None):
        self.stream, self.loop = stream, loop
        self.text = ""
        self.index = 0

    def _put(self, c: Optional[ResponseChunk]) -> None:
        if self.loop is not None and self.loop.is_running():
            self.loop.call_soon_threadsafe(self.stream._q.put_nowait, c)
        else:
            self.stream._q.put_nowait(c)

    def send_delta(self, delta: str, token: Optional[TokenInfo] = None) -> None:
        self.text += delta
        self._put(ResponseChunk(self.stream.request_id, delta, token, self.text, False, None, self.index))
        self.index += 1

    def send_final(self, reason: FinishReason, delta: str = "", token: Optional[TokenInfo] = None) -> None:
        self.text += delta
        self._put(ResponseChunk(self.stream.request_id, delta, token, self.text, True, reason, self.index))

    def send_error(self, msg: str) -> None:
        self._put(ResponseChunk(self.stream.request_id, "", None, self.text, True, FinishReason.error(msg), self.index))


class ResponseBuilder:
    def __init__(self, request_id: str):
        self.r = InferenceResponse(request_id, "")

    def with_text(self, t: str): self.r.text = t; return self
    def with_tokens(self, t: List[TokenInfo]): self.r.tokens = t; return self
    def with_stats(self, s: GenerationStats): self.r.stats = s; return self
    def with_metadata(self, m: ResponseMetadata): self.r.metadata = m; return self
    def with_finish_reason(self, f: FinishReason): self.r.finish_reason, self.r.finished = f, True; return self
    def build(self) -> InferenceResponse: return self.r
