"""``UniLLMInferenceEngine``: the asynchronous serving front end.

The reference engine validates, queues, takes a semaphore permit and then sleeps 10 ms per token
instead of generating (``crates/inference/src/engine.rs:322-379``).  Here the same public surface
(``InferenceEngine`` with ``process_request / process_batch / get_metrics / health_check / shutdown``,
``start / stop / is_running``, ``EngineConfig``, priority queue with expiry, 128-permit concurrency limit,
request timeout, metrics / cleanup workers -- ``lib.rs:22-38``, ``engine.rs:14-230, 414-582``) drives the
real iteration-level ``LLMEngine`` on a dedicated worker thread: requests are tokenised, admitted,
batched continuously with everything else in flight, streamed token by token, and answered with
measured statistics (TTFT, TPOT, cached tokens, queue time).

``BatchProcessor`` / ``BatchOptimizer`` / ``BatchingStrategy`` keep the reference's batch-forming API
(``batch.rs:7-492``) for callers that group requests themselves; they bucket by token count (the
reference compares prompt *character* lengths) and record history that the optimiser really reads.
"""
from __future__ import annotations

import asyncio
import enum
import heapq
import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

from ..config import BatchConfig, MemoryConfig
from ..sampling import SamplingParams
from .metrics import METRICS, InferenceMetrics, PerformanceCollector
from .types import (CacheInfo, EngineHealth, EngineShutdown, FinishReason, GenerationStats, HealthStatus,
                    InferenceError, InferenceRequest, InferenceResponse, InternalError, InvalidRequest, QueueFull,
                    ResourceUsage, ResponseMetadata, ResponseStream, StreamSender, TimeoutError_, TokenInfo)


@dataclass
class ServingModelConfig:
    model_name: str = "default"
    model_path: str = "./models/default"
    max_sequence_length: int = 4096
    vocabulary_size: int = 32000
    num_layers: int = 32
    num_heads: int = 32
    head_dim: int = 128
    hidden_size: int = 4096
    intermediate_size: int = 11008
    dtype: str = "bf16"


@dataclass
class EngineConfig:
    model_config: ServingModelConfig = field(default_factory=ServingModelConfig)
    batch_config: BatchConfig = field(default_factory=BatchConfig)
    memory_config: MemoryConfig = field(default_factory=MemoryConfig)
    max_concurrent_requests: int = 128
    request_timeout_s: float = 300.0
    enable_streaming: bool = True
    enable_metrics_collection: bool = True
    max_queue_size: int = 4096


class InferenceEngine:
    """Interface (``lib.rs:22-38``)."""

    async def process_request(self, request: InferenceRequest) -> InferenceResponse: raise NotImplementedError
    async def process_batch(self, requests: List[InferenceRequest]) -> List[InferenceResponse]: raise NotImplementedError
    async def get_metrics(self) -> InferenceMetrics: raise NotImplementedError
    async def health_check(self) -> EngineHealth: raise NotImplementedError
    async def shutdown(self) -> None: raise NotImplementedError


@dataclass
class _Pending:
    request: InferenceRequest
    future: "asyncio.Future"
    loop: asyncio.AbstractEventLoop
    sender: Optional[StreamSender]
    prompt_ids: List[int]
    submitted: float = field(default_factory=time.monotonic)
    seq_id: Optional[int] = None
    sent_tokens: int = 0
    text: str = ""
    n_decoded: int = 0            # output tokens already turned into text


class UniLLMInferenceEngine(InferenceEngine):
    def __init__(self, llm_engine, tokenizer, config: Optional[EngineConfig] = None):
        self.engine, self.tokenizer = llm_engine, tokenizer
        self.config = config or EngineConfig()
        self.collector = PerformanceCollector()
        self._inbox: "queue.Queue[_Pending]" = queue.Queue()
        self._aborts: "queue.Queue[int]" = queue.Queue()
        self._active: Dict[int, _Pending] = {}
        self._running = False
        self._thread: Optional[threading.Thread] = None
        self._sem: Optional[asyncio.Semaphore] = None
        self._started_at = time.monotonic()
        self._last_error: Optional[str] = None
        self._device_errors = 0
        self._queued = 0

    # ---- lifecycle ----
    def start(self) -> None:
        if self._running:
            return
        self._running = True
        self._started_at = time.monotonic()
        self._thread = threading.Thread(target=self._worker, name="unillm-engine", daemon=True)
        self._thread.start()

    def stop(self) -> None:
        self._running = False
        if self._thread is not None:
            self._thread.join(timeout=30)
            self._thread = None

    def is_running(self) -> bool:
        return self._running

    async def shutdown(self) -> None:
        await asyncio.get_running_loop().run_in_executor(None, self.stop)

    # ---- worker thread: owns the LLMEngine ----
    def _worker(self) -> None:
        eng = self.engine
        last_metrics = 0.0
        while self._running or self._active or not self._inbox.empty():
            try:
                while True:
                    p = self._inbox.get_nowait()
                    self._queued = max(0, self._queued - 1)
                    if p.request.is_expired():
                        self._finish_error(p, TimeoutError_("request expired while queued"))
                        continue
                    try:
                        p.seq_id = eng.add_request(p.prompt_ids, p.request.sampling_params, int(p.request.metadata.priority))
                        self._active[p.seq_id] = p
                        p.request.mark_started()
                    except Exception as e:
                        self._finish_error(p, InvalidRequest(str(e)))
            except queue.Empty:
                pass
            try:
                while True:
                    sid = self._aborts.get_nowait()
                    eng.abort(sid)
            except queue.Empty:
                pass
            if not eng.has_unfinished():
                if not self._running:
                    break
                time.sleep(0.0005)
                continue
            try:
                t0 = time.perf_counter()
                outs = eng.step()
                step_ms = (time.perf_counter() - t0) * 1e3
            except Exception as e:                       # a failed step fails the requests in flight, not the engine
                self._last_error = f"{type(e).__name__}: {e}"
                self._device_errors += 1
                eng._inflight = None                     # whatever was launched is not read back any more
                for sid, p in list(self._active.items()):
                    try:
                        eng.abort(sid)
                    except Exception as e2:              # the abort must not take the worker thread down with it
                        self._last_error = f"{type(e2).__name__}: {e2}"
                    self._finish_error(p, InternalError(self._last_error))
                self._active.clear()
                continue
            for o in outs:
                p = self._active.get(o.seq_id)
                if p is None:
                    continue
                self._on_token(p, o.token, o.finished, o.finish_reason)
            now = time.monotonic()
            for sid, p in list(self._active.items()):
                if p.request.is_expired():
                    eng.abort(sid)
                    self._active.pop(sid, None)
                    self._finish_error(p, TimeoutError_("request timed out"))
            if self.config.enable_metrics_collection and now - last_metrics > 0.25:
                last_metrics = now
                ps = eng.pool.stats()
                rs = eng.radix.stats() if eng.radix is not None else {}
                self.collector.update_engine(queued=self._queued + len(eng.waiting), kv_total=ps["total_blocks"],
                                             kv_used=ps["used_blocks"], batch=len(eng.running), step_ms=step_ms,
                                             hit_tokens=rs.get("hit_tokens", 0), query_tokens=rs.get("query_tokens", 0),
                                             evictions=rs.get("evictions", 0), cached_blocks=rs.get("cached_blocks", 0))

    def _on_token(self, p: _Pending, token: int, finished: bool, reason: Optional[str]) -> None:
        seq = self.engine.seqs[p.seq_id]
        METRICS.token_generated()
        sp = p.request.sampling_params
        # tokens whose values are known: under one-step-ahead scheduling the tail may hold the placeholder of the
        # step in flight
        ids = seq.output_ids
        n = len(ids)
        while n > 0 and ids[n - 1] < 0:
            n -= 1
        if n < p.n_decoded:
            p.n_decoded = n
        # incremental detokenisation: only a window of the latest tokens is decoded, before and after the new ones
        # (a token may complete a multi-byte piece), so the cost per token does not grow with the output length
        w0 = max(0, p.n_decoded - 6)
        old = self.tokenizer.decode(ids[w0:p.n_decoded]) if p.n_decoded > w0 else ""
        new = self.tokenizer.decode(ids[w0:n])
        k = len(old)
        if not new.startswith(old):
            k = 0
            while k < min(len(old), len(new)) and old[k] == new[k]:
                k += 1
        delta = new[k:]
        p.n_decoded = n
        new_text = p.text + delta
        p.text = new_text
        stops = [s for s in sp.stop_sequences if s]
        tail = new_text[-(len(delta) + max(map(len, stops))):] if stops else ""
        stop_hit = next((s for s in stops if s in tail), None)
        if stop_hit is not None and not finished:
            self.engine.abort(p.seq_id)
            p.text = new_text[: new_text.index(stop_hit)]
            finished, reason, delta = True, "stop", ""
        if p.sender is not None:
            ti = TokenInfo(token, delta)
            if finished:
                p.sender.send_final(self._reason(reason), delta, ti)
            else:
                p.sender.send_delta(delta, ti)
        if finished:
            self._active.pop(p.seq_id, None)
            self._finish_ok(p, seq, reason)

    @staticmethod
    def _reason(r: Optional[str]) -> FinishReason:
        return {"length": FinishReason.Length, "stop": FinishReason.stop(), "aborted": FinishReason.aborted()}.get(
            r or "", FinishReason.Completed)

    def _finish_ok(self, p: _Pending, seq, reason: Optional[str]) -> None:
        now = time.perf_counter()
        n_out = len(seq.output_ids)
        ttft = (seq.first_token_time - seq.arrival) * 1e3 if seq.first_token_time else 0.0
        total = (now - seq.arrival) * 1e3
        tpot = (seq.token_times[-1] - seq.token_times[0]) * 1e3 / (n_out - 1) if n_out > 1 else 0.0
        stats = GenerationStats(len(seq.prompt_ids), n_out, len(seq.prompt_ids) + n_out, ttft, total,
                                n_out / (total / 1e3) if total > 0 else 0.0, tpot, seq.num_cached,
                                p.request.queue_time() * 1e3)
        md = ResponseMetadata(self.config.model_config.model_name,
                              cache_info=CacheInfo(seq.num_cached > 0, seq.num_cached, "l1_radix" if seq.num_cached else None),
                              resource_usage=ResourceUsage(preemptions=seq.preemptions))
        text = p.text
        if p.request.metadata.echo:
            text = p.request.text() + text
        resp = InferenceResponse(p.request.request_id, text,
                                 [TokenInfo(t, "") for t in seq.output_ids] if p.request.metadata.logprobs is not None else None,
                                 stats, md, True, self._reason(reason))
        self.collector.record_request_complete(p.request.request_id, total, n_out, ttft, tpot or None, reason or "completed")
        if seq.num_cached:
            METRICS.cache_hit()
        else:
            METRICS.cache_miss()
        p.loop.call_soon_threadsafe(lambda: p.future.done() or p.future.set_result(resp))

    def _finish_error(self, p: _Pending, err: InferenceError) -> None:
        self.collector.record_error(p.request.request_id, err.kind, err.severity, err.msg)
        METRICS.error(err.kind)
        if p.sender is not None:
            p.sender.send_error(err.msg)
        p.loop.call_soon_threadsafe(lambda: p.future.done() or p.future.set_exception(err))

    # ---- async API ----
    def _tokenize(self, request: InferenceRequest) -> List[int]:
        if request.prompt_token_ids is not None:
            return list(request.prompt_token_ids)
        return self.tokenizer.encode_with_special_tokens(request.text(), add_bos=True, add_eos=False)

    async def _submit(self, request: InferenceRequest, stream: Optional[ResponseStream]) -> "asyncio.Future":
        if not self._running:
            raise EngineShutdown("engine is not running")
        try:
            request.validate()
        except InferenceError as e:
            self.collector.record_request_start(request.request_id)
            self.collector.record_error(request.request_id, e.kind, e.severity, e.msg)
            raise
        if self._queued >= self.config.max_queue_size:
            raise QueueFull(f"{self._queued} requests are already queued")
        loop = asyncio.get_running_loop()
        timeout = request.metadata.timeout_s or self.config.request_timeout_s
        if request.context.expires_at is None:
            request.context.expires_at = request.context.created_at + timeout
        fut = loop.create_future()
        sender = StreamSender(stream, loop) if stream is not None else None
        p = _Pending(request, fut, loop, sender, self._tokenize(request))
        self.collector.record_request_start(request.request_id)
        self._queued += 1
        self._inbox.put(p)
        return fut

    async def process_request(self, request: InferenceRequest) -> InferenceResponse:
        if self._sem is None:
            self._sem = asyncio.Semaphore(self.config.max_concurrent_requests)
        timer = METRICS.request_start("process_request")
        async with self._sem:
            try:
                fut = await self._submit(request, None)
                timeout = request.metadata.timeout_s or self.config.request_timeout_s
                resp = await asyncio.wait_for(fut, timeout=timeout + 1.0)
                timer.finish()
                return resp
            except asyncio.TimeoutError:
                timer.finish(error=True)
                raise TimeoutError_("request timed out")
            except Exception:
                timer.finish(error=True)
                raise

    async def process_request_stream(self, request: InferenceRequest) -> ResponseStream:
        """Streaming variant: chunks arrive on the returned stream as tokens are sampled."""
        stream = ResponseStream(request.request_id)
        request.metadata.stream = True
        await self._submit(request, stream)
        return stream

    async def process_batch(self, requests: List[InferenceRequest]) -> List[InferenceResponse]:
        res = await asyncio.gather(*(self.process_request(r) for r in requests), return_exceptions=True)
        out = []
        for r, x in zip(requests, res):
            if isinstance(x, Exception):
                out.append(InferenceResponse(r.request_id, "", finished=True, finish_reason=FinishReason.error(str(x))))
            else:
                out.append(x)
        return out

    async def get_metrics(self) -> InferenceMetrics:
        return self.collector.get_metrics()

    async def health_check(self) -> EngineHealth:
        m = self.collector.get_metrics()
        er = self.collector.error_rate()
        if not self._running:
            st = HealthStatus.Shutdown
        elif self._device_errors > 0 and er > 0.25:
            st = HealthStatus.Unhealthy
        elif er > 0.05 or (m.resources.kv_blocks_total and m.resources.kv_blocks_used / m.resources.kv_blocks_total > 0.97):
            st = HealthStatus.Degraded
        else:
            st = HealthStatus.Healthy
        util = m.resources.kv_blocks_used / m.resources.kv_blocks_total if m.resources.kv_blocks_total else 0.0
        return EngineHealth(st, time.monotonic() - self._started_at, m.requests.in_flight, m.requests.queued, er, util,
                            self._last_error, self._device_errors)

    def generate(self, prompts: List[str], params: Optional[SamplingParams] = None) -> List[InferenceResponse]:
        """Blocking convenience wrapper around ``process_batch``."""
        async def run():
            started = self._running
            if not started:
                self.start()
            try:
                reqs = [InferenceRequest(prompt=p, sampling_params=params or SamplingParams()) for p in prompts]
                return await self.process_batch(reqs)
            finally:
                if not started:
                    await self.shutdown()
        return asyncio.run(run())


# ------------------------------------------------------------------------------------------------
# batch formation API
# ------------------------------------------------------------------------------------------------
class BatchingStrategy(enum.Enum):
    MaxThroughput = "max_throughput"
    MinLatency = "min_latency"
    Balanced = "balanced"
    SequenceLength = "sequence_length"
    CacheAffinity = "cache_affinity"
    Adaptive = "adaptive"


@dataclass
class Batch:
    batch_id: int
    requests: List[InferenceRequest]
    strategy: BatchingStrategy
    estimated_time_ms: float
    priority_score: float
    created_at: float = field(default_factory=time.monotonic)
    started_at: Optional[float] = None


@dataclass
class BatchStats:
    batches_formed: int = 0
    batches_completed: int = 0
    average_batch_size: float = 0.0
    requests_enqueued: int = 0


class BatchProcessor:
    def __init__(self, config: Optional[BatchConfig] = None, token_counter: Optional[Callable[[InferenceRequest], int]] = None):
        self.config = config or BatchConfig()
        self.count = token_counter or (lambda r: len(r.prompt_token_ids) if r.prompt_token_ids is not None else max(1, len(r.text()) // 4))
        self.pending: List[Tuple[int, float, int, InferenceRequest]] = []
        self.active: Dict[int, Batch] = {}
        self._n = 0
        self._next_batch = 1
        self.stats = BatchStats()
        self.history: List[Tuple[float, BatchingStrategy, float, float]] = []    # (time, strategy, tokens/s, latency ms)
        self._oldest: Optional[float] = None

    def enqueue_requests(self, requests: List[InferenceRequest]) -> None:
        for r in requests:
            heapq.heappush(self.pending, (-int(r.metadata.priority), time.monotonic(), self._n, r))
            self._n += 1
        self.stats.requests_enqueued += len(requests)
        if self._oldest is None and requests:
            self._oldest = time.monotonic()

    def choose_strategy(self, seed: InferenceRequest) -> BatchingStrategy:
        md = seed.metadata
        if int(md.priority) >= 3 or md.stream:
            return BatchingStrategy.MinLatency
        if md.cache_key or md.session_id:
            return BatchingStrategy.CacheAffinity
        return BatchingStrategy.SequenceLength if self.count(seed) > 1024 else BatchingStrategy.Balanced

    def estimate_time_ms(self, reqs: List[InferenceRequest]) -> float:
        toks = sum(self.count(r) + r.sampling_params.max_tokens for r in reqs)
        return 5.0 + toks * 0.12

    def form_optimal_batch(self) -> Optional[Batch]:
        if not self.pending:
            return None
        _, _, _, seed = heapq.heappop(self.pending)
        strategy = self.choose_strategy(seed)
        chosen, rest = [seed], []
        n0 = self.count(seed)
        limit = 1 if strategy == BatchingStrategy.MinLatency and int(seed.metadata.priority) >= 3 else self.config.max_batch_size
        while self.pending and len(chosen) < limit:
            item = heapq.heappop(self.pending)
            r = item[3]
            ratio = self.count(r) / max(1, n0)
            same_key = strategy == BatchingStrategy.CacheAffinity and r.generate_cache_key() == seed.generate_cache_key()
            if same_key or 0.7 < ratio < 1.3 or strategy in (BatchingStrategy.MaxThroughput, BatchingStrategy.Balanced):
                chosen.append(r)
            else:
                rest.append(item)
        for item in rest:
            heapq.heappush(self.pending, item)
        b = Batch(self._next_batch, chosen, strategy, self.estimate_time_ms(chosen),
                  sum(int(r.metadata.priority) for r in chosen) / len(chosen))
        self._next_batch += 1
        st = self.stats
        st.batches_formed += 1
        st.average_batch_size += (len(chosen) - st.average_batch_size) / st.batches_formed
        self._oldest = time.monotonic() if self.pending else None
        return b

    def get_next_batch(self) -> Optional[Batch]:
        """A batch when it would be full or the oldest request has waited ``batch_timeout_ms``."""
        if not self.pending:
            return None
        waited = (time.monotonic() - (self._oldest or time.monotonic())) * 1e3
        if len(self.pending) >= self.config.max_batch_size or waited >= self.config.batch_timeout_ms:
            return self.form_optimal_batch()
        return None

    def start_batch(self, b: Batch) -> None:
        b.started_at = time.monotonic()
        self.active[b.batch_id] = b

    def complete_batch(self, batch_id: int, output_tokens: int = 0) -> None:
        b = self.active.pop(batch_id, None)
        if b is None:
            raise InvalidRequest(f"batch {batch_id} is not active")
        dt = max(1e-6, time.monotonic() - (b.started_at or b.created_at))
        self.history.append((time.monotonic(), b.strategy, output_tokens / dt, dt * 1e3))
        self.stats.batches_completed += 1


class BatchOptimizer:
    """Recommends the strategy with the best ``0.7 * throughput - 0.3 * latency`` (both normalised) over the
    last five minutes of the processor's history."""

    def __init__(self, processor: BatchProcessor, window_s: float = 300.0):
        self.p, self.window = processor, window_s

    def recommend(self) -> BatchingStrategy:
        now = time.monotonic()
        rows = [h for h in self.p.history if now - h[0] <= self.window]
        if not rows:
            return BatchingStrategy.Balanced
        mt = max(r[2] for r in rows) or 1.0
        ml = max(r[3] for r in rows) or 1.0
        score: Dict[BatchingStrategy, List[float]] = {}
        for _, s, t, l in rows:
            score.setdefault(s, []).append(0.7 * t / mt - 0.3 * l / ml)
        return max(score, key=lambda s: sum(score[s]) / len(score[s]))
