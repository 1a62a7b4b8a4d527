"""Async serving engine end to end on the CPU backend, request/response types, metrics."""
import asyncio

import pytest
import torch

from unillm_b200.engine.cpu_runner import CpuModelRunner
from unillm_b200.engine.llm_engine import LLMEngine
from unillm_b200.inference import (BatchOptimizer, BatchProcessor, ChatMessage, EngineConfig, FinishReason, HealthStatus,
                                   InferenceRequest, METRICS, PerformanceCollector, RequestBuilder, SamplingParams,
                                   UniLLMInferenceEngine)
from unillm_b200.inference.types import InvalidRequest, INFERENCE_ERROR_VARIANTS
from unillm_b200.config import GenerationConfig
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel
from unillm_b200.scheduler import RequestPriority
from unillm_b200.tokenizer import Tokenizer


def _engine():
    tok = Tokenizer.new()
    cfg = C.LlamaConfig(vocab_size=tok.vocab_size(), hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                        num_attention_heads=4, num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=2)
    runner = CpuModelRunner(m, num_blocks=128, block_size=4, max_model_len=256)
    eng = LLMEngine(runner, num_blocks=128, block_size=4, max_num_seqs=8, max_num_batched_tokens=64, max_model_len=256,
                    eos_token_id=None)
    return m, tok, UniLLMInferenceEngine(eng, tok, EngineConfig())


def test_request_builder_and_validation():
    r = (RequestBuilder.new("hello world").with_temperature(0.5).with_max_tokens(7).with_top_p(0.9).with_top_k(5)
         .with_seed(3).with_priority(RequestPriority.High).with_timeout(10).with_session_id("s1").with_streaming()
         .with_stop_sequences(["x"]).with_tags(["a"]).build())
    r.validate()
    assert r.sampling_params.max_tokens == 7 and r.metadata.stream and r.generate_cache_key().startswith("session:s1:")
    assert not r.is_expired() and r.estimated_complexity() > 0
    with pytest.raises(InvalidRequest):
        RequestBuilder.new("x").with_temperature(3.0).build().validate()
    with pytest.raises(InvalidRequest):
        InferenceRequest().validate()
    chat = InferenceRequest.chat([ChatMessage("user", "hi"), ChatMessage("assistant", "yo")])
    assert chat.conversation_context() == "user: hi\nassistant: yo"
    assert len(INFERENCE_ERROR_VARIANTS) == 9


def test_engine_generates_real_tokens_streams_and_reports():
    m, tok, srv = _engine()

    async def run():
        srv.start()
        assert srv.is_running() and (await srv.health_check()).status == HealthStatus.Healthy
        reqs = [RequestBuilder.new(p).with_temperature(0.0).with_max_tokens(6).build()
                for p in ("hello world", "the quick brown fox", "hello world test")]
        resps = await srv.process_batch(reqs)
        stream = await srv.process_request_stream(RequestBuilder.new("hello world").with_temperature(0.0).with_max_tokens(6).build())
        chunks = [c async for c in stream]
        bad = await srv.process_batch([RequestBuilder.new("x").with_max_tokens(100000).build()])
        metrics = await srv.get_metrics()
        await srv.shutdown()
        return resps, chunks, bad, metrics

    resps, chunks, bad, metrics = asyncio.run(run())
    for p, r in zip(("hello world", "the quick brown fox", "hello world test"), resps):
        ids = tok.encode_with_special_tokens(p, add_bos=True, add_eos=False)
        ref = m.generate_ids(ids, GenerationConfig.greedy(6, eos_token_id=-1))
        assert r.text == tok.decode(ref) and r.finish_reason.kind == "length"
        assert r.stats.completion_tokens == 6 and r.stats.prompt_tokens == len(ids) and r.stats.total_time_ms > 0
    assert chunks[-1].finished and chunks[-1].cumulative_text == resps[0].text and len(chunks) == 6
    assert bad[0].finish_reason.kind == "error"
    assert metrics.requests.completed >= 4 and metrics.requests.failed >= 1 and metrics.performance.latency_ms.p50 > 0
    assert not srv.is_running()
    assert "unillm_requests_total" in srv.collector.export_prometheus()
    assert METRICS.get_stats()["tokens_generated"] >= 24 and "unillm_requests_total" in METRICS.get_prometheus_metrics()


def test_stop_sequence_and_timeout():
    m, tok, srv = _engine()

    async def run():
        srv.start()
        full = await srv.process_request(RequestBuilder.new("hello").with_temperature(0.0).with_max_tokens(8).build())
        words = full.text.split()
        stopped = None
        if len(words) >= 2:
            stopped = await srv.process_request(RequestBuilder.new("hello").with_temperature(0.0).with_max_tokens(8)
                                                .with_stop_sequences([words[1]]).build())
        await srv.shutdown()
        return full, stopped, words

    full, stopped, words = asyncio.run(run())
    if stopped is not None:
        assert stopped.finish_reason.kind == "stop" and words[1] not in stopped.text and full.text.startswith(stopped.text.rstrip())


def test_batch_processor_and_collector():
    bp = BatchProcessor()
    reqs = [RequestBuilder.new("a " * n).build() for n in (10, 11, 12, 400)]
    bp.enqueue_requests(reqs)
    b = bp.form_optimal_batch()
    assert 1 <= len(b.requests) <= 4 and b.estimated_time_ms > 0
    bp.start_batch(b); bp.complete_batch(b.batch_id, output_tokens=100)
    assert BatchOptimizer(bp).recommend() == b.strategy and bp.stats.batches_completed == 1
    pc = PerformanceCollector()
    pc.record_request_start("r1"); pc.record_request_complete("r1", 12.0, 5, ttft_ms=3.0, tpot_ms=2.0)
    pc.record_request_start("r2"); pc.record_error("r2", "timeout", "medium", "late")
    mm = pc.get_metrics()
    assert mm.performance.ttft_ms.p50 == 3.0 and mm.errors.by_type == {"timeout": 1} and pc.error_rate() == 0.5
