"""Tracing spans and the data-parallel replica router."""
import logging

import torch

from unillm_b200.engine.cpu_runner import CpuModelRunner
from unillm_b200.engine.llm_engine import LLMEngine
from unillm_b200.engine.replica import ReplicaRouter, replica_groups
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel
from unillm_b200.sampling import SamplingParams
from unillm_b200.utils import Tracer, span, start_inference_span, start_request_span


def test_spans_nest_and_summarise(caplog):
    t = Tracer()
    with caplog.at_level(logging.DEBUG, logger="unillm_b200.trace"):
        for _ in range(5):
            with t.span("outer", step=1):
                with t.span("inner"):
                    pass
    s = t.summary()
    assert s["outer"]["count"] == 5 and s["inner"]["count"] == 5 and s["outer"]["mean_ms"] >= s["inner"]["mean_ms"]
    assert any('"parent": "outer"' in r.message for r in caplog.records)
    with start_request_span("r1", "generate") as f, start_inference_span("llama", 4) as g:
        assert f["request_id"] == "r1" and g["batch_size"] == 4
    with span("x"):
        pass
    t.reset()
    assert t.summary() == {}


def test_replica_router_balances_and_prefers_cached_prefix():
    assert replica_groups(8, 4) == [[0, 1, 2, 3], [4, 5, 6, 7]]
    cfg = C.LlamaConfig(vocab_size=128, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                        num_key_value_heads=2)
    m = LlamaModel.new(cfg, init="random", seed=3)

    def engine():
        return LLMEngine(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=64), num_blocks=64, block_size=4,
                         max_num_seqs=4, max_num_batched_tokens=32, max_model_len=64)

    r = ReplicaRouter([engine(), engine()])
    g = torch.Generator().manual_seed(0)
    params = SamplingParams(temperature=0.0, max_tokens=4)
    shared = torch.randint(0, 128, (16,), generator=g).tolist()
    a = r.add_request(shared + [1, 2], params)
    b = r.add_request(torch.randint(0, 128, (10,), generator=g).tolist(), params)
    assert r._where[a][0] != r._where[b][0]                  # least loaded: second request goes to the other replica
    out = r.run_to_completion()
    assert len(out[a]) == 4 and len(out[b]) == 4
    c = r.add_request(shared + [9, 9, 9], params)            # its prefix is cached on a's replica
    assert r._where[c][0] == r._where[a][0]
    ref = engine().generate([shared + [9, 9, 9]], params)[0]
    assert r.run_to_completion()[c] == ref
