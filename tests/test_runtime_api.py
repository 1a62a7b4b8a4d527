"""Pipeline, registry cache, benchmark harness, CLI, package exports."""
import json
import os

import pytest
import torch

from unillm_b200.benchmark.harness import (BenchmarkConfig, BenchmarkResults, BenchmarkRunner, EngineBackend, InferenceMetrics,
                                           UniLLMBackend, format_comparison, format_results)
from unillm_b200.config import GenerationConfig
from unillm_b200.models import configs as C
from unillm_b200.models.families import LlamaModel
from unillm_b200.ollama import OllamaRegistry, parse_model_name
from unillm_b200.pipeline import InferencePipelineBuilder
from unillm_b200.types import ConfigurationError, NetworkError


def tiny():
    cfg = C.LlamaConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                        num_key_value_heads=2)
    return LlamaModel.new(cfg, init="random", seed=7)


def test_pipeline_generate_metrics_and_streaming():
    m = tiny()
    pipe = InferencePipelineBuilder().model(m).build()
    cfg = GenerationConfig.greedy(6, eos_token_id=-1)
    text, met = pipe.generate_with_metrics("hi there", cfg)
    assert met.generated_tokens == 6 and met.total_tokens == met.prompt_tokens + 6 and met.tokens_per_second > 0
    streamed = "".join(pipe.generate_streaming("hi there", cfg))
    assert streamed == text
    eng_pipe = InferencePipelineBuilder().model(m).use_engine().build()
    assert eng_pipe.generate("hi there", cfg) == text
    with pytest.raises(ConfigurationError):
        InferencePipelineBuilder().build()


def test_ollama_cache_roundtrip(tmp_path):
    assert parse_model_name("tinyllama") == ("tinyllama", "latest")
    assert parse_model_name("llama3:8b") == ("llama3", "8b")
    reg = OllamaRegistry(cache_dir=str(tmp_path / "c"), registry="http://127.0.0.1:9")
    f = tmp_path / "m.gguf"
    f.write_bytes(b"GGUF" + bytes(100))
    assert not reg.is_cached("toy")
    p = reg.register_local("toy:v1", str(f), copy=True)
    assert os.path.basename(p).startswith("sha256_") and p.endswith(".gguf")
    assert reg.is_cached("toy:v1") and reg.get_cached_path("toy:v1") == p
    infos = reg.list_cached()
    assert len(infos) == 1 and infos[0].name == "toy" and infos[0].tag == "v1" and infos[0].size == 104
    assert reg.pull("toy:v1") == p
    with pytest.raises(NetworkError):
        reg.pull("absent")
    assert reg.delete_cached("toy:v1") and not os.path.exists(p) and not reg.delete_cached("toy:v1")
    layer = OllamaRegistry.model_layer({"layers": [{"mediaType": "application/vnd.ollama.image.license", "digest": "a"},
                                                   {"mediaType": "application/vnd.ollama.image.model", "digest": "b", "size": 3}]})
    assert layer["digest"] == "b"


def test_cache_dir_env(monkeypatch, tmp_path):
    from unillm_b200.ollama import default_cache_dir

    monkeypatch.setenv("UNILLM_CACHE_DIR", str(tmp_path))
    assert default_cache_dir() == os.path.join(str(tmp_path), "ollama")


def test_benchmark_runner_and_aggregate(tmp_path):
    runs = [InferenceMetrics(10.0, 1000.0, n, memory_mb=5.0 + n) for n in (10, 20, 30, 40)]
    r = BenchmarkResults.aggregate("x", 12.0, runs)
    assert r.avg_tokens_per_second == 25.0 and r.p50_tokens_per_second == 30.0 and r.p99_tokens_per_second == 40.0
    assert r.peak_memory_mb == 45.0 and r.runs == 4 and r.avg_ttft_ms == 10.0
    prog = str(tmp_path / "progress.jsonl")
    cfg = BenchmarkConfig("toy", warmup_iterations=1, iterations=2, max_tokens=4, prompts=("a b", "c"), progress_file=prog)
    res = BenchmarkRunner(cfg).run(UniLLMBackend(model=tiny()))
    assert res.runs == 4 and res.total_tokens == 16 and res.avg_tokens_per_second > 0 and res.avg_ttft_ms > 0
    assert sum(1 for _ in open(prog)) == 4
    cfg.iterations = 3
    res2 = BenchmarkRunner(cfg).run(UniLLMBackend(model=tiny()))       # resumes: only 2 new runs
    assert res2.runs == 6 and sum(1 for _ in open(prog)) == 6
    assert "avg tokens/s" in format_results(res) and "diff" in format_comparison(res, res2)


def test_engine_backend():
    from unillm_b200.engine.cpu_runner import CpuModelRunner
    from unillm_b200.engine.llm_engine import LLMEngine

    m = tiny()
    eng = LLMEngine(CpuModelRunner(m, num_blocks=64, block_size=4, max_model_len=64), num_blocks=64, block_size=4,
                    max_num_seqs=4, max_num_batched_tokens=32, max_model_len=64)
    met = EngineBackend(eng, m.tokenizer(), concurrency=3).generate("x y z", 5)
    assert met.tokens_generated == 15 and met.time_to_first_token_ms > 0


def test_cli_models_and_generate(tmp_path, capsys, monkeypatch):
    from unillm_b200.cli import build_parser, main
    from unillm_b200.weights import write_safetensors

    monkeypatch.setenv("UNILLM_CACHE_DIR", str(tmp_path / "cache"))
    assert main(["models"]) == 0
    out = capsys.readouterr().out
    assert "llama" in out and "mixtral" in out
    m = tiny()
    d = tmp_path / "model"
    d.mkdir()
    write_safetensors(str(d / "model.safetensors"), dict(m.export_hf().tensors))
    cfg = {"architectures": ["LlamaForCausalLM"], "vocab_size": 300, "hidden_size": 32, "intermediate_size": 64,
           "num_hidden_layers": 2, "num_attention_heads": 4, "num_key_value_heads": 2}
    (d / "config.json").write_text(json.dumps(cfg))
    assert main(["generate", "-p", "hello", "-m", str(d), "--max-tokens", "4", "--temperature", "0"]) == 0
    assert len(capsys.readouterr().out) > 0
    assert main(["bench", "-m", str(d), "--warmup", "0", "--iterations", "1", "--max-tokens", "3", "--unillm-only"]) == 0
    assert "avg tokens/s" in capsys.readouterr().out
    assert main(["generate", "-p", "x", "-m", "no-such-model-anywhere"]) == 1
    a = build_parser().parse_args(["bench", "--unillm-only"])
    assert a.warmup == 3 and a.iterations == 10 and a.max_tokens == 50 and a.model == "tinyllama:latest"


def test_package_exports():
    import unillm_b200 as u

    for n in u.__all__:
        assert getattr(u, n) is not None


def test_tensor_helpers_and_runtime():
    import unillm_b200 as u

    t = u.Tensor.from_f32_slice([1, 2, 3, 4, 5, 6], [2, 3])
    assert u.Tensor.shape(t) == [2, 3] and u.Tensor.to_vec_f32(u.Tensor.transpose(t)) == [1, 4, 2, 5, 3, 6]
    assert u.Tensor.narrow(t, 1, 1, 2).tolist() == [[2, 3], [5, 6]]
    assert u.Tensor.from_i64_slice([1, 2], [2]).dtype == torch.int64
    r = u.Runtime()
    assert r.devices()[0].kind == "cpu" or str(r.devices()[0]).lower().startswith("cpu")
    assert "unillm_b200" in r.describe()
