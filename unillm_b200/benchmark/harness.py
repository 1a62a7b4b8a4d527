"""Benchmark harness: backend protocol, runner, aggregate statistics, comparison table.

Parity with ``benchmark/runner.rs:13-28,31-37,51-130,134-223``, ``benchmark/metrics.rs:6-37,40-60,78-141`` and
``benchmark/unillm_backend.rs:46-67,69-211``: ``InferenceBackend`` (name / load_model / generate / memory_usage /
unload), ``BenchmarkRunner.run`` (RSS before and after load, warm-up x prompts, measured iterations x prompts,
per-run tokens/s), ``BenchmarkResults.aggregate`` (mean TTFT, mean/p50/p99 tokens/s, mean/peak MB) and the
comparison table.  Two backends ship: ``UniLLMBackend`` (whole-model path: prefill + cached greedy decode, TTFT =
time after prefill) and ``EngineBackend`` (the paged continuous-batching engine, CPU or GPU runner).  The second
arm of the reference's comparison (llama.cpp bindings) is an optional import and reports itself unavailable when
the module is missing.  A run appends one JSON line per measured iteration to a progress file so a long sweep
resumes where it stopped.
"""
from __future__ import annotations

import json
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Dict, List, Optional, Protocol, Sequence

from ..config import GenerationConfig

DEFAULT_PROMPTS = (
    "The capital of France is",
    "Write a short poem about the sea:",
    "Explain in one sentence what a transformer model is:",
)


@dataclass
class BenchmarkConfig:
    model: str = "tinyllama:latest"
    warmup_iterations: int = 3
    iterations: int = 10
    max_tokens: int = 50
    prompts: Sequence[str] = DEFAULT_PROMPTS
    progress_file: Optional[str] = None


@dataclass
class InferenceMetrics:
    time_to_first_token_ms: float
    total_time_ms: float
    tokens_generated: int
    prompt_tokens: int = 0
    memory_mb: float = 0.0

    @property
    def tokens_per_second(self) -> float:
        return self.tokens_generated / (self.total_time_ms / 1e3) if self.total_time_ms > 0 else 0.0


@dataclass
class BenchmarkResults:
    backend: str
    model_load_time_ms: float = 0.0
    avg_ttft_ms: float = 0.0
    avg_tokens_per_second: float = 0.0
    p50_tokens_per_second: float = 0.0
    p99_tokens_per_second: float = 0.0
    avg_memory_mb: float = 0.0
    peak_memory_mb: float = 0.0
    runs: int = 0
    total_tokens: int = 0

    @staticmethod
    def aggregate(backend: str, load_ms: float, runs: List[InferenceMetrics]) -> "BenchmarkResults":
        r = BenchmarkResults(backend, load_ms)
        if not runs:
            return r
        tps = sorted(m.tokens_per_second for m in runs)
        n = len(tps)
        r.runs = n
        r.avg_ttft_ms = sum(m.time_to_first_token_ms for m in runs) / n
        r.avg_tokens_per_second = sum(tps) / n
        r.p50_tokens_per_second = tps[n // 2]
        r.p99_tokens_per_second = tps[min(n - 1, int(n * 0.99))]
        r.avg_memory_mb = sum(m.memory_mb for m in runs) / n
        r.peak_memory_mb = max(m.memory_mb for m in runs)
        r.total_tokens = sum(m.tokens_generated for m in runs)
        return r


class InferenceBackend(Protocol):
    def name(self) -> str: ...
    def load_model(self, path: str) -> None: ...
    def generate(self, prompt: str, max_tokens: int) -> InferenceMetrics: ...
    def memory_usage(self) -> float: ...
    def unload(self) -> None: ...


def rss_mb() -> float:
    try:
        import psutil

        return psutil.Process().memory_info().rss / 2**20
    except Exception:  # pragma: no cover
        import resource

        return resource.getrusage(resource.RUSAGE_SELF).ru_maxrss / 1024.0


class UniLLMBackend:
    """Whole-model backend: prefill once, then one cached forward per token, greedy."""

    def __init__(self, model=None, tokenizer=None, device: str = "cpu"):
        self.model, self.tok, self.device = model, tokenizer, device

    def name(self) -> str:
        return "unillm_b200"

    def load_model(self, path: str) -> None:
        if self.model is not None and not path:
            return
        from ..weights import ModelLoader

        self.model = ModelLoader().load_model(path, device=self.device)
        self.tok = self.model.tokenizer()

    def generate(self, prompt: str, max_tokens: int) -> InferenceMetrics:
        import torch

        tok = self.tok or self.model.tokenizer()
        ids = tok.encode_with_special_tokens(prompt, add_bos=True, add_eos=False)
        m = self.model
        t0 = time.perf_counter()
        cache = m.new_cache() if hasattr(m, "new_cache") else None
        dev = m.device
        out: List[int] = []
        ttft = 0.0
        with torch.no_grad():
            for step in range(max_tokens):
                if cache is not None:
                    feed = ids if step == 0 else out[-1:]
                    logits = m.forward_with_cache(torch.tensor([feed], device=dev), cache)
                else:
                    from ..model_core import ModelInputs

                    logits = m.forward(ModelInputs.text(torch.tensor([ids + out], device=dev))).main_tensor()
                nxt = int(logits[0, -1].argmax())
                if step == 0:
                    ttft = (time.perf_counter() - t0) * 1e3
                out.append(nxt)
        total = (time.perf_counter() - t0) * 1e3
        return InferenceMetrics(ttft, total, len(out), len(ids), self.memory_usage())

    def memory_usage(self) -> float:
        return rss_mb()

    def unload(self) -> None:
        self.model = None


class EngineBackend:
    """The paged engine as a benchmark backend: ``concurrency`` copies of the prompt run as one batch."""

    def __init__(self, engine, tokenizer, concurrency: int = 1):
        self.engine, self.tok, self.concurrency = engine, tokenizer, concurrency

    def name(self) -> str:
        return f"unillm_b200-engine-x{self.concurrency}"

    def load_model(self, path: str) -> None:
        pass

    def generate(self, prompt: str, max_tokens: int) -> InferenceMetrics:
        from ..sampling import SamplingParams

        ids = self.tok.encode_with_special_tokens(prompt, add_bos=True, add_eos=False)
        t0 = time.perf_counter()
        for _ in range(self.concurrency):
            self.engine.add_request(ids, SamplingParams(max_tokens=max_tokens, temperature=0.0, ignore_eos=True))
        n, ttft = 0, 0.0
        while self.engine.has_unfinished():
            outs = self.engine.step()
            if outs and n == 0:
                ttft = (time.perf_counter() - t0) * 1e3
            n += len(outs)
        return InferenceMetrics(ttft, (time.perf_counter() - t0) * 1e3, n, len(ids), self.memory_usage())

    def memory_usage(self) -> float:
        return rss_mb()

    def unload(self) -> None:
        self.engine = None


class LlamaCppBackend:
    """Optional comparison arm; needs the ``llama_cpp`` Python module (n_ctx 2048, n_batch 512, greedy)."""

    def __init__(self):
        self.llm = None

    @staticmethod
    def available() -> bool:
        try:
            import llama_cpp  # noqa: F401

            return True
        except Exception:
            return False

    def name(self) -> str:
        return "llama.cpp"

    def load_model(self, path: str) -> None:
        import llama_cpp

        self.llm = llama_cpp.Llama(model_path=path, n_ctx=2048, n_batch=512, verbose=False)

    def generate(self, prompt: str, max_tokens: int) -> InferenceMetrics:
        t0 = time.perf_counter()
        ttft, n = 0.0, 0
        for _ in self.llm(prompt, max_tokens=max_tokens, temperature=0.0, stream=True):
            if n == 0:
                ttft = (time.perf_counter() - t0) * 1e3
            n += 1
        return InferenceMetrics(ttft, (time.perf_counter() - t0) * 1e3, n, 0, rss_mb())

    def memory_usage(self) -> float:
        return rss_mb()

    def unload(self) -> None:
        self.llm = None


class BenchmarkRunner:
    def __init__(self, config: Optional[BenchmarkConfig] = None):
        self.config = config or BenchmarkConfig()

    def _done(self, backend: str) -> int:
        p = self.config.progress_file
        if not p or not os.path.isfile(p):
            return 0
        return sum(1 for line in open(p) if line.strip() and json.loads(line).get("backend") == backend)

    def _prior(self, backend: str) -> List[InferenceMetrics]:
        p = self.config.progress_file
        if not p or not os.path.isfile(p):
            return []
        out = []
        for line in open(p):
            if line.strip():
                d = json.loads(line)
                if d.get("backend") == backend:
                    out.append(InferenceMetrics(**d["metrics"]))
        return out

    def run(self, backend: InferenceBackend, model_path: str = "") -> BenchmarkResults:
        c = self.config
        before = backend.memory_usage()
        t0 = time.perf_counter()
        backend.load_model(model_path)
        load_ms = (time.perf_counter() - t0) * 1e3
        after = backend.memory_usage()
        for _ in range(c.warmup_iterations):
            for p in c.prompts:
                backend.generate(p, c.max_tokens)
        runs = self._prior(backend.name())
        skip = len(runs)
        k = 0
        for _ in range(c.iterations):
            for p in c.prompts:
                k += 1
                if k <= skip:
                    continue
                m = backend.generate(p, c.max_tokens)
                m.memory_mb = max(m.memory_mb, after) - min(before, after) if m.memory_mb else after - before
                runs.append(m)
                if c.progress_file:
                    with open(c.progress_file, "a") as f:
                        f.write(json.dumps({"backend": backend.name(), "metrics": asdict(m)}) + "\n")
        return BenchmarkResults.aggregate(backend.name(), load_ms, runs)


def format_results(r: BenchmarkResults) -> str:
    rows = [("model load (ms)", r.model_load_time_ms), ("avg TTFT (ms)", r.avg_ttft_ms),
            ("avg tokens/s", r.avg_tokens_per_second), ("p50 tokens/s", r.p50_tokens_per_second),
            ("p99 tokens/s", r.p99_tokens_per_second), ("avg memory (MB)", r.avg_memory_mb),
            ("peak memory (MB)", r.peak_memory_mb), ("runs", r.runs)]
    w = max(len(k) for k, _ in rows)
    return "\n".join([f"== {r.backend} =="] + [f"{k:<{w}}  {v:>12.2f}" for k, v in rows])


def format_comparison(a: BenchmarkResults, b: BenchmarkResults) -> str:
    """Side-by-side table with the relative difference of ``a`` against ``b``."""
    def diff(x, y):
        return f"{(x - y) / y * 100:+.1f}%" if y else "n/a"

    rows = [("model load (ms)", a.model_load_time_ms, b.model_load_time_ms),
            ("avg TTFT (ms)", a.avg_ttft_ms, b.avg_ttft_ms),
            ("avg tokens/s", a.avg_tokens_per_second, b.avg_tokens_per_second),
            ("p50 tokens/s", a.p50_tokens_per_second, b.p50_tokens_per_second),
            ("p99 tokens/s", a.p99_tokens_per_second, b.p99_tokens_per_second),
            ("avg memory (MB)", a.avg_memory_mb, b.avg_memory_mb),
            ("peak memory (MB)", a.peak_memory_mb, b.peak_memory_mb)]
    head = f"{'metric':<18}{a.backend:>22}{b.backend:>22}{'diff':>10}"
    return "\n".join([head, "-" * len(head)] + [f"{k:<18}{x:>22.2f}{y:>22.2f}{diff(x, y):>10}" for k, x, y in rows])
