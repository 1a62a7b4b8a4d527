"""Command line: ``python -m unillm_b200 {generate,models,bench,pull,serve-check}``.

Parity with ``bin/unillm.rs:20-50`` (``generate --prompt/-p --model/-m --max-tokens --temperature``, ``models``),
``bin/test_ollama.rs`` (``pull`` / ``--list-cached``) and ``bin/benchmark_comparison.rs:34-66`` (``bench --model
--warmup --iterations --max-tokens --unillm-only``).  ``--model`` is a registry name (``tinyllama:latest``), a GGUF /
safetensors file or a model directory.  ``UNILLM_LOG_LEVEL`` sets the log level; ``UNILLM_CACHE_DIR`` the cache root.
"""
from __future__ import annotations

import argparse
import logging
import os
import sys
from typing import List, Optional


def _setup_logging() -> None:
    level = os.environ.get("UNILLM_LOG_LEVEL", "info").upper()
    logging.basicConfig(level=getattr(logging, level, logging.INFO), format="%(asctime)s %(levelname)s %(name)s: %(message)s")


def resolve_model_path(model: str) -> str:
    """File or directory as given; otherwise a registry name resolved through the cache (pulling if needed)."""
    if os.path.exists(model):
        return model
    from .ollama import OllamaRegistry

    reg = OllamaRegistry()
    cached = reg.get_cached_path(model)
    if cached:
        return cached

    def prog(done, total):
        pct = 100.0 * done / total if total else 0.0
        print(f"\rdownloading {model}: {done / 2**20:.0f} MB ({pct:.0f}%)", end="", file=sys.stderr)

    path = reg.pull(model, progress=prog)
    print(file=sys.stderr)
    return path


def _load(model: str, device: str):
    from .weights import ModelLoader

    return ModelLoader().load_model(resolve_model_path(model), device=device)


def cmd_generate(a) -> int:
    from .config import GenerationConfig
    from .pipeline import InferencePipelineBuilder

    cuda = a.device.startswith("cuda")
    # for a GPU run the weights are loaded on the host and handed to the kernel runner, which keeps its own bf16
    # copy in kernel layout on the device; a model the runner does not cover is moved to the device as a whole
    model = _load(a.model, "cpu" if cuda else a.device)
    b = InferencePipelineBuilder().model(model).use_engine(a.engine)
    if cuda:
        b = b.device(a.device).engine_options(max_num_seqs=8, max_num_batched_tokens=2048, quantize=a.quantize)
    pipe = b.build()
    if cuda:
        if pipe.engine_note is None:
            print("engine: paged KV + sm_100a kernels", file=sys.stderr)
        else:
            print(f"engine: whole-model path on {a.device} ({pipe.engine_note})", file=sys.stderr)
    cfg = GenerationConfig(max_new_tokens=a.max_tokens, temperature=a.temperature, top_p=a.top_p, top_k=(a.top_k or None),
                           do_sample=a.temperature > 0, seed=a.seed)
    if a.stream:
        for piece in pipe.generate_streaming(a.prompt, cfg):
            print(piece, end="", flush=True)
        print()
    else:
        print(pipe.generate(a.prompt, cfg))
    m = pipe.last_metrics
    print(f"[{m.prompt_tokens} prompt + {m.generated_tokens} new tokens, {m.generation_time_ms:.0f} ms, "
          f"{m.tokens_per_second:.1f} tok/s]", file=sys.stderr)
    return 0


def cmd_models(a) -> int:
    from . import models  # noqa: F401
    from .model_core import registry
    from .ollama import OllamaRegistry

    print("architectures:")
    for n in sorted(registry().supported_architectures()):
        print(f"  {n}")
    cached = OllamaRegistry().list_cached()
    print("cached models:" if cached else "cached models: none")
    for m in cached:
        print(f"  {m.name}:{m.tag}  {m.size / 2**20:.0f} MB  {m.path}")
    return 0


def cmd_pull(a) -> int:
    from .ollama import OllamaRegistry

    reg = OllamaRegistry()
    if a.list_cached:
        for m in reg.list_cached():
            print(f"{m.name}:{m.tag}\t{m.size}\t{m.path}")
        return 0
    if a.file:
        print(reg.register_local(a.model, a.file, copy=a.copy))
        return 0
    print(resolve_model_path(a.model))
    return 0


def cmd_bench(a) -> int:
    from .benchmark.harness import (BenchmarkConfig, BenchmarkRunner, LlamaCppBackend, UniLLMBackend, format_comparison,
                                    format_results)

    path = resolve_model_path(a.model)
    cfg = BenchmarkConfig(a.model, a.warmup, a.iterations, a.max_tokens, progress_file=a.progress_file)
    runner = BenchmarkRunner(cfg)
    ours = None
    if not a.llama_cpp_only:
        ours = runner.run(UniLLMBackend(device=a.device), path)
        print(format_results(ours))
    if not a.unillm_only:
        if not LlamaCppBackend.available():
            print("llama.cpp backend unavailable: python module llama_cpp is not installed", file=sys.stderr)
        else:
            theirs = runner.run(LlamaCppBackend(), path)
            print(format_results(theirs))
            if ours is not None:
                print(format_comparison(ours, theirs))
    return 0


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="unillm_b200", description="B200-native LLM inference")
    sub = p.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate text from a prompt")
    g.add_argument("--prompt", "-p", required=True)
    g.add_argument("--model", "-m", default="tinyllama:latest")
    g.add_argument("--max-tokens", type=int, default=50)
    g.add_argument("--temperature", type=float, default=0.7)
    g.add_argument("--top-p", type=float, default=1.0)
    g.add_argument("--top-k", type=int, default=0)
    g.add_argument("--seed", type=int, default=None)
    g.add_argument("--device", default="cpu")
    g.add_argument("--engine", action="store_true", help="run on the paged continuous-batching engine")
    g.add_argument("--quantize", default=None, choices=["q4_k", "q8_0", "q4_0"],
                   help="--device cuda: keep the projection weights block-quantised on the device")
    g.add_argument("--stream", action="store_true")
    g.set_defaults(fn=cmd_generate)
    m = sub.add_parser("models", help="list architectures and cached models")
    m.set_defaults(fn=cmd_models)
    pl = sub.add_parser("pull", help="fetch a model into the cache, or register a local file")
    pl.add_argument("--model", "-m", default="tinyllama:latest")
    pl.add_argument("--list-cached", action="store_true")
    pl.add_argument("--file", help="register this local GGUF file under --model instead of downloading")
    pl.add_argument("--copy", action="store_true")
    pl.set_defaults(fn=cmd_pull)
    b = sub.add_parser("bench", help="benchmark generation (optionally against llama.cpp)")
    b.add_argument("--model", "-m", default="tinyllama:latest")
    b.add_argument("--warmup", type=int, default=3)
    b.add_argument("--iterations", type=int, default=10)
    b.add_argument("--max-tokens", type=int, default=50)
    b.add_argument("--unillm-only", action="store_true")
    b.add_argument("--llama-cpp-only", action="store_true")
    b.add_argument("--device", default="cpu")
    b.add_argument("--progress-file", default=None)
    b.set_defaults(fn=cmd_bench)
    return p


def main(argv: Optional[List[str]] = None) -> int:
    _setup_logging()
    a = build_parser().parse_args(argv)
    from .types import ModelError

    try:
        return a.fn(a)
    except ModelError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1


if __name__ == "__main__":  # pragma: no cover
    sys.exit(main())
