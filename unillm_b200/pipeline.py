"""``InferencePipeline``: tokenizer + model + sampler in one object, generic over models.

Parity with ``crates/runtime/src/inference.rs:159-388``: ``InferencePipeline(+Builder)``, ``generate(prompt, cfg)``,
``InferenceMetrics{prompt_tokens, generated_tokens, total_tokens, generation_time_ms, tokens_per_second}``.
The reference is hard-wired to LLaMA and re-runs the whole sequence for every token; this one takes any
``Model``, uses its KV-cached path when it has one, offers ``generate_streaming`` (promised by the
reference's docs, ``documentation/docs/api-reference/inference.md:10-34``) and can run on the paged engine
(``use_engine=True``).  With ``device="cuda"`` the paged engine is the one on the sm_100a kernels
(``engine.factory.build_engine``: radix-cached paged KV, tcgen05 GEMMs and attention, device sampling); a model
that the kernel runner does not cover stays on the whole-model path and ``engine_note`` says why.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Iterator, List, Optional, Tuple

from .config import GenerationConfig
from .model_core import Model
from .sampling import SamplingParams
from .tokenizer import Tokenizer
from .types import ConfigurationError, GenerationFailed


@dataclass
class InferenceMetrics:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    total_tokens: int = 0
    generation_time_ms: float = 0.0
    time_to_first_token_ms: float = 0.0
    tokens_per_second: float = 0.0


class InferencePipeline:
    def __init__(self, model: Model, tokenizer: Tokenizer, use_engine: bool = False, device: Optional[str] = None,
                 engine_options: Optional[dict] = None):
        """``device``: ``None`` keeps the model where it is; ``"cuda"`` / ``"cuda:i"`` serves it from the paged engine on
        the GPU kernels when the model qualifies (``use_engine`` is then implied), else moves the whole model there."""
        self.model, self.tokenizer, self.use_engine = model, tokenizer, use_engine
        self.device = device
        self.engine_options = dict(engine_options or {})
        self.engine_kind = "none"        # "gpu-kernels" | "cpu-paged" | "none" once the engine exists
        self.engine_note: Optional[str] = None
        self.last_metrics = InferenceMetrics()
        self._engine = None
        if device is not None and str(device).startswith("cuda"):
            from .engine.factory import why_not_gpu

            self.engine_note = why_not_gpu(model)
            if self.engine_note is None:
                self.use_engine = True
            else:
                import torch

                if torch.cuda.is_available():
                    model.to_device(device)

    def _paged_engine(self):
        if self._engine is None:
            from .engine.factory import build_cpu_engine, build_engine

            want_gpu = self.device is not None and str(self.device).startswith("cuda") and self.engine_note is None
            if want_gpu:
                self._engine = build_engine(self.model, device=self.device, **self.engine_options)
                self.engine_kind = "gpu-kernels"
            else:
                self._engine = build_cpu_engine(self.model)
                self.engine_kind = "cpu-paged"
        return self._engine

    def generate_tokens(self, prompt_ids: List[int], cfg: GenerationConfig,
                        on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        if not prompt_ids:
            raise GenerationFailed("empty prompt")
        t0 = time.perf_counter()
        first = [None]

        def cb(t):
            if first[0] is None:
                first[0] = time.perf_counter()
            if on_token is not None:
                on_token(t)

        if self.use_engine:
            eng = self._paged_engine()
            eng.eos_token_id = cfg.eos_token_id
            sid = eng.add_request(prompt_ids, SamplingParams.from_generation_config(cfg))
            out: List[int] = []
            while eng.has_unfinished():
                for o in eng.step():
                    if o.seq_id == sid and not (o.finished and o.finish_reason == "stop" and o.token == cfg.eos_token_id):
                        out.append(o.token)
                        cb(o.token)
        else:
            out = self.model.generate_ids(prompt_ids, cfg, on_token=cb)
        dt = time.perf_counter() - t0
        self.last_metrics = InferenceMetrics(len(prompt_ids), len(out), len(prompt_ids) + len(out), dt * 1e3,
                                             ((first[0] or time.perf_counter()) - t0) * 1e3, len(out) / dt if dt > 0 else 0.0)
        return out

    def generate(self, prompt: str, cfg: Optional[GenerationConfig] = None) -> str:
        cfg = cfg or GenerationConfig()
        ids = self.tokenizer.encode_with_special_tokens(prompt, add_bos=True, add_eos=False)
        return self.tokenizer.decode(self.generate_tokens(ids, cfg))

    def generate_with_metrics(self, prompt: str, cfg: Optional[GenerationConfig] = None) -> Tuple[str, InferenceMetrics]:
        text = self.generate(prompt, cfg)
        return text, self.last_metrics

    def generate_streaming(self, prompt: str, cfg: Optional[GenerationConfig] = None) -> Iterator[str]:
        """Yields the text delta of every new token."""
        cfg = cfg or GenerationConfig()
        ids = self.tokenizer.encode_with_special_tokens(prompt, add_bos=True, add_eos=False)
        toks: List[int] = []
        prev = ""
        for t in self._iter_tokens(ids, cfg):
            toks.append(t)
            cur = self.tokenizer.decode(toks)
            yield cur[len(prev):]
            prev = cur

    def _iter_tokens(self, ids: List[int], cfg: GenerationConfig) -> Iterator[int]:
        import queue
        import threading

        q: "queue.Queue" = queue.Queue()

        def run():
            try:
                self.generate_tokens(ids, cfg, on_token=q.put)
            finally:
                q.put(None)

        th = threading.Thread(target=run, daemon=True)
        th.start()
        while True:
            t = q.get()
            if t is None:
                break
            yield t
        th.join()


class InferencePipelineBuilder:
    def __init__(self):
        self._model: Optional[Model] = None
        self._tok: Optional[Tokenizer] = None
        self._engine = False
        self._device: Optional[str] = None
        self._engine_options: dict = {}

    def model(self, m: Model) -> "InferencePipelineBuilder":
        self._model = m
        return self

    def tokenizer(self, t: Tokenizer) -> "InferencePipelineBuilder":
        self._tok = t
        return self

    def use_engine(self, flag: bool = True) -> "InferencePipelineBuilder":
        self._engine = flag
        return self

    def device(self, device: Optional[str]) -> "InferencePipelineBuilder":
        self._device = device
        return self

    def engine_options(self, **kw) -> "InferencePipelineBuilder":
        """Keyword arguments of ``engine.factory.build_engine`` (max_num_seqs, max_model_len, num_blocks, ...)."""
        self._engine_options.update(kw)
        return self

    def build(self) -> InferencePipeline:
        if self._model is None:
            raise ConfigurationError("Model is required")
        return InferencePipeline(self._model, self._tok or self._model.tokenizer(), self._engine, self._device,
                                 self._engine_options)
