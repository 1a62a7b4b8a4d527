"""Configuration system: the ``model_config`` decorator and the plain config structs.

``@model_config`` is the Python counterpart of the reference's ``model_config!`` macro
(``crates/runtime/src/model_core.rs:711-759``): it turns a class body of ``name: type = default``
fields into a dataclass with defaults, JSON / dict (de)serialisation, ``architecture()`` (the class
name), ``vocab_size() / hidden_size() / num_layers()`` accessors and ``validate()``.  Like the macro it
requires the fields ``vocab_size``, ``hidden_size`` and ``num_hidden_layers``; ``validate()`` makes the
same three ``> 0`` checks and adds head- and tensor-parallel divisibility checks.

``GenerationConfig`` has the nine fields and defaults of ``model_core.rs:181-207``; unlike the
reference every field is honoured by the samplers.  ``EngineConfig`` / ``BatchConfig`` /
``MemoryConfig`` mirror ``crates/inference/src/engine.rs:40-73`` and ``types.rs:273-319``.
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

from .types import ConfigurationError, ValidationFailed


class ModelConfig:
    """Base of every generated config (the ``ModelConfig`` trait, ``model_core.rs:42-57``)."""

    def architecture(self) -> str:
        return type(self).__name__

    def vocab_size_(self) -> int:
        return int(getattr(self, "vocab_size"))

    def hidden_size_(self) -> int:
        return int(getattr(self, "hidden_size"))

    def num_layers_(self) -> int:
        return int(getattr(self, "num_hidden_layers"))

    def validate(self, tp: int = 1) -> None:
        if self.vocab_size_() <= 0:
            raise ValidationFailed("vocab_size must be > 0")
        if self.hidden_size_() <= 0:
            raise ValidationFailed("hidden_size must be > 0")
        if self.num_layers_() <= 0:
            raise ValidationFailed("num_layers must be > 0")
        nh = getattr(self, "num_attention_heads", None)
        nkv = getattr(self, "num_key_value_heads", None)
        if nh:
            if nkv and nh % nkv != 0:
                raise ValidationFailed(f"num_attention_heads {nh} not divisible by num_key_value_heads {nkv}")
            if tp > 1 and nh % tp != 0:
                raise ValidationFailed(f"num_attention_heads {nh} not divisible by tensor parallel size {tp}")
            if tp > 1 and nkv and nkv % tp != 0 and tp % nkv != 0:
                raise ValidationFailed(f"num_key_value_heads {nkv} incompatible with tensor parallel size {tp}")

    # ---- (de)serialisation -------------------------------------------------------------------
    def to_dict(self) -> Dict[str, Any]:
        return dataclasses.asdict(self)

    def to_json(self, indent: Optional[int] = None) -> str:
        return json.dumps(self.to_dict(), indent=indent)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]):
        names = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in names})

    @classmethod
    def from_json(cls, s: str):
        return cls.from_dict(json.loads(s))

    @classmethod
    def from_hf_config(cls, d: Dict[str, Any]):
        """Build from a HuggingFace ``config.json`` dict; unknown keys are ignored, common aliases mapped."""
        alias = {"n_embd": "hidden_size", "n_layer": "num_hidden_layers", "n_head": "num_attention_heads",
                 "n_positions": "max_position_embeddings", "d_model": "hidden_size", "num_layers": "num_hidden_layers",
                 "layer_norm_epsilon": "layer_norm_eps", "num_local_experts": "num_experts"}
        dd = dict(d)
        names = {f.name for f in fields(cls)}
        for k, v in alias.items():
            if k in d and v in names and v not in d:
                dd[v] = d[k]
        return cls.from_dict(dd)

    @classmethod
    def from_gguf_config(cls, g) -> "ModelConfig":
        """Build from GGUF metadata (``GGUFModelConfig``), like ``LlamaConfig::from_gguf_config``
        (``models_v2/llama.rs:42-55``): only fields the class actually has are overridden."""
        names = {f.name for f in fields(cls)}
        kw = {}
        for k in ("vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "rms_norm_eps", "rope_theta", "max_position_embeddings"):
            if k in names and getattr(g, k, None) is not None:
                kw[k] = getattr(g, k)
        return cls(**kw)

    def replace(self, **kw):
        return dataclasses.replace(self, **kw)


def model_config(cls):
    """Class decorator: ``@model_config class LlamaConfig: vocab_size: int = 32000 ...``"""
    ann = getattr(cls, "__annotations__", {})
    for req in ("vocab_size", "hidden_size", "num_hidden_layers"):
        if req not in ann:
            raise ConfigurationError(f"{cls.__name__}: model_config requires field '{req}'")
    ns = {k: v for k, v in cls.__dict__.items() if k not in ("__dict__", "__weakref__")}
    for k, v in list(ns.items()):
        if k in ann and isinstance(v, (list, dict, set)):
            ns[k] = field(default_factory=(lambda vv=v: type(vv)(vv)))
    new = type(cls.__name__, (ModelConfig,) + tuple(b for b in cls.__bases__ if b is not object), ns)
    new.__module__ = cls.__module__
    new.__qualname__ = cls.__qualname__
    return dataclass(new)


@dataclass
class GenerationConfig:
    max_new_tokens: int = 100
    temperature: float = 1.0
    top_p: float = 0.9
    top_k: Optional[int] = None
    do_sample: bool = True
    repetition_penalty: float = 1.0
    stop_sequences: List[str] = field(default_factory=list)
    eos_token_id: int = 2
    pad_token_id: int = 0
    seed: Optional[int] = None

    @staticmethod
    def greedy(max_new_tokens: int = 100, eos_token_id: int = 2) -> "GenerationConfig":
        return GenerationConfig(max_new_tokens=max_new_tokens, temperature=0.0, do_sample=False, top_p=1.0,
                                eos_token_id=eos_token_id)


@dataclass
class MemoryRequirements:
    """Bytes needed by a model (``model_core.rs:211-220``)."""

    gpu_memory: int = 0
    cpu_memory: int = 0
    kv_cache_memory: int = 0
    peak_memory: int = 0


@dataclass
class BatchConfig:
    max_batch_size: int = 32
    max_sequence_length: int = 4096
    batch_timeout_ms: int = 10
    enable_chunked_prefill: bool = True
    chunk_size: int = 512
    enable_prefix_caching: bool = True
    dynamic_batching: bool = True


@dataclass
class MemoryConfig:
    gpu_memory_fraction: float = 0.9
    kv_cache_block_size: int = 16
    max_kv_cache_blocks: Optional[int] = None
    swap_space_gb: float = 0.0
    cpu_offload: bool = False


@dataclass
class EngineConfig:
    """Serving-engine settings.  The first block mirrors the reference's ``EngineConfig``
    (``crates/inference/src/engine.rs:40-73``); the second block is what a real engine needs."""

    max_concurrent_requests: int = 128
    request_timeout_s: float = 300.0
    enable_streaming: bool = True
    metrics_interval_s: float = 1.0
    cleanup_interval_s: float = 30.0
    batch: BatchConfig = field(default_factory=BatchConfig)
    memory: MemoryConfig = field(default_factory=MemoryConfig)
    # ---- execution ----
    tensor_parallel_size: int = 1
    expert_parallel_size: int = 1
    block_size: int = 16
    num_kv_blocks: Optional[int] = None       # None: size from gpu_memory_fraction
    max_num_seqs: int = 256
    max_num_batched_tokens: int = 8192
    max_model_len: int = 8192
    enable_prefix_caching: bool = True
    enable_chunked_prefill: bool = True
    scheduling_policy: str = "fcfs"           # fcfs | longest_prefix_match | cache_aware | gpu_memory_optimized | adaptive
    use_cuda_graphs: bool = True
    fused_collectives: bool = True            # False: NCCL + separate GEMMs (the library baseline)
    seed: int = 0
    dtype: str = "bf16"
    device: str = "auto"

    def validate(self) -> None:
        if self.block_size <= 0 or self.block_size & (self.block_size - 1):
            raise ValidationFailed("block_size must be a power of two")
        if self.tensor_parallel_size < 1 or self.expert_parallel_size < 1:
            raise ValidationFailed("parallel sizes must be >= 1")
        if self.max_num_seqs < 1 or self.max_num_batched_tokens < 1:
            raise ValidationFailed("max_num_seqs / max_num_batched_tokens must be >= 1")
        if not (0.0 < self.memory.gpu_memory_fraction <= 1.0):
            raise ValidationFailed("gpu_memory_fraction must be in (0, 1]")
