"""Core model abstractions: ``Model``, ``ModelInputs`` / ``ModelOutputs``, ``ModelWeights``, the model
registry, and the generic mixture-of-experts layer.

Parity with the reference (``crates/runtime/src/model_core.rs``): the ``Model`` trait's seven methods
(``:15-39``), the four input variants and five output variants with their constructors and
``main_tensor`` (``:61-120, 282-367``), ``ModelWeights`` keyed by HuggingFace tensor names with
``get / require / tensor_names / to_device`` (``:124-138, 369-502``), ``ModelFactory`` / ``ModelRegistry``
/ ``registry()`` (``:223-279``; here the registry is actually populated, by ``unillm_b200.models``),
and ``MoELayer`` / ``MoEExpert`` / ``MoEConfig`` / ``RouterType`` (``:516-703``).

Differences by design: linear weights stay in the on-disk ``[out, in]`` layout (the reference
transposes every Linear at load); ``generate`` is implemented once here on top of ``forward`` and the
shared sampler (the reference copies a greedy/temperature loop into every model file).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional

import torch

from .config import GenerationConfig, MemoryRequirements, ModelConfig
from .types import Device, GenerationFailed, InvalidInput, LoadingError, UnsupportedOperation


# ------------------------------------------------------------------------------------------------
# Inputs / outputs
# ------------------------------------------------------------------------------------------------
@dataclass
class ModelInputs:
    """Tagged union of the four input kinds; build with the class-method constructors."""

    kind: str                                   # "text" | "image" | "multimodal" | "audio"
    input_ids: Optional[torch.Tensor] = None
    attention_mask: Optional[torch.Tensor] = None
    position_ids: Optional[torch.Tensor] = None
    pixel_values: Optional[torch.Tensor] = None
    image_mask: Optional[torch.Tensor] = None
    input_features: Optional[torch.Tensor] = None
    decoder_input_ids: Optional[torch.Tensor] = None

    @classmethod
    def text(cls, input_ids: torch.Tensor) -> "ModelInputs":
        return cls("text", input_ids=_as_2d(input_ids))

    @classmethod
    def text_with_mask(cls, input_ids: torch.Tensor, attention_mask: torch.Tensor) -> "ModelInputs":
        return cls("text", input_ids=_as_2d(input_ids), attention_mask=attention_mask)

    @classmethod
    def image(cls, pixel_values: torch.Tensor, image_mask: Optional[torch.Tensor] = None) -> "ModelInputs":
        return cls("image", pixel_values=pixel_values, image_mask=image_mask)

    @classmethod
    def multimodal(cls, input_ids: torch.Tensor, pixel_values: Optional[torch.Tensor] = None,
                   attention_mask: Optional[torch.Tensor] = None,
                   image_mask: Optional[torch.Tensor] = None) -> "ModelInputs":
        return cls("multimodal", input_ids=_as_2d(input_ids), pixel_values=pixel_values,
                   attention_mask=attention_mask, image_mask=image_mask)

    @classmethod
    def audio(cls, input_features: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
              decoder_input_ids: Optional[torch.Tensor] = None) -> "ModelInputs":
        return cls("audio", input_features=input_features, attention_mask=attention_mask,
                   decoder_input_ids=decoder_input_ids)

    def _primary(self) -> torch.Tensor:
        for t in (self.input_ids, self.pixel_values, self.input_features):
            if t is not None:
                return t
        raise InvalidInput("empty ModelInputs")

    def batch_size(self) -> int:
        return int(self._primary().shape[0])

    def sequence_length(self) -> int:
        if self.input_ids is not None:
            return int(self.input_ids.shape[1])
        t = self._primary()
        return int(t.shape[-1]) if self.kind == "audio" else int(t.shape[1])


def _as_2d(ids: torch.Tensor) -> torch.Tensor:
    ids = torch.as_tensor(ids)
    return ids.unsqueeze(0) if ids.dim() == 1 else ids


@dataclass
class ModelOutputs:
    """Tagged union of the five output kinds."""

    kind: str                                   # "logits" | "embeddings" | "multimodal" | "sequence" | "clip"
    logits: Optional[torch.Tensor] = None
    hidden_states: Optional[torch.Tensor] = None
    embeddings_: Optional[torch.Tensor] = None
    pooled: Optional[torch.Tensor] = None
    text_logits: Optional[torch.Tensor] = None
    image_logits: Optional[torch.Tensor] = None
    text_embeddings: Optional[torch.Tensor] = None
    image_embeddings: Optional[torch.Tensor] = None
    encoder_hidden_states: Optional[torch.Tensor] = None
    decoder_hidden_states: Optional[torch.Tensor] = None
    logits_per_text: Optional[torch.Tensor] = None
    logits_per_image: Optional[torch.Tensor] = None
    text_embeds: Optional[torch.Tensor] = None
    image_embeds: Optional[torch.Tensor] = None

    @classmethod
    def from_logits(cls, logits, hidden_states=None) -> "ModelOutputs":
        return cls("logits", logits=logits, hidden_states=hidden_states)

    @classmethod
    def embeddings(cls, embeddings, pooled=None) -> "ModelOutputs":
        return cls("embeddings", embeddings_=embeddings, pooled=pooled)

    @classmethod
    def multimodal(cls, text_logits=None, image_logits=None, text_embeddings=None, image_embeddings=None):
        return cls("multimodal", text_logits=text_logits, image_logits=image_logits,
                   text_embeddings=text_embeddings, image_embeddings=image_embeddings)

    @classmethod
    def sequence(cls, logits, encoder_hidden_states=None, decoder_hidden_states=None) -> "ModelOutputs":
        return cls("sequence", logits=logits, encoder_hidden_states=encoder_hidden_states,
                   decoder_hidden_states=decoder_hidden_states)

    @classmethod
    def clip(cls, logits_per_text, logits_per_image, text_embeds, image_embeds) -> "ModelOutputs":
        return cls("clip", logits_per_text=logits_per_text, logits_per_image=logits_per_image,
                   text_embeds=text_embeds, image_embeds=image_embeds)

    def main_tensor(self) -> torch.Tensor:
        if self.kind in ("logits", "sequence"):
            return self.logits
        if self.kind == "embeddings":
            return self.embeddings_
        if self.kind == "clip":
            return self.logits_per_text
        for t in (self.text_logits, self.image_logits, self.text_embeddings, self.image_embeddings):
            if t is not None:
                return t
        raise InvalidInput("empty ModelOutputs")


# ------------------------------------------------------------------------------------------------
# Weights
# ------------------------------------------------------------------------------------------------
@dataclass
class WeightMetadata:
    architecture: str = "unknown"
    total_params: int = 0
    format: str = "unknown"
    dtype: str = "unknown"
    extra: Dict[str, Any] = field(default_factory=dict)


@dataclass
class QuantizedTensor:
    """A GGUF block-quantised 2-D weight kept in its on-disk encoding (``simd/quant/block.rs:235-377``)."""

    data: torch.Tensor          # uint8, raw blocks, row-major over [rows, cols/block]
    qtype: int                  # GGML type id (2 = Q4_0, 8 = Q8_0, 12 = Q4_K, 14 = Q6_K)
    shape: tuple                # logical (rows, cols)

    def dequantize(self, dtype=torch.float32) -> torch.Tensor:
        from .weights.gguf import dequantize_blocks

        return dequantize_blocks(self.data, self.qtype, self.shape).to(dtype)


class ModelWeights:
    """Tensors by HuggingFace name.  Linear weights are ``[out_features, in_features]``."""

    def __init__(self, tensors: Optional[Dict[str, torch.Tensor]] = None, metadata: Optional[WeightMetadata] = None):
        self.tensors: Dict[str, torch.Tensor] = dict(tensors or {})
        self.metadata = metadata or WeightMetadata()
        self.gguf_config = None
        self.gguf_tokenizer = None
        self.quantized_tensors: Dict[str, QuantizedTensor] = {}

    def get(self, name: str) -> Optional[torch.Tensor]:
        return self.tensors.get(name)

    def require(self, name: str) -> torch.Tensor:
        t = self.tensors.get(name)
        if t is None:
            raise LoadingError(f"required weight '{name}' not found ({len(self.tensors)} tensors loaded)")
        return t

    def first(self, *names: str) -> Optional[torch.Tensor]:
        """First present alias."""
        for n in names:
            t = self.tensors.get(n)
            if t is not None:
                return t
        return None

    def get_quantized(self, name: str) -> Optional[QuantizedTensor]:
        return self.quantized_tensors.get(name)

    def has_quantized(self, name: str) -> bool:
        return name in self.quantized_tensors

    def tensor_names(self) -> List[str]:
        return sorted(self.tensors.keys())

    def insert(self, name: str, t: torch.Tensor) -> None:
        self.tensors[name] = t

    def total_params(self) -> int:
        return sum(int(t.numel()) for t in self.tensors.values())

    def to_device(self, device, dtype: Optional[torch.dtype] = None) -> "ModelWeights":
        dev = device.to_torch() if isinstance(device, Device) else torch.device(device)
        for k, t in list(self.tensors.items()):
            if dtype is not None and t.is_floating_point():
                self.tensors[k] = t.to(device=dev, dtype=dtype)
            else:
                self.tensors[k] = t.to(dev)
        for q in self.quantized_tensors.values():
            q.data = q.data.to(dev)
        return self

    def __len__(self) -> int:
        return len(self.tensors)

    def __contains__(self, name: str) -> bool:
        return name in self.tensors

    def __repr__(self) -> str:
        return (f"ModelWeights({len(self.tensors)} tensors, {len(self.quantized_tensors)} quantized, "
                f"arch={self.metadata.architecture}, format={self.metadata.format})")


# ------------------------------------------------------------------------------------------------
# Model
# ------------------------------------------------------------------------------------------------
class Model:
    """Uniform model interface.  Subclasses implement ``_init_params`` / ``_load`` / ``forward``."""

    config_class: type = ModelConfig

    def __init__(self, config):
        config.validate()
        self._config = config
        self.device = torch.device("cpu")
        self.dtype = torch.float32
        self._tokenizer = None

    # -- construction --
    @classmethod
    def new(cls, config=None, *, init: str = "zeros", seed: int = 0, dtype=torch.float32, device="cpu"):
        """Fresh model.  ``init='zeros'`` matches the reference's ``new`` (zero-filled tensors);
        ``init='random'`` draws N(0, initializer_range) -- used by the benchmarks and oracles."""
        m = cls(config if config is not None else cls.config_class())
        m._init_params(init=init, seed=seed, dtype=dtype, device=torch.device(device))
        m.device, m.dtype = torch.device(device), dtype
        return m

    @classmethod
    def from_weights(cls, config, weights: ModelWeights, *, dtype=None, device=None):
        m = cls(config)
        m._load(weights, dtype=dtype, device=device)
        return m

    def _init_params(self, init, seed, dtype, device):  # pragma: no cover - abstract
        raise NotImplementedError

    def _load(self, weights, dtype=None, device=None):  # pragma: no cover - abstract
        raise NotImplementedError

    # -- inference --
    def forward(self, inputs: ModelInputs) -> ModelOutputs:  # pragma: no cover - abstract
        raise NotImplementedError

    def __call__(self, inputs: ModelInputs) -> ModelOutputs:
        return self.forward(inputs)

    def config(self):
        return self._config

    def parameters(self) -> Dict[str, torch.Tensor]:
        """Name -> tensor for everything the model owns (HF names)."""
        return {}

    def memory_requirements(self) -> MemoryRequirements:
        nbytes = sum(t.numel() * t.element_size() for t in self.parameters().values())
        c = self._config
        kv = 0
        nh = getattr(c, "num_attention_heads", 0)
        if nh:
            nkv = getattr(c, "num_key_value_heads", nh) or nh
            hd = getattr(c, "head_dim", None) or (c.hidden_size // nh)
            ctx = getattr(c, "max_position_embeddings", 2048)
            kv = 2 * c.num_hidden_layers * nkv * hd * ctx * 2
        on_gpu = self.device.type == "cuda"
        return MemoryRequirements(gpu_memory=nbytes if on_gpu else 0, cpu_memory=0 if on_gpu else nbytes,
                                  kv_cache_memory=kv, peak_memory=nbytes + kv + nbytes // 10)

    def to_device(self, device, dtype=None) -> "Model":
        dev = device.to_torch() if isinstance(device, Device) else torch.device(device)
        self._move(dev, dtype)
        self.device = dev
        if dtype is not None:
            self.dtype = dtype
        return self

    def _move(self, dev, dtype):  # pragma: no cover - abstract
        raise NotImplementedError

    # -- tokenizer + generation --
    def set_tokenizer(self, tok) -> None:
        self._tokenizer = tok

    def tokenizer(self):
        if self._tokenizer is None:
            from .tokenizer import Tokenizer

            self._tokenizer = Tokenizer.new()
        return self._tokenizer

    def generate(self, prompt: str, config: Optional[GenerationConfig] = None) -> str:
        """Text in, text out.  Uses the KV-cached path when the model provides one."""
        cfg = config or GenerationConfig()
        tok = self.tokenizer()
        ids = tok.encode_with_special_tokens(prompt, add_bos=True, add_eos=False)
        out = self.generate_ids(ids, cfg)
        return tok.decode(out)

    def generate_ids(self, prompt_ids: List[int], cfg: GenerationConfig,
                     on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        from .sampling import Sampler

        if len(prompt_ids) == 0:
            raise GenerationFailed("empty prompt")
        sampler = Sampler(seed=cfg.seed)
        ids = list(prompt_ids)
        new: List[int] = []
        vocab = self._config.vocab_size_()
        cache = self.new_cache() if hasattr(self, "new_cache") else None
        for step in range(cfg.max_new_tokens):
            if cache is not None:
                feed = ids if step == 0 else ids[-1:]
                logits = self.forward_with_cache(torch.tensor([feed], device=self.device), cache)
            else:
                logits = self.forward(ModelInputs.text(torch.tensor([ids], device=self.device))).main_tensor()
            row = logits[0, -1].float().cpu()
            nxt = sampler.sample(row[:vocab], cfg, history=ids)
            if nxt == cfg.eos_token_id:
                break
            ids.append(nxt)
            new.append(nxt)
            if on_token is not None:
                on_token(nxt)
            if cfg.stop_sequences and self._tokenizer is not None:
                text = self._tokenizer.decode(new)
                if any(s and s in text for s in cfg.stop_sequences):
                    break
        return new


# ------------------------------------------------------------------------------------------------
# Registry
# ------------------------------------------------------------------------------------------------
class ModelFactory:
    """Creates models of one or more architectures from a JSON config."""

    def __init__(self, model_cls: type, architectures: Iterable[str]):
        self.model_cls = model_cls
        self._archs = [a for a in architectures]

    def create_model(self, config_json: Optional[str] = None, **kw) -> Model:
        cfg_cls = self.model_cls.config_class
        cfg = cfg_cls.from_json(config_json) if config_json else cfg_cls()
        return self.model_cls.new(cfg, **kw)

    def supported_architectures(self) -> List[str]:
        return list(self._archs)

    def supports(self, architecture: str) -> bool:
        return architecture.lower() in (a.lower() for a in self._archs)


class ModelRegistry:
    def __init__(self):
        self.factories: Dict[str, ModelFactory] = {}

    def register(self, architecture: str, factory: ModelFactory) -> None:
        self.factories[architecture.lower()] = factory

    def create_model(self, architecture: str, config_json: Optional[str] = None, **kw) -> Model:
        f = self.factories.get(architecture.lower())
        if f is None:
            raise UnsupportedOperation(f"Unsupported architecture: {architecture}")
        return f.create_model(config_json, **kw)

    def get(self, architecture: str) -> Optional[ModelFactory]:
        return self.factories.get(architecture.lower())

    def supported_architectures(self) -> List[str]:
        return sorted(self.factories.keys())

    def supports(self, architecture: str) -> bool:
        return architecture.lower() in self.factories


_REGISTRY = ModelRegistry()


def registry() -> ModelRegistry:
    """Global registry, populated when ``unillm_b200.models`` is imported."""
    return _REGISTRY


# ------------------------------------------------------------------------------------------------
# Generic mixture of experts
# ------------------------------------------------------------------------------------------------
class RouterType(enum.Enum):
    TopK = "top_k"
    ExpertChoice = "expert_choice"
    Soft = "soft"


@dataclass
class MoEConfig:
    num_experts: int = 8
    num_experts_per_tok: int = 2
    hidden_size: int = 4096
    intermediate_size: int = 14336
    router_type: RouterType = RouterType.TopK
    normalize_topk: bool = True      # softmax over the k selected logits (Mixtral); False: softmax over all, then pick
    activation: str = "silu"


class MoEExpert:
    """SwiGLU MLP expert; weights in ``[out, in]`` layout: gate/up ``[I, H]``, down ``[H, I]``."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, activation: str = "silu"):
        self.gate, self.up, self.down, self.activation = gate, up, down, activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        from .tensor_core import ops_fn

        g = ops_fn.linear(x, self.gate)
        u = ops_fn.linear(x, self.up)
        return ops_fn.linear((ops_fn.act(g, self.activation).float() * u.float()).to(x.dtype), self.down)


class MoELayer:
    """Router + experts.  ``route`` reproduces ``model_core.rs:583-604`` (logits -> top-k -> softmax over
    the k selected); ``forward`` groups tokens per expert instead of the reference's per-token loop."""

    def __init__(self, config: MoEConfig, router_weight: torch.Tensor, experts: List[MoEExpert]):
        self.config, self.router_weight, self.experts = config, router_weight, experts

    def route(self, x: torch.Tensor):
        logits = torch.nn.functional.linear(x.float(), self.router_weight.float())
        k = self.config.num_experts_per_tok
        if self.config.router_type == RouterType.Soft:
            w = torch.softmax(logits, dim=-1)
            idx = torch.arange(logits.shape[-1], device=x.device).expand_as(w)
            return w, idx
        if self.config.normalize_topk:
            v, idx = torch.topk(logits, k, dim=-1)
            w = torch.softmax(v, dim=-1)
        else:
            p = torch.softmax(logits, dim=-1)
            w, idx = torch.topk(p, k, dim=-1)
        return w, idx

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        x2 = x.reshape(-1, shape[-1])
        w, idx = self.route(x2)
        out = torch.zeros_like(x2, dtype=torch.float32)
        for e, expert in enumerate(self.experts):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            y = expert.forward(x2[tok])
            out.index_add_(0, tok, y.float() * w[tok, slot].unsqueeze(-1))
        return out.to(x.dtype).reshape(shape)
