"""Shared value types: errors, dtypes, devices, feature flags, generation statistics.

Parity with the reference: ``ModelError`` has the same 15 variants as
``crates/runtime/src/types.rs:406-450``; ``DataType`` covers the 7 dtypes of
``crates/runtime/src/tensor_core.rs:28-36`` plus ``Int4`` from the legacy enum
(``types.rs:36-55``); ``Device`` is ``tensor_core.rs:40-44`` with the ``auto / is_gpu / index``
helpers that the reference only documents (``documentation/docs/user-guide/configuration.md:143-160``);
``ModelFeature`` is ``types.rs:554-583``; ``WeightFormat`` adds ``Sharded`` (``types.rs:513-523``).
"""
from __future__ import annotations

import enum
from dataclasses import dataclass, field
from typing import Optional

import torch


class ModelError(Exception):
    """Base error.  Each variant is a subclass so callers can catch one or all."""

    prefix = "Model error"

    def __init__(self, msg: str = ""):
        super().__init__(f"{self.prefix}: {msg}")
        self.msg = msg


def _variant(name: str, prefix: str):
    return type(name, (ModelError,), {"prefix": prefix})


InitializationFailed = _variant("InitializationFailed", "Initialization failed")
ComputationFailed = _variant("ComputationFailed", "Computation failed")
InvalidInput = _variant("InvalidInput", "Invalid input")
DeviceError = _variant("DeviceError", "Device error")
MemoryError_ = _variant("MemoryError_", "Memory error")
UnsupportedOperation = _variant("UnsupportedOperation", "Unsupported operation")
GenerationFailed = _variant("GenerationFailed", "Generation failed")
ValidationFailed = _variant("ValidationFailed", "Validation failed")
ServerError = _variant("ServerError", "Server error")
LoadingError = _variant("LoadingError", "Loading error")
ConfigurationError = _variant("ConfigurationError", "Configuration error")
NetworkError = _variant("NetworkError", "Network error")
FileSystemError = _variant("FileSystemError", "File system error")
CommunicationError = _variant("CommunicationError", "Communication error")
RuntimeError_ = _variant("RuntimeError_", "Runtime error")

MODEL_ERROR_VARIANTS = (
    InitializationFailed, ComputationFailed, InvalidInput, DeviceError, MemoryError_, UnsupportedOperation,
    GenerationFailed, ValidationFailed, ServerError, LoadingError, ConfigurationError, NetworkError,
    FileSystemError, CommunicationError, RuntimeError_,
)


class DataType(enum.Enum):
    F32 = "f32"
    F16 = "f16"
    BF16 = "bf16"
    I32 = "i32"
    I64 = "i64"
    I8 = "i8"
    Bool = "bool"
    Int4 = "int4"

    def size_bytes(self) -> float:
        return {"f32": 4, "f16": 2, "bf16": 2, "i32": 4, "i64": 8, "i8": 1, "bool": 1, "int4": 0.5}[self.value]

    def to_torch(self) -> torch.dtype:
        m = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16, "i32": torch.int32,
             "i64": torch.int64, "i8": torch.int8, "bool": torch.bool}
        if self.value not in m:
            raise UnsupportedOperation(f"{self} has no torch dtype")
        return m[self.value]

    @staticmethod
    def from_torch(dt: torch.dtype) -> "DataType":
        m = {torch.float32: DataType.F32, torch.float16: DataType.F16, torch.bfloat16: DataType.BF16,
             torch.int32: DataType.I32, torch.int64: DataType.I64, torch.int8: DataType.I8, torch.bool: DataType.Bool,
             torch.float64: DataType.F32, torch.uint8: DataType.I8}
        if dt not in m:
            raise UnsupportedOperation(f"no DataType for {dt}")
        return m[dt]


@dataclass(frozen=True)
class Device:
    """``Device.CPU`` or ``Device.CUDA(i)``.  (Metal exists in the reference as a Candle feature flag only.)"""

    kind: str = "cpu"
    ordinal: int = 0

    CPU = None  # filled below

    @staticmethod
    def CUDA(i: int = 0) -> "Device":
        return Device("cuda", i)

    @staticmethod
    def auto() -> "Device":
        return Device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else Device("cpu", 0)

    def is_gpu(self) -> bool:
        return self.kind == "cuda"

    def index(self) -> int:
        return self.ordinal

    def to_torch(self) -> torch.device:
        return torch.device("cpu") if self.kind == "cpu" else torch.device(f"cuda:{self.ordinal}")

    @staticmethod
    def from_torch(d) -> "Device":
        d = torch.device(d)
        return Device("cpu", 0) if d.type == "cpu" else Device("cuda", d.index or 0)

    def __str__(self) -> str:
        return "CPU" if self.kind == "cpu" else f"CUDA({self.ordinal})"


Device.CPU = Device("cpu", 0)


class ModelFeature(enum.Enum):
    FlashAttention = "flash_attention"
    GroupedQueryAttention = "gqa"
    RoPE = "rope"
    RMSNorm = "rms_norm"
    LayerNorm = "layer_norm"
    SwiGLU = "swiglu"
    GELU = "gelu"
    PrefixCaching = "prefix_caching"
    ChunkedPrefill = "chunked_prefill"
    DynamicBatching = "dynamic_batching"
    ContinuousBatching = "continuous_batching"
    LongContext = "long_context"
    SlidingWindow = "sliding_window"
    Quantization = "quantization"
    LoRA = "lora"


class WeightFormat(enum.Enum):
    SafeTensors = "SafeTensors"
    PyTorch = "PyTorch"
    GGUF = "GGUF"
    Sharded = "Sharded"


@dataclass
class GenerationStats:
    prompt_tokens: int = 0
    generated_tokens: int = 0
    total_tokens: int = 0
    total_time_ms: float = 0.0
    time_to_first_token_ms: float = 0.0
    tokens_per_second: float = 0.0
    finish_reason: Optional[str] = None
    extra: dict = field(default_factory=dict)

    def finalize(self) -> "GenerationStats":
        self.total_tokens = self.prompt_tokens + self.generated_tokens
        if self.total_time_ms > 0:
            self.tokens_per_second = self.generated_tokens / (self.total_time_ms / 1000.0)
        return self
