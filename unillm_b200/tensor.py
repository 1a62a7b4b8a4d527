"""Tensor helpers with the reference's names.

The reference wraps candle tensors in its own ``Tensor`` (shape / dtype / device + storage,
``crates/runtime/src/tensor_core.rs:15-24``) with ``from_f32_slice`` (``:470``), ``from_i64_slice`` (``:481``),
``to_vec_f32`` (``:492``), ``reshape`` (``:357``), ``narrow`` (``:380``), ``transpose`` (``:501``) and
``transpose_dims`` (``:512``).  Here ``torch.Tensor`` *is* the tensor type; this module offers the same constructors
and accessors as thin functions so that code written against the reference's names has a home.  ``Runtime`` is the
reference's empty placeholder struct (``lib.rs:71-87``) given a little content: version, device inventory and the
native libraries' build state.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from .types import DataType, Device


class Tensor:
    """Namespace of constructors / accessors over ``torch.Tensor`` (not a wrapper type)."""

    @staticmethod
    def from_f32_slice(data: Sequence[float], shape: Sequence[int], device: str = "cpu") -> torch.Tensor:
        t = torch.tensor(list(data), dtype=torch.float32, device=device)
        return t.reshape(*shape)

    @staticmethod
    def from_i64_slice(data: Sequence[int], shape: Sequence[int], device: str = "cpu") -> torch.Tensor:
        return torch.tensor(list(data), dtype=torch.int64, device=device).reshape(*shape)

    @staticmethod
    def zeros(shape: Sequence[int], dtype: DataType = DataType.F32, device: str = "cpu") -> torch.Tensor:
        return torch.zeros(*shape, dtype=dtype.to_torch() if hasattr(dtype, "to_torch") else dtype, device=device)

    @staticmethod
    def to_vec_f32(t: torch.Tensor) -> List[float]:
        return t.detach().float().cpu().reshape(-1).tolist()

    @staticmethod
    def reshape(t: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
        return t.reshape(*shape)

    @staticmethod
    def narrow(t: torch.Tensor, dim: int, start: int, length: int) -> torch.Tensor:
        return t.narrow(dim, start, length)

    @staticmethod
    def transpose(t: torch.Tensor) -> torch.Tensor:
        return t.transpose(-1, -2)

    @staticmethod
    def transpose_dims(t: torch.Tensor, d0: int, d1: int) -> torch.Tensor:
        return t.transpose(d0, d1)

    @staticmethod
    def shape(t: torch.Tensor) -> List[int]:
        return list(t.shape)

    @staticmethod
    def device(t: torch.Tensor) -> Device:
        return Device.from_torch(t.device)


class Runtime:
    """Process-level facts: package version, visible devices, whether the native libraries are built."""

    def __init__(self):
        from . import __version__

        self.version = __version__

    def devices(self) -> List[Device]:
        out = [Device.from_torch(torch.device("cpu"))]
        if torch.cuda.is_available():
            out += [Device.from_torch(torch.device("cuda", i)) for i in range(torch.cuda.device_count())]
        return out

    def native_libraries(self) -> dict:
        from .ops import _native as N

        return {"cuda": N.cuda_lib_path().exists(), "host": N.host_lib_path().exists()}

    def describe(self) -> str:
        libs = self.native_libraries()
        return f"unillm_b200 {self.version}: {len(self.devices()) - 1} CUDA device(s), cuda kernels built: {libs['cuda']}, host runtime built: {libs['host']}"


ModelResult = object   # the reference's Result<T, ModelError>: here functions return T or raise a ModelError subclass
