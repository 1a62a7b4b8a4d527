"""Block-quantised (GGUF) weights: host oracle, host vector kernels and the CUDA dequantise / GEMV kernels.

* ``dequantize_host`` / ``qgemv_host``: the C++ scalar oracle (``csrc/quant/quant_ref.cpp``).
* ``SimdBackend``: the host vector kernels (``csrc/simd/simd_backend.cpp``), the counterpart of the reference's
  ``SimdBackend`` trait (``crates/runtime/src/simd/mod.rs:103-201``) and of ``get_simd_backend`` (``:234``).
* ``dequantize_cuda`` / ``qgemv_cuda``: ``csrc/quant/quant.cu``.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from ..weights.gguf import BLOCK

QTYPES = (2, 3, 6, 8, 12, 14)


def _host():
    from . import _native as N

    lib = N.host_lib()
    if not getattr(lib, "_quant_bound", False):
        vp, i32, i64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float
        lib.ubq_dequantize.argtypes, lib.ubq_dequantize.restype = [vp, vp, i64, i32], i32
        lib.ubq_gemv.argtypes, lib.ubq_gemv.restype = [vp, vp, vp, i32, i32, i32, i32], i32
        lib.ubs_backend_level.restype = i32
        lib.ubs_backend_name.restype = C.c_char_p
        lib.ubs_force_level.argtypes = [i32]
        lib.ubs_set_threads.argtypes = [i32]
        lib.ubs_dot.argtypes, lib.ubs_dot.restype = [vp, vp, i64], f32
        for n in ("ubs_add", "ubs_mul", "ubs_fused_swiglu"):
            getattr(lib, n).argtypes = [vp, vp, vp, i64]
        lib.ubs_silu.argtypes = [vp, vp, i64]
        lib.ubs_rms_norm.argtypes = [vp, vp, vp, i64, i64, f32]
        lib.ubs_softmax.argtypes = [vp, vp, i64, i64]
        lib.ubs_apply_rope.argtypes = [vp, vp, i64, i32, i32, i32, f32]
        lib.ubs_q_gemm.argtypes, lib.ubs_q_gemm.restype = [vp, vp, vp, i32, i32, i32, i32], i32
        lib.ubs_q_gemv.argtypes, lib.ubs_q_gemv.restype = [vp, vp, vp, i32, i32, i32], i32
        lib._quant_bound = True
    return lib


def _bytes(blocks) -> np.ndarray:
    a = blocks.cpu().numpy() if isinstance(blocks, torch.Tensor) else np.asarray(blocks)
    return np.ascontiguousarray(a).view(np.uint8).reshape(-1)


def _check(qtype: int, n: int) -> None:
    if qtype not in QTYPES:
        raise ValueError(f"unsupported ggml type {qtype}")
    if n % BLOCK[qtype][0]:
        raise ValueError(f"{n} elements is not a multiple of the block size {BLOCK[qtype][0]}")


def dequantize_host(blocks, qtype: int, n_elems: int) -> torch.Tensor:
    _check(qtype, n_elems)
    raw = _bytes(blocks)
    out = np.empty(n_elems, dtype=np.float32)
    rc = _host().ubq_dequantize(raw.ctypes.data, out.ctypes.data, n_elems, qtype)
    if rc != 0:
        raise RuntimeError(f"ubq_dequantize failed ({rc})")
    return torch.from_numpy(out)


def qgemv_host(blocks, x: torch.Tensor, N_: int, qtype: int) -> torch.Tensor:
    """``x`` [M, K] fp32 -> [M, N] with the scalar oracle."""
    x = x.float().contiguous()
    M, K = x.shape
    _check(qtype, K)
    raw = _bytes(blocks)
    out = torch.empty(M, N_, dtype=torch.float32)
    rc = _host().ubq_gemv(raw.ctypes.data, x.data_ptr(), out.data_ptr(), M, N_, K, qtype)
    if rc != 0:
        raise RuntimeError(f"ubq_gemv failed ({rc})")
    return out


class SimdBackend:
    """Host vector kernels over fp32 torch tensors (contiguous)."""

    def __init__(self, force_level: Optional[int] = None):
        self.lib = _host()
        if force_level is not None:
            self.lib.ubs_force_level(force_level)

    @property
    def name(self) -> str:
        return self.lib.ubs_backend_name().decode()

    @property
    def level(self) -> int:
        return self.lib.ubs_backend_level()

    @staticmethod
    def _c(t: torch.Tensor) -> torch.Tensor:
        return t.float().contiguous()

    def dot(self, a, b) -> float:
        a, b = self._c(a), self._c(b)
        return float(self.lib.ubs_dot(a.data_ptr(), b.data_ptr(), a.numel()))

    def _bin(self, fn, a, b):
        a, b = self._c(a), self._c(b)
        out = torch.empty_like(a)
        fn(out.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel())
        return out

    def add(self, a, b): return self._bin(self.lib.ubs_add, a, b)
    def mul(self, a, b): return self._bin(self.lib.ubs_mul, a, b)
    def fused_swiglu(self, gate, up): return self._bin(self.lib.ubs_fused_swiglu, gate, up)

    def silu(self, x):
        x = self._c(x)
        out = torch.empty_like(x)
        self.lib.ubs_silu(out.data_ptr(), x.data_ptr(), x.numel())
        return out

    def rms_norm(self, x, w, eps: float = 1e-6):
        x, w = self._c(x), self._c(w)
        out = torch.empty_like(x)
        self.lib.ubs_rms_norm(out.data_ptr(), x.data_ptr(), w.data_ptr(), x.numel() // x.shape[-1], x.shape[-1], eps)
        return out

    def rms_norm_inplace(self, x, w, eps: float = 1e-6):
        self.lib.ubs_rms_norm(x.data_ptr(), x.data_ptr(), self._c(w).data_ptr(), x.numel() // x.shape[-1], x.shape[-1], eps)
        return x

    def softmax(self, x):
        x = self._c(x)
        out = torch.empty_like(x)
        self.lib.ubs_softmax(out.data_ptr(), x.data_ptr(), x.numel() // x.shape[-1], x.shape[-1])
        return out

    def softmax_inplace(self, x):
        self.lib.ubs_softmax(x.data_ptr(), x.data_ptr(), x.numel() // x.shape[-1], x.shape[-1])
        return x

    def apply_rope(self, x, positions, rot_dim: Optional[int] = None, theta: float = 10000.0):
        """``x`` [tokens, heads, head_dim] fp32, rotated in place (half-split pairing)."""
        pos = positions.to(torch.int32).contiguous()
        T, H, D = x.shape
        self.lib.ubs_apply_rope(x.data_ptr(), pos.data_ptr(), T, H, D, rot_dim or D, theta)
        return x

    def q_gemm(self, blocks, x, N_: int, qtype: int):
        x = self._c(x)
        M, K = x.shape
        _check(qtype, K)
        raw = _bytes(blocks)
        out = torch.empty(M, N_, dtype=torch.float32)
        if self.lib.ubs_q_gemm(raw.ctypes.data, x.data_ptr(), out.data_ptr(), M, N_, K, qtype) != 0:
            raise RuntimeError("ubs_q_gemm failed")
        return out

    def q_gemv(self, blocks, x, N_: int, qtype: int):
        return self.q_gemm(blocks, x.reshape(1, -1), N_, qtype)[0]

    def set_threads(self, n: int) -> None:
        """Worker threads of the tiled quantised GEMM (0 = all hardware threads, at most 16)."""
        self.lib.ubs_set_threads(int(n))

    q4_gemm, q4_gemv = q_gemm, q_gemv


_backend: Optional[SimdBackend] = None


def get_simd_backend() -> SimdBackend:
    global _backend
    if _backend is None:
        _backend = SimdBackend()
    return _backend


# ---- CUDA ----
def _cuda():
    from . import _native as N

    lib = N.cuda_lib()
    if not getattr(lib, "_quant_bound", False):
        vp, i32 = N.vp, N.i32
        lib.ub_dequant.argtypes, lib.ub_dequant.restype = [vp, vp, C.c_longlong, i32, vp], i32
        lib.ub_qgemv.argtypes, lib.ub_qgemv.restype = [vp, vp, vp, i32, i32, i32, i32, vp], i32
        lib._quant_bound = True
    return lib, N


def dequantize_cuda(blocks_dev: torch.Tensor, qtype: int, shape) -> torch.Tensor:
    """uint8 CUDA tensor of raw blocks -> bf16 tensor of ``shape``."""
    n = int(np.prod(shape))
    _check(qtype, n)
    lib, N = _cuda()
    out = torch.empty(n, dtype=torch.bfloat16, device=blocks_dev.device)
    N.check(lib.ub_dequant(blocks_dev.data_ptr(), out.data_ptr(), n, qtype,
                           torch.cuda.current_stream(blocks_dev.device).cuda_stream), "ub_dequant")
    return out.view(*shape)


def dequantize_cuda_into(blocks_dev: torch.Tensor, qtype: int, out: torch.Tensor) -> torch.Tensor:
    """Expands raw blocks into the given contiguous bf16 tensor (no allocation: usable inside a captured graph)."""
    n = out.numel()
    _check(qtype, n)
    if out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise ValueError("out must be a contiguous bfloat16 tensor")
    lib, N = _cuda()
    N.check(lib.ub_dequant(blocks_dev.data_ptr(), out.data_ptr(), n, qtype,
                           torch.cuda.current_stream(blocks_dev.device).cuda_stream), "ub_dequant")
    return out


def qgemv_cuda(blocks_dev: torch.Tensor, x: torch.Tensor, N_: int, qtype: int) -> torch.Tensor:
    """``x`` bf16 [M <= 8, K] times the quantised [N, K] matrix -> bf16 [M, N]."""
    x = x.contiguous()
    M, K = x.shape
    _check(qtype, K)
    lib, N = _cuda()
    out = torch.empty(M, N_, dtype=torch.bfloat16, device=x.device)
    N.check(lib.ub_qgemv(blocks_dev.data_ptr(), x.data_ptr(), out.data_ptr(), M, N_, K, qtype,
                         torch.cuda.current_stream(x.device).cuda_stream), "ub_qgemv")
    return out
