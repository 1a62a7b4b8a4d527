"""Tensor operation layer: the ``TensorOps`` interface, its CPU and CUDA implementations, the global
dispatcher ``ops()`` and the ``ops_fn`` functional namespace that model code calls.

Parity with the reference (``crates/runtime/src/tensor_core.rs``): ``TensorOps`` has the same 24
primitive + 3 fused methods (``:179-296``); ``ops_fn`` exposes the same 32 free functions
(``:1632-1824``) including the three mask builders (``:1751-1781``).  ``torch.Tensor`` is the tensor
type (the reference wraps Candle tensors, ``:15-24``); shapes follow the reference, except that
linear weights keep the on-disk ``[out, in]`` layout and go through :func:`ops_fn.linear`.

Dispatch: CPU tensors use ``CpuTensorOps`` (plain fp32-accurate PyTorch, the numerical oracle);
CUDA bf16 tensors use ``CudaTensorOps`` whose hot methods call the hand-written sm_100a kernels in
``unillm_b200.ops.cuda_ops`` (the reference's ``GpuTensorOpsImpl`` forwards everything to the CPU,
``:1504-1629``).
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .types import InvalidInput, UnsupportedOperation


class TensorOps:
    """Interface; every method takes and returns ``torch.Tensor``."""

    # --- 24 primitives ---
    def matmul(self, a, b): raise NotImplementedError
    def add(self, a, b): raise NotImplementedError
    def sub(self, a, b): raise NotImplementedError
    def mul(self, a, b): raise NotImplementedError
    def scale(self, x, s): raise NotImplementedError
    def clamp(self, x, lo, hi): raise NotImplementedError
    def exp(self, x): raise NotImplementedError
    def tanh(self, x): raise NotImplementedError
    def sigmoid(self, x): raise NotImplementedError
    def gelu(self, x): raise NotImplementedError
    def silu(self, x): raise NotImplementedError
    def softmax(self, x, dim=-1): raise NotImplementedError
    def attention(self, q, k, v, mask=None, scale=None): raise NotImplementedError
    def layer_norm(self, x, w, b=None, eps=1e-5): raise NotImplementedError
    def rms_norm(self, x, w, eps=1e-6): raise NotImplementedError
    def embedding(self, ids, table): raise NotImplementedError
    def topk(self, x, k, dim=-1): raise NotImplementedError
    def conv1d(self, x, w, b=None, stride=1, padding=0): raise NotImplementedError
    def normalize(self, x, p=2.0, dim=-1): raise NotImplementedError
    def concat(self, xs, dim=0): raise NotImplementedError
    def gather(self, x, dim, index): raise NotImplementedError
    def scatter(self, x, dim, index, src): raise NotImplementedError
    def zeros(self, shape, dtype=torch.float32, device="cpu"): raise NotImplementedError
    def randn(self, shape, dtype=torch.float32, device="cpu"): raise NotImplementedError
    # --- 3 fused ---
    def flash_attention(self, q, k, v, scale=None, causal=True): raise NotImplementedError
    def fused_swiglu(self, gate, up): raise NotImplementedError
    def fused_residual_rms_norm(self, x, residual, w, eps=1e-6): raise NotImplementedError


class CpuTensorOps(TensorOps):
    """Plain PyTorch; math in fp32 for half-precision inputs.  Works on any device, used as the oracle."""

    @staticmethod
    def _up(x):
        return x.float() if x.dtype in (torch.bfloat16, torch.float16) else x

    def matmul(self, a, b):
        # (M,K)@(K,N); (B,M,K)@(K,N); (B,M,K)@(B,K,N); (M,K)@(B,K,N) -- torch.matmul broadcasting covers all four
        return torch.matmul(a, b)

    def add(self, a, b): return a + b
    def sub(self, a, b): return a - b
    def mul(self, a, b): return a * b
    def scale(self, x, s): return x * s
    def clamp(self, x, lo, hi): return torch.clamp(x, lo, hi)
    def exp(self, x): return torch.exp(self._up(x)).to(x.dtype)
    def tanh(self, x): return torch.tanh(self._up(x)).to(x.dtype)
    def sigmoid(self, x): return torch.sigmoid(self._up(x)).to(x.dtype)
    def gelu(self, x): return F.gelu(self._up(x)).to(x.dtype)
    def silu(self, x): return F.silu(self._up(x)).to(x.dtype)
    def softmax(self, x, dim=-1): return torch.softmax(self._up(x), dim=dim).to(x.dtype)

    def attention(self, q, k, v, mask=None, scale=None):
        """``softmax(q k^T * scale, masked) v``; ``mask`` is 1/0 (1 = visible) broadcastable to the scores."""
        d = q.shape[-1]
        scale = scale if scale is not None else 1.0 / math.sqrt(d)
        s = torch.matmul(self._up(q), self._up(k).transpose(-1, -2)) * scale
        if mask is not None:
            s = s.masked_fill(mask.to(s.device) == 0, -1e9)
        p = torch.softmax(s, dim=-1)
        return torch.matmul(p, self._up(v)).to(q.dtype)

    def layer_norm(self, x, w, b=None, eps=1e-5):
        xf = self._up(x)
        y = F.layer_norm(xf, (x.shape[-1],), None if w is None else self._up(w), None if b is None else self._up(b), eps)
        return y.to(x.dtype)

    def rms_norm(self, x, w, eps=1e-6):
        xf = self._up(x)
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        if w is not None:
            y = y * self._up(w)
        return y.to(x.dtype)

    def embedding(self, ids, table): return F.embedding(ids.long(), table)

    def topk(self, x, k, dim=-1):
        v, i = torch.topk(x, k, dim=dim)
        return v, i

    def conv1d(self, x, w, b=None, stride=1, padding=0):
        return F.conv1d(x, w, b, stride=stride, padding=padding)

    def normalize(self, x, p=2.0, dim=-1): return F.normalize(self._up(x), p=p, dim=dim).to(x.dtype)
    def concat(self, xs, dim=0): return torch.cat(list(xs), dim=dim)
    def gather(self, x, dim, index): return torch.gather(x, dim, index.long())
    def scatter(self, x, dim, index, src): return x.scatter(dim, index.long(), src)

    def scatter_add(self, x, dim, index, src): return x.scatter_add(dim, index.long(), src)

    def zeros(self, shape, dtype=torch.float32, device="cpu"): return torch.zeros(*shape, dtype=dtype, device=device)
    def randn(self, shape, dtype=torch.float32, device="cpu"): return torch.randn(*shape, dtype=dtype, device=device)

    def flash_attention(self, q, k, v, scale=None, causal=True):
        """``[B, H, Sq, D]`` inputs; with ``causal`` query i sees keys ``<= Sk - Sq + i``.  No L x L mask is
        materialised on the host (the reference builds one, ``tensor_core.rs:1347-1371``)."""
        d = q.shape[-1]
        scale = scale if scale is not None else 1.0 / math.sqrt(d)
        qf, kf, vf = self._up(q), self._up(k), self._up(v)
        if kf.shape[1] != qf.shape[1]:
            g = qf.shape[1] // kf.shape[1]
            kf, vf = kf.repeat_interleave(g, dim=1), vf.repeat_interleave(g, dim=1)
        sq, sk = qf.shape[-2], kf.shape[-2]
        mask = None
        if causal:
            mask = torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq)
        y = F.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, scale=scale)
        return y.to(q.dtype)

    def fused_swiglu(self, gate, up):
        return (F.silu(self._up(gate)) * self._up(up)).to(gate.dtype)

    def fused_residual_rms_norm(self, x, residual, w, eps=1e-6):
        """Returns ``(rms_norm(x + residual), x + residual)``."""
        h = x + residual
        return self.rms_norm(h, w, eps), h


class CudaTensorOps(CpuTensorOps):
    """bf16 CUDA tensors: hot ops on the sm_100a kernels, the rest on torch CUDA ops."""

    @staticmethod
    def _k():
        from .ops import cuda_ops

        return cuda_ops

    @staticmethod
    def _fast(x):
        return x.is_cuda and x.dtype == torch.bfloat16

    def linear(self, x, w, b=None, act=None, residual=None):
        if self._fast(x) and self._fast(w) and x.shape[-1] % 8 == 0:
            lead = x.shape[:-1]
            x2 = x.reshape(-1, x.shape[-1])
            if x2.stride(-1) != 1 or x2.stride(0) % 8 != 0:
                x2 = x2.contiguous()
            r2 = None if residual is None else residual.reshape(-1, residual.shape[-1]).contiguous()
            y = self._k().gemm_tn(x2, w if w.stride(-1) == 1 else w.contiguous(), bias=b, act=act, residual=r2)
            return y.reshape(*lead, y.shape[-1])
        y = F.linear(x, w, b)
        if act is not None:
            y = _ACT_TORCH[act](y)
        return y if residual is None else y + residual

    def matmul(self, a, b):
        # Activations @ pre-transposed weight [K, N] (reference convention): route through the TN GEMM.
        if self._fast(a) and self._fast(b) and b.dim() == 2 and a.shape[-1] % 8 == 0 and b.shape[0] % 8 == 0:
            return self.linear(a, b.t().contiguous())
        return torch.matmul(a, b)

    def gelu(self, x): return self._k().eltwise(x, "gelu") if self._fast(x) else super().gelu(x)
    def silu(self, x): return self._k().eltwise(x, "silu") if self._fast(x) else super().silu(x)
    def sigmoid(self, x): return self._k().eltwise(x, "sigmoid") if self._fast(x) else super().sigmoid(x)
    def tanh(self, x): return self._k().eltwise(x, "tanh") if self._fast(x) else super().tanh(x)
    def exp(self, x): return self._k().eltwise(x, "exp") if self._fast(x) else super().exp(x)
    def scale(self, x, s): return self._k().eltwise(x, None, float(s)) if self._fast(x) else super().scale(x, s)

    def add(self, a, b):
        if self._fast(a) and self._fast(b) and a.shape == b.shape:
            return self._k().add(a, b)
        return a + b

    def sub(self, a, b):
        if self._fast(a) and self._fast(b) and a.shape == b.shape:
            return self._k().add(a, b, 1.0, -1.0)
        return a - b

    def layer_norm(self, x, w, b=None, eps=1e-5):
        if self._fast(x):
            return self._k().norm(x, w, bias=b, eps=eps, kind="layer").reshape(x.shape)
        return super().layer_norm(x, w, b, eps)

    def rms_norm(self, x, w, eps=1e-6):
        if self._fast(x):
            return self._k().norm(x, w, eps=eps, kind="rms").reshape(x.shape)
        return super().rms_norm(x, w, eps)

    def fused_residual_rms_norm(self, x, residual, w, eps=1e-6):
        if self._fast(x) and self._fast(residual):
            y, h = self._k().norm(x, w, residual=residual.contiguous(), eps=eps, kind="rms", want_residual_out=True)
            return y.reshape(x.shape), h.reshape(x.shape)
        return super().fused_residual_rms_norm(x, residual, w, eps)

    def fused_swiglu(self, gate, up):
        if self._fast(gate) and self._fast(up):
            return self._k().act_mul(torch.cat([gate, up], dim=-1), "silu")
        return super().fused_swiglu(gate, up)

    def embedding(self, ids, table):
        if self._fast(table):
            return self._k().embed_gather(ids.reshape(-1), table).reshape(*ids.shape, table.shape[1])
        return super().embedding(ids, table)

    def normalize(self, x, p=2.0, dim=-1):
        if self._fast(x) and p == 2.0 and dim in (-1, x.dim() - 1):
            return self._k().l2_normalize(x)
        return super().normalize(x, p, dim)

    def softmax(self, x, dim=-1):
        if self._fast(x) and dim in (-1, x.dim() - 1):
            return self._k().softmax_rows(x)
        return super().softmax(x, dim)

    def _attn_ok(self, q, k, v):
        return (self._fast(q) and self._fast(k) and self._fast(v) and q.dim() == 4 and k.dim() == 4 and
                q.shape[-1] in (64, 128) and q.shape[1] % k.shape[1] == 0 and k.shape == v.shape)

    def attention(self, q, k, v, mask=None, scale=None):
        # no mask: the paged attention kernels on dense pages; an explicit mask keeps the torch path
        if mask is None and self._attn_ok(q, k, v):
            return self._k().dense_attention(q, k, v, causal=False, scale=scale)
        return super().attention(q, k, v, mask, scale)

    def flash_attention(self, q, k, v, scale=None, causal=True):
        if self._attn_ok(q, k, v):
            return self._k().dense_attention(q, k, v, causal=causal, scale=scale)
        return super().flash_attention(q, k, v, scale, causal)

    def conv1d(self, x, w, b=None, stride=1, padding=0):
        if self._fast(x):
            from .models.simple import conv1d

            return conv1d(x, w, b, stride=stride, padding=padding)      # window rows x filter matrix on the tcgen05 GEMM
        return super().conv1d(x, w, b, stride, padding)


_ACT_TORCH = {
    "silu": F.silu, "swish": F.silu, "gelu": F.gelu, "relu": F.relu, "sigmoid": torch.sigmoid, "tanh": torch.tanh,
    "gelu_tanh": lambda t: F.gelu(t, approximate="tanh"), "gelu_new": lambda t: F.gelu(t, approximate="tanh"),
    "gelu_pytorch_tanh": lambda t: F.gelu(t, approximate="tanh"),
    "quick_gelu": lambda t: t * torch.sigmoid(1.702 * t), "relu2": lambda t: F.relu(t) ** 2,
    "softplus": F.softplus, "exp": torch.exp, "none": lambda t: t, None: lambda t: t,
}

_CPU_OPS = CpuTensorOps()
_CUDA_OPS = CudaTensorOps()


class TensorOpsDispatcher:
    """Picks the implementation from the first tensor argument's device (``tensor_core.rs:622-822``)."""

    def get_ops(self, t) -> TensorOps:
        if isinstance(t, torch.Tensor) and t.is_cuda:
            return _CUDA_OPS
        return _CPU_OPS

    def __getattr__(self, name):
        def call(*args, **kw):
            probe = args[0]
            if isinstance(probe, (list, tuple)) and probe and isinstance(probe[0], torch.Tensor):
                probe = probe[0]
            return getattr(self.get_ops(probe), name)(*args, **kw)

        return call


_DISPATCH = TensorOpsDispatcher()


def ops() -> TensorOpsDispatcher:
    """Global dispatcher (``tensor_core.rs:1497-1502``)."""
    return _DISPATCH


class _OpsFn:
    """``ops_fn::*`` -- the 32 free functions of the reference plus ``linear`` / activation lookup."""

    def matmul(self, a, b): return ops().matmul(a, b)
    def add(self, a, b): return ops().add(a, b)
    def zeros(self, shape, dtype=torch.float32, device="cpu"): return _CPU_OPS.zeros(shape, dtype, device)
    def randn(self, shape, dtype=torch.float32, device="cpu"): return _CPU_OPS.randn(shape, dtype, device)
    def layer_norm(self, x, w, b=None, eps=1e-5): return ops().layer_norm(x, w, b, eps)
    def embedding(self, ids, table): return ops().get_ops(table).embedding(ids, table)
    def silu(self, x): return ops().silu(x)
    def mul(self, a, b): return ops().mul(a, b)
    def attention(self, q, k, v, mask=None, scale=None): return ops().attention(q, k, v, mask, scale)
    def gelu(self, x): return ops().gelu(x)
    def exp(self, x): return ops().exp(x)
    def normalize(self, x, p=2.0, dim=-1): return ops().normalize(x, p, dim)
    def concat(self, xs, dim=0): return ops().concat(xs, dim)
    def rms_norm(self, x, w, eps=1e-6): return ops().rms_norm(x, w, eps)
    def scale(self, x, s): return ops().scale(x, s)
    def transpose(self, x): return x.transpose(-1, -2)
    def transpose_dims(self, x, d0, d1): return x.transpose(d0, d1)
    def sigmoid(self, x): return ops().sigmoid(x)
    def topk(self, x, k, dim=-1): return ops().topk(x, k, dim)
    def conv1d(self, x, w, b=None, stride=1, padding=0): return ops().conv1d(x, w, b, stride, padding)
    def tanh(self, x): return ops().tanh(x)
    def sub(self, a, b): return ops().sub(a, b)
    def clamp(self, x, lo, hi): return ops().clamp(x, lo, hi)
    def gather(self, x, dim, index): return ops().gather(x, dim, index)
    def scatter(self, x, dim, index, src): return ops().scatter(x, dim, index, src)
    def softmax(self, x, dim=-1): return ops().softmax(x, dim)

    def causal_mask(self, n: int, device="cpu") -> torch.Tensor:
        """1/0 lower-triangular ``[n, n]`` (``tensor_core.rs:1751-1762``)."""
        return torch.ones(n, n, device=device).tril()

    def sliding_window_mask(self, n: int, window: int, device="cpu") -> torch.Tensor:
        """1 where ``|i - j| < window`` (``tensor_core.rs:1764-1776``)."""
        i = torch.arange(n, device=device)
        return ((i[:, None] - i[None, :]).abs() < window).float()

    def causal_sliding_window_mask(self, n: int, window: int, device="cpu") -> torch.Tensor:
        """1 where ``j <= i`` and ``i - j < window`` (``tensor_core.rs:1778-1795``)."""
        i = torch.arange(n, device=device)
        d = i[:, None] - i[None, :]
        return ((d >= 0) & (d < window)).float()

    def flash_attention(self, q, k, v, scale=None, causal=True): return ops().flash_attention(q, k, v, scale, causal)
    def fused_swiglu(self, gate, up): return ops().fused_swiglu(gate, up)
    def fused_residual_rms_norm(self, x, residual, w, eps=1e-6): return ops().fused_residual_rms_norm(x, residual, w, eps)

    # ---- additions used by the model zoo ----
    def linear(self, x, w, b=None, act=None, residual=None):
        """``act(x @ w^T + b) + residual`` with ``w`` in ``[out, in]`` layout."""
        if x.is_cuda:
            return _CUDA_OPS.linear(x, w, b, act, residual)
        y = F.linear(x, w, b)
        if act is not None:
            y = _ACT_TORCH[act](y)
        return y if residual is None else y + residual

    def activation(self, name: Optional[str]):
        if name not in _ACT_TORCH:
            raise UnsupportedOperation(f"unknown activation {name!r}")
        return _ACT_TORCH[name]

    def act(self, x, name):
        if x.is_cuda and x.dtype == torch.bfloat16 and name in ("gelu", "silu", "relu", "relu2", "quick_gelu",
                                                                 "gelu_tanh", "gelu_new", "gelu_pytorch_tanh",
                                                                 "sigmoid", "tanh", "softplus"):
            return _CUDA_OPS._k().eltwise(x, name)
        xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
        return _ACT_TORCH[name](xf).to(x.dtype)


ops_fn = _OpsFn()

OPS_FN_REFERENCE_NAMES = (
    "matmul", "add", "zeros", "randn", "layer_norm", "embedding", "silu", "mul", "attention", "gelu", "exp",
    "normalize", "concat", "rms_norm", "scale", "transpose", "transpose_dims", "sigmoid", "topk", "conv1d", "tanh",
    "sub", "clamp", "gather", "scatter", "softmax", "causal_mask", "sliding_window_mask",
    "causal_sliding_window_mask", "flash_attention", "fused_swiglu", "fused_residual_rms_norm",
)
