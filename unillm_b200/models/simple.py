"""Base class and building blocks for the architectures that are not plain decoder stacks (state-space, RWKV,
Griffin, encoders, encoder-decoders, vision, audio).

Parameters live in ``self.p`` under their on-disk (HF / GGUF-mapped) names, so loading and exporting are the
identity; ``param_shapes`` is the single source of truth for names and shapes.  All tensor math goes through
``ops_fn`` (CPU fp32 oracle or the CUDA kernels, picked from the tensor) and ``ops.recurrent``.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from ..model_core import Model, ModelWeights
from ..tensor_core import ops_fn
from ..types import LoadingError


def _f(x: torch.Tensor) -> torch.Tensor:
    return x if x.dtype == torch.float32 else x.float()


class ParamModel(Model):
    #: strict loading raises on a missing tensor; skeleton families of the reference load what is there
    strict = True

    def param_shapes(self) -> Dict[str, tuple]:  # pragma: no cover - abstract
        raise NotImplementedError

    @staticmethod
    def is_norm_scale(name: str, shape: tuple) -> bool:
        """1-D ``<module>.weight`` of a normalisation module (named *norm* / *ln*): starts at one."""
        if len(shape) != 1 or not name.endswith(".weight"):
            return False
        mod = name[:-len(".weight")].rsplit(".", 1)[-1].lower()
        return "norm" in mod or mod.startswith("ln") or mod in ("gamma",)

    def special_init(self, name: str, shape: tuple, g: torch.Generator) -> Optional[torch.Tensor]:
        """Hook for parameters whose random init is not N(0, std) (decays, A_log, ...)."""
        return None

    def _init_params(self, init="zeros", seed=0, dtype=torch.float32, device=torch.device("cpu")):
        g = torch.Generator(device="cpu").manual_seed(seed)
        std = getattr(self._config, "initializer_range", 0.02)
        self.p: Dict[str, torch.Tensor] = {}
        for name, shape in self.param_shapes().items():
            if init == "zeros":
                t = torch.zeros(shape)
            else:
                t = self.special_init(name, shape, g)
                if t is None:
                    if self.is_norm_scale(name, shape):
                        t = torch.ones(shape)
                    elif name.endswith(".bias"):
                        t = torch.zeros(shape)
                    else:
                        t = torch.randn(shape, generator=g) * std
            self.p[name] = t.to(dtype).to(device)
        self.device, self.dtype = device, dtype

    def _load(self, weights: ModelWeights, dtype=None, device=None):
        dtype = dtype or torch.float32
        dev = torch.device(device) if device is not None else torch.device("cpu")
        self.p = {}
        for name, shape in self.param_shapes().items():
            t = None
            for alias in self.aliases(name):
                t = weights.get(alias)
                if t is None:
                    q = weights.get_quantized(alias)
                    t = q.dequantize() if q is not None else None
                if t is not None:
                    break
            if t is None:
                if self.strict:
                    raise LoadingError(f"{type(self).__name__}: missing tensor {name}")
                t = torch.zeros(shape)
            if tuple(t.shape) != tuple(shape):
                if t.numel() == math.prod(shape):
                    t = t.reshape(shape)
                else:
                    raise LoadingError(f"{type(self).__name__}: {name} has shape {tuple(t.shape)}, expected {tuple(shape)}")
            self.p[name] = t.to(dtype).to(dev)
        self.device, self.dtype = dev, dtype

    def aliases(self, name: str):
        """On-disk spellings tried in order for parameter ``name``."""
        return (name,)

    def export_hf(self) -> ModelWeights:
        return ModelWeights({k: v.detach().clone() for k, v in self.p.items()})

    def parameters(self) -> Dict[str, torch.Tensor]:
        return dict(self.p)

    def _move(self, dev, dtype):
        self.p = {k: v.to(device=dev, dtype=dtype or v.dtype) for k, v in self.p.items()}

    # ---- small helpers over self.p ----
    def lin(self, x: torch.Tensor, name: str, act: Optional[str] = None) -> torch.Tensor:
        return ops_fn.linear(x, self.p[name + ".weight"], self.p.get(name + ".bias"), act=act)

    def ln(self, x: torch.Tensor, name: str, eps: float = 1e-5) -> torch.Tensor:
        return ops_fn.layer_norm(x, self.p[name + ".weight"], self.p.get(name + ".bias"), eps)

    def rms(self, x: torch.Tensor, name: str, eps: float = 1e-6, offset_one: bool = False) -> torch.Tensor:
        w = self.p[name + ".weight"]
        return ops_fn.rms_norm(x, (w.float() + 1.0).to(w.dtype) if offset_one else w, eps)


def mha(x_q: torch.Tensor, x_kv: torch.Tensor, wq, bq, wk, bk, wv, bv, wo, bo, num_heads: int, *, causal: bool = False,
        num_kv_heads: Optional[int] = None, bias: Optional[torch.Tensor] = None, scale: Optional[float] = None,
        cache: Optional[dict] = None, rope=None, window: int = 0, head_dim: Optional[int] = None) -> torch.Tensor:
    """Multi-head attention over [B, T, H] inputs.  ``cache`` (dict with optional 'k', 'v') makes it incremental;
    ``bias`` is an additive [1|B, heads, Tq, Tk] term (T5 relative positions); ``rope`` = (cos, sin) tables
    [max_pos, rot/2] applied at absolute positions."""
    B, Tq, _ = x_q.shape
    nkv = num_kv_heads or num_heads
    q = ops_fn.linear(x_q, wq, bq)
    k = ops_fn.linear(x_kv, wk, bk)
    v = ops_fn.linear(x_kv, wv, bv)
    D = head_dim or q.shape[-1] // num_heads
    q = q.view(B, Tq, num_heads, D).transpose(1, 2)
    k = k.view(B, -1, nkv, D).transpose(1, 2)
    v = v.view(B, -1, nkv, D).transpose(1, 2)
    past = 0
    if cache is not None and cache.get("k") is not None:
        past = cache["k"].shape[2]
    if rope is not None:
        cos, sin = rope
        q = apply_rope(q, cos, sin, past)
        k = apply_rope(k, cos, sin, past)
    if cache is not None:
        if cache.get("k") is not None:
            k = torch.cat([cache["k"], k], 2)
            v = torch.cat([cache["v"], v], 2)
        cache["k"], cache["v"] = k, v
    if (q.is_cuda and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and D in (64, 128) and bias is None
            and not window and num_heads % nkv == 0):
        # bf16 on the GPU: the paged attention kernels of the serving engine on dense pages (tcgen05 for head size
        # 128, warp MMA for 64), grouped heads indexed in the kernel instead of being copied
        from ..ops import cuda_ops as K

        o = K.dense_attention(q, k, v, causal=bool(causal), scale=scale if scale is not None else D ** -0.5)
        o = o.transpose(1, 2).reshape(B, Tq, num_heads * D)
        return ops_fn.linear(o, wo, bo)
    if nkv != num_heads:
        k = k.repeat_interleave(num_heads // nkv, 1)
        v = v.repeat_interleave(num_heads // nkv, 1)
    Tk = k.shape[2]
    s = torch.matmul(_f(q), _f(k).transpose(-1, -2)) * (scale if scale is not None else D ** -0.5)
    if bias is not None:
        s = s + _f(bias)
    if causal or window:
        qi = torch.arange(Tk - Tq, Tk, device=s.device)[:, None]
        ki = torch.arange(Tk, device=s.device)[None, :]
        m = ki > qi if causal else torch.zeros(Tq, Tk, dtype=torch.bool, device=s.device)
        if window:
            m = m | (ki <= qi - window)
        s = s.masked_fill(m, float("-inf"))
    o = torch.matmul(torch.softmax(s, -1), _f(v)).to(x_q.dtype)
    o = o.transpose(1, 2).reshape(B, Tq, num_heads * D)
    return ops_fn.linear(o, wo, bo)


def rope_tables(max_pos: int, rot_dim: int, theta: float = 10000.0, device="cpu"):
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None]
    return ang.cos(), ang.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, offset: int = 0) -> torch.Tensor:
    """Half-split rotation of the first ``2*cos.shape[1]`` features of ``x`` [B, heads, T, D]."""
    T = x.shape[2]
    r = cos.shape[1] * 2
    c, s = cos[offset:offset + T].to(x.device)[None, None], sin[offset:offset + T].to(x.device)[None, None]
    xr, rest = _f(x[..., :r]), x[..., r:]
    a, b = xr[..., :r // 2], xr[..., r // 2:]
    out = torch.cat([a * c - b * s, b * c + a * s], -1).to(x.dtype)
    return torch.cat([out, rest], -1) if rest.shape[-1] else out


_IMPLICIT_CONV = {"ok": True}
_CONV_FILTERS: dict = {}


def _filter_matrix(w: torch.Tensor) -> torch.Tensor:
    """``w [O, C, k]`` as the GEMM operand ``[O, k * C]`` whose columns run tap-major (tap j, channel c), cached per
    weight tensor."""
    key = (w.data_ptr(), tuple(w.shape), w.dtype, str(w.device))
    m = _CONV_FILTERS.get(key)
    if m is None:
        if len(_CONV_FILTERS) > 256:
            _CONV_FILTERS.clear()
        m = _CONV_FILTERS[key] = w.permute(0, 2, 1).reshape(w.shape[0], -1).to(torch.bfloat16).contiguous()
    return m


def conv1d(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, stride: int = 1, padding: int = 0,
           groups: int = 1, dilation: int = 1) -> torch.Tensor:
    """[B, C, L] convolution.

    bf16 CUDA inputs with ``groups == 1``, ``dilation == 1`` and a channel count that is a multiple of 8 run as an
    IMPLICIT GEMM on the tcgen05 kernel: the input is laid out once channel-last and zero-padded, and the window matrix
    ``[windows, k * C]`` is never built -- window t is the ``k * C`` consecutive elements that start at row ``t * stride``,
    so the matrix is an overlapping strided view (row stride ``stride * C``) that the GEMM's TMA descriptor walks
    directly.  Batch elements are padded to a whole number of windows; the few windows that straddle two batch elements
    are computed and dropped.  Grouped convolutions run one such GEMM per group; dilated convolutions still build the
    window matrix before the GEMM; everything else is an fp32 convolution (audio stems on CPU, single-channel
    waveforms, depthwise filters)."""
    if (x.is_cuda and x.dtype == torch.bfloat16 and groups > 1 and dilation == 1 and w.shape[1] % 8 == 0
            and x.shape[1] == groups * w.shape[1] and w.shape[0] % groups == 0 and _IMPLICIT_CONV["ok"]):
        # grouped (e.g. the positional convolution of wav2vec2 / HuBERT: 16 groups of 48 channels, 128 taps): one implicit
        # GEMM per group over that group's channels
        Og = w.shape[0] // groups
        outs = [conv1d(x[:, gi * w.shape[1]:(gi + 1) * w.shape[1]], w[gi * Og:(gi + 1) * Og],
                       None if b is None else b[gi * Og:(gi + 1) * Og], stride=stride, padding=padding)
                for gi in range(groups)]
        return torch.cat(outs, dim=1)
    if x.is_cuda and x.dtype == torch.bfloat16 and groups == 1 and (w.shape[1] * w.shape[2]) % 8 == 0:
        from ..ops import cuda_ops as K

        B, Cc, L = x.shape
        O, _, k = w.shape
        bias = None if b is None else b.to(torch.bfloat16)
        if dilation == 1 and Cc % 8 == 0 and _IMPLICIT_CONV["ok"]:
            Lp = L + 2 * padding
            Lo = (Lp - k) // stride + 1
            R = -(-Lp // stride)                                   # windows per batch element, the straddling ones included
            buf = x.new_zeros(B * R * stride + k, Cc)              # channel-last, padded; k spare rows behind the last window
            buf[:B * R * stride].view(B, R * stride, Cc)[:, padding:padding + L] = x.transpose(1, 2)
            win = buf.as_strided((B * R, k * Cc), (stride * Cc, 1))
            try:
                y = K.gemm_tn(win, _filter_matrix(w), bias=bias)
                return y.view(B, R, O)[:, :Lo].transpose(1, 2).contiguous()
            except RuntimeError:
                _IMPLICIT_CONV["ok"] = False                       # the descriptor was refused: window matrix from here on
        xp = F.pad(x, (padding, padding)) if padding else x
        span = dilation * (k - 1) + 1
        Lo = (xp.shape[-1] - span) // stride + 1
        idx = (torch.arange(Lo, device=x.device) * stride)[:, None] + (torch.arange(k, device=x.device) * dilation)[None]
        cols = xp[:, :, idx].permute(0, 2, 1, 3).reshape(B * Lo, Cc * k).contiguous()      # [B*Lo, C*k]
        y = K.linear(cols, w.reshape(O, Cc * k).to(torch.bfloat16).contiguous(), bias)
        return y.view(B, Lo, O).transpose(1, 2).contiguous()
    return F.conv1d(_f(x), _f(w), None if b is None else _f(b), stride=stride, padding=padding, groups=groups,
                    dilation=dilation).to(x.dtype)


def conv_transpose1d(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor] = None, stride: int = 1) -> torch.Tensor:
    """[B, C_in, L] transposed convolution with filters ``w [C_in, C_out, k]`` (torch layout), no padding:
    output length ``(L - 1) * stride + k``.  bf16 CUDA inputs run as one tensor-core GEMM -- every input frame times
    the filter matrix ``[C_out * k, C_in]`` gives that frame's ``k`` output taps for all channels -- followed by an
    overlap-add of the taps (``F.fold``); everything else is the fp32 torch operator."""
    Ci, Co, k = w.shape
    if x.is_cuda and x.dtype == torch.bfloat16 and Ci % 8 == 0:
        from ..ops import cuda_ops as K

        B, _, L = x.shape
        rows = x.transpose(1, 2).reshape(B * L, Ci).contiguous()                       # [B*L, C_in]
        wm = w.permute(1, 2, 0).reshape(Co * k, Ci).to(torch.bfloat16).contiguous()    # row (o, t) = w[:, o, t]
        taps = K.linear(rows, wm, None)                                                # [B*L, C_out*k]
        cols = taps.view(B, L, Co * k).transpose(1, 2).float()                         # [B, C_out*k, L]
        Lo = (L - 1) * stride + k
        y = F.fold(cols, output_size=(1, Lo), kernel_size=(1, k), stride=(1, stride)).view(B, Co, Lo)
        if b is not None:
            y = y + b.float()[None, :, None]
        return y.to(x.dtype)
    return F.conv_transpose1d(_f(x), _f(w), None if b is None else _f(b), stride=stride).to(x.dtype)
