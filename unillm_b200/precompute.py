"""Precomputed position tables: RoPE cos/sin, causal masks, sliding-window masks.

Parity with ``crates/runtime/src/precompute.rs``: ``RoPECache(head_dim, max_seq, base)`` holds cos/sin
``[max_seq, head_dim/2]`` with ``get(len)`` / ``get_range(start, end)`` (``:29-147``);
``CausalMaskCache`` holds an additive 0 / -inf mask with ``get`` and ``get_broadcast -> [1, 1, L, L]``
(``:153-218``); ``SlidingWindowMaskCache(window)`` (``:224-289``).  The reference never uses these from
its models; here the CPU oracle decoder does, and the device kernels compute the same quantities on
the fly (``csrc/norm_rope/rope_kv_append.cu``), so the tables double as their test oracle.
RoPE scaling variants: ``linear`` (positions divided by a factor, CodeLlama) and ``llama3``.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def rope_inv_freq(rotary_dim: int, base: float, llama3: Optional[Tuple[float, float, float, float]] = None) -> torch.Tensor:
    inv = base ** (-torch.arange(0, rotary_dim // 2, dtype=torch.float64) * 2.0 / rotary_dim)
    if llama3 is not None:
        factor, low, high, orig = llama3
        wavelen = 2 * math.pi / inv
        low_wl, high_wl = orig / low, orig / high
        smooth = (orig / wavelen - low) / (high - low)
        mid = (1 - smooth) * inv / factor + smooth * inv
        inv = torch.where(wavelen > low_wl, inv / factor, torch.where(wavelen >= high_wl, mid, inv))
    return inv.float()


class RoPECache:
    def __init__(self, head_dim: int, max_seq_len: int = 2048, base: float = 10000.0, *, rotary_dim: Optional[int] = None,
                 position_scale: float = 1.0, llama3: Optional[Tuple[float, float, float, float]] = None,
                 device="cpu"):
        self.head_dim, self.max_seq_len, self.base = head_dim, max_seq_len, base
        self.rotary_dim = rotary_dim if rotary_dim is not None else head_dim
        inv = rope_inv_freq(self.rotary_dim, base, llama3).to(device)
        pos = torch.arange(max_seq_len, dtype=torch.float32, device=device) * position_scale
        ang = pos[:, None] * inv[None, :]
        self.cos, self.sin = ang.cos(), ang.sin()

    def get(self, seq_len: int):
        return self.cos[:seq_len], self.sin[:seq_len]

    def get_range(self, start: int, end: int):
        return self.cos[start:end], self.sin[start:end]

    def at(self, positions: torch.Tensor):
        return self.cos[positions.long()], self.sin[positions.long()]


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: Optional[int] = None,
               interleaved: bool = False) -> torch.Tensor:
    """x ``[..., T, H, D]``; cos/sin ``[T, rd/2]``.  Half-split pairs ``(i, i + rd/2)`` like the reference
    (``simd/arch/scalar.rs:112-153``) or adjacent pairs when ``interleaved``."""
    rd = rotary_dim if rotary_dim is not None else x.shape[-1]
    half = rd // 2
    xf = x.float()
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    out = xf.clone()
    if interleaved:
        x0, x1 = xf[..., 0:rd:2], xf[..., 1:rd:2]
        out[..., 0:rd:2] = x0 * c - x1 * s
        out[..., 1:rd:2] = x1 * c + x0 * s
    else:
        x0, x1 = xf[..., :half], xf[..., half:rd]
        out[..., :half] = x0 * c - x1 * s
        out[..., half:rd] = x1 * c + x0 * s
    return out.to(x.dtype)


class CausalMaskCache:
    def __init__(self, max_seq_len: int = 2048, device="cpu"):
        self.max_seq_len = max_seq_len
        m = torch.full((max_seq_len, max_seq_len), float("-inf"), device=device)
        self.mask = torch.triu(m, diagonal=1)

    def get(self, seq_len: int) -> torch.Tensor:
        return self.mask[:seq_len, :seq_len]

    def get_broadcast(self, seq_len: int) -> torch.Tensor:
        return self.get(seq_len)[None, None]


class SlidingWindowMaskCache:
    def __init__(self, window: int, max_seq_len: int = 2048, device="cpu"):
        self.window, self.max_seq_len = window, max_seq_len
        i = torch.arange(max_seq_len, device=device)
        d = i[:, None] - i[None, :]
        vis = (d >= 0) & (d < window)
        self.mask = torch.where(vis, 0.0, float("-inf"))

    def get(self, seq_len: int) -> torch.Tensor:
        return self.mask[:seq_len, :seq_len]

    def get_broadcast(self, seq_len: int) -> torch.Tensor:
        return self.get(seq_len)[None, None]


def alibi_slopes(num_heads: int) -> torch.Tensor:
    """Standard ALiBi head slopes (``models_v2/bloom.rs:226-252``, ``baichuan.rs:427-459``)."""
    def pow2(n):
        start = 2.0 ** (-(2.0 ** -(math.log2(n) - 3)))
        return [start * (start ** i) for i in range(n)]

    if math.log2(num_heads).is_integer():
        s = pow2(num_heads)
    else:
        c = 2 ** math.floor(math.log2(num_heads))
        s = pow2(c) + pow2(2 * c)[0::2][: num_heads - c]
    return torch.tensor(s, dtype=torch.float32)
