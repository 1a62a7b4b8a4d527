"""Host-side samplers and sampling parameters.

``Sampler`` offers the reference's ``sample_greedy / sample_temperature / sample_top_p / softmax``
(``crates/runtime/src/inference.rs:15-156``) plus top-k and the repetition penalty that the reference
declares in ``GenerationConfig`` but never reads.  Random draws come from Philox4x32-10 keyed by
``(seed, step, row)`` -- the same generator as the device sampler (``csrc/sample/sample.cu``), so a
host run and a device run with the same seed make the same choices (up to floating-point ties).
``GreedySampler`` mirrors ``crates/runtime/src/sampler.rs:7-68``.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from .config import GenerationConfig

_M32 = 0xFFFFFFFF


def philox_uniform(seed: int, step: int, row: int) -> float:
    """First output word of Philox4x32-10 with counter (step_lo, step_hi, row, 0), mapped to [0, 1)."""
    c = [step & _M32, (step >> 32) & _M32, row & _M32, 0]
    k = [seed & _M32, (seed >> 32) & _M32]
    for _ in range(10):
        p0 = 0xD2511F53 * c[0]
        p1 = 0xCD9E8D57 * c[2]
        hi0, lo0 = (p0 >> 32) & _M32, p0 & _M32
        hi1, lo1 = (p1 >> 32) & _M32, p1 & _M32
        c = [hi1 ^ c[1] ^ k[0], lo1, hi0 ^ c[3] ^ k[1], lo0]
        k = [(k[0] + 0x9E3779B9) & _M32, (k[1] + 0xBB67AE85) & _M32]
    return (c[0] >> 8) * (1.0 / 16777216.0)


@dataclass
class SamplingParams:
    """Per-request sampling settings (``crates/inference/src/types.rs:57-78``)."""

    temperature: float = 1.0
    top_p: float = 1.0
    top_k: Optional[int] = None
    max_tokens: int = 100
    stop_sequences: List[str] = field(default_factory=list)
    stop_token_ids: List[int] = field(default_factory=list)
    seed: Optional[int] = None
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    ignore_eos: bool = False

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0

    @staticmethod
    def from_generation_config(g: GenerationConfig) -> "SamplingParams":
        t = g.temperature if g.do_sample else 0.0
        return SamplingParams(temperature=t, top_p=g.top_p, top_k=g.top_k, max_tokens=g.max_new_tokens,
                              stop_sequences=list(g.stop_sequences), seed=g.seed,
                              repetition_penalty=g.repetition_penalty)


class Sampler:
    def __init__(self, seed: Optional[int] = None):
        self.seed = 0 if seed is None else int(seed)
        self.step = 0

    # ---- reference API ----
    @staticmethod
    def softmax(logits: torch.Tensor) -> torch.Tensor:
        return torch.softmax(logits.float(), dim=-1)

    @staticmethod
    def sample_greedy(logits: torch.Tensor) -> int:
        return int(torch.argmax(logits.float()).item())

    def sample_temperature(self, logits: torch.Tensor, temperature: float) -> int:
        if temperature <= 0:
            return self.sample_greedy(logits)
        p = self.softmax(logits / temperature)
        return self._draw(p)

    def sample_top_p(self, logits: torch.Tensor, top_p: float, temperature: float = 1.0) -> int:
        """Sort descending, keep the smallest prefix whose mass reaches ``top_p``, renormalise, draw."""
        if temperature <= 0:
            return self.sample_greedy(logits)
        p = self.softmax(logits / temperature)
        sp, si = torch.sort(p, descending=True, stable=True)
        cum = torch.cumsum(sp, 0)
        cut = int(torch.searchsorted(cum, torch.tensor(top_p * float(cum[-1]))).item()) + 1
        cut = max(1, min(cut, p.numel()))
        kept = sp[:cut] / sp[:cut].sum()
        return int(si[self._draw(kept)].item())

    def sample_top_k(self, logits: torch.Tensor, k: int, temperature: float = 1.0) -> int:
        if temperature <= 0:
            return self.sample_greedy(logits)
        v, i = torch.topk(logits.float(), min(k, logits.numel()))
        return int(i[self._draw(self.softmax(v / temperature))].item())

    # ---- combined entry point ----
    def sample(self, logits: torch.Tensor, cfg, history: Optional[Sequence[int]] = None) -> int:
        """``cfg`` is a ``GenerationConfig`` or ``SamplingParams``."""
        sp = cfg if isinstance(cfg, SamplingParams) else SamplingParams.from_generation_config(cfg)
        x = logits.float().clone()
        if sp.repetition_penalty != 1.0 and history:
            idx = torch.tensor(sorted(set(int(t) for t in history if 0 <= int(t) < x.numel())), dtype=torch.long)
            if idx.numel():
                v = x[idx]
                x[idx] = torch.where(v > 0, v / sp.repetition_penalty, v * sp.repetition_penalty)
        if (sp.presence_penalty or sp.frequency_penalty) and history:
            counts = torch.bincount(torch.tensor([t for t in history if 0 <= t < x.numel()], dtype=torch.long),
                                    minlength=x.numel()).float()
            x = x - sp.frequency_penalty * counts - sp.presence_penalty * (counts > 0).float()
        if sp.greedy:
            return self.sample_greedy(x)
        x = x / sp.temperature
        k = sp.top_k if sp.top_k and sp.top_k > 0 else 0
        if k == 0 and sp.top_p < 1.0:
            k = min(1024, x.numel())
        if k:
            v, i = torch.topk(x, min(k, x.numel()))
            order = torch.argsort(-v, stable=True)
            v, i = v[order], i[order]
            p = torch.softmax(v, 0)
            if sp.top_p < 1.0:
                cum = torch.cumsum(p, 0)
                cut = int((cum >= sp.top_p * float(cum[-1])).nonzero()[0].item()) + 1
                p, i = p[:cut] / p[:cut].sum(), i[:cut]
            return int(i[self._draw(p)].item())
        return self._draw(torch.softmax(x, 0))

    def _draw(self, probs: torch.Tensor) -> int:
        u = philox_uniform(self.seed, self.step, 0)
        self.step += 1
        cum = torch.cumsum(probs.double(), 0)
        target = u * float(cum[-1])
        idx = int(torch.searchsorted(cum, torch.tensor(target, dtype=torch.float64), right=True).item())
        return min(idx, probs.numel() - 1)


class GreedySampler:
    """Argmax over the last dimension (``crates/runtime/src/sampler.rs:22-67``)."""

    def sample(self, logits: torch.Tensor) -> int:
        return int(torch.argmax(logits.reshape(-1, logits.shape[-1])[-1].float()).item())

    def sample_batch(self, logits: torch.Tensor) -> List[int]:
        x = logits if logits.dim() == 2 else logits[:, -1, :]
        return torch.argmax(x.float(), dim=-1).tolist()
