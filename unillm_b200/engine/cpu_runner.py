"""``CpuModelRunner``: the engine's step interface (``StepBatch`` in, sampled ids out) on the CPU in
fp32 over a paged KV cache.  It shares parameters and per-layer math with ``DecoderModel`` (the
oracle), so an engine run on this backend is the token-exact reference for the GPU runner, and it is
the backend of the CPU benchmark configuration (TinyLlama architecture, paged KV with block size 16).
Works on any torch device; every op is a plain torch op.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..models.decoder import DecoderModel
from ..precompute import RoPECache, alibi_slopes, apply_rope
from ..sampling import Sampler, SamplingParams
from ..tensor_core import ops_fn
from .runner import StepBatch


class CpuModelRunner:
    def __init__(self, model: DecoderModel, *, num_blocks: int, block_size: int = 16, max_model_len: int = 8192):
        self.model, self.spec = model, model.spec
        s = self.spec
        self.block_size, self.num_blocks, self.max_model_len = block_size, num_blocks, max_model_len
        dev, dt = model.device, model.dtype
        self.k_cache = [torch.zeros(num_blocks, s.num_kv_heads, block_size, s.head_dim, dtype=dt, device=dev)
                        for _ in range(s.num_layers)]
        self.v_cache = [torch.zeros_like(k) for k in self.k_cache]
        self._rope: Optional[RoPECache] = None
        self._alibi = alibi_slopes(s.num_heads).to(dev) if s.pos == "alibi" else None
        self.launches = 0
        self.h2d_bytes = self.d2h_bytes = 0
        self._sampler = Sampler()

    def _rope_at(self, positions: torch.Tensor):
        s = self.spec
        need = int(positions.max()) + 1
        if self._rope is None or self._rope.max_seq_len < need:
            self._rope = RoPECache(s.head_dim, max(need, 4096), s.rope_theta, rotary_dim=s.rd,
                                   position_scale=s.rope_pos_scale, llama3=s.rope_llama3, device=self.model.device)
        return self._rope.at(positions)

    def _attention(self, i: int, h: torch.Tensor, b: StepBatch, pos: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
        s, m = self.spec, self.model
        L = f"layers.{i}."
        T = h.shape[0]
        qkv = ops_fn.linear(h, m.p[L + "wqkv"], m.p.get(L + "bqkv"))
        q, k, v = qkv.split([s.q_size, s.kv_size, s.kv_size], dim=-1)
        q = q.reshape(T, s.num_heads, s.head_dim)
        k = k.reshape(T, s.num_kv_heads, s.head_dim)
        v = v.reshape(T, s.num_kv_heads, s.head_dim)
        if s.qk_norm:
            q = ops_fn.rms_norm(q, m.p[L + "q_norm"], s.norm_eps)
            k = ops_fn.rms_norm(k, m.p[L + "k_norm"], s.norm_eps)
        if s.pos == "rope" and s.rd > 0:
            cos, sin = self._rope_at(pos)
            q = apply_rope(q, cos, sin, s.rd, s.rope_interleaved)
            k = apply_rope(k, cos, sin, s.rd, s.rope_interleaved)
        ok = slots >= 0
        blk, off = slots[ok] // self.block_size, slots[ok] % self.block_size
        self.k_cache[i][blk, :, off] = k[ok]
        self.v_cache[i][blk, :, off] = v[ok]
        out = torch.empty(T, s.num_heads, s.head_dim, dtype=h.dtype, device=h.device)
        scale = s.attn_scale if s.attn_scale is not None else 1.0 / math.sqrt(s.head_dim)
        g = s.num_heads // s.num_kv_heads
        row = 0
        q_lens = [1] * b.num_decode + list(b.prefill_q_lens)
        for si, ql in enumerate(q_lens):
            kv_len = b.seq_lens[si]
            bt = torch.as_tensor(b.block_tables[si][: (kv_len + self.block_size - 1) // self.block_size],
                                 device=h.device, dtype=torch.long)
            kk = self.k_cache[i][bt].permute(1, 0, 2, 3).reshape(s.num_kv_heads, -1, s.head_dim)[:, :kv_len]
            vv = self.v_cache[i][bt].permute(1, 0, 2, 3).reshape(s.num_kv_heads, -1, s.head_dim)[:, :kv_len]
            if g > 1:
                kk, vv = kk.repeat_interleave(g, 0), vv.repeat_interleave(g, 0)
            qq = q[row:row + ql].transpose(0, 1).float()              # [H, ql, D]
            qpos = torch.arange(kv_len - ql, kv_len, device=h.device)[:, None]
            kpos = torch.arange(kv_len, device=h.device)[None, :]
            vis = kpos <= qpos
            if s.window > 0:
                vis = vis & (kpos > qpos - s.window)
            bias = torch.zeros(ql, kv_len, device=h.device).masked_fill(~vis, float("-inf"))
            if self._alibi is not None:
                bias = bias[None] + self._alibi[:, None, None] * (kpos - qpos)[None].float()
            y = F.scaled_dot_product_attention(qq[None], kk.float()[None], vv.float()[None],
                                               attn_mask=bias if bias.dim() == 2 else bias[None], scale=scale)[0]
            out[row:row + ql] = y.transpose(0, 1).to(h.dtype)
            row += ql
        return ops_fn.linear(out.reshape(T, s.q_size), m.p[L + "wo"], m.p.get(L + "bo"))

    @torch.no_grad()
    def forward_logits(self, b: StepBatch) -> torch.Tensor:
        s, m = self.spec, self.model
        dev = m.device
        ids = torch.as_tensor(b.token_ids, dtype=torch.long, device=dev)
        pos = torch.as_tensor(b.positions, dtype=torch.long, device=dev)
        slots = torch.as_tensor(b.slot_mapping, dtype=torch.long, device=dev)
        x = m.p["embed"][ids]
        if s.embed_proj_dim:
            x = ops_fn.linear(x, m.p["project_in"])
        if s.embed_scale != 1.0:
            x = (x.float() * s.embed_scale).to(x.dtype)
        if s.pos == "learned":
            x = x + m.p["pos_embed"][pos + s.learned_pos_offset]
        if s.embed_norm:
            x = ops_fn.layer_norm(x, m.p["embed_norm.w"], m.p["embed_norm.b"], s.norm_eps)
        rs = s.residual_scale
        for i in range(s.num_layers):
            L = f"layers.{i}."
            if s.post_ln:
                x = m._norm(x + self._attention(i, x, b, pos, slots) * rs, L + "ln1")
                x = m._norm(x + m._mlp(i, x[None])[0] * rs, L + "ln2")
                continue
            h = m._norm(x, L + "ln1")
            a = self._attention(i, h, b, pos, slots)
            if s.parallel_residual:
                m_in = h if s.parallel_shared_norm else m._norm(x, L + "ln2")
                x = x + (a + m._mlp(i, m_in[None])[0]) * rs
            else:
                x = x + a * rs
                x = x + m._mlp(i, m._norm(x, L + "ln2")[None])[0] * rs
        rows = torch.as_tensor(b.sample_rows, dtype=torch.long, device=dev)
        xs = x[rows]
        if s.final_norm:
            xs = m._norm(xs, "final_norm", layer_level=False)
        return m.lm_logits(xs)

    def execute(self, b: StepBatch) -> List[int]:
        if not b.sample_rows:
            self.forward_logits(b)
            return []
        logits = self.forward_logits(b).float().cpu()
        out = []
        for r in range(logits.shape[0]):
            t = b.temperature[r] if b.temperature is not None else 0.0
            if t <= 0:
                out.append(int(torch.argmax(logits[r])))
            else:
                sp = SamplingParams(temperature=t, top_p=b.top_p[r] if b.top_p else 1.0,
                                    top_k=b.top_k[r] if b.top_k else None)
                smp = Sampler(seed=b.seed)
                smp.step = b.step
                # row index enters the Philox counter like on the device
                from ..sampling import philox_uniform
                smp._draw = (lambda probs, _r=r, _s=smp: _draw_row(probs, b.seed, b.step, _r))
                out.append(smp.sample(logits[r], sp))
        return out

    def launch(self, b: StepBatch) -> int:
        if b.token_src is not None:
            # input tokens that the previous step sampled and the engine has not read yet
            prev = self._pending
            for r, k in enumerate(b.token_src):
                if k >= 0:
                    b.token_ids[r] = prev[k]
        self._pending = self.execute(b)
        return len(self._pending)

    def pending(self):
        return self._pending

    def fetch(self, handle=None) -> List[int]:
        return self._pending if handle is None else handle


def _draw_row(probs: torch.Tensor, seed: int, step: int, row: int) -> int:
    from ..sampling import philox_uniform

    u = philox_uniform(seed, step, row)
    cum = torch.cumsum(probs.double(), 0)
    idx = int(torch.searchsorted(cum, torch.tensor(u * float(cum[-1]), dtype=torch.float64), right=True))
    return min(idx, probs.numel() - 1)


class TpCpuModelRunner(CpuModelRunner):
    """The CPU runner, tensor parallel over a ``torch.distributed`` (gloo) group: attention heads, KV heads, the MLP
    width and the vocabulary are divided over the ranks exactly as ``RunnerWeights`` divides them for the GPU runner,
    the row-parallel outputs (attention output projection, MLP down projection) are summed with ``all_reduce`` and the
    vocabulary shards' logits are gathered.  It exists for the host-side tests of the distributed engine (sharding
    math, failure detection, recovery at a smaller tensor-parallel size): every rank runs the same ``LLMEngine`` on the
    same request stream, like the GPU ranks do.  Dense decoder models with a sequential or parallel residual."""

    def __init__(self, model: DecoderModel, rank: int, world: int, group=None, *, num_blocks: int, block_size: int = 16,
                 max_model_len: int = 8192):
        import copy
        import dataclasses

        from .runner import RunnerWeights

        s = model.spec
        if s.moe is not None or s.embed_proj_dim:
            raise ValueError("TpCpuModelRunner covers dense decoder models")
        self.rank, self.world, self.group = rank, world, group
        w = RunnerWeights(s, model.p, "cpu", rank, world)
        shard = copy.copy(model)
        shard.spec = dataclasses.replace(s, num_heads=w.hq, num_kv_heads=w.hkv, tie_embeddings=False)
        shard.p = {k: v.to(model.dtype) for k, v in w.t.items()}
        shard._rope = shard._alibi = None
        inner_mlp = shard._mlp

        def mlp(i, x):
            return self._sum(inner_mlp(i, x))

        def lm_logits(x):
            y = ops_fn.linear(x, shard.p["lm_head"], shard.p.get("lm_head_bias"))
            if s.logit_scale != 1.0:
                y = (y.float() * s.logit_scale).to(y.dtype)
            return self._gather_cols(y)

        shard._mlp, shard.lm_logits = mlp, lm_logits
        super().__init__(shard, num_blocks=num_blocks, block_size=block_size, max_model_len=max_model_len)
        if s.pos == "alibi":
            self._alibi = alibi_slopes(s.num_heads)[rank * w.hq:(rank + 1) * w.hq].to(model.device)

    def _sum(self, y: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            import torch.distributed as dist

            y = y.contiguous()
            dist.all_reduce(y, group=self.group)
        return y

    def _gather_cols(self, y: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return y
        import torch.distributed as dist

        parts = [torch.empty_like(y) for _ in range(self.world)]
        dist.all_gather(parts, y.contiguous(), group=self.group)
        return torch.cat(parts, dim=-1)

    def _attention(self, i, h, b, pos, slots):
        return self._sum(super()._attention(i, h, b, pos, slots))
