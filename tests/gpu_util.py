"""Helpers for GPU kernel tests: random paged caches and fp32 reference attention."""
import math

import torch


def make_paged_cache(num_seqs, seq_lens, Hkv, D, block_size=16, extra_blocks=7, device="cuda", seed=0):
    """Random K/V in a paged cache with a shuffled block table.  Returns dense copies for reference."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    max_len = max(seq_lens)
    max_blocks = (max_len + block_size - 1) // block_size
    total_blocks = sum((l + block_size - 1) // block_size for l in seq_lens) + extra_blocks
    perm = torch.randperm(total_blocks, generator=g)
    k_cache = torch.zeros(total_blocks, Hkv, block_size, D, dtype=torch.bfloat16)
    v_cache = torch.zeros_like(k_cache)
    bt = torch.zeros(num_seqs, max_blocks, dtype=torch.int32)
    dense_k, dense_v = [], []
    nxt = 0
    for s, l in enumerate(seq_lens):
        k = (torch.randn(l, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
        v = (torch.randn(l, Hkv, D, generator=g) * 0.5).to(torch.bfloat16)
        dense_k.append(k)
        dense_v.append(v)
        nb = (l + block_size - 1) // block_size
        for b in range(nb):
            blk = int(perm[nxt]); nxt += 1
            bt[s, b] = blk
            n = min(block_size, l - b * block_size)
            k_cache[blk, :, :n] = k[b * block_size:b * block_size + n].transpose(0, 1)
            v_cache[blk, :, :n] = v[b * block_size:b * block_size + n].transpose(0, 1)
    return (k_cache.to(device), v_cache.to(device), bt.to(device),
            torch.tensor(seq_lens, dtype=torch.int32, device=device), dense_k, dense_v)


def ref_attention(q, k, v, *, causal_offset=None, window=0, alibi=None, scale=None, kv_start=0):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] (cpu, any dtype) -> (out fp32 [Tq, Hq, D], lse [Tq, Hq]).
    Query i sits at kv position causal_offset + i (None = bidirectional)."""
    q, k, v = q.float(), k.float(), v.float()
    Tq, Hq, D = q.shape
    Tk, Hkv, _ = k.shape
    G = Hq // Hkv
    k = k.repeat_interleave(G, dim=1)
    v = v.repeat_interleave(G, dim=1)
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    s = torch.einsum("qhd,khd->hqk", q, k) * scale
    kpos = torch.arange(Tk)[None, :]
    qpos = (torch.arange(Tq)[:, None] + (causal_offset if causal_offset is not None else Tk - Tq))
    mask = torch.ones(Tq, Tk, dtype=torch.bool)
    if causal_offset is not None:
        mask &= kpos <= qpos
    if window > 0:
        mask &= kpos > qpos - window
    mask &= kpos >= kv_start
    if alibi is not None:
        s = s + alibi.float()[:, None, None] * (kpos - qpos)[None].float()
    s = s.masked_fill(~mask[None], float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    out = torch.einsum("hqk,khd->qhd", p, v)
    return out, lse.transpose(0, 1)
