"""``GpuModelRunner``: executes one engine step of a decoder model on one B200 with the hand-written
sm_100a kernels and a paged KV cache.

Per layer (tensor-parallel rank view):

    norm (K5)  ->  QKV GEMM (K1, tcgen05)  ->  RoPE + KV append (K6)  ->  paged attention (K3 prefill rows,
    K4 decode rows, optional cascade over a radix-shared prefix)  ->  o_proj GEMM with the residual add in
    its epilogue  ->  norm  ->  gate/up GEMM with SwiGLU in its epilogue (K2)  ->  down GEMM + residual

then final norm on the rows that are sampled, the (vocab-parallel) lm_head GEMM and the device sampler
(K8).  Token metadata for a step arrives as ONE packed int32 buffer copied from pinned host memory;
pure-decode steps are captured in CUDA graphs keyed by (padded batch, shared-prefix length).

Tensor parallelism (``TpContext``): column-parallel QKV / gate-up, row-parallel o / down, KV heads and
the vocabulary sharded.  With ``fused=True`` the two reductions per layer run inside the GEMM and norm
kernels over NVSwitch peer memory (GEMM epilogue pushes rows to the owning rank = reduce-scatter, the
norm kernel sums the partials, normalises its token shard and pushes it to every rank = all-gather,
and the next GEMM's TMA producer waits on the arrival counters); with ``fused=False`` the same math uses
NCCL all-reduce between library-style separate kernels -- the measured baseline.

Reference counterpart: the per-token loop of ``UniLLMBackend::generate`` / ``LlamaModelV2::forward_with_cache``
(``crates/runtime/src/benchmark/unillm_backend.rs:69-211``, ``models_v2/llama.rs:421-464, 654-680,
1027-1156``), which is batch-1, CPU-only and uses a contiguous cache.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch

from ..models.spec import DecoderSpec
from ..ops import cuda_ops as K
from ..precompute import alibi_slopes
from ..types import InvalidInput, UnsupportedOperation


class DeviceStepError(RuntimeError):
    """A kernel of a launched step recorded a problem in the device error word (a bounded wait that gave up, an
    out-of-range block-table entry or slot): the step's sampled ids are garbage and must not be used."""

    NAMES = {1: "mbarrier wait timed out", 2: "flag wait timed out (peer or producer missing)",
             3: "index out of range", 4: "bad argument"}

    def __init__(self, code: int, detail: int):
        super().__init__(f"device error {code} ({self.NAMES.get(code, '?')}), detail {detail}")
        self.code, self.detail = code, detail


@dataclass
class StepBatch:
    """Host-side description of one engine step (built by the scheduler).

    Token rows are ordered: first the ``num_decode`` decode sequences (one row each), then the prefill
    chunks.  ``seq_lens`` is the KV length of each sequence after this step's tokens are appended."""

    token_ids: List[int]
    positions: List[int]
    slot_mapping: List[int]
    num_decode: int
    seq_lens: List[int]
    block_tables: List[List[int]]
    prefill_q_lens: List[int] = field(default_factory=list)
    sample_rows: List[int] = field(default_factory=list)
    shared_prefix_len: int = 0          # tokens of KV that ALL decode sequences share (whole blocks)
    prefill_shares_prefix: bool = False  # the prefill chunks start at or after that prefix and share its blocks too
    # sampling (per sampled row); None = greedy
    temperature: Optional[List[float]] = None
    top_p: Optional[List[float]] = None
    top_k: Optional[List[int]] = None
    seed: int = 0
    step: int = 0
    # per decode row: index (in sample order) of the PREVIOUS step's output that is this row's input token, or -1
    # when ``token_ids`` already holds it.  Lets a step be launched before the host has read the previous
    # step's samples.
    token_src: Optional[List[int]] = None


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n]


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n]


class QWeight:
    """A projection weight kept block-quantised on the device (ggml block layout, rows independent): what the
    reference keeps as ``QMatMul`` for ``*_proj`` / ``lm_head`` tensors of a GGUF checkpoint
    (``crates/runtime/src/weight_loader_core.rs:554-584``, used at ``models_v2/llama.rs:1184-1195``)."""

    __slots__ = ("blocks", "qtype", "shape")

    def __init__(self, blocks: torch.Tensor, qtype: int, shape):
        self.blocks, self.qtype, self.shape = blocks, qtype, tuple(shape)

    def nbytes(self) -> int:
        return self.blocks.numel()


QUANT_NAMES = {"q4_0": 2, "q8_0": 8, "q4_k": 12}


class RunnerWeights:
    """Device weights of one rank in kernel layout (bf16, fused QKV / gate-up, TP-sharded)."""

    def __init__(self, spec: DecoderSpec, params: Dict[str, torch.Tensor], device, rank: int = 0, world: int = 1,
                 expert_parallel: bool = False):
        self.spec, self.rank, self.world = spec, rank, world
        s = spec
        self._set_ep(expert_parallel)
        if s.num_heads % world != 0:
            raise InvalidInput(f"{s.num_heads} heads not divisible by tensor parallel size {world}")
        self.hq = s.num_heads // world
        self.hkv, self.kv_lo = self.kv_layout(s.num_kv_heads, rank, world)
        D = s.head_dim

        def kv_rows(t):
            """Rows (or elements) of this rank's KV heads inside a [num_kv_heads * D, ...] tensor."""
            return t[self.kv_lo * D:(self.kv_lo + self.hkv) * D]

        def dev(t):
            return t.to(device=device, dtype=torch.bfloat16).contiguous()

        self.t: Dict[str, torch.Tensor] = {}
        p = params
        self.t["embed"] = dev(p["embed"])
        for n in ("pos_embed", "embed_norm.w", "embed_norm.b", "final_norm.w", "final_norm.b", "project_in", "project_out"):
            if n in p:
                self.t[n] = dev(p[n])
        lm = p["embed"] if s.tie_embeddings else p["lm_head"]
        if s.vocab_size % world != 0:
            raise InvalidInput(f"vocab {s.vocab_size} not divisible by tensor parallel size {world}")
        self.vocab_shard = s.vocab_size // world
        self.t["lm_head"] = dev(shard_rows(lm, rank, world)) if (world > 1 or not s.tie_embeddings) else self.t["embed"]
        if "lm_head_bias" in p:
            self.t["lm_head_bias"] = dev(shard_rows(p["lm_head_bias"], rank, world))
        for i in range(s.num_layers):
            L = f"layers.{i}."
            for n in ("ln1.w", "ln1.b", "ln2.w", "ln2.b", "q_norm", "k_norm"):
                if L + n in p:
                    self.t[L + n] = dev(p[L + n])
            wqkv = p[L + "wqkv"]
            q, k, v = wqkv.split([s.q_size, s.kv_size, s.kv_size], dim=0)
            self.t[L + "wqkv"] = dev(torch.cat([shard_rows(q, rank, world), kv_rows(k), kv_rows(v)], 0))
            if L + "bqkv" in p:
                qb, kb, vb = p[L + "bqkv"].split([s.q_size, s.kv_size, s.kv_size])
                self.t[L + "bqkv"] = dev(torch.cat([shard_rows(qb, rank, world), kv_rows(kb), kv_rows(vb)]))
            self.t[L + "wo"] = dev(shard_cols(p[L + "wo"], rank, world))
            if L + "bo" in p:
                self.t[L + "bo"] = dev(p[L + "bo"] if rank == 0 else torch.zeros_like(p[L + "bo"]))
            if L + "w_gate_up" in p:
                g, u = p[L + "w_gate_up"].chunk(2, 0)
                self.t[L + "w_gate_up"] = dev(torch.cat([shard_rows(g, rank, world), shard_rows(u, rank, world)], 0))
            if L + "w_up" in p:
                self.t[L + "w_up"] = dev(shard_rows(p[L + "w_up"], rank, world))
                if L + "b_up" in p:
                    self.t[L + "b_up"] = dev(shard_rows(p[L + "b_up"], rank, world))
            if L + "w_down" in p:
                self.t[L + "w_down"] = dev(shard_cols(p[L + "w_down"], rank, world))
                if L + "b_down" in p:
                    self.t[L + "b_down"] = dev(p[L + "b_down"] if rank == 0 else torch.zeros_like(p[L + "b_down"]))
            if L + "router" in p:
                # experts: tensor-parallel inside each expert here; expert-parallel layouts are built by MoeRunner
                self.t[L + "router"] = dev(p[L + "router"])
                gu = p[L + "experts_gate_up"]
                E = gu.shape[0]
                if self.ep:
                    # expert parallel: whole experts [expert_lo, expert_lo + experts_local) live here
                    lo, hi = self.expert_lo, self.expert_lo + self.experts_local
                    self.t[L + "experts_gate_up"] = dev(gu[lo:hi])
                    self.t[L + "experts_down"] = dev(p[L + "experts_down"][lo:hi])
                elif s.moe.gated:
                    g, u = gu.chunk(2, 1)
                    n = g.shape[1] // world
                    gu = torch.cat([g[:, rank * n:(rank + 1) * n], u[:, rank * n:(rank + 1) * n]], 1)
                else:
                    n = gu.shape[1] // world
                    gu = gu[:, rank * n:(rank + 1) * n]
                if not self.ep:
                    self.t[L + "experts_gate_up"] = dev(gu)
                    dn = p[L + "experts_down"]
                    n = dn.shape[2] // world
                    self.t[L + "experts_down"] = dev(dn[:, :, rank * n:(rank + 1) * n])
                if L + "shared_gate_up" in p:
                    g, u = p[L + "shared_gate_up"].chunk(2, 0)
                    self.t[L + "shared_gate_up"] = dev(torch.cat([shard_rows(g, rank, world), shard_rows(u, rank, world)], 0))
                    self.t[L + "shared_down"] = dev(shard_cols(p[L + "shared_down"], rank, world))

    @staticmethod
    def kv_layout(num_kv_heads: int, rank: int, world: int) -> Tuple[int, int]:
        """(KV heads held by ``rank``, index of the first one).  When the ranks divide the KV heads every rank holds
        its share; when there are more ranks than KV heads (``world`` a multiple of them) every KV head is replicated
        on ``world / num_kv_heads`` consecutive ranks, whose query heads are exactly that head's group -- the
        reference expands grouped heads by copying them (``crates/runtime/src/models_v2/llama.rs:1073-1087``)."""
        if num_kv_heads % world == 0:
            n = num_kv_heads // world
            return n, rank * n
        if world % num_kv_heads == 0:
            return 1, rank // (world // num_kv_heads)
        raise UnsupportedOperation(f"{num_kv_heads} KV heads cannot be divided over or replicated on {world} ranks")

    def _set_ep(self, expert_parallel: bool) -> None:
        """Expert parallelism applies when asked for, with more than one rank and an expert count the ranks divide."""
        m = self.spec.moe
        self.ep = bool(expert_parallel and self.world > 1 and m is not None and m.num_experts % self.world == 0)
        self.experts_local = m.num_experts // self.world if self.ep else (m.num_experts if m is not None else 0)
        self.expert_lo = self.rank * self.experts_local if self.ep else 0

    @staticmethod
    def random(spec: DecoderSpec, device, rank: int = 0, world: int = 1, seed: int = 0,
               expert_parallel: bool = False) -> "RunnerWeights":
        """Random-init weights generated directly on the device, shard by shard (no host copy): the
        benchmark path for 8B-70B architectures.  Every rank draws the same full-size tensor for a given
        name from a per-tensor seed and keeps its shard, so TP=1 and TP=N hold the same model."""
        self = RunnerWeights.__new__(RunnerWeights)
        self.spec, self.rank, self.world = spec, rank, world
        s = spec
        self._set_ep(expert_parallel)
        self.hq = s.num_heads // world
        self.hkv, self.kv_lo = self.kv_layout(s.num_kv_heads, rank, world)
        self.vocab_shard = s.vocab_size // world
        self.t = {}
        H, I = s.hidden_size, s.intermediate_size
        std = s.initializer_range
        counter = [0]

        def rnd(rows, cols, row0=0, nrows=None, col0=0, ncols=None):
            """Rows [row0, row0+nrows) x cols [col0, col0+ncols) of a virtual [rows, cols] N(0, std) matrix."""
            counter[0] += 1
            nrows = rows if nrows is None else nrows
            ncols = cols if ncols is None else ncols
            g = torch.Generator(device=device).manual_seed(seed * 1000003 + counter[0])
            # generate in row blocks so that a shard equals the same rows of the full matrix
            out = torch.empty(nrows, ncols, dtype=torch.bfloat16, device=device)
            blk = 1024
            for r in range(0, rows, blk):
                rr = min(blk, rows - r)
                lo, hi = max(r, row0), min(r + rr, row0 + nrows)
                g.manual_seed((seed * 1000003 + counter[0]) * 65537 + r)
                if lo >= hi:
                    continue
                full = torch.randn(rr, cols, generator=g, device=device, dtype=torch.float32) * std
                out[lo - row0:hi - row0] = full[lo - r:hi - r, col0:col0 + ncols].to(torch.bfloat16)
            return out

        ones = lambda n: torch.ones(n, dtype=torch.bfloat16, device=device)
        self.t["embed"] = rnd(s.vocab_size, H)
        self.t["final_norm.w"] = ones(H)
        vs = self.vocab_shard
        if s.tie_embeddings:
            self.t["lm_head"] = self.t["embed"][rank * vs:(rank + 1) * vs] if world > 1 else self.t["embed"]
        else:
            self.t["lm_head"] = rnd(s.vocab_size, H, rank * vs, vs)
        qs, ks = s.q_size // world, self.hkv * s.head_dim
        k0 = self.kv_lo * s.head_dim
        for i in range(s.num_layers):
            L = f"layers.{i}."
            self.t[L + "ln1.w"], self.t[L + "ln2.w"] = ones(H), ones(H)
            q = rnd(s.q_size, H, rank * qs, qs)
            k = rnd(s.kv_size, H, k0, ks)
            v = rnd(s.kv_size, H, k0, ks)
            self.t[L + "wqkv"] = torch.cat([q, k, v], 0)
            self.t[L + "wo"] = rnd(H, s.q_size, 0, H, rank * qs, qs)
            if s.layer_is_moe(i):
                m = s.moe
                self.t[L + "router"] = rnd(m.num_experts, H)
                # tensor parallel inside every expert, or (expert parallel) whole experts of this rank
                Ie = m.intermediate_size if self.ep else m.intermediate_size // world
                c0 = 0 if self.ep else rank * Ie
                gu = torch.empty(self.experts_local, 2 * Ie, H, dtype=torch.bfloat16, device=device)
                dn = torch.empty(self.experts_local, H, Ie, dtype=torch.bfloat16, device=device)
                for e in range(m.num_experts):
                    mine = self.expert_lo <= e < self.expert_lo + self.experts_local
                    if not mine:
                        counter[0] += 3           # keep the per-tensor seeds aligned across ranks
                        continue
                    j = e - self.expert_lo
                    gu[j, :Ie] = rnd(m.intermediate_size, H, c0, Ie)
                    gu[j, Ie:] = rnd(m.intermediate_size, H, c0, Ie)
                    dn[j] = rnd(H, m.intermediate_size, 0, H, c0, Ie)
                self.t[L + "experts_gate_up"], self.t[L + "experts_down"] = gu, dn
            else:
                Is = I // world
                g = rnd(I, H, rank * Is, Is)
                u = rnd(I, H, rank * Is, Is)
                self.t[L + "w_gate_up"] = torch.cat([g, u], 0)
                self.t[L + "w_down"] = rnd(H, I, 0, H, rank * Is, Is)
        return self

    def quantize(self, qtype="q4_k") -> "RunnerWeights":
        """Re-encodes every projection matrix (QKV, attention output, MLP, ``lm_head``; not embeddings, norms, routers
        or expert stacks) as ggml blocks of ``qtype`` on the device and drops the bf16 copy.  Decode-sized GEMMs
        (<= 8 token rows) then stream the blocks through the quantised GEMV kernel; larger ones expand the matrix into
        a scratch buffer first and run the tensor-core GEMM.  Rows are quantised independently along K, so sharded
        and fused matrices quantise like their parts.  Returns self."""
        from ..weights.gguf import BLOCK, quantize_blocks

        qt = QUANT_NAMES[qtype] if isinstance(qtype, str) else int(qtype)
        be = BLOCK[qt][0]
        tied = self.t.get("lm_head") is self.t.get("embed")
        for name, w in list(self.t.items()):
            leaf = name.rsplit(".", 1)[-1]
            if leaf not in ("wqkv", "wo", "w_gate_up", "w_up", "w_down", "lm_head") or isinstance(w, QWeight):
                continue
            if w.dim() != 2 or w.shape[1] % be or w.shape[1] % 8:
                continue                     # K is not a whole number of blocks: this matrix stays bf16
            if name == "lm_head" and tied:
                w = w.clone()                # the embedding keeps its bf16 table
            raw = quantize_blocks(w.float().cpu(), qt)
            self.t[name] = QWeight(torch.from_numpy(raw.copy()).to(w.device), qt, w.shape)
        self.quantized = qtype if isinstance(qtype, str) else str(qt)
        return self

    def dequantized_copy(self) -> "RunnerWeights":
        """The same weights with every quantised matrix expanded to bf16 (the values the quantised kernels compute
        with): the reference run for accuracy checks of the quantised path."""
        import copy

        from ..ops.quant import dequantize_cuda

        o = copy.copy(self)
        o.t = {k: (dequantize_cuda(v.blocks, v.qtype, v.shape) if isinstance(v, QWeight) else v) for k, v in self.t.items()}
        o.quantized = None
        return o

    def nbytes(self) -> int:
        seen, n = set(), 0
        for t in self.t.values():
            if isinstance(t, QWeight):
                n += t.nbytes()
                continue
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()
        return n


class TpContext:
    """Tensor-parallel plumbing of one rank: NCCL group for the baseline path, and (when fused) the
    symmetric buffers + counters that the fused kernels use.  ``world == 1`` needs none of it."""

    def __init__(self, rank: int = 0, world: int = 1, group=None, fused: bool = False):
        self.rank, self.world, self.group, self.fused = rank, world, group, fused and world > 1
        self.comm = None   # unillm_b200.dist.fused.FusedComm when fused

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.world > 1:
            if self.comm is not None and self.comm.can_all_reduce(t):
                return self.comm.all_reduce(t)        # decode-sized message: one-shot exchange over peer memory
            import torch.distributed as dist

            dist.all_reduce(t, group=self.group)
        return t

    def all_gather_cat(self, t: torch.Tensor, dim: int = -1) -> torch.Tensor:
        if self.world == 1:
            return t
        import torch.distributed as dist

        outs = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(outs, t.contiguous(), group=self.group)
        return torch.cat(outs, dim=dim)


class StepPacker:
    """Packs a ``StepBatch`` into one int32 staging buffer (host-only logic, numpy views)."""

    def __init__(self, buf: torch.Tensor, max_blocks_per_seq: int):
        self.meta_host = buf
        self.np = buf.numpy()
        self.META_INTS = buf.numel()
        self.max_blocks_per_seq = max_blocks_per_seq

    @staticmethod
    def _bucket(n: int) -> int:
        b = 1
        while b < n:
            b <<= 1
        return b

    def pack(self, b: StepBatch, bucketed: bool = False, token_src: Optional[List[int]] = None):
        """Writes the step's integer metadata into the pinned buffer and returns the layout
        (name -> (offset, length)); one H2D copy moves all of it.

        With ``bucketed`` the batch is padded to a shape from a small set so that a captured CUDA graph
        can be replayed: decode rows to a power of two, prefill tokens to a multiple of 128 (the padding
        forms a dummy sequence that writes no KV), prefill sequences to a power of two (empty dummies),
        and every decode row plus the last row of every prefill sequence is sampled."""
        D = b.num_decode
        nseq = len(b.seq_lens)
        P = nseq - D
        mb = self.max_blocks_per_seq
        q_lens = list(b.prefill_q_lens)
        p_lens = list(b.seq_lens[D:])
        Tp = sum(q_lens)
        Dp, Pp, tpad = D, P, 0
        if bucketed:
            Dp = self._bucket(D) if D else 0
            if P:
                tpad = (-Tp) % 128
                Pp = self._bucket(P + (1 if tpad else 0))
                if tpad:
                    q_lens.append(tpad)
                    p_lens.append(tpad)
                q_lens += [0] * (Pp - len(q_lens))
                p_lens += [0] * (Pp - len(p_lens))
        pad = Dp - D
        h = self.np
        off = 0
        lay = {}

        def put(name, vals):
            nonlocal off
            n = len(vals)
            if off + n > self.META_INTS:
                raise InvalidInput("step metadata exceeds the staging buffer")
            if n:
                h[off:off + n] = vals
            lay[name] = (off, n)
            off += (n + 3) // 4 * 4     # keep every array 16-byte aligned

        # decode rows first (padded rows point at slot -1 / block 0 / length 1 so kernels stay in bounds)
        put("token_ids", b.token_ids[:D] + [0] * pad + b.token_ids[D:] + [0] * tpad)
        put("positions", b.positions[:D] + [0] * pad + b.positions[D:] + [0] * tpad)
        put("slot_mapping", b.slot_mapping[:D] + [-1] * pad + b.slot_mapping[D:] + [-1] * tpad)
        put("seq_lens_d", b.seq_lens[:D] + [1] * pad)
        if token_src is not None:
            # device index of each decode row's input token inside the previous step's sampled ids (-1 = uploaded)
            put("token_src", list(token_src[:D]) + [-1] * pad)
        nbt = (Dp + Pp) * mb
        if off + nbt > self.META_INTS:
            raise InvalidInput("step metadata exceeds the staging buffer")
        bt = h[off:off + nbt].reshape(Dp + Pp, mb)
        # only the entries below each sequence's length are ever read; rows of padded sequences are zeroed
        for i, row in enumerate(b.block_tables):
            bt[i if i < D else i + pad, :len(row)] = row
        if pad:
            bt[D:Dp, 0] = 0
        if Pp > P:
            bt[Dp + P:, :(128 // 16) + 1] = 0      # the dummy sequence is shorter than 128 tokens
        lay["block_tables"] = (off, nbt)
        off += (nbt + 3) // 4 * 4
        put("seq_lens_p", p_lens)
        qs = [0]
        for ql in q_lens:
            qs.append(qs[-1] + ql)
        put("q_start", qs)
        if bucketed:
            rows = list(range(Dp)) + [Dp + max(qs[j + 1] - 1, 0) for j in range(Pp)]
            sel = []
            for r in b.sample_rows:
                if r < D:
                    sel.append(r)
                else:
                    # r is the last row of some prefill sequence j: find it from the unpadded prefix sums
                    j = next(jj for jj in range(P) if D + qs[jj + 1] - 1 == r)
                    sel.append(Dp + j)
            lay["_sel"] = sel
        else:
            rows = [r if r < D else r + pad for r in b.sample_rows]
            lay["_sel"] = list(range(len(rows)))
        put("sample_rows", rows)
        lay["_T"], lay["_D"], lay["_Dp"], lay["_P"], lay["_S"] = Dp + Tp + tpad, D, Dp, Pp, len(rows)
        mq = max(q_lens) if q_lens else 0
        lay["_max_q"] = self._bucket(mq) if (bucketed and mq) else mq
        lay["_used"] = off
        return lay



class _OpTimer:
    def __init__(self, runner, name):
        self.r, self.name = runner, name

    def __enter__(self):
        if self.r.profile and not self.r._graph_mode:
            self.a = torch.cuda.Event(enable_timing=True)
            self.a.record()
        else:
            self.a = None

    def __exit__(self, *exc):
        if self.a is not None:
            b = torch.cuda.Event(enable_timing=True)
            b.record()
            self.r._prof_events.append((self.name, self.a, b))
        return False


class GpuModelRunner:
    META_INTS = 1 << 20   # capacity of the packed per-step metadata buffer (int32 words)

    def __init__(self, spec: DecoderSpec, weights: RunnerWeights, *, num_blocks: int, block_size: int = 16,
                 max_num_seqs: int = 256, max_num_batched_tokens: int = 8192, max_model_len: int = 8192,
                 tp: Optional[TpContext] = None, device=None, use_cuda_graphs: bool = True):
        if spec.norm not in ("rms", "layer") or spec.post_ln or spec.embed_proj_dim:
            raise UnsupportedOperation("this spec is served by the generic model path, not the fused runner")
        self.spec, self.w = spec, weights
        self.tp = tp or TpContext()
        self.device = torch.device(device if device is not None else f"cuda:{torch.cuda.current_device()}")
        self.block_size, self.num_blocks = block_size, num_blocks
        self.max_num_seqs, self.max_tokens, self.max_model_len = max_num_seqs, max_num_batched_tokens, max_model_len
        self.max_blocks_per_seq = (max_model_len + block_size - 1) // block_size
        # NCCL collectives inside a captured graph stalled on this stack; the baseline path launches eagerly
        self.use_cuda_graphs = use_cuda_graphs and (self.tp.world == 1 or self.tp.fused)
        s, dev = spec, self.device
        hkv, D = weights.hkv, s.head_dim
        self.k_cache = [torch.zeros(num_blocks, hkv, block_size, D, dtype=torch.bfloat16, device=dev)
                        for _ in range(s.num_layers)]
        self.v_cache = [torch.zeros(num_blocks, hkv, block_size, D, dtype=torch.bfloat16, device=dev)
                        for _ in range(s.num_layers)]
        self.alibi = None
        if s.pos == "alibi":
            sl = alibi_slopes(s.num_heads)
            self.alibi = sl[weights.rank * weights.hq:(weights.rank + 1) * weights.hq].to(dev)
        # packed metadata: pinned host staging + device mirror with fixed addresses (graph friendly)
        # two staging buffers: the next step may be packed while the copy of the previous one is still queued
        self.meta_hosts = [torch.zeros(self.META_INTS, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self.packers = [StepPacker(h, self.max_blocks_per_seq) for h in self.meta_hosts]
        self._flip = 0
        self.meta_dev = torch.empty(self.META_INTS, dtype=torch.int32, device=dev)
        self.fmeta_hosts = [torch.empty(4 * max_num_seqs, dtype=torch.float32, pin_memory=True) for _ in range(2)]
        self.fmeta_dev = torch.empty(4 * max_num_seqs, dtype=torch.float32, device=dev)
        self.out_ids_dev = torch.zeros(4 * max_num_seqs, dtype=torch.int32, device=dev)
        self.out_ids_hosts = [torch.zeros(4 * max_num_seqs, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        # the per-device error word travels back with every step's sampled ids (same stream, no extra synchronisation)
        self.err_hosts = [torch.zeros(2, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._out_events = [torch.cuda.Event(), torch.cuda.Event()]
        self._sel: List[int] = []
        self._handle = None
        self.attn_scratch = torch.empty(max_num_seqs * weights.hq * 16 * (D + 2), dtype=torch.float32, device=dev)
        self.prefix_scratch = None     # workspace of the key-split shared-prefix pass, allocated on first use
        self._deq_scratch = None       # bf16 expansion of one quantised matrix at a time (quantised weights, > 8 rows)
        if getattr(weights, "quantized", None):
            big = max((int(v.shape[0]) * int(v.shape[1]) for v in weights.t.values() if isinstance(v, QWeight)), default=0)
            self._deq_scratch = torch.empty(big, dtype=torch.bfloat16, device=dev) if big else None
        self.overlap_suffix = os.environ.get("UB_ATTN_OVERLAP", "1") != "0"
        self._side = None
        self.graphs: Dict[tuple, tuple] = {}
        self.profile = False
        self._prof_events = []
        self._graph_mode = False
        self.launches = 0          # kernels of this library launched so far (counted on the host)
        self.captures = 0          # CUDA-graph captures so far (each costs an eager run, a synchronize and the capture)
        self.capture_new_graphs = True   # False: a step shape without a graph runs as plain launches instead
        self.eager_steps = 0       # graphable steps that ran as plain launches for that reason
        self.wait_s = 0.0          # host time spent blocked in fetch() waiting for the device
        self.fused_steps = 0       # tensor-parallel steps that ran the fused (peer-memory) path / the NCCL path
        self.unfused_steps = 0
        self.h2d_bytes = 0
        self.d2h_bytes = 0
        self._layout = None
        self._last_fused = False

    # ------------------------------------------------------------------------------------------
    # metadata packing
    # ------------------------------------------------------------------------------------------
    def _pack(self, b: StepBatch, bucketed: bool = False):
        src = None
        if b.token_src is not None:
            prev = self._sel            # sample order -> index in out_ids_dev, of the step launched before this one
            src = [prev[k] if k >= 0 else -1 for k in b.token_src]
        self._flip ^= 1
        pk = self.packers[self._flip]
        lay = pk.pack(b, bucketed, token_src=src)
        lay["_host"] = pk.meta_host
        return lay

    def _feed_sampled_ids(self, lay) -> None:
        """Decode rows whose input token was sampled by the previous step take it from the device buffer of that
        step's samples (the host may not have read them yet).  Runs right after the upload and outside the captured
        graph: the step itself then only reads its own metadata and can be replayed (graph capture runs it more
        than once) without seeing the samples it has just written."""
        if "token_src" not in lay:
            return
        src = self._view(lay, "token_src")
        d = self._view(lay, "token_ids")[:src.numel()]
        prev = self.out_ids_dev.index_select(0, src.clamp(min=0))
        d.copy_(torch.where(src >= 0, prev, d))

    def _view(self, lay, name):
        o, n = lay[name]
        return self.meta_dev[o:o + n]

    def _upload(self, lay):
        n = lay["_used"]
        self.meta_dev[:n].copy_(lay["_host"][:n], non_blocking=True)
        self.h2d_bytes += n * 4
        self._feed_sampled_ids(lay)

    # ------------------------------------------------------------------------------------------
    # layer math
    # ------------------------------------------------------------------------------------------
    def _prof(self, name: str):
        """Context manager timing one op with CUDA events when profiling is on (eager mode only)."""
        return _OpTimer(self, name)

    def profile_report(self) -> Dict[str, float]:
        """Milliseconds per op name accumulated since profiling was switched on (synchronises)."""
        torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for name, a, b in self._prof_events:
            out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self._prof_events = []
        return out

    def _norm(self, x, name, residual=None, want_h=False):
        s, t = self.spec, self.w.t
        self.launches += 1
        with self._prof("norm"):
            return self._norm_impl(x, name, residual, want_h)

    def _norm_impl(self, x, name, residual=None, want_h=False):
        s, t = self.spec, self.w.t
        return K.norm(x, t[name + ".w"], bias=t.get(name + ".b"), residual=residual, eps=s.norm_eps,
                      kind="rms" if s.norm == "rms" else "layer", weight_offset_one=s.norm_weight_offset_one,
                      want_residual_out=want_h)

    def _gemm(self, x, w, tag="gemm", **kw):
        self.launches += 1
        with self._prof(f"{tag}[{x.shape[0]}x{w.shape[0]}x{w.shape[1]}]"):
            if isinstance(w, QWeight):
                return self._qgemm(x, w, **kw)
            return K.gemm_tn(x, w, **kw)

    def _qgemm(self, x, w: "QWeight", **kw):
        """GEMM against a block-quantised matrix.  Up to 8 token rows: the quantised GEMV kernel (the weight stream is
        4.5 - 8.5 bits per value) followed by the small epilogue kernels; more rows, or a fused collective: the matrix
        is expanded into the runner's scratch buffer and the tensor-core GEMM runs on that."""
        from ..ops import quant as Q

        M = x.shape[0]
        N_, Kd = w.shape
        plain = kw.get("rs") is None and kw.get("ag") is None and kw.get("out") is None
        if M <= 8 and plain and x.is_contiguous():
            y = Q.qgemv_cuda(w.blocks, x, N_, w.qtype)
            self.launches += 1
            dual = kw.get("dual_rows", 0)
            scale = kw.get("out_scale", 1.0)
            if dual:
                y = K.act_mul(y, kw.get("act") or "silu")
            else:
                if kw.get("bias") is not None or scale != 1.0:
                    yf = y.float() * scale
                    if kw.get("bias") is not None:
                        yf = yf + kw["bias"].float()
                    y = yf.to(torch.bfloat16)
                if kw.get("act"):
                    y = K.eltwise(y, kw["act"])
            if kw.get("residual") is not None:
                y = K.add(y, kw["residual"])
            if kw.get("out_dtype", torch.bfloat16) == torch.float32:
                y = y.float()
            return y
        need = N_ * Kd
        if self._deq_scratch is None or self._deq_scratch.numel() < need:
            self._deq_scratch = torch.empty(need, dtype=torch.bfloat16, device=self.device)
        dense = self._deq_scratch[:need].view(N_, Kd)
        Q.dequantize_cuda_into(w.blocks, w.qtype, dense)
        self.launches += 1
        return K.gemm_tn(x, dense, **kw)

    def _attention(self, i, qkv, lay, shared_prefix_len):
        """qkv [T, (hq + 2 hkv) * D] already rotated and appended -> attention output [T, hq * D]."""
        s, w = self.spec, self.w
        D, hq, hkv = s.head_dim, w.hq, w.hkv
        T, Dp, P = lay["_T"], lay["_Dp"], lay["_P"]
        q = qkv.view(T, hq + 2 * hkv, D)[:, :hq]           # strided view: row stride (hq + 2 hkv) * D
        out = torch.empty(T, hq, D, dtype=torch.bfloat16, device=qkv.device)
        kc, vc = self.k_cache[i], self.v_cache[i]
        bt = self._view(lay, "block_tables").view(Dp + P, self.max_blocks_per_seq)
        scale = s.attn_scale
        cascade = shared_prefix_len >= 4 * self.block_size and Dp >= 8
        # prefill rows join the cascade when their chunks start after the shared prefix and share its blocks
        pp = cascade and P > 0 and lay.get("_pp", False) and s.window == 0 and self.alibi is None
        if cascade:
            # one GEMM-shaped pass of all queries over the shared prefix blocks, one pass per sequence over the
            # unique suffixes, then a merge of the two partials
            R = T if pp else Dp
            # the suffix kernels fold the prefix partial into their output themselves (head dim 128, page 16, no
            # window / ALiBi); otherwise a separate merge kernel combines the two partials
            fused = D == 128 and self.block_size == 16 and s.window == 0 and self.alibi is None
            lse_a = torch.empty(R, hq, dtype=torch.float32, device=qkv.device)
            oa = torch.empty(R, hq, D, dtype=torch.bfloat16, device=qkv.device)
            kvs = self._prefix_splits(R, shared_prefix_len)
            with self._prof("attn_shared_prefix"):
                K.attn_prefill(q[:R], kc, vc, bt[:1], self._prefix_len_dev(shared_prefix_len), self._q_start_all(R),
                               R, scale=scale, causal=False, window=0, alibi_slopes=None, out=oa, lse=lse_a,
                               return_lse=True, kv_splits=kvs, scratch=self.prefix_scratch if kvs > 1 else None)
            if kvs > 1:
                self.launches += 1
            if fused:
                # The suffix pass of the prefill chunks is a handful of CTAs whose time is all latency; it runs beside
                # the decode rows' suffix pass on a second stream (both only read the prefix partial).
                side = self._side_stream() if (pp and self.overlap_suffix) else None
                if side is not None:
                    cur = torch.cuda.current_stream()
                    side.wait_stream(cur)
                    with torch.cuda.stream(side):
                        with self._prof("attn_prefill_suffix"):
                            K.attn_prefill(q[Dp:], kc, vc, bt[Dp:], self._view(lay, "seq_lens_p"),
                                           self._view(lay, "q_start"), lay["_max_q"], scale=scale, causal=True,
                                           kv_start=shared_prefix_len, out=out[Dp:], merge=(oa[Dp:], lse_a[Dp:]))
                    self.launches += 1
                with self._prof("attn_decode_suffix"):
                    K.attn_decode(q[:Dp], kc, vc, bt[:Dp], self._view(lay, "seq_lens_d"), scale=scale,
                                  kv_start=shared_prefix_len, out=out[:Dp], splits=1, merge=(oa[:Dp], lse_a[:Dp]))
                if side is not None:
                    cur.wait_stream(side)
                elif pp:
                    with self._prof("attn_prefill_suffix"):
                        K.attn_prefill(q[Dp:], kc, vc, bt[Dp:], self._view(lay, "seq_lens_p"), self._view(lay, "q_start"),
                                       lay["_max_q"], scale=scale, causal=True, kv_start=shared_prefix_len, out=out[Dp:],
                                       merge=(oa[Dp:], lse_a[Dp:]))
                    self.launches += 1
                self.launches += 2
            else:
                lse_b = torch.empty(R, hq, dtype=torch.float32, device=qkv.device)
                ob = torch.empty(R, hq, D, dtype=torch.bfloat16, device=qkv.device)
                with self._prof("attn_decode_suffix"):
                    K.attn_decode(q[:Dp], kc, vc, bt[:Dp], self._view(lay, "seq_lens_d"), scale=scale, window=s.window,
                                  kv_start=shared_prefix_len, alibi_slopes=self.alibi, out=ob[:Dp], lse=lse_b[:Dp],
                                  return_lse=True, splits=1)
                if pp:
                    with self._prof("attn_prefill_suffix"):
                        K.attn_prefill(q[Dp:], kc, vc, bt[Dp:], self._view(lay, "seq_lens_p"), self._view(lay, "q_start"),
                                       lay["_max_q"], scale=scale, causal=True, kv_start=shared_prefix_len, out=ob[Dp:],
                                       lse=lse_b[Dp:], return_lse=True)
                    self.launches += 1
                with self._prof("attn_merge"):
                    K.attn_merge(oa, lse_a, ob, lse_b, out=out[:R])
                self.launches += 3
        elif Dp > 0:
            with self._prof("attn_decode"):
                K.attn_decode(q[:Dp], kc, vc, bt[:Dp], self._view(lay, "seq_lens_d"), scale=scale, window=s.window,
                              alibi_slopes=self.alibi, out=out[:Dp], scratch=self.attn_scratch,
                              max_seq_len=self.max_model_len if self._graph_mode else int(self._max_len_d))
            self.launches += 1
        if P > 0 and not pp:
            with self._prof("attn_prefill"):
                K.attn_prefill(q[Dp:], kc, vc, bt[Dp:], self._view(lay, "seq_lens_p"), self._view(lay, "q_start"),
                               lay["_max_q"], scale=scale, causal=True, window=s.window, alibi_slopes=self.alibi,
                               out=out[Dp:])
            self.launches += 1
        return out.view(T, hq * D)

    def _side_stream(self):
        if self._side is None:
            self._side = torch.cuda.Stream(device=self.device)
        return self._side

    PREFIX_SPLIT_ROWS = 160 * 128     # (query row, head) pairs x splits the key-split workspace can hold

    def _prefix_splits(self, R: int, prefix_len: int) -> int:
        """Key splits of the shared-prefix pass.  The pass has one CTA per 128 packed (token, head-of-group) rows and KV
        head; a tensor-parallel rank with one KV head and a few hundred rows would keep a fraction of the SMs busy while
        every CTA walks the whole prefix, so the key tiles are divided until about one wave of CTAs exists."""
        s, w = self.spec, self.w
        if s.head_dim != 128 or self.block_size != 16 or s.window or self.alibi is not None:
            return 1
        G = w.hq // w.hkv
        if 128 % G:
            return 1
        ctas = -(-R // (128 // G)) * w.hkv
        n = min(prefix_len // 128, 148 // max(ctas, 1), 8)
        while n > 1 and n * R * w.hq > self.PREFIX_SPLIT_ROWS:
            n -= 1
        if n > 1 and self.prefix_scratch is None:
            self.prefix_scratch = torch.empty(K.attn_prefill_split_scratch_floats(self.PREFIX_SPLIT_ROWS, 1, 128, 1),
                                              dtype=torch.float32, device=self.device)
        return max(n, 1)

    def _prefix_len_dev(self, n: int) -> torch.Tensor:
        c = getattr(self, "_plen_cache", None)
        if c is None:
            c = self._plen_cache = {}
        if n not in c:
            c[n] = torch.tensor([n], dtype=torch.int32, device=self.device)
        return c[n]

    def _q_start_all(self, n: int) -> torch.Tensor:
        c = getattr(self, "_qsa_cache", None)
        if c is None:
            c = self._qsa_cache = {}
        if n not in c:
            c[n] = torch.tensor([0, n], dtype=torch.int32, device=self.device)
        return c[n]

    def _mlp(self, i, h, residual):
        s, t = self.spec, self.w.t
        L = f"layers.{i}."
        tp = self.tp
        if s.layer_is_moe(i):
            from .moe_runner import moe_forward

            return moe_forward(self, i, h, residual)
        if s.mlp == "gated":
            I = t[L + "w_gate_up"].shape[0] // 2
            a = self._gemm(h, t[L + "w_gate_up"], dual_rows=I, act=s.act)
        else:
            a = self._gemm(h, t[L + "w_up"], bias=t.get(L + "b_up"), act=s.act)
        if tp.world == 1:
            return self._gemm(a, t[L + "w_down"], bias=t.get(L + "b_down"), residual=residual)
        y = self._gemm(a, t[L + "w_down"], bias=t.get(L + "b_down"))
        tp.all_reduce(y)
        self.launches += 1
        return K.add(y, residual)

    def _forward_tokens(self, lay, shared_prefix_len: int) -> torch.Tensor:
        """Runs all layers on the packed step; returns the sampled token ids tensor (device, [S])."""
        s, t, tp = self.spec, self.w.t, self.tp
        T = lay["_T"]
        self._final_norm_done = False
        if self._fused_ok(T):
            self._last_fused = True
            return self._forward_tokens_fused(lay, shared_prefix_len)
        self._last_fused = False
        ids = self._view(lay, "token_ids")
        pos = self._view(lay, "positions")
        slots = self._view(lay, "slot_mapping")
        x = K.embed_gather(ids, t["embed"], scale=s.embed_scale)
        self.launches += 1
        if s.pos == "learned":
            x = x + t["pos_embed"][(pos + s.learned_pos_offset).long()]
        if s.embed_norm:
            x = K.norm(x, t["embed_norm.w"], bias=t["embed_norm.b"], eps=s.norm_eps, kind="layer")
        rs = s.residual_scale
        for i in range(s.num_layers):
            L = f"layers.{i}."
            h = self._norm(x, L + "ln1")
            qkv = self._gemm(h, t[L + "wqkv"], bias=t.get(L + "bqkv"))
            with self._prof("rope_kv_append"):
                K.rope_kv_append(qkv, pos, slots, self.k_cache[i], self.v_cache[i], num_q_heads=self.w.hq,
                                 num_kv_heads=self.w.hkv, head_dim=s.head_dim,
                                 rotary_dim=s.rd if s.pos == "rope" else 0, theta=s.rope_theta,
                                 pos_scale=s.rope_pos_scale, interleaved=s.rope_interleaved,
                                 q_norm_w=t.get(L + "q_norm"), k_norm_w=t.get(L + "k_norm"), norm_eps=s.norm_eps,
                                 llama3_scaling=s.rope_llama3)
            self.launches += 1
            a = self._attention(i, qkv, lay, shared_prefix_len)
            if s.parallel_residual:
                m_in = h if s.parallel_shared_norm else self._norm(x, L + "ln2")
                o = self._gemm(a, t[L + "wo"], bias=t.get(L + "bo"))
                m = self._mlp_noresid(i, m_in)
                y = K.add(o, m)
                if tp.world > 1:
                    tp.all_reduce(y)
                x = K.add(x, y, 1.0, rs)
                self.launches += 2
                continue
            if tp.world == 1 and rs == 1.0:
                x = self._gemm(a, t[L + "wo"], bias=t.get(L + "bo"), residual=x)
            else:
                o = self._gemm(a, t[L + "wo"], bias=t.get(L + "bo"))
                tp.all_reduce(o)
                x = K.add(x, o, 1.0, rs)
                self.launches += 1
            h2 = self._norm(x, L + "ln2")
            if rs == 1.0:
                x = self._mlp(i, h2, x)
            else:
                m = self._mlp_noresid(i, h2)
                if tp.world > 1:
                    tp.all_reduce(m)
                x = K.add(x, m, 1.0, rs)
                self.launches += 1
        return x

    # ------------------------------------------------------------------------------------------
    # fused tensor-parallel path (F1 / F3)
    # ------------------------------------------------------------------------------------------
    def _fused_ok(self, T: int) -> bool:
        s, tp = self.spec, self.tp
        return (tp.fused and tp.comm is not None and T % tp.world == 0 and T // tp.world <= tp.comm.max_rows
                and not s.parallel_residual and s.residual_scale == 1.0 and s.pos != "learned"
                and not s.embed_norm and s.final_norm
                and (s.moe is None or (s.moe.num_shared_experts == 0 and not s.moe.dense_parallel)))

    def _forward_tokens_fused(self, lay, shared_prefix_len: int) -> torch.Tensor:
        """Same math as ``_forward_tokens`` with the residual stream sharded by token rows between the two
        GEMM pairs of every layer: o_proj / down_proj epilogues push rows to their owner (reduce-scatter),
        the norm kernel sums, normalises and pushes to everyone (all-gather), and the next GEMM waits on
        the arrival counters inside its TMA producer.  No NCCL call, no separate reduction kernel."""
        s, t, tp = self.spec, self.w.t, self.tp
        c, W, r = tp.comm, tp.world, tp.rank
        T = lay["_T"]
        R = T // W
        H = s.hidden_size
        ids = self._view(lay, "token_ids")
        pos = self._view(lay, "positions")
        slots = self._view(lay, "slot_mapping")
        x_full = K.embed_gather(ids, t["embed"], scale=s.embed_scale)
        self.launches += 1
        xr = x_full[r * R:(r + 1) * R]                      # this rank's rows of the residual stream
        h_full = self._norm(x_full, "layers.0.ln1")         # layer 0 normalises all rows locally
        kind = "rms" if s.norm == "rms" else "layer"
        dense = [i for i in range(s.num_layers) if not s.layer_is_moe(i)]
        I_loc = 0
        if dense:
            L0 = f"layers.{dense[0]}."
            I_loc = (t[L0 + "w_gate_up"].shape[0] // 2) if s.mlp == "gated" else t[L0 + "w_up"].shape[0]
        rs0_out = c.rs_local_tensor(0, R)
        rs1_out = c.rs_local_tensor(1, R)
        ag_args = None
        # whole experts per rank and a dispatch area in the symmetric buffer: route locally, send pairs, not all rows
        self._moe_sparse = bool(s.moe is not None and self.w.ep and c.has_moe_dispatch and
                                os.environ.get("UB_MOE_SPARSE", "1") != "0")
        for i in range(s.num_layers):
            L = f"layers.{i}."
            qkv = self._gemm(h_full, t[L + "wqkv"], bias=t.get(L + "bqkv"), ag=ag_args, tag="gemm_ag" if ag_args else "gemm")
            with self._prof("rope_kv_append"):
                K.rope_kv_append(qkv, pos, slots, self.k_cache[i], self.v_cache[i], num_q_heads=self.w.hq,
                                 num_kv_heads=self.w.hkv, head_dim=s.head_dim,
                                 rotary_dim=s.rd if s.pos == "rope" else 0, theta=s.rope_theta,
                                 pos_scale=s.rope_pos_scale, interleaved=s.rope_interleaved,
                                 q_norm_w=t.get(L + "q_norm"), k_norm_w=t.get(L + "k_norm"), norm_eps=s.norm_eps,
                                 llama3_scaling=s.rope_llama3)
            self.launches += 1
            a = self._attention(i, qkv, lay, shared_prefix_len)
            # o_proj: partial rows go straight to their owner's receive slot
            self._gemm(a, t[L + "wo"], bias=t.get(L + "bo"), out=rs0_out.view(W * R, H)[:T], rs=c.gemm_rs(0, R),
                       tag="gemm_rs")
            sparse = s.layer_is_moe(i) and self._moe_sparse
            if sparse:
                # F5 / F6: this rank normalises and routes its own rows only; each (token, expert) pair travels to the
                # rank of its expert and its weighted output comes back into slot k of the combine area
                from .moe_runner import moe_sparse

                with self._prof("norm_rs"):
                    h_own, xr = K.norm(rs0_out, t[L + "ln2.w"], bias=t.get(L + "ln2.b"), residual=xr, eps=s.norm_eps,
                                       kind=kind, weight_offset_one=s.norm_weight_offset_one, want_residual_out=True, T=R,
                                       rs=c.norm_rs(0, rows_per_rank=R), reset=c.reset_after_ag(1))
                self.launches += 1
                moe_sparse(self, i, h_own, c, R)
                last = i == s.num_layers - 1
                nname = "final_norm" if last else f"layers.{i + 1}.ln1"
                with self._prof("norm_rs_ag"):
                    _, xr = K.norm(c.moe_comb_tensor(R), t[nname + ".w"], bias=t.get(nname + ".b"), residual=xr,
                                   eps=s.norm_eps, kind=kind, weight_offset_one=s.norm_weight_offset_one,
                                   want_residual_out=True, no_out=True, T=R, rs=c.norm_comb(), ag=c.norm_ag(0),
                                   reset=c.reset_after_ag(0))
                self.launches += 1
                h_full = c.ag_local_tensor(0, T)
                ag_args = c.gemm_ag(0, R)
                continue
            # sum partials + residual, normalise own rows, push to every rank's gather area 1
            with self._prof("norm_rs_ag"):
                _, xr = K.norm(rs0_out, t[L + "ln2.w"], bias=t.get(L + "ln2.b"), residual=xr, eps=s.norm_eps, kind=kind,
                               weight_offset_one=s.norm_weight_offset_one, want_residual_out=True, no_out=True, T=R,
                               rs=c.norm_rs(0, rows_per_rank=R), ag=c.norm_ag(1), reset=c.reset_after_ag(1))
            self.launches += 1
            h2 = c.ag_local_tensor(1, T)
            if s.layer_is_moe(i):
                # F5: the all-gather of the normalised rows is the dispatch (every rank sees every token and keeps
                # the pairs of its own experts); F6: the combine kernel stores partial rows into their owners' slots
                from ..dist.fused import AG1
                from .moe_runner import moe_partial

                K.wait_flags(c.local_flag_ptr(AG1), W, 1, self.device)
                self.launches += 1
                moe_partial(self, i, h2, None, combine_rs=c.gemm_rs(1, R))
            else:
                if s.mlp == "gated":
                    act = self._gemm(h2, t[L + "w_gate_up"], dual_rows=I_loc, act=s.act, ag=c.gemm_ag(1, R), tag="gemm_ag")
                else:
                    act = self._gemm(h2, t[L + "w_up"], bias=t.get(L + "b_up"), act=s.act, ag=c.gemm_ag(1, R), tag="gemm_ag")
                self._gemm(act, t[L + "w_down"], bias=t.get(L + "b_down"), out=rs1_out.view(W * R, H)[:T],
                           rs=c.gemm_rs(1, R), tag="gemm_rs")
            last = i == s.num_layers - 1
            nname = "final_norm" if last else f"layers.{i + 1}.ln1"
            with self._prof("norm_rs_ag"):
                _, xr = K.norm(rs1_out, t[nname + ".w"], bias=t.get(nname + ".b"), residual=xr, eps=s.norm_eps, kind=kind,
                               weight_offset_one=s.norm_weight_offset_one, want_residual_out=True, no_out=True, T=R,
                               rs=c.norm_rs(1, rows_per_rank=R), ag=c.norm_ag(0), reset=c.reset_after_ag(0))
            self.launches += 1
            h_full = c.ag_local_tensor(0, T)
            ag_args = c.gemm_ag(0, R)
        # the final-normed rows of all ranks arrive in gather area 0; wait for them before the row gather
        from ..dist.fused import AG0

        K.wait_flags(c.local_flag_ptr(AG0), W, 1, self.device)
        self.launches += 1
        self._final_norm_done = True
        return h_full

    def _mlp_noresid(self, i, h, dense_only=False):
        s, t = self.spec, self.w.t
        L = f"layers.{i}."
        if s.layer_is_moe(i) and not dense_only:
            from .moe_runner import moe_partial

            return moe_partial(self, i, h, None)
        if s.mlp == "gated":
            I = t[L + "w_gate_up"].shape[0] // 2
            a = self._gemm(h, t[L + "w_gate_up"], dual_rows=I, act=s.act)
        else:
            a = self._gemm(h, t[L + "w_up"], bias=t.get(L + "b_up"), act=s.act)
        return self._gemm(a, t[L + "w_down"], bias=t.get(L + "b_down"))

    def _logits_and_sample(self, x, lay, b: Optional[StepBatch], fl) -> torch.Tensor:
        s, t, tp = self.spec, self.w.t, self.tp
        S = lay["_S"]
        rows = self._view(lay, "sample_rows")
        xs = x.index_select(0, rows.long()) if S != x.shape[0] else x
        if s.final_norm and not self._final_norm_done:
            xs = self._norm(xs, "final_norm")
        logits = self._gemm(xs, t["lm_head"], bias=t.get("lm_head_bias"), out_scale=s.logit_scale)
        out = self.out_ids_dev[:S]
        greedy = fl is None
        if tp.world == 1:
            if greedy:
                K.sample(logits, out_ids=out)
            else:
                K.sample(logits, temperature=fl["temperature"], top_p=fl["top_p"], top_k=fl["top_k"],
                         seed=fl["seed"], step=fl["step"], out_ids=out)
            self.launches += 1
            return out
        if greedy:
            ids, vals = K.sample(logits, vocab_offset=tp.rank * self.w.vocab_shard, return_vals=True)
            if tp.comm is not None and S <= 2048:
                tp.comm.argmax_merge(vals, ids, out)     # F4: exchange over peer memory, no NCCL call
                self.launches += 2
                return out
            allv = tp.all_gather_cat(vals[None], dim=0)
            alli = tp.all_gather_cat(ids[None], dim=0)
            K.argmax_merge(allv.contiguous(), alli.contiguous(), out=out)
            self.launches += 2
            return out
        kc = fl.get("cand_k", 0)
        if tp.comm is not None and kc and tp.comm.can_gather_pairs(S, kc) and os.environ.get("UB_SAMPLE_PAIRS", "1") != "0":
            # F4s: every shard hands in the best `kc` entries of each row (after temperature), the pairs are gathered
            # over peer memory and every rank draws the same token from them -- the whole-vocabulary logits stay put
            cv, ci = K.sample(logits, temperature=fl["temperature"], top_p=fl["top_p"], top_k=fl["top_k"], seed=fl["seed"],
                              step=fl["step"], vocab_offset=tp.rank * self.w.vocab_shard, candidates=kc)
            av, ai = tp.comm.gather_pairs(cv, ci)
            K.sample(av, temperature=fl["temperature"], top_p=fl["top_p"], top_k=fl["top_k"], seed=fl["seed"],
                     step=fl["step"], out_ids=out, id_map=ai)
            self.launches += 3
            return out
        if (tp.comm is not None and fl.get("whole_vocab") and tp.comm.can_gather_pairs(S, 1) and S <= 2048
                and os.environ.get("UB_SAMPLE_PAIRS", "1") != "0"):
            # F4s, temperature only: every shard reports its maximum and its mass, all ranks work out which shard the
            # draw falls into and where, that shard picks the token and the winner is merged like a greedy one
            st = K.sample(logits, temperature=fl["temperature"], seed=fl["seed"], step=fl["step"], stats=True)
            mv, sv = tp.comm.gather_pairs(st[:, :1].contiguous(), st[:, 1:].contiguous().view(torch.int32))
            owner, local = K.vocab_shard_targets(mv, sv.view(torch.float32), fl["uniform"])
            local = torch.where(owner == tp.rank, local, torch.full_like(local, -1.0)).contiguous()
            ids, vals = K.sample(logits, temperature=fl["temperature"], seed=fl["seed"], step=fl["step"],
                                 vocab_offset=tp.rank * self.w.vocab_shard, target=local, return_vals=True)
            tp.comm.argmax_merge(vals, ids, out)
            self.launches += 4
            return out
        full = tp.all_gather_cat(logits, dim=-1)
        K.sample(full, temperature=fl["temperature"], top_p=fl["top_p"], top_k=fl["top_k"], seed=fl["seed"],
                 step=fl["step"], out_ids=out)
        self.launches += 1
        return out

    # ------------------------------------------------------------------------------------------
    # step execution
    # ------------------------------------------------------------------------------------------
    @staticmethod
    def _bucket(n: int) -> int:
        b = 1
        while b < n:
            b <<= 1
        return b

    @staticmethod
    def candidate_count(temperature, top_k, top_p) -> int:
        """Candidates per row and vocabulary shard that a tensor-parallel draw has to exchange: the largest ``top_k`` of
        the batch, or the 1024 survivors that a top-p draw keeps; greedy rows need one.  0 = some row samples from the
        whole vocabulary (pure temperature), so the logits have to be gathered."""
        cand = 1
        for i, t in enumerate(temperature):
            if t <= 0:
                continue
            k = top_k[i] if top_k is not None and top_k[i] else 0
            p = top_p[i] if top_p is not None else 1.0
            k = min(k, 1024) if k > 0 else (1024 if p < 1.0 else 0)
            if k == 0:
                return 0
            cand = max(cand, k)
        return cand

    def _sampling_tensors(self, b: StepBatch, S: int):
        if b.temperature is None or all(t <= 0 for t in b.temperature):
            return None
        f = self.fmeta_hosts[self._flip]
        f[:S] = torch.as_tensor(b.temperature, dtype=torch.float32)
        f[S:2 * S] = torch.as_tensor(b.top_p if b.top_p is not None else [1.0] * S, dtype=torch.float32)
        self.fmeta_dev[:2 * S].copy_(f[:2 * S], non_blocking=True)
        self.h2d_bytes += 8 * S
        tk = None
        if b.top_k is not None and any(k and k > 0 for k in b.top_k):
            tk = torch.as_tensor([k or 0 for k in b.top_k], dtype=torch.int32).to(self.device, non_blocking=True)
            self.h2d_bytes += 4 * S
        cand = self.candidate_count(b.temperature, b.top_k, b.top_p)
        # temperature-only rows everywhere: the draw from the whole vocabulary can be split over the shards; it needs the
        # uniform number of every row (the device sampler's Philox stream, evaluated here)
        whole = cand == 0 and all(t > 0 for t in b.temperature) and (b.top_k is None or not any(b.top_k)) and \
            (b.top_p is None or all(p >= 1.0 for p in b.top_p)) and self.tp.world > 1
        uni = None
        if whole:
            from ..sampling import philox_uniform

            uni = torch.tensor([philox_uniform(b.seed, b.step, r) for r in range(S)], dtype=torch.float32).to(self.device)
        return {"temperature": self.fmeta_dev[:S], "top_p": self.fmeta_dev[S:2 * S], "top_k": tk, "seed": b.seed,
                "step": b.step, "cand_k": cand, "whole_vocab": whole, "uniform": uni}

    MAX_GRAPHS = 96

    def launch(self, b: StepBatch) -> int:
        """Uploads the step's metadata and enqueues all kernels on the current stream.  Returns the number of
        sampled rows; ``fetch`` reads them back."""
        D = b.num_decode
        if len(b.token_ids) > self.max_tokens + self.max_num_seqs:
            raise InvalidInput("step exceeds max_num_batched_tokens")
        greedy = b.temperature is None or all(t <= 0 for t in b.temperature)
        graphable = self.use_cuda_graphs and greedy and len(b.token_ids) > 0
        self._max_len_d = max(b.seq_lens[:D]) if D else 0
        if graphable:
            lay = self._pack(b, bucketed=True)
            lay["_pp"] = b.prefill_shares_prefix
            key = (lay["_Dp"], lay["_P"], lay["_T"], lay["_max_q"], b.shared_prefix_len, b.prefill_shares_prefix)
            g = self.graphs.get(key)
            self._graph_mode = True
            self._upload(lay)
            if g is None and self.capture_new_graphs and len(self.graphs) < self.MAX_GRAPHS:
                # one eager run (sets kernel attributes, warms the allocator), then capture
                self._forward_and_sample(lay, b.shared_prefix_len, None)
                torch.cuda.current_stream().synchronize()
                before = self.launches
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._forward_and_sample(lay, b.shared_prefix_len, None)
                g = self.graphs[key] = (graph, self.launches - before, self._last_fused)
                self.captures += 1
            if g is not None:
                g[0].replay()
                self.launches += g[1]
                self._count_step(g[2])
            else:
                # a shape without a graph while captures are off (or the graph table is full): the padded step runs
                # as plain launches -- slower than a replay, but without the synchronisation a capture needs
                self._forward_and_sample(lay, b.shared_prefix_len, None)
                self._count_step(self._last_fused)
                self.eager_steps += 1
            return self._queue_readback(lay["_sel"])
        self._graph_mode = False
        lay = self._pack(b, bucketed=False)
        lay["_pp"] = b.prefill_shares_prefix
        self._upload(lay)
        fl = None if greedy else self._sampling_tensors(b, lay["_S"])
        self._forward_and_sample(lay, b.shared_prefix_len, fl)
        self._count_step(self._last_fused)
        return self._queue_readback(lay["_sel"])

    def _count_step(self, fused: bool) -> None:
        if self.tp.world > 1:
            if fused:
                self.fused_steps += 1
            else:
                self.unfused_steps += 1

    def _queue_readback(self, sel: List[int]) -> int:
        """Queues the device -> pinned host copy of the sampled ids behind the step and records an event; the
        returned handle of ``pending()`` stays valid while one later step is launched."""
        self._sel = sel
        n = (max(sel) + 1) if sel else 0
        host, ev, err = self.out_ids_hosts[self._flip], self._out_events[self._flip], self.err_hosts[self._flip]
        if n:
            host[:n].copy_(self.out_ids_dev[:n], non_blocking=True)
            self.d2h_bytes += 4 * n
        err.copy_(K.err_word(self.device), non_blocking=True)
        self.d2h_bytes += 8
        ev.record()
        self._handle = (ev, host, n, sel, err)
        return len(sel)

    def pending(self):
        """Handle of the step launched last; pass it to ``fetch`` after launching the next step."""
        return self._handle

    def _forward_and_sample(self, lay, shared_prefix_len, fl):
        x = self._forward_tokens(lay, shared_prefix_len)
        if lay["_S"] > 0:
            self._logits_and_sample(x, lay, None, fl)

    def fetch(self, handle=None) -> List[int]:
        """Waits for a launched step (the last one by default) and returns its sampled ids from pinned memory."""
        ev, host, n, sel, err = handle if handle is not None else self._handle
        t0 = time.perf_counter()
        ev.synchronize()
        self.wait_s += time.perf_counter() - t0
        code, detail = err.tolist()
        if code != 0:
            raise DeviceStepError(code, detail)
        if not sel:
            return []
        vals = host[:n].tolist()
        return [vals[i] for i in sel]

    def execute(self, b: StepBatch) -> List[int]:
        self.launch(b)
        return self.fetch()

    def reset_after_error(self) -> None:
        """After a ``DeviceStepError``: waits for the device, clears the error word and (tensor parallel, fused path)
        zeroes the arrival counters on every rank -- a collective call, every rank of the group has to make it."""
        torch.cuda.synchronize(self.device)
        K.err_word(self.device).zero_()
        K.gemm_streamk_reset(self.device)
        for e in self.err_hosts:
            e.zero_()
        if self.tp.comm is not None:
            self.tp.comm.reset()
        torch.cuda.synchronize(self.device)

    def kv_cache_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.k_cache) * 2

    def logits_for(self, b: StepBatch) -> torch.Tensor:
        """Test hook: full logits [S, vocab_shard] of a step (eager, no sampling)."""
        self._graph_mode = False
        self._max_len_d = max(b.seq_lens[:b.num_decode]) if b.num_decode else 0
        lay = self._pack(b, bucketed=False)
        lay["_pp"] = b.prefill_shares_prefix
        self._upload(lay)
        x = self._forward_tokens(lay, b.shared_prefix_len)
        rows = self._view(lay, "sample_rows")
        xs = x.index_select(0, rows.long())
        if self.spec.final_norm and not self._final_norm_done:
            xs = self._norm(xs, "final_norm")
        return self._gemm(xs, self.w.t["lm_head"], bias=self.w.t.get("lm_head_bias"), out_scale=self.spec.logit_scale,
                          out_dtype=torch.float32)
