"""Symmetric-memory plumbing for the fused tensor-parallel kernels.

``FusedComm`` owns, on every rank, one symmetric allocation (same layout on all ranks, mapped into
every peer's address space by ``dist.symm_heap.SymmetricHeap`` -- the library's own heap over the CUDA
virtual-memory API, with an NVSwitch multicast view where the GPUs have one -- or, as a fallback,
through ``torch.distributed._symmetric_memory``) that holds

  * two reduce-scatter receive areas ``rs[k]``  : ``[world][rows_per_rank][H]`` bf16 -- slot ``[src]`` is
    written by rank ``src``'s GEMM epilogue (F1), read by the local norm kernel;
  * two all-gather areas ``ag[k]``              : ``[world * rows_per_rank][H]`` bf16 -- rows of rank
    ``src`` are written by ``src``'s norm kernel (F3 producer), read by the local GEMM's TMA loads;
  * the arrival counters of both.

Counter protocol: a producing launch tells a peer ONCE that all of its rows have arrived: its CTAs arrive
on a counter in local memory and the last one bumps the peer's counter (``publish_to_peers`` in
``csrc/common/ptx.cuh``), so a consumer waits for ``world`` arrivals on a reduce-scatter counter and for one
arrival on each per-source all-gather counter, and a use costs ``world`` remote atomics per rank instead of
``CTAs x world``.  Peer counters only count up during a use and are zeroed between uses by a kernel that
the layer pipeline orders after their last reader and before their next writer (the norm kernel
that follows, see ``csrc/norm/norm.cu``); the local arrival counters are zeroed by the CTA that arrives last.  The counters are laid out so that each norm kernel's reset
set is one consecutive run: ``[ag0 x 8][rs1]`` and ``[ag1 x 8][rs0]``.  All device waits are bounded;
after a reported timeout call :meth:`reset` on every rank before the next step.

The reference has no collective or peer-memory code at all; the library baseline that this replaces
is ``TpContext.all_reduce`` (NCCL) in ``unillm_b200/engine/runner.py``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional

import torch

MAXR = 8
# counter indices (uint32 words) inside the flag area
AG0, RS1, AG1, RS0 = 0, 8, 16, 24
FLAG_WORDS = 512
AR_ROUND, AR_DONE = 44, 45               # one-shot all-reduce: exchanges completed, CTAs finished (both local)
AR_FLAGS = 64                            # ... and its 64 per-CTA arrival counters (words 64..127)
AR_ROWS = 32                             # token rows the one-shot all-reduce area holds (decode-sized messages)
ARGMAX_FLAG, ARGMAX_ROUND = 32, 33     # counter of the greedy merge and its (local) round word
LOCAL_RS0, LOCAL_RS1, LOCAL_AG0, LOCAL_AG1 = 40, 41, 42, 43   # local arrival counters of the producing launches
AR_CTA_ROUNDS, SG_CTA_ROUNDS = 192, 256  # per-CTA exchange counts of the two one-shot kernels (local, 64 words each)
SG_ROUND, SG_DONE = 49, 50               # pair gather of vocabulary-parallel sampling: exchanges completed, CTAs finished
SG_FLAGS = 128                           # ... and its 64 per-CTA arrival counters (words 128..191)
SG_PAIRS = 32768                         # (value, id) pairs per rank and exchange the gather area holds (rows x k)
DISP_FLAG, DISP_ROUND, LOCAL_DISP = 46, 47, 48   # sparse MoE dispatch: arrivals (peers), uses so far and CTA counter (local)
ARGMAX_ROWS = 2048                      # sampled rows per step the merge area can hold


@dataclass
class _Area:
    offset: int      # bytes from the start of the symmetric buffer
    nbytes: int


class FusedComm:
    def __init__(self, rank: int, world: int, hidden: int, max_tokens: int, buf: torch.Tensor, peer_ptrs: List[int],
                 handle=None, group=None, mc_ptr: int = 0, moe_top_k: int = 0, moe_experts: int = 0):
        self.rank, self.world, self.H = rank, world, hidden
        self.max_rows = (max_tokens + world - 1) // world
        self.buf, self.peer_ptrs, self.handle, self.group = buf, peer_ptrs, handle, group
        # address of the NVSwitch multicast view of the buffer (0: none).  With it the reduce-scatter becomes "every
        # rank keeps its partial rows in its own buffer, the owner reads them summed by the switch" and the all-gather
        # one multimem.st per 16 bytes instead of `world` peer stores.
        self.mc_ptr = mc_ptr
        self.multimem = bool(mc_ptr) and os.environ.get("UB_MULTIMEM", "1") != "0"
        # The reduce-scatter has two forms on a multicast heap.  "pull" (default): partial rows stay local and the owner
        # reads them summed by the switch, all of the NVLink time sits in the consumer.  "push" (UB_MULTIMEM_RS=0): the
        # GEMM epilogue stores rows into the owners' slots as its tiles finish, so the transfer overlaps the tiles
        # still being computed; the all-gather keeps its multicast stores either way.
        self.multimem_rs = self.multimem and os.environ.get("UB_MULTIMEM_RS", "1") != "0"
        self.heap = None
        slot = world * self.max_rows * hidden * 2
        self.rs = [_Area(0, slot), _Area(slot, slot)]
        self.ag = [_Area(2 * slot, slot), _Area(3 * slot, slot)]
        self.flags = _Area(4 * slot, FLAG_WORDS * 4)
        am = 2 * world * ARGMAX_ROWS * 4
        self.am_vals = _Area(4 * slot + FLAG_WORDS * 4, am)
        self.am_ids = _Area(4 * slot + FLAG_WORDS * 4 + am, am)
        self.ar_elems = AR_ROWS * hidden                       # bf16 elements per rank slot of the one-shot all-reduce
        self.ar_slots = _Area(self.am_ids.offset + am, 2 * world * self.ar_elems * 2)
        end0 = self.ar_slots.offset + self.ar_slots.nbytes
        sg = 2 * world * SG_PAIRS * 4
        self.sg_vals = _Area(end0, sg)
        self.sg_ids = _Area(end0 + sg, sg)
        # sparse expert-parallel MoE (F5 / F6): receive rows [world][cap][H] with their metadata and the count header,
        # and the combine area [K][rows][H]; sized for cap = max_rows * K
        self.moe_top_k, self.moe_experts = moe_top_k, moe_experts
        end = self.sg_ids.offset + self.sg_ids.nbytes
        if moe_top_k:
            pairs = world * self.max_rows * moe_top_k
            self.disp_rows = _Area(end, pairs * hidden * 2)
            self.disp_meta = _Area(self.disp_rows.offset + self.disp_rows.nbytes, pairs * 16)
            self.disp_counts = _Area(self.disp_meta.offset + self.disp_meta.nbytes, (max(moe_experts, 1) * 4 + 255) // 256 * 256)
            self.comb = _Area(self.disp_counts.offset + self.disp_counts.nbytes, moe_top_k * self.max_rows * hidden * 2)
        self.device = buf.device

    @staticmethod
    def nbytes(world: int, hidden: int, max_tokens: int, moe_top_k: int = 0, moe_experts: int = 0) -> int:
        rows = (max_tokens + world - 1) // world
        n = (4 * world * rows * hidden * 2 + FLAG_WORDS * 4 + 2 * (2 * world * ARGMAX_ROWS * 4) +
             2 * world * AR_ROWS * hidden * 2 + 2 * (2 * world * SG_PAIRS * 4))
        if moe_top_k:
            pairs = world * rows * moe_top_k
            n += pairs * hidden * 2 + pairs * 16 + (max(moe_experts, 1) * 4 + 255) // 256 * 256 + moe_top_k * rows * hidden * 2
        return n

    @staticmethod
    def _moe_shape(spec, world: int):
        """(top_k, experts) when the model's routed experts can be spread whole over ``world`` ranks, else (0, 0)."""
        m = getattr(spec, "moe", None)
        if m is None or world < 2 or m.num_experts % world or m.num_experts > 256:
            return 0, 0
        return m.top_k, m.num_experts

    @classmethod
    def create(cls, spec, rank: int, world: int, group, max_tokens: int, device, heap: Optional[str] = None) -> "FusedComm":
        """``heap``: "own" (the library's symmetric heap, multicast when available), "torch"
        (``torch.distributed._symmetric_memory``) or None = "own" with "torch" as the fallback when the own heap
        cannot be set up on this box; ``UB_SYMM_HEAP`` overrides.  All ranks take the same branch."""
        import torch.distributed as dist

        group = group if group is not None else dist.group.WORLD
        heap = os.environ.get("UB_SYMM_HEAP") or heap
        mk, me = cls._moe_shape(spec, world)
        n = cls.nbytes(world, spec.hidden_size, max_tokens, mk, me)
        if heap != "torch":
            from .symm_heap import SymmetricHeap

            ok, err, h = 1, "", None
            try:
                mc = None if os.environ.get("UB_MULTIMEM", "1") != "0" else False
                h = SymmetricHeap.create(n, rank, world, group, device, multicast=mc)
            except Exception as e:      # noqa: BLE001 - every rank has to learn about it and fall back together
                ok, err = 0, repr(e)[:200]
            # the agreement runs on the group's own kind of tensor (a gloo control group takes host tensors)
            flag = torch.tensor([ok], dtype=torch.int32, device=device if dist.get_backend(group) == "nccl" else "cpu")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if int(flag[0]) == 1:
                c = cls(rank, world, spec.hidden_size, max_tokens, h.tensor()[:n], list(h.peer_ptrs), None, group, h.mc_ptr,
                        moe_top_k=mk, moe_experts=me)
                c.heap = h
                return c
            if heap == "own":
                raise RuntimeError(f"own symmetric heap unavailable: {err or 'another rank failed'}")
            if h is not None:
                h._closed = True         # a partial set-up on this rank: leave it to process exit
        import torch.distributed._symmetric_memory as symm

        buf = symm.empty(n, dtype=torch.uint8, device=device)
        hd = symm.rendezvous(buf, group)
        buf.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group)
        return cls(rank, world, spec.hidden_size, max_tokens, buf, [int(p) for p in hd.buffer_ptrs], hd, group,
                   moe_top_k=mk, moe_experts=me)

    def close(self) -> None:
        """Collective: releases the own heap (multicast binding first); a no-op for the torch-backed buffer."""
        if self.heap is not None:
            self.heap.close()
            self.heap = None

    @classmethod
    def emulated(cls, world: int, hidden: int, max_tokens: int, device, moe_top_k: int = 0,
                 moe_experts: int = 0) -> List["FusedComm"]:
        """All ranks on ONE device (tests): plain buffers whose addresses stand in for peer mappings.  Kernels of
        different emulated ranks must then be launched producer-before-consumer on one stream."""
        n = cls.nbytes(world, hidden, max_tokens, moe_top_k, moe_experts)
        bufs = [torch.zeros(n, dtype=torch.uint8, device=device) for _ in range(world)]
        ptrs = [b.data_ptr() for b in bufs]
        return [cls(r, world, hidden, max_tokens, bufs[r], ptrs, moe_top_k=moe_top_k, moe_experts=moe_experts)
                for r in range(world)]

    # ---- address helpers ----
    def _peer(self, r: int, area: _Area, extra: int = 0) -> int:
        return self.peer_ptrs[r] + area.offset + extra

    def flag_ptr(self, r: int, word: int) -> int:
        return self.peer_ptrs[r] + self.flags.offset + 4 * word

    def local_flag_ptr(self, word: int) -> int:
        return self.buf.data_ptr() + self.flags.offset + 4 * word

    def rs_local(self, k: int) -> int:
        return self.buf.data_ptr() + self.rs[k].offset

    def ag_local_tensor(self, k: int, rows: int) -> torch.Tensor:
        a = self.ag[k]
        return self.buf[a.offset:a.offset + rows * self.H * 2].view(torch.bfloat16).view(rows, self.H)

    def rs_local_tensor(self, k: int, rows_per_rank: int) -> torch.Tensor:
        a = self.rs[k]
        n = self.world * rows_per_rank * self.H
        return self.buf[a.offset:a.offset + n * 2].view(torch.bfloat16).view(self.world, rows_per_rank, self.H)

    # ---- kernel argument dicts ----
    def gemm_rs(self, k: int, rows_per_rank: int) -> dict:
        """F1 producer arguments: push rows into rank ``owner``'s ``rs[k]`` slot of this rank."""
        # multicast mode: the partial rows stay in this rank's own rs[k] area (peer_out all null); the owners read them
        # summed through the multicast address
        outs = [0] * self.world if self.multimem_rs else [self._peer(r, self.rs[k]) for r in range(self.world)]
        return {"world": self.world, "rank": self.rank, "rows_per_rank": rows_per_rank, "peer_out": outs,
                "peer_flag": [self.flag_ptr(r, RS0 if k == 0 else RS1) for r in range(self.world)],
                "local_count": self.local_flag_ptr(LOCAL_RS0 if k == 0 else LOCAL_RS1), "local_out": self.rs_local(k)}

    def norm_rs(self, k: int, signals: int = 0, rows_per_rank: int = 0) -> dict:
        """F1 consumer arguments: wait for one arrival per source rank (``signals`` overrides the count), then sum the
        ``world`` slots of ``rs[k]`` -- or, in multicast mode, read this rank's ``rows_per_rank`` rows of the partial
        buffer through the multicast address (the switch sums the ranks' copies)."""
        d = {"world": self.world, "flag": self.local_flag_ptr(RS0 if k == 0 else RS1),
             "signals_per_use": signals or self.world}
        if self.multimem_rs:
            if rows_per_rank <= 0:
                raise ValueError("multicast reduce-scatter needs rows_per_rank")
            d["multimem_x"] = self.mc_ptr + self.rs[k].offset + self.rank * rows_per_rank * self.H * 2
        return d

    def norm_ag(self, k: int) -> dict:
        """F3 producer arguments: push normalised rows into every rank's ``ag[k]`` and bump their counter for us."""
        base = AG0 if k == 0 else AG1
        return {"world": self.world, "rank": self.rank,
                "peer_out": [self._peer(r, self.ag[k]) for r in range(self.world)],
                "peer_flag": [self.flag_ptr(r, base + self.rank) for r in range(self.world)],
                "local_count": self.local_flag_ptr(LOCAL_AG0 if k == 0 else LOCAL_AG1),
                "mc_out": (self.mc_ptr + self.ag[k].offset) if self.multimem else 0}

    def gemm_ag(self, k: int, rows_per_rank: int) -> dict:
        """F3 consumer arguments: the token rows of source rank ``s`` are ready when counter ``s`` shows its one arrival."""
        base = AG0 if k == 0 else AG1
        return {"world": self.world, "rows_per_rank": rows_per_rank, "flags": self.local_flag_ptr(base),
                "signals_per_use": 1}

    # ---- sparse expert-parallel MoE (F5 / F6) ----
    @property
    def has_moe_dispatch(self) -> bool:
        return bool(self.moe_top_k)

    def moe_dispatch_args(self) -> dict:
        """Send side of the dispatch: every rank's receive rows, metadata, count header and arrival counter."""
        W = self.world
        return {"world": W, "rank": self.rank,
                "peer_rows": [self._peer(r, self.disp_rows) for r in range(W)],
                "peer_meta": [self._peer(r, self.disp_meta) for r in range(W)],
                "peer_counts": [self._peer(r, self.disp_counts) for r in range(W)],
                "peer_flag": [self.flag_ptr(r, DISP_FLAG) for r in range(W)],
                "local_count": self.local_flag_ptr(LOCAL_DISP)}

    def moe_recv_args(self) -> dict:
        base = self.buf.data_ptr()
        return {"counts": base + self.disp_counts.offset, "meta": base + self.disp_meta.offset,
                "flag": self.local_flag_ptr(DISP_FLAG), "round": self.local_flag_ptr(DISP_ROUND)}

    def moe_recv_rows(self, rows: int) -> torch.Tensor:
        """This rank's receive buffer as ``[rows, H]`` (``rows = world * cap``)."""
        a = self.disp_rows
        return self.buf[a.offset:a.offset + rows * self.H * 2].view(torch.bfloat16).view(rows, self.H)

    def moe_return_args(self) -> dict:
        """Send side of the combine: every rank's combine area; arrivals count on the second reduce-scatter counter,
        which the norm kernels already zero between uses."""
        W = self.world
        return {"world": W, "peer_comb": [self._peer(r, self.comb) for r in range(W)],
                "peer_flag": [self.flag_ptr(r, RS1) for r in range(W)],
                "local_count": self.local_flag_ptr(LOCAL_RS1)}

    def moe_comb_tensor(self, rows_per_rank: int) -> torch.Tensor:
        """This rank's combine area as ``[K, rows_per_rank, H]``: slot k holds every own token's k-th expert output."""
        a = self.comb
        n = self.moe_top_k * rows_per_rank * self.H
        return self.buf[a.offset:a.offset + n * 2].view(torch.bfloat16).view(self.moe_top_k, rows_per_rank, self.H)

    def norm_comb(self) -> dict:
        """Consumer arguments for a norm kernel that sums the combine area: K slots, one arrival per rank."""
        return {"world": self.moe_top_k, "flag": self.local_flag_ptr(RS1), "signals_per_use": self.world}

    def reset_after_ag(self, k: int) -> tuple:
        """Counters a norm kernel may zero: the all-gather counters it does NOT feed plus the reduce-scatter
        counter it does NOT read -- ``k`` is the all-gather area this norm kernel pushes into."""
        # norm pushing into ag1 (post-attention) resets [ag0 x 8][rs1]; norm pushing into ag0 resets [ag1 x 8][rs0]
        base = AG0 if k == 1 else AG1
        return (self.local_flag_ptr(base), 9)

    def argmax_merge(self, vals: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
        """F4: global greedy winners from per-shard (value, id) pairs, exchanged through peer memory."""
        import ctypes as C

        from ..ops import _native as N
        from ..ops import cuda_ops

        rows = vals.numel()
        a = N.UbArgmaxMergeArgs()
        a.vals, a.ids, a.out_ids = vals.data_ptr(), ids.data_ptr(), out.data_ptr()
        for r in range(self.world):
            a.peer_vals[r] = self._peer(r, self.am_vals)
            a.peer_ids[r] = self._peer(r, self.am_ids)
            a.peer_flags[r] = self.flag_ptr(r, ARGMAX_FLAG)
        a.my_vals = self.buf.data_ptr() + self.am_vals.offset
        a.my_ids = self.buf.data_ptr() + self.am_ids.offset
        a.my_flag, a.round = self.local_flag_ptr(ARGMAX_FLAG), self.local_flag_ptr(ARGMAX_ROUND)
        a.world, a.rank, a.rows, a.max_rows = self.world, self.rank, rows, ARGMAX_ROWS
        a.err = cuda_ops.err_word(self.device).data_ptr()
        N.check(N.cuda_lib().ub_tp_argmax_merge(C.byref(a), torch.cuda.current_stream(self.device).cuda_stream),
                "ub_tp_argmax_merge")
        return out

    def all_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """F1s: in-place sum of a small contiguous bf16 tensor (at most ``AR_ROWS`` rows of the hidden size) over the
        ranks, through peer memory -- no NCCL call, capturable in a CUDA graph."""
        import ctypes as C

        from ..ops import _native as N
        from ..ops import cuda_ops

        n = t.numel()
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or n % 8 or n > self.ar_elems:
            raise ValueError("one-shot all-reduce takes a contiguous bf16 tensor of at most AR_ROWS x hidden elements")
        a = N.UbAllReduceArgs()
        a.in_, a.out = t.data_ptr(), t.data_ptr()
        for r in range(self.world):
            a.peer_slots[r] = self._peer(r, self.ar_slots)
            a.peer_flags[r] = self.flag_ptr(r, AR_FLAGS)
        a.my_slots = self.buf.data_ptr() + self.ar_slots.offset
        a.my_flags = self.local_flag_ptr(AR_FLAGS)
        a.round, a.done_count = self.local_flag_ptr(AR_ROUND), self.local_flag_ptr(AR_DONE)
        a.cta_rounds, a.max_n = self.local_flag_ptr(AR_CTA_ROUNDS), self.ar_elems
        a.world, a.rank, a.n = self.world, self.rank, n
        a.err = cuda_ops.err_word(self.device).data_ptr()
        N.check(N.cuda_lib().ub_allreduce_oneshot(C.byref(a), torch.cuda.current_stream(self.device).cuda_stream),
                "ub_allreduce_oneshot")
        return t

    def can_gather_pairs(self, rows: int, k: int) -> bool:
        return 0 < rows * k <= SG_PAIRS

    def gather_pairs(self, vals: torch.Tensor, ids: torch.Tensor):
        """F4s: ``vals`` / ``ids`` [rows, k] (fp32 / int32) of every rank -> ([rows, world * k], [rows, world * k]) in rank
        order, identical on every rank, through peer memory (no NCCL call)."""
        import ctypes as C

        from ..ops import _native as N
        from ..ops import cuda_ops

        rows, k = vals.shape
        if vals.dtype != torch.float32 or ids.dtype != torch.int32 or not vals.is_contiguous() or not ids.is_contiguous() \
                or not self.can_gather_pairs(rows, k):
            raise ValueError("gather_pairs takes contiguous fp32 / int32 [rows, k] with rows * k <= SG_PAIRS")
        ov = torch.empty(rows, self.world * k, dtype=torch.float32, device=self.device)
        oi = torch.empty(rows, self.world * k, dtype=torch.int32, device=self.device)
        a = N.UbPairGatherArgs()
        a.vals, a.ids, a.out_vals, a.out_ids = vals.data_ptr(), ids.data_ptr(), ov.data_ptr(), oi.data_ptr()
        for r in range(self.world):
            a.peer_vals[r] = self._peer(r, self.sg_vals)
            a.peer_ids[r] = self._peer(r, self.sg_ids)
            a.peer_flags[r] = self.flag_ptr(r, SG_FLAGS)
        a.my_vals = self.buf.data_ptr() + self.sg_vals.offset
        a.my_ids = self.buf.data_ptr() + self.sg_ids.offset
        a.my_flags = self.local_flag_ptr(SG_FLAGS)
        a.round, a.done_count = self.local_flag_ptr(SG_ROUND), self.local_flag_ptr(SG_DONE)
        a.cta_rounds = self.local_flag_ptr(SG_CTA_ROUNDS)
        a.world, a.rank, a.rows, a.k, a.cap = self.world, self.rank, rows, k, SG_PAIRS
        a.err = cuda_ops.err_word(self.device).data_ptr()
        lib = N.cuda_lib()
        lib.ub_pair_gather_oneshot.restype = C.c_int
        N.check(lib.ub_pair_gather_oneshot(C.byref(a), torch.cuda.current_stream(self.device).cuda_stream),
                "ub_pair_gather_oneshot")
        return ov, oi

    def can_all_reduce(self, t: torch.Tensor) -> bool:
        return t.dtype == torch.bfloat16 and t.is_contiguous() and t.numel() % 8 == 0 and t.numel() <= self.ar_elems

    def reset(self) -> None:
        """Zero all counters (host side); call on every rank, then barrier, after a reported device timeout."""
        a = self.flags
        self.buf[a.offset:a.offset + a.nbytes].zero_()
        torch.cuda.synchronize(self.device)
        if self.group is not None:
            import torch.distributed as dist

            dist.barrier(self.group)
