"""``LLMEngine``: the iteration-level serving loop -- request queue, continuous batching with chunked
prefill, radix prefix reuse over the paged block pool, preemption by recomputation, and one call into a
model runner per step.

The reference has the pieces but never connects them: its scheduler forms batches once
(``crates/scheduler/src/lib.rs:271-323``), its KV crate only does bookkeeping and its engine sleeps
instead of running a model (``crates/inference/src/engine.rs:322-379``).  Here every step:

  1. running sequences that finished prefill get one decode token each (a new block when they cross a
     block boundary; if the pool is empty the radix tree evicts unlocked leaves, then the youngest
     running sequence is preempted and later recomputed);
  2. the remaining token budget goes to prefill chunks -- first to sequences already in flight, then to
     waiting requests in policy order, whose longest cached prefix (whole blocks) is taken from the radix
     tree instead of being recomputed;
  3. blocks that this step fills completely are published to the radix tree at scheduling time, so a
     request admitted in the same step can already share them (the KV append of every layer runs before
     that layer's attention);
  4. the runner executes the packed step and returns one sampled token per finished prefill / decode row.

With ``async_scheduling`` the host runs one step ahead of the device: step N + 1 is scheduled, packed and launched
while step N executes.  Lengths and block tables of N + 1 do not depend on the token values of N, so the engine
appends a placeholder per sampled sequence, lets the runner feed the sampled ids from device memory into the
next step, and reads the real values one step later.  Finishes by length are known in advance; a stop token is
noticed one step late (that sequence's extra row is dropped).  Preemption, abort and snapshot first wait for
the step in flight.

Every rank of a tensor-parallel group runs this loop on the same request stream and takes identical
decisions (it is deterministic), so no per-step control traffic is needed.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable, Deque, Dict, List, Optional, Sequence, Tuple

from ..kv.block_pool import BlockPool, RadixTree
from ..sampling import SamplingParams
from ..types import InvalidInput, MemoryError_
from .runner import DeviceStepError, StepBatch

WAITING, RUNNING, FINISHED, ABORTED = "waiting", "running", "finished", "aborted"


@dataclass(eq=False)
class Sequence:
    seq_id: int
    prompt_ids: List[int]
    params: SamplingParams
    priority: int = 0
    arrival: float = field(default_factory=time.perf_counter)
    output_ids: List[int] = field(default_factory=list)
    blocks: List[int] = field(default_factory=list)
    num_computed: int = 0            # tokens whose KV is in the cache
    num_cached: int = 0              # of those, how many came from the radix tree
    published_blocks: int = 0        # leading blocks already offered to the radix tree
    radix_node: int = 0
    status: str = WAITING
    finish_reason: Optional[str] = None
    first_token_time: Optional[float] = None
    finish_time: Optional[float] = None
    token_times: List[float] = field(default_factory=list)
    preemptions: int = 0
    pending_src: int = -1            # sample index, in the step in flight, of the token that output_ids[pending_at] awaits
    pending_at: int = -1
    _blocks_np: Optional[object] = field(default=None, repr=False)

    def blocks_array(self):
        """Block table as an int32 array (the packer copies rows from it); every change of ``blocks`` drops it."""
        c = self._blocks_np
        if c is None or len(c) != len(self.blocks):
            import numpy as np

            c = self._blocks_np = np.asarray(self.blocks, dtype=np.int32)
        return c

    @property
    def tokens(self) -> List[int]:
        return self.prompt_ids + self.output_ids

    @property
    def total_len(self) -> int:
        return len(self.prompt_ids) + len(self.output_ids)

    @property
    def prefill_done(self) -> bool:
        return self.num_computed >= self.total_len - 1 and len(self.output_ids) > 0


@dataclass
class StepOutput:
    seq_id: int
    token: int
    finished: bool
    finish_reason: Optional[str] = None


@dataclass
class EngineStats:
    steps: int = 0
    prefill_tokens: int = 0
    decode_tokens: int = 0
    cached_tokens: int = 0
    preemptions: int = 0
    finished: int = 0
    generated_tokens: int = 0
    device_errors: int = 0           # steps dropped because a kernel reported a problem in the device error word


class LLMEngine:
    def __init__(self, runner, *, num_blocks: int, block_size: int = 16, max_num_seqs: int = 256,
                 max_num_batched_tokens: int = 8192, max_model_len: int = 8192, enable_prefix_caching: bool = True,
                 enable_chunked_prefill: bool = True, eos_token_id: Optional[int] = None,
                 policy: Optional[Callable[[List[Sequence]], List[Sequence]]] = None, seed: int = 0,
                 async_scheduling: bool = False):
        self.runner = runner
        self.block_size = block_size
        self.pool = BlockPool(num_blocks, block_size)
        self.radix = RadixTree(self.pool) if enable_prefix_caching else None
        self.max_num_seqs, self.max_tokens, self.max_model_len = max_num_seqs, max_num_batched_tokens, max_model_len
        self.chunked = enable_chunked_prefill
        self.eos_token_id = eos_token_id
        self.policy = policy
        self.seed = seed
        self.waiting: Deque[Sequence] = deque()
        self.running: List[Sequence] = []
        self.seqs: Dict[int, Sequence] = {}
        self._next_id = 0
        self.stats = EngineStats()
        self.async_scheduling = async_scheduling
        self._inflight = None       # (plan, runner handle) of the launched step whose samples are not read yet
        self._late: List[StepOutput] = []   # outputs of a step that had to be waited for outside ``step``
        self.max_device_errors = 3  # consecutive failed steps after which the error is raised to the caller
        self._consecutive_errors = 0
        self.step_events = None     # optional (start, end) CUDA events recorded around the runner launch
        self.tracer = None          # optional unillm_b200.utils.Tracer: spans around schedule / launch / fetch / process

    # ------------------------------------------------------------------------------------------
    def add_request(self, prompt_ids: Sequence[int], params: Optional[SamplingParams] = None, priority: int = 0,
                    seq_id: Optional[int] = None) -> int:
        if len(prompt_ids) == 0:
            raise InvalidInput("empty prompt")
        params = params or SamplingParams()
        if len(prompt_ids) + params.max_tokens > self.max_model_len:
            raise InvalidInput(f"prompt ({len(prompt_ids)}) + max_tokens ({params.max_tokens}) exceeds "
                               f"max_model_len {self.max_model_len}")
        sid = self._next_id if seq_id is None else seq_id
        self._next_id = max(self._next_id, sid) + 1
        s = Sequence(sid, list(prompt_ids), params, priority)
        self.seqs[sid] = s
        self.waiting.append(s)
        return sid

    def abort(self, seq_id: int) -> bool:
        s = self.seqs.get(seq_id)
        if s is None or s.status in (FINISHED, ABORTED):
            return False
        self._late.extend(self._drain())
        if s.status in (FINISHED, ABORTED):
            return False
        if s.status == RUNNING:
            self.running.remove(s)
        else:
            self.waiting.remove(s)
        self._release(s, publish=False)
        s.status, s.finish_reason, s.finish_time = ABORTED, "aborted", time.perf_counter()
        return True

    def has_unfinished(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None or self._late)

    # ------------------------------------------------------------------------------------------
    # block management
    # ------------------------------------------------------------------------------------------
    def _alloc(self, n: int) -> Optional[List[int]]:
        if n <= 0:
            return []
        got = self.pool.try_allocate(n)
        if got is None and self.radix is not None:
            self.radix.evict(n - self.pool.num_free())
            got = self.pool.try_allocate(n)
        return got

    def _release(self, s: Sequence, publish: bool) -> None:
        if publish and self.radix is not None:
            self._publish(s, s.num_computed)
        for b in s.blocks:
            self.pool.free(b)
        s.blocks = []
        s._blocks_np = None
        if self.radix is not None and s.radix_node:
            self.radix.unlock(s.radix_node)
        s.radix_node = 0
        s.published_blocks = 0

    def _publish(self, s: Sequence, upto_tokens: int) -> None:
        """Offer the blocks that are completely filled by the first ``upto_tokens`` tokens to the radix tree."""
        nb = min(upto_tokens // self.block_size, len(s.blocks))
        if self.radix is None or nb <= s.published_blocks:
            return
        self.radix.insert(s.tokens[: nb * self.block_size], s.blocks[:nb])
        s.published_blocks = nb

    def _preempt_one(self, keep: Sequence) -> bool:
        """Free the blocks of the youngest running sequence other than ``keep``; it is recomputed later."""
        if self._inflight is not None:
            # a preempted sequence is recomputed from its token list: all of its tokens must be known first
            self._late.extend(self._drain())
        for cand in reversed(self.running):
            if cand is not keep and cand.status == RUNNING:
                self.running.remove(cand)
                self._release(cand, publish=True)
                cand.num_computed = cand.num_cached = 0
                cand.status = WAITING
                cand.preemptions += 1
                self.stats.preemptions += 1
                self.waiting.appendleft(cand)
                return True
        return False

    def _ensure_blocks(self, s: Sequence, upto_tokens: int) -> bool:
        need = (upto_tokens + self.block_size - 1) // self.block_size - len(s.blocks)
        while need > 0:
            got = self._alloc(need)
            if got is not None:
                s.blocks.extend(got)
                s._blocks_np = None
                return True
            if not self._preempt_one(s):
                return False
        return True

    # ------------------------------------------------------------------------------------------
    # scheduling
    # ------------------------------------------------------------------------------------------
    def _admit(self, s: Sequence) -> None:
        """Look up the longest cached prefix of a waiting sequence and take references on its blocks."""
        s.blocks, s.num_computed, s.num_cached, s.published_blocks = [], 0, 0, 0
        s._blocks_np = None
        if self.radix is None:
            return
        toks = s.tokens
        blocks, node = self.radix.match_prefix(toks[: len(toks) - 1])   # at least one token is always computed
        if blocks:
            for b in blocks:
                self.pool.incref(b)
            self.radix.lock(node)
            s.blocks = list(blocks)
            s._blocks_np = None
            s.radix_node = node
            s.num_computed = s.num_cached = len(blocks) * self.block_size
            s.published_blocks = len(blocks)

    def schedule(self) -> Tuple[Optional[StepBatch], List[Tuple[Sequence, int, bool]]]:
        """Returns the packed step and, per scheduled sequence, (sequence, tokens this step, samples?)."""
        bs = self.block_size
        decode: List[Sequence] = []
        # membership in self.running is the same thing as status == RUNNING (preemption flips the status)
        for s in list(self.running):
            if s.status != RUNNING or not s.prefill_done:
                continue                      # includes sequences preempted while making room for an earlier one
            if s.pending_src >= 0 and (len(s.output_ids) >= s.params.max_tokens or s.total_len >= self.max_model_len):
                continue                      # its last token is in flight; it finishes when that step is read
            if not self._ensure_blocks(s, s.total_len):
                continue
            decode.append(s)
        decode = [s for s in decode if s.status == RUNNING]
        in_decode = {id(s) for s in decode}
        budget = self.max_tokens - len(decode)
        chunks: List[Tuple[Sequence, int]] = []
        for s in list(self.running):
            if s.status != RUNNING or budget <= 0 or id(s) in in_decode or s.prefill_done:
                continue
            left = s.total_len - s.num_computed
            n = min(left, budget) if self.chunked else left
            if n <= 0 or n > budget:
                continue
            if self._ensure_blocks(s, s.num_computed + n):
                chunks.append((s, n))
                budget -= n
        # making room may have preempted sequences that were already picked above
        decode = [s for s in decode if s.status == RUNNING]
        chunks = [(s, n) for s, n in chunks if s.status == RUNNING]
        budget = self.max_tokens - len(decode) - sum(n for _, n in chunks)
        # from here on nothing is preempted, so blocks filled by this step can be published now
        for s, n in chunks:
            self._publish(s, s.num_computed + n)
        order = list(self.waiting)
        if self.policy is not None:
            order = self.policy(order)
        for s in order:
            if budget <= 0 or len(self.running) >= self.max_num_seqs:
                break
            self._admit(s)
            remaining = s.total_len - s.num_computed
            n = min(remaining, budget) if self.chunked else remaining
            if n > budget or not self._ensure_blocks_no_preempt(s, s.num_computed + n):
                self._release(s, publish=False)
                s.num_computed = s.num_cached = 0
                break
            self.waiting.remove(s)
            s.status = RUNNING
            self.running.append(s)
            self.stats.cached_tokens += s.num_cached
            chunks.append((s, n))
            budget -= n
            self._publish(s, s.num_computed + n)
        if not decode and not chunks:
            return None, []
        token_ids: List[int] = []
        positions: List[int] = []
        slots: List[int] = []
        seq_lens: List[int] = []
        tables: List[List[int]] = []
        sample_rows: List[int] = []
        plan: List[Tuple[Sequence, int, bool]] = []
        token_src: Optional[List[int]] = None
        if decode:
            positions = [len(s.prompt_ids) + len(s.output_ids) - 1 for s in decode]
            if self._inflight is not None:
                token_src = [s.pending_src for s in decode]
                token_ids = [0 if s.pending_src >= 0 else s.output_ids[-1] for s in decode]
            else:
                token_ids = [s.output_ids[-1] for s in decode]
            slots = [s.blocks[p // bs] * bs + p % bs for s, p in zip(decode, positions)]
            seq_lens = [p + 1 for p in positions]
            tables = [s.blocks_array() for s in decode]
            sample_rows = list(range(len(decode)))
            plan = [(s, 1, True) for s in decode]
        q_lens: List[int] = []
        for s, n in chunks:
            a, b = s.num_computed, s.num_computed + n
            npr = len(s.prompt_ids)
            if b <= npr:
                token_ids.extend(s.prompt_ids[a:b])
            else:
                token_ids.extend(s.tokens[a:b])
            positions.extend(range(a, b))
            blk = s.blocks
            slots.extend([blk[p // bs] * bs + p % bs for p in range(a, b)])
            seq_lens.append(s.num_computed + n)
            tables.append(s.blocks_array())
            q_lens.append(n)
            done = s.num_computed + n >= s.total_len
            if done:
                sample_rows.append(len(token_ids) - 1)
            plan.append((s, n, done))
        shared = self._shared_prefix(decode) if len(decode) >= 8 else 0
        # prefill chunks can join the shared-prefix pass when they start at or after the prefix and reuse its blocks
        nshared = shared // bs
        pfx_ok = bool(chunks) and shared > 0 and all(
            s.num_computed >= shared and s.blocks[:nshared] == decode[0].blocks[:nshared] for s, _ in chunks)
        sampled = [s for s, _, smp in plan if smp]
        greedy = all(s.params.greedy for s in sampled)
        batch = StepBatch(token_ids, positions, slots, len(decode), seq_lens, tables, q_lens, sample_rows, shared,
                          prefill_shares_prefix=pfx_ok, seed=self.seed, step=self.stats.steps, token_src=token_src)
        if not greedy:
            batch.temperature = [s.params.temperature for s in sampled]
            batch.top_p = [s.params.top_p for s in sampled]
            batch.top_k = [s.params.top_k or 0 for s in sampled]
        return batch, plan

    def _ensure_blocks_no_preempt(self, s: Sequence, upto_tokens: int) -> bool:
        need = (upto_tokens + self.block_size - 1) // self.block_size - len(s.blocks)
        if need <= 0:
            return True
        got = self._alloc(need)
        if got is None:
            return False
        s.blocks.extend(got)
        s._blocks_np = None
        return True

    def _shared_prefix(self, decode: List[Sequence]) -> int:
        """Number of leading tokens (whole blocks) whose blocks are identical in all decode sequences."""
        first = decode[0].blocks
        n = min(min(len(s.blocks) for s in decode), min((s.total_len - 1) // self.block_size for s in decode))
        for s in decode:
            if n == 0:
                break
            if s.blocks[:n] != first[:n]:          # list slices compare at C speed; shrink only on mismatch
                k = 0
                while k < n and s.blocks[k] == first[k]:
                    k += 1
                n = k
        return n * self.block_size

    # ------------------------------------------------------------------------------------------
    # stepping
    # ------------------------------------------------------------------------------------------
    def step(self) -> List[StepOutput]:
        tr = self.tracer
        if tr is None:
            return self._step()
        with tr.span("engine.step"):
            return self._step(tr)

    def _step(self, tr=None) -> List[StepOutput]:
        if tr is not None:
            with tr.span("engine.schedule"):
                batch, plan = self.schedule()
        else:
            batch, plan = self.schedule()
        if batch is None:
            outs = self._late + self._drain()
            self._late = []
            if not outs and self.waiting and not self.running:
                raise MemoryError_("a waiting request does not fit in the KV cache even when it is empty")
            return outs
        ev = self.step_events
        if ev is not None:
            ev[0].record()
        if tr is not None:
            with tr.span("engine.launch", tokens=len(batch.token_ids), decode=batch.num_decode):
                self.runner.launch(batch)
        else:
            self.runner.launch(batch)
        if ev is not None:
            ev[1].record()
            self.step_events = None          # consumed: a caller that times steps sets a fresh pair per step
        if not self.async_scheduling:
            if tr is not None:
                with tr.span("engine.fetch"):
                    ids = self._fetch(None)
                if ids is None:
                    return []
                with tr.span("engine.process"):
                    return self._finalize(self._advance(plan), ids)
            ids = self._fetch(None)
            if ids is None:
                return []
            return self._finalize(self._advance(plan), ids)
        # one step ahead: this step is in flight; read the one launched before it
        prev = self._inflight
        self._inflight = (self._advance(plan), self.runner.pending())
        outs, self._late = self._late, []
        if prev is not None:
            if tr is not None:
                with tr.span("engine.fetch"):
                    ids = self._fetch(prev[1])
                if ids is not None:
                    with tr.span("engine.process"):
                        outs.extend(self._finalize(prev[0], ids))
            else:
                ids = self._fetch(prev[1])
                if ids is not None:
                    outs.extend(self._finalize(prev[0], ids))
        return outs

    def _fetch(self, handle) -> Optional[List[int]]:
        """Sampled ids of a launched step, or None when the device reported an error for it: then the step's
        results are dropped and every running sequence is queued for recomputation (``_on_device_error``)."""
        try:
            ids = self.runner.fetch(handle) if handle is not None else self.runner.fetch()
        except DeviceStepError as e:
            self._on_device_error(e)
            return None
        self._consecutive_errors = 0
        return ids

    def _on_device_error(self, exc: DeviceStepError) -> None:
        """A bounded device wait gave up or an index was out of range: nothing the failed step (or the step launched
        after it, which consumed its samples) produced can be trusted.  Their tokens are dropped, the KV blocks of all
        running sequences go back to the pool WITHOUT being offered to the prefix cache, the cache itself is emptied
        (blocks were published at scheduling time), and the sequences wait to be prefilled again from their token
        history.  The runner clears the error word and, under tensor parallelism, the arrival counters on every rank.
        The reference only has request time-outs (``crates/inference/src/engine.rs:238-264``)."""
        self.stats.device_errors += 1
        self._consecutive_errors += 1
        self._inflight = None
        reset = getattr(self.runner, "reset_after_error", None)
        if reset is not None:
            reset()
        for s in self.running:
            while s.output_ids and s.output_ids[-1] < 0:      # placeholders of the dropped steps
                s.output_ids.pop()
            s.pending_src = s.pending_at = -1
            self._release(s, publish=False)
            s.num_computed = s.num_cached = 0
            s.status = WAITING
        self.waiting.extendleft(reversed(self.running))
        self.running = []
        if self.radix is not None:
            self.radix.clear()
        if self._consecutive_errors > self.max_device_errors:
            raise exc

    def flush(self) -> List[StepOutput]:
        """Outputs of the step still in flight under ``async_scheduling`` (empty otherwise); afterwards every token
        launched so far has been read back."""
        outs, self._late = self._late + self._drain(), []
        return outs

    def _drain(self) -> List[StepOutput]:
        """Waits for the step in flight (if any) and applies its results."""
        prev, self._inflight = self._inflight, None
        if prev is None:
            return []
        ids = self._fetch(prev[1])
        return [] if ids is None else self._finalize(prev[0], ids)

    def _advance(self, plan) -> List[Tuple[Sequence, int, bool, int]]:
        """Bookkeeping that does not need the sampled values: computed lengths move on and every sampled sequence
        gets a placeholder token.  Returns the plan with the placeholder's index in ``output_ids``."""
        self.stats.steps += 1
        out = []
        k = 0
        for s, n, sampled in plan:
            s.num_computed += n
            if n == 1 and len(s.output_ids) > 0 and sampled:
                self.stats.decode_tokens += 1
            else:
                self.stats.prefill_tokens += n
            at = -1
            if sampled:
                at = len(s.output_ids)
                s.output_ids.append(-1)
                s.pending_src, s.pending_at = k, at
                k += 1
            out.append((s, n, sampled, at))
        return out

    def _finalize(self, plan, ids: List[int]) -> List[StepOutput]:
        now = time.perf_counter()
        outs: List[StepOutput] = []
        k = 0
        for s, n, sampled, at in plan:
            if not sampled:
                continue
            tok = int(ids[k])
            k += 1
            if s.status != RUNNING:
                continue                  # stopped or aborted while this row was already in flight
            s.output_ids[at] = tok
            if s.pending_at == at:
                s.pending_src = s.pending_at = -1
            s.token_times.append(now)
            if s.first_token_time is None:
                s.first_token_time = now
            self.stats.generated_tokens += 1
            reason = None
            p = s.params
            if not p.ignore_eos and self.eos_token_id is not None and tok == self.eos_token_id:
                reason = "stop"
            elif tok in p.stop_token_ids:
                reason = "stop"
            elif at + 1 >= p.max_tokens:
                reason = "length"
            elif len(s.prompt_ids) + at + 1 >= self.max_model_len:
                reason = "length"
            if reason is not None:
                del s.output_ids[at + 1:]          # a placeholder of the step launched meanwhile
                s.pending_src = s.pending_at = -1
                s.num_computed = min(s.num_computed, s.total_len)
                s.status, s.finish_reason, s.finish_time = FINISHED, reason, now
                self.running.remove(s)
                self._release(s, publish=True)
                self.stats.finished += 1
            outs.append(StepOutput(s.seq_id, tok, reason is not None, reason))
        return outs

    def run_to_completion(self, max_steps: int = 1 << 30) -> Dict[int, List[int]]:
        n = 0
        while self.has_unfinished() and n < max_steps:
            self.step()
            n += 1
        return {sid: s.output_ids for sid, s in self.seqs.items()}

    def generate(self, prompts: Sequence[Sequence[int]], params: Optional[SamplingParams] = None) -> List[List[int]]:
        ids = [self.add_request(p, params) for p in prompts]
        self.run_to_completion()
        return [self.seqs[i].output_ids for i in ids]

    # ------------------------------------------------------------------------------------------
    # snapshot / restore: the request log is the durable state, KV is recomputed
    # ------------------------------------------------------------------------------------------
    def snapshot(self) -> dict:
        """JSON-serialisable state of every unfinished request (prompt, tokens generated so far, sampling settings)
        plus the finished ones' outputs.  The KV cache and the radix tree are not saved: after ``restore`` the
        engine prefills prompt + generated tokens again (greedy requests then continue with identical tokens)."""
        import dataclasses

        self._late.extend(self._drain())
        reqs = []
        for s in self.seqs.values():
            reqs.append({"id": s.seq_id, "prompt": list(s.prompt_ids), "output": list(s.output_ids), "priority": s.priority,
                         "params": dataclasses.asdict(s.params), "status": s.status, "finish_reason": s.finish_reason})
        return {"version": 1, "next_id": self._next_id, "eos_token_id": self.eos_token_id, "seed": self.seed,
                "stats": dataclasses.asdict(self.stats), "requests": reqs}

    def restore(self, snap: dict) -> List[int]:
        """Re-creates the requests of ``snapshot()`` in a fresh engine; returns the ids that were requeued."""
        if snap.get("version") != 1:
            raise InvalidInput("unknown snapshot version")
        if self.seqs:
            raise InvalidInput("restore needs an engine without requests")
        self.eos_token_id = snap.get("eos_token_id", self.eos_token_id)
        requeued = []
        for r in snap["requests"]:
            params = SamplingParams(**r["params"])
            s = Sequence(r["id"], list(r["prompt"]), params, r.get("priority", 0))
            s.output_ids = list(r["output"])
            self.seqs[s.seq_id] = s
            if r["status"] in (FINISHED, ABORTED):
                s.status, s.finish_reason = r["status"], r.get("finish_reason")
                continue
            if s.output_ids:
                # decode again from the full token history: the last generated token is the next input
                s.num_computed = 0
            self.waiting.append(s)
            requeued.append(s.seq_id)
        self._next_id = max(snap.get("next_id", 0), max(self.seqs, default=-1) + 1)
        return requeued
