"""Recovery that runs: a tensor-parallel serving loop that notices a dead rank between steps, re-forms a smaller
group from the survivors and finishes the requests there.

What survives a failure is the request log -- prompts and the tokens generated so far (``LLMEngine.snapshot``); KV
is recomputed.  The loop on every rank:

  1. before each step, ``StepGate.wait`` publishes "I am at step k" in the store and returns once every live rank
     has published it; a rank whose heartbeat has stopped raises ``RankFailure`` here, i.e. on the host and BEFORE
     the step's collectives are issued (a collective is never started with a peer known to be gone);
  2. the engine step (the same deterministic ``LLMEngine`` on every rank);
  3. on ``RankFailure`` (or a collective that ended with an error because the peer died inside it): take the
     snapshot, compute ``RecoveryPlan`` -- the largest tensor-parallel size the surviving ranks and the head counts
     allow --, leave the old process group, rendezvous with the other survivors under a new store prefix
     (``gen<N>``), rebuild runner and engine at the new size through the caller's ``build_engine`` and ``restore``
     the snapshot.  Survivors that the smaller group has no place for return with ``role == "spare"``.

The reference has no notion of a worker (only request time-outs, ``crates/inference/src/engine.rs:238-264``), so
there is no counterpart; the recovery contract (requeue prompt + generated tokens, drop KV and the radix tree) is
the one a multi-GPU engine needs.  Failures are made on the host only (``FaultInjector``); the loop itself is
device-agnostic and is exercised with gloo ranks on the CPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from .health import FailureDetector, FaultInjector, Heartbeat, RankFailure, RecoveryPlan, StepWatchdog, _get_int


class StepGate:
    """Host-side rendezvous before a step: every rank publishes the step it is about to run and waits until all live
    ranks have published it.  A dead peer (heartbeat) ends the wait with ``RankFailure``."""

    def __init__(self, store, rank: int, ranks: List[int], detector: FailureDetector, prefix: str = "gate",
                 poll_s: float = 0.001, timeout_s: float = 60.0):
        self.store, self.rank, self.ranks, self.det = store, rank, list(ranks), detector
        self.prefix, self.poll_s, self.timeout_s = prefix, poll_s, timeout_s

    def wait(self, step: int) -> None:
        self.store.set(f"{self.prefix}/{self.rank}", str(step))
        t0 = time.monotonic()
        while True:
            self.det.check()
            if all(_get_int(self.store, f"{self.prefix}/{r}") >= step for r in self.ranks):
                return
            if time.monotonic() - t0 > self.timeout_s:
                late = [r for r in self.ranks if _get_int(self.store, f"{self.prefix}/{r}") < step]
                raise RankFailure(late, f"did not reach step {step} within {self.timeout_s:.0f} s")
            time.sleep(self.poll_s)


@dataclass
class ElasticResult:
    role: str                                   # "finished" | "spare" | "exited"
    outputs: Dict[int, List[int]] = field(default_factory=dict)
    generations: int = 1                        # process groups this rank has been part of
    final_world: int = 0
    final_rank: int = -1
    recovered_from: List[List[int]] = field(default_factory=list)   # dead ranks of every recovery
    steps: int = 0


def serve_elastic(rank: int, world: int, store, build_engine: Callable[[int, int, object], object],
                  requests: List[dict], *, num_heads: int, num_kv_heads: int, hb_interval: float = 0.05,
                  hb_timeout: float = 1.0, injector: Optional[FaultInjector] = None, backend: str = "gloo",
                  collective_timeout_s: float = 10.0, max_generations: int = 4) -> ElasticResult:
    """Runs ``requests`` (dicts with ``id``, ``prompt``, ``params`` = ``SamplingParams``) to completion on the ranks
    ``0..world-1`` that share ``store``, surviving rank failures as described in the module docstring.

    ``build_engine(rank_in_group, group_size, process_group)`` returns a fresh ``LLMEngine`` for that layout.
    ``rank`` / ``world`` are the ORIGINAL numbering: heartbeats, the step gate and the injector use it throughout."""
    import datetime

    import torch.distributed as dist

    hb = Heartbeat(store, rank, world, interval=hb_interval, timeout=hb_timeout).start()
    inj = injector or FaultInjector(hb)
    inj.hb = hb
    res = ElasticResult("finished")
    members = list(range(world))                 # original ranks of the current group, in group-rank order
    snapshot = None
    try:
        for gen in range(max_generations):
            if rank not in members:
                res.role = "spare"
                return res
            g_rank, g_world = members.index(rank), len(members)
            pg_store = dist.PrefixStore(f"gen{gen}", store)
            dist.init_process_group(backend, store=pg_store, rank=g_rank, world_size=g_world,
                                    timeout=datetime.timedelta(seconds=collective_timeout_s))
            group = dist.group.WORLD
            res.generations, res.final_world, res.final_rank = gen + 1, g_world, g_rank
            dead: List[int] = []
            try:
                eng = build_engine(g_rank, g_world, group)
                if snapshot is None:
                    for r in requests:
                        eng.add_request(r["prompt"], r["params"], seq_id=r["id"])
                else:
                    eng.restore(snapshot)
                # only the members of this group are watched from here on
                det = FailureDetector(_MemberView(hb, members), StepWatchdog(hb, max_lag=1 << 30))
                gate = StepGate(store, rank, members, det, prefix=f"gate{gen}")
                step = 0
                while eng.has_unfinished():
                    inj.before_step(res.steps, rank)          # may raise SystemExit / RankFailure on this rank
                    hb.set_step(res.steps)
                    gate.wait(step)
                    try:
                        eng.step()
                    except RankFailure:
                        raise
                    except RuntimeError as e:                 # a collective that lost its peer mid-flight
                        time.sleep(hb_timeout + 2 * hb_interval)
                        gone = [r for r in hb.dead_ranks() if r in members]
                        if not gone:
                            raise
                        raise RankFailure(gone, f"collective failed: {str(e)[:80]}")
                    step += 1
                    res.steps += 1
                res.outputs = {sid: list(s.output_ids) for sid, s in eng.seqs.items()}
                return res
            except RankFailure as e:
                dead = [r for r in e.ranks if r in members]
                if rank in dead or not dead:
                    raise
                snapshot = eng.snapshot()
                res.recovered_from.append(dead)
            finally:
                try:
                    dist.destroy_process_group()
                except Exception:
                    pass
            plan = RecoveryPlan.make(len(members), [members.index(r) for r in dead], num_heads, num_kv_heads)
            if plan.new_world == 0:
                raise RankFailure(dead, "no tensor-parallel size fits the surviving ranks")
            keep = sorted(plan.new_ranks, key=plan.new_ranks.get)          # group ranks that stay, in their new order
            members = [members[i] for i in keep]
        raise RankFailure([], f"gave up after {max_generations} process groups")
    except SystemExit:
        res.role = "exited"
        return res
    finally:
        hb.stop()


class _MemberView:
    """A ``Heartbeat`` restricted to the members of the current group (ranks that already left are not reported again)."""

    def __init__(self, hb: Heartbeat, members: List[int]):
        self._hb, self._members = hb, set(members)
        self.rank, self.world = hb.rank, hb.world

    def dead_ranks(self) -> List[int]:
        return [r for r in self._hb.dead_ranks() if r in self._members]

    def steps(self) -> Dict[int, int]:
        return {r: s for r, s in self._hb.steps().items() if r in self._members}

    def observe(self):
        return self._hb.observe()
