"""Data-parallel replicas: several independent engines (each possibly tensor-parallel) behind one router.

When ``world / tp > 1`` the GPUs form ``world / tp`` replica groups; every request goes to the least-loaded
replica (fewest unfinished tokens), and a replica's radix cache is preferred when it already holds the request's
prefix.  The reference has no notion of replicas (``ScheduleInfo.gpu_id`` is always 0,
``crates/scheduler/src/intelligent_scheduler.rs:709-716``).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

from ..sampling import SamplingParams


def replica_groups(world: int, tp: int) -> List[List[int]]:
    """Ranks of each replica: consecutive blocks of ``tp`` ranks (NVSwitch makes every grouping equivalent)."""
    if tp <= 0 or world % tp != 0:
        raise ValueError(f"world {world} is not a multiple of the tensor-parallel size {tp}")
    return [list(range(g * tp, (g + 1) * tp)) for g in range(world // tp)]


class ReplicaRouter:
    def __init__(self, engines: Sequence, prefix_affinity: bool = True):
        if not engines:
            raise ValueError("at least one engine")
        self.engines = list(engines)
        self.prefix_affinity = prefix_affinity
        self._where: Dict[int, Tuple[int, int]] = {}     # global id -> (replica, local id)
        self._next = 0

    def load(self, i: int) -> int:
        e = self.engines[i]
        return sum(s.total_len + s.params.max_tokens - len(s.output_ids) for s in list(e.running) + list(e.waiting))

    def _cached(self, i: int, prompt: Sequence[int]) -> int:
        e = self.engines[i]
        if e.radix is None or len(prompt) < 2:
            return 0
        blocks, _ = e.radix.match_prefix(list(prompt[:-1]))
        return len(blocks) * e.block_size

    def pick(self, prompt: Sequence[int]) -> int:
        loads = [self.load(i) for i in range(len(self.engines))]
        if self.prefix_affinity:
            hits = [self._cached(i, prompt) for i in range(len(self.engines))]
            best_hit = max(hits)
            if best_hit > 0:
                # a cached prefix is worth its tokens of prefill work, as long as the replica is not far busier
                cands = [i for i, h in enumerate(hits) if h == best_hit]
                i = min(cands, key=lambda j: loads[j])
                if loads[i] - min(loads) <= 4 * best_hit:
                    return i
        return min(range(len(loads)), key=lambda j: loads[j])

    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None, priority: int = 0) -> int:
        i = self.pick(prompt)
        local = self.engines[i].add_request(prompt, params, priority)
        gid = self._next
        self._next += 1
        self._where[gid] = (i, local)
        return gid

    def has_unfinished(self) -> bool:
        return any(e.has_unfinished() for e in self.engines)

    def step(self) -> List[Tuple[int, object]]:
        """One step of every replica that has work; returns (global id, StepOutput) pairs."""
        back = {v: k for k, v in self._where.items()}
        outs = []
        for i, e in enumerate(self.engines):
            if e.has_unfinished():
                for o in e.step():
                    outs.append((back[(i, o.seq_id)], o))
        return outs

    def run_to_completion(self) -> Dict[int, List[int]]:
        while self.has_unfinished():
            self.step()
        return {gid: self.engines[i].seqs[local].output_ids for gid, (i, local) in self._where.items()}
