"""Rank failure detection, step watchdog, host-side fault injection and recovery planning.

The reference detects failures of requests only (time-outs, expiry, ``FinishReason::{Aborted,Error,Timeout}``,
``crates/inference/src/engine.rs:238-264``); it has no notion of a worker.  A multi-GPU engine needs one more layer:

* ``Heartbeat``: every rank bumps a counter in a key-value store (``torch.distributed.TCPStore`` or any object with
  ``set`` / ``get`` / ``add``) from a daemon thread and publishes the engine step it is at.  Observers judge a peer
  by the *local* time at which they last saw its counter change, so clocks of different hosts never get compared.
* ``StepWatchdog``: ranks must execute the same step sequence; a rank that falls more than ``max_lag`` steps behind
  or stops advancing while others wait is reported.
* ``FailureDetector``: combines both, plus the device error word that bounded waits of the fused kernels set (the
  kernels give up after a deadline and return a status instead of hanging).
* ``FaultInjector``: failures are made on the host only: muted heartbeats, a rank that raises or exits between steps,
  delayed control messages, a peer told not to signal (a launch parameter), allocator exhaustion.  Nothing here
  makes a GPU fault, trap or hang.
* ``RecoveryPlan``: what survives a failure is the request log (prompt + generated tokens); KV is recomputed.  The
  plan picks the next smaller tensor-parallel size the model supports and lists what to requeue.
"""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence


class RankFailure(RuntimeError):
    """Raised on the host of a rank that is told to fail, and by observers that found a dead peer."""

    def __init__(self, ranks: Sequence[int], reason: str):
        super().__init__(f"rank(s) {list(ranks)} failed: {reason}")
        self.ranks, self.reason = list(ranks), reason


class DictStore:
    """In-process stand-in for a TCPStore (single-process tests, world size 1)."""

    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k: str, v) -> None:
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k: str) -> bytes:
        with self._lock:
            return self._d[k]

    def add(self, k: str, n: int) -> int:
        with self._lock:
            v = int(self._d.get(k, b"0")) + n
            self._d[k] = str(v).encode()
            return v

    def check(self, keys: List[str]) -> bool:
        with self._lock:
            return all(k in self._d for k in keys)


def _get_int(store, key: str, default: int = -1) -> int:
    try:
        if hasattr(store, "check") and not store.check([key]):
            return default
        return int(store.get(key))
    except Exception:
        return default


@dataclass
class PeerView:
    counter: int = -1
    step: int = -1
    last_change: float = field(default_factory=time.monotonic)
    ever_seen: bool = False


class Heartbeat:
    def __init__(self, store, rank: int, world: int, interval: float = 0.2, timeout: float = 1.0, prefix: str = "hb",
                 startup_grace: float = 30.0):
        """``timeout``: a peer whose counter has not moved for this long is dead.  ``startup_grace``: a peer that has
        never published a beat yet (its process is still starting) is given this long before it counts as dead."""
        self.store, self.rank, self.world = store, rank, world
        self.interval, self.timeout, self.prefix = interval, timeout, prefix
        self.startup_grace = max(startup_grace, timeout)
        self.muted = False                      # fault injection: stop publishing
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._views = {r: PeerView() for r in range(world)}
        self._step = 0

    def _key(self, what: str, r: int) -> str:
        return f"{self.prefix}/{what}/{r}"

    def beat(self) -> None:
        if not self.muted:
            self.store.add(self._key("ctr", self.rank), 1)

    def set_step(self, step: int) -> None:
        self._step = step
        if not self.muted:
            self.store.set(self._key("step", self.rank), str(step))

    def start(self) -> "Heartbeat":
        self.beat()
        self.set_step(self._step)

        def loop():
            while not self._stop.wait(self.interval):
                try:
                    self.beat()
                except Exception:
                    return
        self._thread = threading.Thread(target=loop, daemon=True, name=f"heartbeat-{self.rank}")
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2 * self.interval + 1)

    def observe(self) -> Dict[int, PeerView]:
        now = time.monotonic()
        for r, v in self._views.items():
            c = _get_int(self.store, self._key("ctr", r))
            if c != v.counter:
                v.counter, v.last_change, v.ever_seen = c, now, v.ever_seen or c >= 0
            v.step = _get_int(self.store, self._key("step", r), v.step)
        return self._views

    def dead_ranks(self) -> List[int]:
        now = time.monotonic()
        return [r for r, v in self.observe().items() if r != self.rank and
                now - v.last_change > (self.timeout if v.ever_seen else self.startup_grace)]

    def steps(self) -> Dict[int, int]:
        return {r: v.step for r, v in self.observe().items()}


class StepWatchdog:
    """All ranks run the same step sequence; a rank more than ``max_lag`` steps behind the front is lagging, and a
    front that has not moved for ``stall_timeout`` seconds is a stall."""

    def __init__(self, hb: Heartbeat, max_lag: int = 2, stall_timeout: float = 5.0):
        self.hb, self.max_lag, self.stall_timeout = hb, max_lag, stall_timeout
        self._front, self._front_time = -1, time.monotonic()

    def lagging(self) -> List[int]:
        s = self.hb.steps()
        front = max(s.values())
        if front != self._front:
            self._front, self._front_time = front, time.monotonic()
        return [r for r, v in s.items() if front - v > self.max_lag]

    def stalled(self) -> bool:
        self.lagging()
        return time.monotonic() - self._front_time > self.stall_timeout


@dataclass
class HealthReport:
    healthy: bool
    dead: List[int] = field(default_factory=list)
    lagging: List[int] = field(default_factory=list)
    device_error: Optional[str] = None
    stalled: bool = False

    def status(self) -> str:
        if self.dead or self.device_error:
            return "unhealthy"
        return "degraded" if (self.lagging or self.stalled) else "healthy"


class FailureDetector:
    def __init__(self, hb: Heartbeat, watchdog: Optional[StepWatchdog] = None,
                 device_error_check: Optional[Callable[[], Optional[str]]] = None):
        self.hb, self.watchdog, self.device_error_check = hb, watchdog or StepWatchdog(hb), device_error_check

    def poll(self) -> HealthReport:
        dead = self.hb.dead_ranks()
        lag = [r for r in self.watchdog.lagging() if r not in dead]
        err = self.device_error_check() if self.device_error_check else None
        return HealthReport(not (dead or err), dead, lag, err, self.watchdog.stalled())

    def check(self) -> None:
        """Called between steps, before the next launch: raises if a peer is gone or a bounded device wait timed out."""
        rep = self.poll()
        if rep.dead:
            raise RankFailure(rep.dead, "no heartbeat")
        if rep.device_error:
            raise RankFailure([], f"device wait gave up: {rep.device_error}")


def cuda_error_word_check(device=None) -> Callable[[], Optional[str]]:
    """Adapter from the kernels' per-device error word to ``FailureDetector``: returns a description or None."""
    def check() -> Optional[str]:
        from ..ops import cuda_ops

        try:
            cuda_ops.check_device_errors(device)
        except RuntimeError as e:
            return str(e)
        return None
    return check


class FaultInjector:
    """Host-side failures for tests and drills."""

    def __init__(self, hb: Optional[Heartbeat] = None):
        self.hb = hb
        self.fail_step: Optional[int] = None
        self.exit_step: Optional[int] = None
        self.delay_s = 0.0
        self.skip_signal = False          # passed to fused launches: this rank's kernels do not bump peer counters
        self.alloc_fail_after: Optional[int] = None
        self._allocs = 0

    def mute_heartbeat(self, on: bool = True) -> None:
        if self.hb is not None:
            self.hb.muted = on

    def fail_at_step(self, step: int) -> None:
        self.fail_step = step

    def exit_at_step(self, step: int) -> None:
        self.exit_step = step

    def delay_control(self, seconds: float) -> None:
        self.delay_s = seconds

    def exhaust_allocator_after(self, n: int) -> None:
        self.alloc_fail_after = n

    def on_alloc(self) -> bool:
        """True if this allocation should be refused."""
        self._allocs += 1
        return self.alloc_fail_after is not None and self._allocs > self.alloc_fail_after

    def before_step(self, step: int, rank: int) -> None:
        """Engine hook between steps (no kernels or collectives of this rank are in flight here)."""
        if self.delay_s:
            time.sleep(self.delay_s)
        if self.fail_step is not None and step >= self.fail_step:
            self.mute_heartbeat()
            raise RankFailure([rank], "injected failure")
        if self.exit_step is not None and step >= self.exit_step:
            self.mute_heartbeat()
            raise SystemExit(17)


@dataclass
class RecoveryPlan:
    survivors: List[int]
    new_world: int
    new_ranks: Dict[int, int]                    # old rank -> new rank for the ranks that stay
    requeue: List[dict] = field(default_factory=list)

    @staticmethod
    def make(world: int, dead: Iterable[int], num_heads: int, num_kv_heads: int, requests: Iterable[dict] = ()) -> "RecoveryPlan":
        """Largest tensor-parallel size <= survivors that divides the head counts (KV heads may also be replicated when
        the size is a multiple of them)."""
        dead = set(dead)
        survivors = [r for r in range(world) if r not in dead]
        n = len(survivors)
        size = 0
        for cand in range(n, 0, -1):
            if num_heads % cand == 0 and (num_kv_heads % cand == 0 or cand % num_kv_heads == 0):
                size = cand
                break
        keep = survivors[:size]
        reqs = [dict(prompt=list(r["prompt"]) + list(r.get("output", [])), done=len(r.get("output", [])),
                     max_tokens=r["max_tokens"] - len(r.get("output", [])), id=r.get("id"))
                for r in requests if r["max_tokens"] - len(r.get("output", [])) > 0]
        return RecoveryPlan(survivors, size, {old: new for new, old in enumerate(keep)}, reqs)
