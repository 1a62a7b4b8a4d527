"""Multi-GPU runtime: fused compute+collective plumbing (``fused``), rank health / recovery (``health``), launch
helpers (``launch``)."""
from .health import (DictStore, FailureDetector, FaultInjector, Heartbeat, HealthReport, RankFailure, RecoveryPlan,
                     StepWatchdog)
